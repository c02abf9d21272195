#!/usr/bin/env python
"""Benchmark of the activation-compression hot path on B200.

  python bench.py --gpus N --steps K --warmup W            this library (CUDA kernels, C ABI)
  python bench.py --impl reference --gpus N --steps K ...   the reference's own implementation of the path: its
                                                            unmodified CUDA kernels (built into oracle/_ref/) in
                                                            the reference's op chain on one GPU; without them, the
                                                            CPU restatement of its math on the host cores
  python bench.py --workload cfg3 --n_bits 4 --kept_frac 0.25   the reference drivers' knobs (--n_bits, --kept_frac,
                                                            --act_fp: mem_speed_bench/arxiv/train_full_batch.py:44-48)

Metric: full-batch GNN epoch/s (the reference's own throughput definition,
mem_speed_bench/arxiv/train_full_batch.py:251-267: one epoch = zero_grad, forward, loss, backward,
optimizer step over the whole graph).  Default workload: the 3-layer GraphSAGE on a synthetic
2,449,029-node power-law graph, INT2 activations with kept_frac 0.125 -- the configuration the
1/2/4/8-GPU scaling is quoted on; node rows are partitioned across the N ranks (strong scaling).
One JSON line is printed by rank 0; it also carries the pack / unpack kernel bandwidths against the
HBM roofline, the roofline of the dominant kernel, the CPU baseline and the end-to-end (host buffers)
number.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per edge and operand column, from one ncu capture of
# each SpMM entry point on a case a few GB small: the kernel sweep's R-MAT graph of 1,200,000 nodes / 62.9 M edges
# (operand 10x larger than L2), all launches of one call added (row kernel, long-row pieces, their reduction).
#   K = 256 (128-column tiles):              9.98 GB per call  -> 0.62 bytes per edge and column
#   K = 32 (narrow-operand kernel, routed):  0.80 GB per call  -> 0.40 bytes per edge and column
# `traffic` of the roofline block is this figure times the edges x columns of an average launch of the run: an
# estimate that assumes DRAM bytes grow with the gathered volume once the operand is far larger than L2 (a
# capture of the full 2.45 M-node graph gave 0.64 for K = 256).
SPMM_DRAM_BYTES_PER_EDGE_COLUMN = {"exact_spmm_split": 0.62, "exact_spmm": 0.62, "exact_spmm_split_routed": 0.40}


def apply_knobs(c, args):
    """The reference drivers' command-line knobs onto a workload and the global config
    (mem_speed_bench/arxiv/train_full_batch.py:120-137): --act_fp turns activation compression off but keeps the
    random projection when --kept_frac < 1; otherwise activations are saved at --n_bits with --kept_frac."""
    from exact_b200 import config
    c = dict(c)
    if args.n_bits is not None:
        c["bits"] = args.n_bits
    if args.kept_frac is not None:
        c["kept_frac"] = args.kept_frac
    if args.no_compress:          # comparison run of this benchmark: no compression and no projection
        c["kept_frac"] = 1.0
    act_fp = bool(args.act_fp or args.no_compress)
    # train_full_batch.py:123-129: fp32 activations without projection train the unwrapped model
    c["use_qmodule"] = not (act_fp and c["kept_frac"] == 1.0)
    config.compress_activation = not act_fp
    config.activation_compression_bits = [c["bits"]]
    config.kept_frac = c["kept_frac"]
    c["act_fp"] = act_fp
    return c


def workload_name(c, nodes):
    prec = "fp32act" if c.get("act_fp") else f"int{c['bits']}"
    return (f"{c['model']}{c['layers']}_{nodes}n_{c['feats']}f_{c['hidden']}h_{c['classes']}c_{prec}"
            f"_kf{c['kept_frac']}")


def packed_stream_sha256(packed, world, rank, dev):
    """SHA-256 of a packed activation stream over all ranks in row order (rank 0 returns the digest, the others
    None).  Row shards are multiples of 8 rows, so the concatenation of the shards' streams is the stream a
    single GPU produces; each shard's last byte is the one the reference allocates and never writes."""
    import hashlib

    import torch
    import torch.distributed as dist
    if packed is None:
        return None
    body = packed.view(torch.uint8)[:-1].contiguous()
    if world == 1:
        return hashlib.sha256(body.cpu().numpy().tobytes()).hexdigest()
    sizes = torch.zeros(world, dtype=torch.int64, device=dev)
    sizes[rank] = body.numel()
    dist.all_reduce(sizes)
    sizes = [int(v) for v in sizes.tolist()]
    pad = torch.zeros(max(sizes), dtype=torch.uint8, device=dev)
    pad[:body.numel()] = body
    allb = torch.empty(world * max(sizes), dtype=torch.uint8, device=dev)
    dist.all_gather_into_tensor(allb, pad)
    if rank != 0:
        return None
    h = hashlib.sha256()
    host = allb.cpu().numpy()
    for r in range(world):
        h.update(host[r * max(sizes):r * max(sizes) + sizes[r]].tobytes())
    return h.hexdigest()


# ----------------------------------------------------------------------------------------------------
def run_b200(args):
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import exact_b200
    from exact_b200 import QModule, _lib, config, graphs, models
    from exact_b200 import dist as xdist
    from exact_b200.cpp_extension import quantization as Q

    rank, world, local = xdist.init_process_group_from_env()
    assert world == args.gpus or world == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = torch.device("cuda", local)
    c = apply_knobs(graphs.CONFIGS[args.workload], args)
    nodes = args.nodes or c["nodes"]
    hbm_peak, peak_kind = measured_peaks()

    # ---- synthetic inputs (same seed on every rank) --------------------------------------------------
    t0 = time.time()
    full = graphs.build_graph(c, seed=0, device=dev, nodes=None if nodes == c["nodes"] else nodes)
    if c["gcn_norm"]:
        full = exact_b200.gcn_norm(full, add_self_loops=False)
    n = full.size(0)
    nnz = full.nnz()
    reduce = "mean" if c["model"] == "sage" else "sum"
    if world > 1:
        adj = xdist.shard_graph(full, reduce, rank, world)
        r0, r1 = adj.row_start, adj.row_end
    else:
        full.fill_cache_()
        full.to_int32_()
        full.storage.transposed(reduce)   # the SpMM backward's structure, built once
        adj, r0, r1 = full, 0, n
        config.row_offset = 0
    del full
    torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(1)
    # features live in pinned host memory (the end-to-end leg copies them in every step); every rank draws the
    # whole matrix from the same seed and keeps its rows, so that every world size trains on the same data
    x_host = torch.empty((r1 - r0, c["feats"]), dtype=torch.float32).pin_memory()
    gd = torch.Generator(device=dev).manual_seed(1)
    x_dev = torch.randn((n, c["feats"]), device=dev, generator=gd)[r0:r1].clone()
    torch.cuda.empty_cache()
    x_host.copy_(x_dev)
    y = torch.randint(c["classes"], (n,), generator=g)[r0:r1].to(dev)
    torch.manual_seed(0)
    cls = models.GCN if c["model"] == "gcn" else models.SAGE
    config.manual_seed(0)
    config.compact_gather = not args.dense_gather
    config.compact_operand = not args.dense_gather
    config.peer_exchange = not args.no_peer_exchange
    config.column_split_aggregation = False if args.row_split else (True if args.column_split else None)
    config.routed_aggregation_output = bool(args.routed_output)
    if args.min_slice_columns is not None:
        config.aggregation_min_slice_columns = args.min_slice_columns
    if args.result_chunks is not None:
        config.aggregation_result_chunks = args.result_chunks
    config.cache_constant_gather = False   # every timed step exchanges its input features again
    net = cls(c["feats"], c["hidden"], c["classes"], c["layers"], dropout=c["dropout"], batch_norm=c["batch_norm"])
    net = (QModule(net) if c["use_qmodule"] else net).to(dev).train()
    opt = torch.optim.Adam(net.parameters(), lr=0.002)
    params = list(net.parameters())
    setup_s = time.time() - t0

    def step(x):
        opt.zero_grad(set_to_none=True)
        out = net(x, adj)
        # per-row losses summed by a parallel reduction (the fused "sum" reduction of nll_loss runs in one block)
        loss = F.cross_entropy(out, y, reduction="none").sum() / n
        loss.backward()
        xdist.allreduce_gradients(params)
        opt.step()
        return loss

    def global_loss(loss):
        """The loss over all rows (each rank holds the sum over its own, already divided by n)."""
        t = loss.detach().clone()
        if world > 1:
            dist.all_reduce(t)
        return t

    # ---- evidence that every world size trains the same model: the first compressed activation of the
    # first step (INT2 codes of layer 1's projected input) hashed over all ranks in row order, and the loss
    first = {}

    def grab(quantized, randmat):
        if "packed" not in first and quantized[1] is not None:
            first["packed"] = quantized[0].detach().clone()

    config.quantized_hook = grab
    loss0 = global_loss(step(x_dev))
    config.quantized_hook = None
    stream_sha = packed_stream_sha256(first.get("packed"), world, rank, dev)
    loss0 = float(loss0.item())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident leg ---------------------------------------------------------------------
    for _ in range(max(args.warmup - 1, 0)):   # the step above was the first warm-up step
        step(x_dev)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.LAUNCHES
    _lib.LIBRARY_CALLS.clear()
    _lib.TIMER = _lib.KernelTimer()
    torch.cuda.reset_peak_memory_stats(dev)
    timed_losses = []
    ms = timed(lambda: timed_losses.append(step(x_dev)), args.steps)
    # torch's allocator plus the exchange buffers the library allocates itself for the peers to write into
    peak_mem = torch.cuda.max_memory_allocated(dev) + xdist.PeerBuffers.peak_allocated_bytes
    loss_first = float(global_loss(timed_losses[0]).item())
    loss_last = float(global_loss(timed_losses[-1]).item())
    del timed_losses
    exact_b200.check_status(dev, force=True)
    ksum = _lib.TIMER.summary()
    _lib.TIMER = None
    launches = _lib.LAUNCHES - launches0
    library_calls = {k: round(v / args.steps, 2) for k, v in sorted(_lib.LIBRARY_CALLS.items())}

    # ---- end-to-end leg: features come from pinned host memory, the loss goes back to the host ------
    # Every step copies its features host -> device and reads its loss back.  The copy of step i+1 runs on a
    # second stream while step i computes (two device buffers), as an input pipeline would do it; the first
    # copy and every later one lie inside the timed region.
    bufs = [torch.empty_like(x_dev), torch.empty_like(x_dev)]
    copy_stream = torch.cuda.Stream(device=dev)
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    freed = [torch.cuda.Event(), torch.cuda.Event()]
    state = {"i": 0, "primed": False}

    def issue_copy(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[slot])      # the step that last read this buffer has finished
            bufs[slot].copy_(x_host, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_step():
        slot = state["i"] & 1
        if not state["primed"]:
            issue_copy(slot)
            state["primed"] = True
        issue_copy(slot ^ 1)                          # next step's features, overlapping this step
        torch.cuda.current_stream().wait_event(ready[slot])
        loss = step(bufs[slot])
        freed[slot].record(torch.cuda.current_stream())
        state["i"] += 1
        return loss.item()

    for e in freed:
        e.record(torch.cuda.current_stream())
    e2e_step()
    _lib.HOST_CLOCK = [0, 0]
    ms_e2e = timed(e2e_step, args.steps)
    host_ns, host_calls = _lib.HOST_CLOCK
    _lib.HOST_CLOCK = None
    clocks = sampler.stop() if rank == 0 else None

    # ---- pack / unpack kernels against the HBM roofline (first half of the metric) -------------------
    kern = {}
    if rank == 0 and not args.no_kernels:
        kern = kernel_bandwidths(torch, Q, _lib, dev, hbm_peak, workload_shape=(r1 - r0, c["hidden"]))

    exchange = "none"
    if world > 1:
        exchange = adj.describe_exchange() + ", input features exchanged every step"
        adj.close()
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    roofline = roofline_of_dominant_kernel(ksum, ms, args.steps, hbm_peak, peak_kind)
    cpu = None
    if args.gpus == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(c, args.cpu_nodes)
    value = args.steps / (ms * 1e-3)
    line = {
        "metric": "full_batch_gnn_epoch_per_s", "value": round(value, 4), "unit": "epoch/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(c, n), "nodes": n, "directed_edges": nnz, "parallelism": f"rows/{world}",
                   "activations": "uncompressed (comparison run)" if args.no_compress else "compressed",
                   "exchange": exchange,
                   "l2": "inputs larger than L2" if n * c["hidden"] * 4 > 126e6 else "working set fits L2",
                   "setup_s": round(setup_s, 1)},
        "e2e": {"value": round(args.steps / (ms_e2e * 1e-3), 4), "unit": "epoch/s",
                "h2d_bytes_per_step": x_host.numel() * 4 * world, "d2h_bytes_per_step": 4 * world},
        "gpu_launches": launches,
        "loss_first": loss_first, "loss_last": loss_last, "loss_step0": loss0, "packed_stream_sha256": stream_sha,
        "peak_device_memory_GB": round(peak_mem / 1e9, 2),   # rank 0, device-resident leg (graph, features, training state)
        "kernel_ms_per_step": {k: round(v["ms"] / args.steps, 3) for k, v in sorted(ksum.items())},
        "library_gemm_calls_per_step": library_calls,
        # host side of this library's calls during the end-to-end leg (rank 0): the binding plus the C entry point
        # (argument checks, descriptor encoding, launch), not the device time
        "host": {"calls_per_step": round(host_calls / args.steps, 1),
                 "us_per_call": round(host_ns / max(host_calls, 1) / 1e3, 2),
                 "ms_per_step": round(host_ns / args.steps / 1e6, 3)},
        "roofline": roofline, "kernels": kern, "cpu_baseline": cpu, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def roofline_of_dominant_kernel(ksum, ms_total, steps, hbm_peak, peak_kind):
    """Roofline block for the entry point with the most device time in the timed region.

    HBM-bound kernels: `achieved` = bytes that must cross HBM at least once (the operand in the form the kernel
    reads it, the indices, the output) / mean launch time, so that `frac` cannot exceed 1 by counting cache hits;
    for the gathers `l2_side_GB/s` gives the bytes requested from L2 when no source row is reused (the
    reference's kernel moves exactly those).  The dense-layer GEMM is tensor-bound: tf32 flop issued (three
    MMAs per product) against half the measured bf16 peak."""
    if not ksum:
        return None
    name, r = max(ksum.items(), key=lambda kv: kv[1]["ms"])
    per_ms = r["ms"] / r["launches"]
    sec = per_ms * 1e-3
    common = {"kernel": name, "launches_per_step": r["launches"] / steps, "ms_per_launch": round(per_ms, 4),
              "share_of_step": round(r["ms"] / ms_total, 4)}
    if name == "exact_linear_forward":
        peak = None
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak = float(json.load(f)["bf16_tflops_sustained"]) / 2.0
            kind = "measured bf16 sustained / 2 (tf32 runs at half the bf16 rate)"
        except Exception:
            peak, kind = 1400.0 / 2.0, "fallback bf16 sustained / 2"
        achieved = r["flops"] / r["launches"] / sec / 1e12
        return dict(common, bound="tensor", achieved=round(achieved, 1), peak=peak, peak_kind=kind, unit="TFLOP/s",
                    frac=round(achieved / peak, 4), traffic=None,
                    flops_model="6*M*K*N tf32 flop per call: every fp32 product is three tf32 MMAs (head*head, "
                                "tail*head, head*tail)")
    achieved = r["bytes"] / r["launches"] / sec / 1e9
    out = dict(common, bound="hbm", achieved=round(achieved, 1), peak=hbm_peak, peak_kind=peak_kind, unit="GB/s",
               frac=round(achieved / hbm_peak, 4))
    if name.startswith("exact_spmm"):
        out["l2_side_GB/s"] = round(r["l2_bytes"] / r["launches"] / sec / 1e9, 1)
        per = SPMM_DRAM_BYTES_PER_EDGE_COLUMN.get(name)
        units = r.get("edge_columns", 0) / r["launches"]
        out["traffic"] = None if per is None or not units else round(per * units)
        out["traffic_GB/s"] = None if out["traffic"] is None else round(out["traffic"] / sec / 1e9, 1)
        out["traffic_note"] = ("DRAM bytes per edge and column measured by ncu on a 1.2 M-node case of the kernel "
                               "sweep, times the edges x columns of an average launch here")
        out["bytes_model"] = "operand rows + indices + output, each once"
    else:
        out["traffic"] = None
    return out


def _pack_unpack_fractions(torch, Q, dev, hbm_peak, N, D, reps):
    out = {}
    gen = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(N, D, device=dev, generator=gen).relu_()
    for bits in (1, 2, 4, 8):
        pk, sb, mb = Q.quantize_pack(x, bits, seed=1, offset=0)
        pack_bytes = N * D * 4 + (pk.numel() - 1) + 4 * N
        unpack_bytes = (pk.numel() - 1) + 4 * N + N * D * 4
        for kind, call, nbytes in (("pack", lambda: Q.quantize_pack(x, bits, seed=1, offset=0), pack_bytes),
                                   ("unpack", lambda: Q.unpack_single_precision(pk, bits, sb, mb, N, D), unpack_bytes)):
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                call()
            b.record()
            torch.cuda.synchronize()
            gbs = nbytes * reps / (a.elapsed_time(b) * 1e-3) / 1e9
            out[f"{kind}_int{bits}"] = {"GB/s": round(gbs, 1), "frac": round(gbs / hbm_peak, 4)}
    out["shape"] = f"{N}x{D} fp32"
    return out


def reference_kernel_times(torch, dev, hbm_peak, reps):
    """The reference's own unmodified CUDA kernels (oracle/_ref/, checker side) timed on this GPU beside this
    library's: pack_single_precision + the two torch reductions that feed it (what quantize_activation runs,
    exact/exact/ops.py:61-83), unpack_single_precision, and spmm_mean_fw on a 300,000-node R-MAT graph with
    K = 256.  Same algorithmic byte counts as the lines above.  None when oracle/_ref/ is not built."""
    try:
        from oracle import ref_chain as RC
        if not RC.available():
            return None
        rq, rs = RC._mods()
    except Exception:
        return None
    from exact_b200 import graphs
    from exact_b200.cpp_extension import spmm as S

    def timeit(call, n):
        for _ in range(2):
            call()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            call()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e-3 / n

    out = {}
    N, D = 1_000_000, 128
    gen = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(N, D, device=dev, generator=gen).relu_()
    for bits in (1, 2, 4, 8):
        q = RC.quantize_activation(x, bits)
        G = q[0].numel() - 1
        sec_p = timeit(lambda: RC.quantize_activation(x, bits), max(reps // 2, 5))
        sec_u = timeit(lambda: RC.dequantize_activation(q, (N, D)), max(reps // 2, 5))
        gp, gu = (N * D * 4 + G + 4 * N) / sec_p / 1e9, (G + 4 * N + N * D * 4) / sec_u / 1e9
        out[f"quantize_activation_int{bits}"] = {"GB/s": round(gp, 1), "frac": round(gp / hbm_peak, 4)}
        out[f"dequantize_activation_int{bits}"] = {"GB/s": round(gu, 1), "frac": round(gu / hbm_peak, 4)}
    out["shape"] = f"{N}x{D} fp32"
    del x, q
    nodes, K = 300_000, 256
    adj = graphs.rmat(nodes, int(nodes * 50 / 2), 0, dev, self_loops=False)
    rowptr, col, _ = adj.csr()
    xs = torch.randn(nodes, K, device=dev, generator=gen)
    sec_ref = timeit(lambda: rs.spmm_mean_fw(None, rowptr, col, None, None, None, None, xs), 5)
    r32, c32 = rowptr.to(torch.int32), col.to(torch.int32)
    sec_own = timeit(lambda: S._spmm(r32, c32, None, xs, "mean"), 5)
    ref_out = rs.spmm_mean_fw(None, rowptr, col, None, None, None, None, xs)
    own_out = S._spmm(r32, c32, None, xs, "mean")
    short = (rowptr[1:] - rowptr[:-1]) <= 256     # rows one warp sums in CSR order in both kernels
    out["spmm_mean_rmat300k_K256"] = {
        "reference_ms": round(sec_ref * 1e3, 4), "this_library_ms": round(sec_own * 1e3, 4),
        "rows_up_to_256_edges_equal_bitwise": bool(torch.equal(ref_out[short], own_out[short])),
        "edges": int(col.numel())}
    return out


def kernel_bandwidths(torch, Q, _lib, dev, hbm_peak, N=1_000_000, D=128, reps=20, workload_shape=None):
    """Achieved GB/s of the fused quantise+pack and of unpack+dequantise, INT{1,2,4,8}, fp32 in, on a
    10^6 x 128 activation (512 MB: larger than L2) and on the workload's own hidden-activation shape, CUDA
    events on the launching stream."""
    out = _pack_unpack_fractions(torch, Q, dev, hbm_peak, N, D, reps)
    if workload_shape is not None:
        out["workload_shape"] = _pack_unpack_fractions(torch, Q, dev, hbm_peak, workload_shape[0], workload_shape[1],
                                                       max(reps // 2, 5))
    gen = torch.Generator(device=dev).manual_seed(4)
    # the two tensor-core kernels of the projection pair at 10^6 x 256 <-> k = 32, INT2
    from exact_b200.ops import _rademacher
    N2, D2, k2 = 1_000_000, 256, 32
    x2 = torch.randn(N2, D2, device=dev, generator=gen)
    R = _rademacher(D2, k2, dev, torch.float32, seed=1, offset=0)
    pk, sb, mb = Q.rp_quantize_pack(x2, R, 2, seed=1, offset=1)
    cases = (("rp_pack_int2_256to32", lambda: Q.rp_quantize_pack(x2, R, 2, seed=1, offset=1),
              N2 * D2 * 4 + D2 * k2 * 4 + (pk.numel() - 1) + 4 * N2),
             ("unpack_rp_int2_32to256", lambda: Q.unpack_dequant_rp(pk, 2, sb, mb, N2, R),
              (pk.numel() - 1) + 4 * N2 + D2 * k2 * 4 + N2 * D2 * 4))
    for name, call, nbytes in cases:
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            call()
        b.record()
        torch.cuda.synchronize()
        sec = a.elapsed_time(b) * 1e-3 / reps
        out[name] = {"GB/s": round(nbytes / sec / 1e9, 1), "frac": round(nbytes / sec / 1e9 / hbm_peak, 4),
                     "TFLOP/s": round(2.0 * N2 * D2 * k2 / sec / 1e12, 1)}
    del x2, pk
    ref = reference_kernel_times(torch, dev, hbm_peak, reps)
    if ref is not None:
        out["ref_cuda"] = ref
    # the dense-layer GEMM (tf32 head/tail split, three MMAs per tile) against the library's fp32 GEMM
    from exact_b200.cpp_extension import backward_func as B
    M3, K3, N3 = 1_000_000, 256, 256
    a3 = torch.randn(M3, K3, device=dev, generator=gen)
    w3 = torch.randn(N3, K3, device=dev, generator=gen)
    times = {}
    for name, call in (("tc", lambda: B.linear_forward(a3, w3)), ("lib", lambda: torch.nn.functional.linear(a3, w3))):
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            call()
        b.record()
        torch.cuda.synchronize()
        times[name] = a.elapsed_time(b) * 1e-3 / reps
    out["linear_tf32x3_1Mx256x256"] = {"ms": round(times["tc"] * 1e3, 4), "library_fp32_ms": round(times["lib"] * 1e3, 4),
                                       "fp32_equiv_TFLOP/s": round(2.0 * M3 * K3 * N3 / times["tc"] / 1e12, 1),
                                       "tensor_TFLOP/s": round(6.0 * M3 * K3 * N3 / times["tc"] / 1e12, 1)}
    return out


# ----------------------------------------------------------------------------------------------------
def cpu_epoch(c, nodes, steps, warmup):
    """Times the CPU restatement (oracle/ + torch CPU GEMMs) of one training epoch on a graph of
    `nodes` nodes with the workload's mean degree; returns seconds per step."""
    import torch

    import oracle
    from oracle import gnn as O
    from exact_b200 import graphs, gcn_norm, models

    oracle.build()
    torch.set_num_threads(os.cpu_count())
    adj = graphs.build_graph(c, seed=0, device="cpu", nodes=nodes)
    if c["gcn_norm"]:
        adj = gcn_norm(adj, add_self_loops=False)
    n = adj.size(0)
    rowptr, col, val = adj.csr()
    adj_np = (rowptr.numpy(), col.numpy(), None if val is None else val.numpy())
    g = torch.Generator().manual_seed(1)
    x = torch.randn(n, c["feats"], generator=g)
    y = torch.randint(c["classes"], (n,), generator=g)
    torch.manual_seed(0)
    cls = models.GCN if c["model"] == "gcn" else models.SAGE
    ref_model = cls(c["feats"], c["hidden"], c["classes"], c["layers"], dropout=c["dropout"], batch_norm=c["batch_norm"])
    params = {}
    for k, v in ref_model.state_dict().items():
        if "running" in k or "num_batches" in k:
            continue
        params[k] = v.t().contiguous() if (c["model"] == "gcn" and k.endswith("weight") and v.dim() == 2) else v
    cfg = O.Cfg(c["bits"], c["kept_frac"], True, seed=0)
    times = []
    for i in range(warmup + steps):
        t = time.perf_counter()
        O.train_step(cfg, c["model"], params, x, adj_np, y, c["layers"], c["batch_norm"], c["dropout"])
        if i >= warmup:
            times.append(time.perf_counter() - t)
    return sum(times) / len(times), n, adj.nnz()


def cpu_baseline(c, cpu_nodes):
    """The CPU restatement timed on two bounded samples (the second half the size of the first), so that the
    scaling to the full graph by node count is checked rather than assumed."""
    sec, n, nnz = cpu_epoch(c, cpu_nodes, steps=1, warmup=1)
    sec2, n2, _ = cpu_epoch(c, cpu_nodes // 2, steps=1, warmup=1)
    scale = c["nodes"] / n
    return {"value": round(1.0 / (sec * scale), 6), "unit": "epoch/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"one epoch on a {n}-node / {nnz}-edge graph of the same mean degree took {sec:.2f} s on the "
                      f"host ({sec2:.2f} s at {n2} nodes: {sec / sec2:.2f}x the time for {n / n2:.2f}x the nodes); "
                      f"scaled by {scale:.1f}x nodes to the full graph"}


def reference_gpu_epoch(c, nodes, steps, warmup):
    """Seconds per training step of the reference's own op chain on cuda:0 (oracle/ref_chain.py: the reference's
    unmodified pack / unpack / SpMM kernels, torch.min/max, torch.matmul, F.linear, Adam), same graph, features,
    labels and model shape as this library's arm.  SAGE workloads only."""
    import torch
    import torch.nn.functional as F

    from oracle import ref_chain as RC
    from exact_b200 import graphs, models

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    full = graphs.build_graph(c, seed=0, device=dev, nodes=None if nodes == c["nodes"] else nodes)
    n = full.size(0)
    rowptr, col, _ = full.csr()
    graph = RC.Graph(rowptr, col)
    nnz = int(col.numel())
    del full, rowptr, col
    torch.cuda.empty_cache()
    gd = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn((n, c["feats"]), device=dev, generator=gd)
    g = torch.Generator().manual_seed(1)
    y = torch.randint(c["classes"], (n,), generator=g).to(dev)
    torch.manual_seed(0)
    model = models.SAGE(c["feats"], c["hidden"], c["classes"], c["layers"], dropout=c["dropout"], batch_norm=False)
    params = {k: torch.nn.Parameter(v.to(dev)) for k, v in model.state_dict().items()}
    opt = torch.optim.Adam(list(params.values()), lr=0.002)
    cfg = {"bits": c["bits"], "kept_frac": c["kept_frac"]}

    def step():
        opt.zero_grad(set_to_none=True)
        out = RC.sage_forward(params, x, graph, c["layers"], c["dropout"], cfg)
        loss = F.nll_loss(F.log_softmax(out, dim=-1), y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = step()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e-3 / steps, n, nnz, float(loss.item())


def run_reference(args):
    """The reference arm.  The reference implements this path only as CUDA kernels, so "the reference's own
    implementation" is those kernels, compiled unmodified into oracle/_ref/, driven by the reference's op chain
    on ONE GPU (it has no multi-GPU mode) on the full workload.  Without a GPU or without oracle/_ref/ (and for
    the GCN workloads, whose chain is not restated) the arm times the CPU restatement of the reference's math
    (oracle/) with all host threads on a bounded sample, at two sample sizes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from exact_b200 import graphs

    class _A:
        n_bits, kept_frac, act_fp, no_compress = args.n_bits, args.kept_frac, False, False
    c = apply_knobs(graphs.CONFIGS[args.workload], _A)
    nodes = args.nodes or c["nodes"]
    line = {"impl": "reference", "metric": "full_batch_gnn_epoch_per_s", "unit": "epoch/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(c, nodes), "nodes": nodes}}
    gpu_chain = False
    try:
        from oracle import ref_chain
        gpu_chain = ref_chain.available() and c["model"] == "sage" and not args.cpu_reference
    except Exception:
        gpu_chain = False
    if gpu_chain:
        sec, n, nnz, loss = reference_gpu_epoch(c, nodes, args.steps, max(args.warmup, 1))
        value = 1.0 / sec
        line.update({"value": round(value, 6), "ms_per_step": round(sec * 1e3, 2), "reference_loss": loss,
                     "reference_device": "cuda:0 (one GPU: the reference has no multi-GPU mode)",
                     "cpu_baseline": {"value": round(value, 6), "unit": "epoch/s", "cores": 1, "kind": "reference",
                                      "sample": f"{args.steps} epochs of the full {n}-node / {nnz}-edge workload through "
                                                "the reference's op chain with its own unmodified CUDA kernels "
                                                "(pack, unpack, SpMM) on one GPU of this box, driven by one host "
                                                "thread; ReLU / dropout are torch's (the reference's mask kernels "
                                                "write out of bounds at these sizes and are not run)"},
                     "e2e": {"value": round(value, 6), "unit": "epoch/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0}})
        line["config"]["directed_edges"] = nnz
        print(json.dumps(line), flush=True)
        return
    sec, n, nnz = cpu_epoch(c, args.cpu_nodes, steps=args.steps, warmup=min(args.warmup, 1))
    sec2, n2, _ = cpu_epoch(c, args.cpu_nodes // 2, steps=1, warmup=1)
    scale = nodes / n
    value = 1.0 / (sec * scale)
    sample = (f"{args.steps} epochs on a {n}-node / {nnz}-edge sample of the workload ({sec:.2f} s each; {sec2:.2f} s at "
              f"{n2} nodes: {sec / sec2:.2f}x the time for {n / n2:.2f}x the nodes), scaled by {scale:.1f}x nodes")
    line.update({"value": round(value, 6), "ms_per_step": round(sec * scale * 1e3, 1),
                 "cpu_baseline": {"value": round(value, 6), "unit": "epoch/s", "cores": os.cpu_count(), "kind": "port",
                                  "sample": sample},
                 "e2e": {"value": round(value, 6), "unit": "epoch/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg4", choices=["cfg1", "cfg2", "cfg3", "cfg4"])
    ap.add_argument("--nodes", type=int, default=None, help="shrink the graph to this many nodes (same mean degree)")
    ap.add_argument("--cpu-nodes", type=int, default=200000, help="nodes of the bounded sample the CPU baseline runs")
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-compress", action="store_true",
                    help="comparison run: activations saved uncompressed (config.compress_activation = False)")
    ap.add_argument("--dense-gather", action="store_true", help="N > 1: exchange dense rows (no zero compaction)")
    ap.add_argument("--no-peer-exchange", action="store_true",
                    help="N > 1: exchange through the collective library only (no rank writes a peer's memory)")
    ap.add_argument("--column-split", action="store_true",
                    help="N > 1: feature-parallel aggregation at every N (default: from 8 ranks on)")
    ap.add_argument("--row-split", action="store_true",
                    help="N > 1: aggregate on row shards of the adjacency (exchange whole operand rows) instead of "
                         "switching to column slices around each aggregation")
    ap.add_argument("--routed-output", action="store_true",
                    help="N > 1: the SpMM of the feature-parallel aggregation stores its result rows straight into "
                         "their owners' buffers instead of a local result followed by a scatter kernel")
    ap.add_argument("--min-slice-columns", type=int, default=None,
                    help="N > 1: config.aggregation_min_slice_columns (narrow operands of the feature-parallel "
                         "aggregation are cut into fewer, wider column slices times row blocks)")
    ap.add_argument("--result-chunks", type=int, default=None,
                    help="N > 1: config.aggregation_result_chunks (pieces a rank's row block of the feature-parallel "
                         "aggregation is summed in; each piece's stores overlap the next piece's sums)")
    ap.add_argument("--cpu-reference", action="store_true",
                    help="--impl reference: time the CPU restatement even when the reference's CUDA kernels are built")
    # the reference drivers' knobs (mem_speed_bench/arxiv/train_full_batch.py:44-48)
    ap.add_argument("--n_bits", type=int, default=None, choices=[1, 2, 4, 8])
    ap.add_argument("--kept_frac", type=float, default=None)
    ap.add_argument("--act_fp", action="store_true",
                    help="keep activations in fp32 (compression off; the projection still applies when --kept_frac < 1)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
