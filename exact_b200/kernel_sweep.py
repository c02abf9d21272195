"""Kernel sweep: achieved GB/s of the pack / unpack (and SpMM) kernels against the HBM roofline over
bit widths, row counts, column counts and input dtypes (the kernel-level benchmark configuration).

  python -m exact_b200.kernel_sweep                          # default grid, one JSON line per case
  python -m exact_b200.kernel_sweep --op pack --N 1000000 --D 128 --bits 2 --reps 3   # one case (for ncu)
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m exact_b200.kernel_sweep --sharded \
      --N 10000000 --D 128 256 --bits 2                      # row-sharded over the GPUs of one node

Timing: CUDA events on the launching stream, 3 warm-up launches, inputs larger than L2 or an L2 flush
between launches (a 256 MB write) when they are not."""
import argparse
import json
import os

import torch

from . import _lib
from .cpp_extension import quantization as Q
from .cpp_extension import spmm as S


def _peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def _time(call, reps, flush):
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        if flush is not None:
            flush.fill_(1.0)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # The device spins for about 0.2 ms while the host enqueues the call: the interval between the two
        # events is then the kernel's, not the host's time to reach the launch (tens of microseconds of
        # Python and ctypes, a third of a 0.1 ms kernel).
        torch.cuda._sleep(400_000)
        a.record()
        call()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
    ms.sort()
    return ms[len(ms) // 2]


def run_case(op, N, D, bits, dtype, reps, noise):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(N, D, device=dev, generator=g).relu_().to(dtype)
    eb = x.element_size()
    flush = torch.empty(64 * 1024 * 1024, device=dev) if N * D * eb < 256e6 else None
    u = torch.rand(N, D, device=dev, generator=g) if noise else None
    pk, sb, mb = Q.quantize_pack(x, bits, noise=u, seed=1, offset=0)
    G = pk.numel() - 1
    if op == "pack":
        nbytes = N * D * eb + G + 4 * N + (N * D * 4 if noise else 0)
        call = lambda: Q.quantize_pack(x, bits, noise=u, seed=1, offset=0)
    elif op == "unpack":
        nbytes = G + 4 * N + N * D * 4
        call = lambda: Q.unpack_single_precision(pk, bits, sb, mb, N, D)
    else:
        raise ValueError(op)
    ms = _time(call, reps, flush)
    peak, kind = _peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"op": op, "N": N, "D": D, "bits": bits, "dtype": str(dtype).replace("torch.", ""),
            "supplied_noise": bool(noise), "ms": round(ms, 4), "GB/s": round(gbs, 1), "frac": round(gbs / peak, 4),
            "peak": peak, "peak_kind": kind}


def run_rp(N, D, kept_frac, bits, reps):
    """Fused projection + pack (tcgen05): HBM GB/s on the algorithmic bytes and TFLOP/s of the GEMM."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(N, D, device=dev, generator=g).relu_()
    k = int(kept_frac * D + 0.999)
    if not Q.rp_supported(D, k):
        return {"op": "rp_pack", "N": N, "D": D, "k": k, "bits": bits, "skipped": "shape not taken by the fused kernel"}
    from .ops import _rademacher
    R = _rademacher(D, k, dev, torch.float32, seed=1, offset=0)
    flush = torch.empty(64 * 1024 * 1024, device=dev) if N * D * 4 < 256e6 else None
    call = lambda: Q.rp_quantize_pack(x, R, bits, seed=1, offset=1)
    ms = _time(call, reps, flush)
    wpt = 8 // bits
    nbytes = N * D * 4 + D * k * 4 + ((N + wpt - 1) // wpt) * k + 4 * N
    peak, kind = _peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"op": "rp_pack", "N": N, "D": D, "k": k, "bits": bits, "ms": round(ms, 4), "GB/s": round(gbs, 1),
            "frac": round(gbs / peak, 4), "TFLOP/s": round(2.0 * N * D * k / (ms * 1e-3) / 1e12, 2), "peak": peak,
            "peak_kind": kind}


def run_unpack_rp(N, D, kept_frac, bits, reps):
    """Fused unpack + dequantise + transpose projection (tcgen05): GB/s on the algorithmic bytes."""
    dev = torch.device("cuda")
    k = int(kept_frac * D + 0.999)
    if not Q.unpack_rp_supported(D, k):
        return {"op": "unpack_rp", "N": N, "D": D, "k": k, "bits": bits, "skipped": "shape not taken by the fused kernel"}
    g = torch.Generator(device=dev).manual_seed(0)
    y = torch.randn(N, k, device=dev, generator=g)
    pk, sb, mb = Q.quantize_pack(y, bits, seed=1, offset=0)
    from .ops import _rademacher
    R = _rademacher(D, k, dev, torch.float32, seed=1, offset=0)
    flush = torch.empty(64 * 1024 * 1024, device=dev) if N * D * 4 < 256e6 else None
    call = lambda: Q.unpack_dequant_rp(pk, bits, sb, mb, N, R)
    ms = _time(call, reps, flush)
    nbytes = (pk.numel() - 1) + 4 * N + D * k * 4 + N * D * 4
    peak, kind = _peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"op": "unpack_rp", "N": N, "D": D, "k": k, "bits": bits, "ms": round(ms, 4), "GB/s": round(gbs, 1),
            "frac": round(gbs / peak, 4), "TFLOP/s": round(2.0 * N * D * k / (ms * 1e-3) / 1e12, 2), "peak": peak,
            "peak_kind": kind}


def run_linear(M, K, N, reps):
    """Dense-layer GEMM (tf32 head/tail split, tcgen05) against the library fp32 GEMM: ms, TFLOP/s, error vs fp64."""
    from .cpp_extension import backward_func as B
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    a = torch.randn(M, K, device=dev, generator=g)
    w = torch.randn(N, K, device=dev, generator=g)
    b = torch.randn(N, device=dev, generator=g)
    flush = torch.empty(64 * 1024 * 1024, device=dev) if M * (K + N) * 4 < 256e6 else None
    ms = _time(lambda: B.linear_forward(a, w, b), reps, flush)
    ms_lib = _time(lambda: torch.nn.functional.linear(a, w, b), reps, flush)
    rows = min(M, 20000)
    ref = a[:rows].double() @ w.double().t() + b.double()
    err = float((B.linear_forward(a, w, b)[:rows].double() - ref).norm() / ref.norm())
    err_lib = float((torch.nn.functional.linear(a, w, b)[:rows].double() - ref).norm() / ref.norm())
    nbytes = 4 * (M * K + N * K + M * N)
    peak, kind = _peak()
    return {"op": "linear", "M": M, "K": K, "N": N, "ms": round(ms, 4), "library_fp32_ms": round(ms_lib, 4),
            "TFLOP/s": round(2.0 * M * K * N / (ms * 1e-3) / 1e12, 1),
            "tensor_TFLOP/s": round(6.0 * M * K * N / (ms * 1e-3) / 1e12, 1),
            "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1), "frac_hbm": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4),
            "rel_err_vs_fp64": err, "library_rel_err_vs_fp64": err_lib, "peak_kind": kind}


def run_grad_weight(N, O, k, bits, reps):
    """g^T . dequantise([Xq_a | Xq_b]) (two packed activations of k columns, one pass over g) against the route
    it replaces: two unpacks and two batched library GEMMs."""
    from .cpp_extension import backward_func as B
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(0)
    g = torch.randn(N, O, device=dev, generator=gen)
    qs = []
    for s in (1, 2):
        x = torch.randn(N, k, device=dev, generator=gen)
        pk, sb, mb = Q.quantize_pack(x, bits, seed=s, offset=0)
        qs.append((pk, bits, sb, mb))
    ms = _time(lambda: B.grad_weight_from_packed(g, qs[0], k, qs[1], k), reps, None)

    def old():
        for q in qs:
            B.rows_reduce_mm(g, Q.unpack_single_precision(q[0], bits, q[2], q[3], N, k))
    ms_old = _time(old, reps, None)
    nbytes = 4 * N * O + 2 * (N * k * bits // 8 + 4 * N)
    peak, kind = _peak()
    return {"op": "grad_weight_from_packed", "N": N, "O": O, "k": [k, k], "bits": bits, "ms": round(ms, 4),
            "unpack_plus_library_gemm_ms": round(ms_old, 4), "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1),
            "frac": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4), "TFLOP/s": round(4.0 * N * O * k / (ms * 1e-3) / 1e12, 1),
            "peak": peak, "peak_kind": kind}


def run_bn_bwd(N, D, bits, reps):
    """Batch-norm backward read from the packed input (two passes over g and the packed bytes, one write) against
    the route it replaces: unpack to fp32, then ATen's backward on the reconstruction."""
    from .cpp_extension import backward_func as B
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(N, D, device=dev, generator=gen)
    g = torch.randn(N, D, device=dev, generator=gen)
    w = torch.randn(D, device=dev, generator=gen)
    rm, rv = torch.zeros(D, device=dev), torch.ones(D, device=dev)
    _, mean, invstd = torch.ops.aten.native_batch_norm(x, w, None, rm, rv, True, 0.1, 1e-5)
    pk, sb, mb = Q.quantize_pack(x, bits, seed=1, offset=0)
    q = (pk, bits, sb, mb)
    del x
    ms = _time(lambda: B.batch_norm_backward_from_packed(g, q, w, rm, rv, mean, invstd, True, 1e-5, [True, True, True]),
               reps, None)

    def old():
        xh = Q.unpack_single_precision(pk, bits, sb, mb, N, D)
        torch.ops.aten.native_batch_norm_backward(g, xh, w, rm, rv, mean, invstd, True, 1e-5, [True, True, True])
    ms_old = _time(old, reps, None)
    nbytes = 12 * N * D + 2 * (N * D * bits // 8 + 4 * N)
    peak, kind = _peak()
    return {"op": "bn_backward_from_packed", "N": N, "D": D, "bits": bits, "ms": round(ms, 4),
            "unpack_plus_aten_ms": round(ms_old, 4), "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1),
            "frac": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4), "peak": peak, "peak_kind": kind}


def run_rowops(N, D, reps):
    """D^-1 g and g.sum(0) in one pass over g against the framework's broadcast multiply + column reduction."""
    from .cpp_extension import backward_func as B
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(0)
    g = torch.randn(N, D, device=dev, generator=gen)
    inv = torch.rand(N, device=dev, generator=gen)
    ms = _time(lambda: B.rows_scale_colsum(g, inv, want_scaled=True, want_colsum=True), reps, None)
    ms_old = _time(lambda: (g * inv.unsqueeze(1), g.sum(0)), reps, None)
    nbytes = 8 * N * D
    peak, kind = _peak()
    return {"op": "rows_scale_colsum", "N": N, "D": D, "ms": round(ms, 4), "multiply_plus_sum_ms": round(ms_old, 4),
            "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1), "frac": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4),
            "peak": peak, "peak_kind": kind}


def run_mask(N, D, p, reps):
    """ReLU + dropout of a hidden layer in one pass (forward) and its backward: GB/s on 8 bytes + 1 bit per element."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(N, D, device=dev, generator=g).requires_grad_()
    gout = torch.randn(N, D, device=dev, generator=g)
    n = N * D
    nbytes = 8 * n + n // 8
    y = Q.act_quantized_relu_dropout(x, p, True)
    ms_fw = _time(lambda: Q.act_quantized_relu_dropout(x, p, True), reps, None)
    ms_bw = _time(lambda: torch.autograd.grad(y, x, gout, retain_graph=True), reps, None)
    peak, kind = _peak()
    out = []
    for name, ms in (("relu_dropout_forward", ms_fw), ("relu_dropout_backward", ms_bw)):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out.append({"op": name, "N": N, "D": D, "p": p, "ms": round(ms, 4), "GB/s": round(gbs, 1),
                    "frac": round(gbs / peak, 4), "peak": peak, "peak_kind": kind})
    return out


def run_spmm(nodes, avg_deg, K, reps, reduce, density=None, regroup=False):
    """Mean / sum aggregation over an R-MAT graph.  `density`: the share of non-zero entries of the dense
    operand; below 1 the packing of the operand into compact rows and its expansion back (the two kernels
    around the peer exchange of a row-sharded run) are timed too."""
    from . import graphs
    from .cpp_extension import rows as RW
    dev = torch.device("cuda")
    adj = graphs.rmat(nodes, int(nodes * avg_deg / 2), 0, dev, self_loops=False)
    adj.to_int32_()
    rowptr, col, _ = adj.csr()
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(nodes, K, device=dev, generator=g)
    if density is not None and density < 1.0:
        x = x * (torch.rand(nodes, K, device=dev, generator=g) < density)
    nnz = col.numel()
    peak, kind = _peak()
    out = []
    if density is not None and density < 1.0 and K <= 256:
        cr = RW.crows_pack(x)
        cr.density = density
        dense = torch.empty_like(x)
        compact_bytes = nodes * (16 + int(density * K) * 5)
        for name, call in (("crows_pack", lambda: RW.crows_pack(x, out=cr)),
                           ("crows_unpack", lambda: RW.crows_unpack(cr, nodes, out=dense))):
            ms = _time(call, reps, None)
            nb = nodes * K * 4 + compact_bytes
            out.append({"op": name, "nodes": nodes, "K": K, "density": density, "ms": round(ms, 4),
                        "GB/s": round(nb / (ms * 1e-3) / 1e9, 1), "frac": round(nb / (ms * 1e-3) / 1e9 / peak, 4),
                        "peak": peak, "peak_kind": kind})
    ms = _time(lambda: S._spmm(rowptr, col, None, x, reduce, regroup=regroup), reps, None)
    must = nodes * K * 4 + nnz * 4 + (nodes + 1) * 4 + nodes * K * 4
    l2 = nnz * K * 4 + nnz * 4 + (nodes + 1) * 4 + nodes * K * 4
    out.append({"op": "spmm_" + reduce, "nodes": nodes, "nnz": nnz, "K": K, "density": density, "regroup": regroup,
                "ms": round(ms, 4), "GB/s": round(must / (ms * 1e-3) / 1e9, 1),
                "frac": round(must / (ms * 1e-3) / 1e9 / peak, 4), "l2_side_GB/s": round(l2 / (ms * 1e-3) / 1e9, 1),
                "peak": peak, "peak_kind": kind})
    return out


def run_sharded(op, N, D, bits, kept_frac, reps):
    """Row-sharded kernel sweep: every rank runs the kernel on its shard of the N rows (a multiple of 8 rows,
    noise keyed by global rows), the aggregate is bytes of all ranks / slowest rank's time (no collective on
    the data path), and rank 0 checks that the shards' packed streams and statistics, concatenated in rank
    order, are the bytes one GPU produces for the whole matrix (SHA-256 of both)."""
    import hashlib

    import torch.distributed as dist

    from . import dist as xdist
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    shard = xdist.shard_rows(N, world)
    r0, r1 = min(rank * shard, N), min(rank * shard + shard, N)
    n = r1 - r0

    def rows(a, b):   # rows [a, b) of the synthetic matrix (every rank draws the same whole matrix and slices it)
        g = torch.Generator(device=dev).manual_seed(1234)
        full = torch.randn(N, D, device=dev, generator=g).relu_()
        return full[a:b].contiguous()

    x = rows(r0, r1)
    k = D if kept_frac >= 1.0 else int(kept_frac * D + 0.999)
    if op == "rp_pack":
        from .ops import _rademacher
        R = _rademacher(D, k, dev, torch.float32, seed=1, offset=0)
        call = lambda t, off: Q.rp_quantize_pack(t, R, bits, seed=1, offset=1, row_offset=off)
        nbytes = n * D * 4 + D * k * 4 + ((n + 8 // bits - 1) // (8 // bits)) * k + 4 * n
    else:
        call = lambda t, off: Q.quantize_pack(t, bits, seed=1, offset=1, row_offset=off)
        nbytes = n * D * 4 + ((n + 8 // bits - 1) // (8 // bits)) * D + 4 * n
    flush = torch.empty(64 * 1024 * 1024, device=dev) if n * D * 4 < 256e6 else None
    ms = torch.tensor([_time(lambda: call(x, r0), reps, flush)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tot = torch.tensor([float(nbytes)], device=dev, dtype=torch.float64)
    dist.all_reduce(tot)
    pk, sb, mb = call(x, r0)
    body = torch.cat([pk.view(torch.uint8)[:-1], sb.view(torch.uint8), mb.view(torch.uint8)])
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
    peak, kind = _peak()
    parts = [allb[r * max(sizes):r * max(sizes) + sizes[r]].cpu() for r in range(world)]
    # split each rank's bytes back into stream / scale / min and concatenate per kind in rank order
    streams, scales, mins = [], [], []
    for r, part in enumerate(parts):
        nr = min(r * shard + shard, N) - min(r * shard, N)
        streams.append(part[:part.numel() - 4 * nr])
        scales.append(part[part.numel() - 4 * nr:part.numel() - 2 * nr])
        mins.append(part[part.numel() - 2 * nr:])
    sharded = hashlib.sha256(torch.cat(streams + scales + mins).numpy().tobytes()).hexdigest()
    del x
    torch.cuda.empty_cache()
    pk1, sb1, mb1 = call(rows(0, N), 0)
    whole = hashlib.sha256(torch.cat([pk1.view(torch.uint8)[:-1].cpu(), sb1.view(torch.uint8).cpu(),
                                      mb1.view(torch.uint8).cpu()]).numpy().tobytes()).hexdigest()
    gbs = float(tot.item()) / (float(ms.item()) * 1e-3) / 1e9
    return {"op": op, "sharded_over": world, "N": N, "D": D, "k": k, "bits": bits, "ms_slowest_rank": round(float(ms.item()), 4),
            "aggregate_GB/s": round(gbs, 1), "frac_of_n_peaks": round(gbs / (peak * world), 4), "peak_per_gpu": peak,
            "peak_kind": kind, "shard_streams_equal_one_gpu_stream": sharded == whole, "sha256": whole}


def main_sharded(a):
    """torchrun entry of the row-sharded sweep: pack and fused projection + pack over N x D x bits x kept_frac."""
    import torch.distributed as dist

    from . import dist as xdist
    rank, world, _ = xdist.init_process_group_from_env()
    assert world > 1, "--sharded runs under torchrun with more than one rank"
    for N in a.N:
        for D in a.D:
            if N * D * 4 > a.max_bytes:
                continue
            for bits in a.bits:
                for kf in [1.0] + list(a.kept_frac):
                    op = "pack" if kf >= 1.0 else "rp_pack"
                    if op == "rp_pack" and not Q.rp_supported(D, int(kf * D + 0.999)):
                        continue
                    r = run_sharded(op, N, D, bits, kf, a.reps)
                    if r is not None:
                        print(json.dumps(r), flush=True)
                    torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "pack", "unpack", "spmm", "rp_pack", "unpack_rp", "linear", "mask", "grad_weight", "bn_bwd", "rowops"])
    ap.add_argument("--kept-frac", type=float, nargs="*", default=[0.5, 0.125])
    ap.add_argument("--N", type=int, nargs="*", default=[100_000, 1_000_000, 10_000_000])
    ap.add_argument("--D", type=int, nargs="*", default=[64, 128, 256, 602])
    ap.add_argument("--bits", type=int, nargs="*", default=[1, 2, 4, 8])
    ap.add_argument("--dtype", nargs="*", default=["float32", "bfloat16"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--noise", action="store_true", help="supply the noise tensor instead of drawing Philox noise")
    ap.add_argument("--nodes", type=int, default=1_000_000)
    ap.add_argument("--avg-deg", type=float, default=50.0)
    ap.add_argument("--K", type=int, nargs="*", default=[256])
    ap.add_argument("--regroup", action="store_true",
                    help="--op spmm: accept a regrouped per-row sum (operands of at most 64 columns then take "
                         "several edges per load instruction, as the column slices of a row-sharded run do)")
    ap.add_argument("--density", type=float, default=None,
                    help="--op spmm: share of non-zero operand entries; below 1 the compact-rows pack / unpack are timed too")
    ap.add_argument("--max-bytes", type=float, default=12e9, help="skip cases whose input exceeds this")
    ap.add_argument("--sharded", action="store_true",
                    help="row-sharded sweep of pack and fused projection + pack; launch with torchrun on 2, 4 or 8 GPUs")
    a = ap.parse_args()
    _lib.load()
    if a.sharded:
        main_sharded(a)
        return
    if a.op == "spmm":
        for K in a.K:
            for r in run_spmm(a.nodes, a.avg_deg, K, a.reps, "mean", a.density, a.regroup):
                print(json.dumps(r), flush=True)
        return
    if a.op == "grad_weight":
        for N in a.N:
            for bits in a.bits:
                print(json.dumps(run_grad_weight(N, 256, 32, bits, a.reps)), flush=True)
        return
    if a.op == "rowops":
        for N in a.N:
            for D in a.D:
                if N * D * 4 <= a.max_bytes:
                    print(json.dumps(run_rowops(N, D, a.reps)), flush=True)
        return
    if a.op == "bn_bwd":
        for N in a.N:
            for D in a.D:
                if N * D * 4 > a.max_bytes or D % 4:
                    continue
                for bits in a.bits:
                    print(json.dumps(run_bn_bwd(N, D, bits, a.reps)), flush=True)
        return
    if a.op == "mask":
        for N in a.N:
            for D in a.D:
                if N * D * 4 > a.max_bytes:
                    continue
                for r in run_mask(N, D, 0.5, a.reps):
                    print(json.dumps(r), flush=True)
        return
    if a.op == "linear":
        for M in a.N:
            for K in a.D:
                for N in a.K:
                    print(json.dumps(run_linear(M, K, N, a.reps)), flush=True)
        return
    if a.op == "unpack_rp":
        for N in a.N:
            for D in a.D:
                if N * D * 4 > a.max_bytes:
                    continue
                for kf in a.kept_frac:
                    for bits in a.bits:
                        print(json.dumps(run_unpack_rp(N, D, kf, bits, a.reps)), flush=True)
                torch.cuda.empty_cache()
        return
    if a.op == "rp_pack":
        for N in a.N:
            for D in a.D:
                if N * D * 4 > a.max_bytes:
                    continue
                for kf in a.kept_frac:
                    for bits in a.bits:
                        print(json.dumps(run_rp(N, D, kf, bits, a.reps)), flush=True)
                torch.cuda.empty_cache()
        return
    ops = ["pack", "unpack"] if a.op == "all" else [a.op]
    for dt in a.dtype:
        dtype = getattr(torch, dt)
        for N in a.N:
            for D in a.D:
                if N * D * 4 > a.max_bytes:
                    continue
                for bits in a.bits:
                    for op in ops:
                        if op == "unpack" and dtype != torch.float32:
                            continue
                        print(json.dumps(run_case(op, N, D, bits, dtype, a.reps, a.noise)), flush=True)
                torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
