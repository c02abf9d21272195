"""One rank of a row-sharded training run of the quantised 3-layer GraphSAGE, for test_dist_gpu.py.

Several of these processes share one GPU (backend gloo, collectives staged through the host), so the whole
multi-rank path -- shards, noise keyed by global rows, the exchange before every aggregation (ranks writing
their compact rows into each other's buffers, or the collective fallback), the gradient all-reduce -- runs
on a box with a single device.  Writes losses, first-step gradients, final parameters and the first packed
activation stream of this rank to <out>/w<world>_<name>_r<rank>.pt."""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--name", default="run")
    ap.add_argument("--nodes", type=int, default=4000)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--peer", type=int, default=1)
    ap.add_argument("--compact", type=int, default=1)
    ap.add_argument("--colsplit", type=int, default=1)
    ap.add_argument("--routed", type=int, default=0)
    ap.add_argument("--overlap", type=int, default=0)
    ap.add_argument("--slicemajor", type=int, default=0)
    ap.add_argument("--minslice", type=int, default=0)
    ap.add_argument("--chunks", type=int, default=1)
    a = ap.parse_args()

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from exact_b200 import QModule, config, graphs, models
    from exact_b200 import dist as xdist

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    if a.world > 1:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(a.port)
        dist.init_process_group("gloo", rank=a.rank, world_size=a.world)
    c = dict(graphs.CONFIGS["cfg4"])
    full = graphs.build_graph(c, seed=0, device=dev, nodes=a.nodes)
    n = full.size(0)
    config.peer_exchange = bool(a.peer)
    config.compact_operand = bool(a.compact)
    config.column_split_aggregation = bool(a.colsplit)
    config.routed_aggregation_output = bool(a.routed)
    config.overlap_exchange = bool(a.overlap)
    config.slice_major_result = bool(a.slicemajor)
    config.aggregation_min_slice_columns = a.minslice
    config.aggregation_result_chunks = a.chunks
    config.cache_constant_gather = False
    if a.world > 1:
        adj = xdist.shard_graph(full, "mean", a.rank, a.world)
        r0, r1 = adj.row_start, adj.row_end
    else:
        full.fill_cache_()
        full.to_int32_()
        adj, r0, r1 = full, 0, n
        config.row_offset = 0
    g = torch.Generator().manual_seed(1)
    x = torch.randn(n, c["feats"], generator=g)[r0:r1].to(dev)
    y = torch.randint(c["classes"], (n,), generator=g)[r0:r1].to(dev)
    torch.manual_seed(0)
    config.compress_activation = True
    config.activation_compression_bits = [c["bits"]]
    config.kept_frac = c["kept_frac"]
    config.manual_seed(0)
    net = QModule(models.SAGE(c["feats"], c["hidden"], c["classes"], c["layers"], dropout=c["dropout"],
                              batch_norm=False)).to(dev).train()
    opt = torch.optim.Adam(net.parameters(), lr=0.01)
    params = list(net.parameters())
    first = {}

    def hook(quantized, randmat):
        if "packed" not in first:
            first["packed"] = quantized[0].detach().clone()
            first["scale"] = quantized[2].detach().clone()
            first["min"] = quantized[3].detach().clone()

    config.quantized_hook = hook
    losses, grads0 = [], None
    for step in range(a.steps):
        opt.zero_grad(set_to_none=True)
        out = net(x, adj)
        loss = F.cross_entropy(out, y, reduction="none").sum() / n
        loss.backward()
        xdist.allreduce_gradients(params)
        total = loss.detach().clone()
        if a.world > 1:
            xdist.all_reduce(total)
        losses.append(float(total.item()))
        if step == 0:
            grads0 = [p.grad.detach().cpu().clone() for p in params]
        opt.step()
        config.quantized_hook = None
    from exact_b200 import check_status
    check_status(force=True)
    forms = {}
    form = getattr(adj, "_operand_form", None) if a.world > 1 else None
    if form is not None:
        forms = {k: (v[0], v[2]) for k, v in form.state.items()}
    peers_used = bool(getattr(adj, "_peers", None)) or bool(getattr(adj, "_col_bufs", None))
    exchange = adj.describe_exchange() if a.world > 1 else "none"
    col_keys = sorted(getattr(adj, "_col_bufs", {}).keys()) if a.world > 1 else []
    torch.save({"losses": losses, "grads0": grads0, "params": [p.detach().cpu() for p in params],
                "packed": first["packed"].cpu()[:-1], "scale": first["scale"].cpu(), "min": first["min"].cpu(),
                "rows": (r0, r1), "forms": forms, "peers_used": peers_used, "exchange": exchange,
                "col_keys": col_keys},
               os.path.join(a.out, f"w{a.world}_{a.name}_r{a.rank}.pt"))
    if a.world > 1:
        adj.close()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
