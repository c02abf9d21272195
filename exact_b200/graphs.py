"""Seeded synthetic graphs with the shapes of the benchmark configurations.  They stand in for the
public datasets the reference's drivers load (mem_speed_bench/data.py:11-58), which are not
available offline: only node / edge / feature / class counts are taken from those datasets.

All generators run with torch ops on the device they are given (CPU for the oracle-side tests, CUDA
for the benchmark) and return a SparseTensor with int64 indices sorted by (row, col)."""
import torch

from .sparse import SparseTensor


def _symmetric_csr(src, dst, n, self_loops):
    keep = src != dst
    src, dst = src[keep], dst[keep]
    row = torch.cat([src, dst])
    col = torch.cat([dst, src])
    if self_loops:
        loop = torch.arange(n, device=row.device, dtype=row.dtype)
        row = torch.cat([row, loop])
        col = torch.cat([col, loop])
    key = torch.unique(row * n + col)  # sorted, duplicates removed
    row = torch.div(key, n, rounding_mode="floor")
    col = key - row * n
    return SparseTensor(row=row, col=col, value=None, sparse_sizes=(n, n), is_sorted=True)


def erdos_renyi(n, avg_degree, seed, device="cpu", self_loops=True):
    """G(n, m) with m = n * avg_degree / 2 undirected edges, symmetrised (mean degree ~avg_degree
    after symmetrisation), optional self-loops."""
    g = torch.Generator(device=device).manual_seed(seed)
    m = int(n * avg_degree / 2)
    src = torch.randint(n, (m,), generator=g, device=device, dtype=torch.int64)
    dst = torch.randint(n, (m,), generator=g, device=device, dtype=torch.int64)
    return _symmetric_csr(src, dst, n, self_loops)


def _rmat_edges(n, m, g, device, a, b, c, chunk):
    scale = max(1, (n - 1).bit_length())
    srcs, dsts = [], []
    done = 0
    while done < m:
        k = min(chunk, m - done)
        src = torch.zeros(k, dtype=torch.int64, device=device)
        dst = torch.zeros(k, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(k, generator=g, device=device)
            src_bit = (r >= a + b).to(torch.int64)                                   # quadrants c, d
            dst_bit = (((r >= a) & (r < a + b)) | (r >= a + b + c)).to(torch.int64)  # quadrants b, d
            src = (src << 1) | src_bit
            dst = (dst << 1) | dst_bit
        srcs.append(src % n)
        dsts.append(dst % n)
        done += k
    return torch.cat(srcs), torch.cat(dsts)


def rmat(n, n_undirected, seed, device="cpu", a=0.57, b=0.19, c=0.19, self_loops=True, chunk=1 << 24):
    """R-MAT power-law graph (Chakrabarti, Zhan, Faloutsos 2004) on 2^ceil(log2 n) ids folded onto n
    nodes by modulo and relabelled by a fixed permutation (so hubs are spread over row shards),
    symmetrised, duplicates removed, optional self-loops.  Duplicate samples are topped up (at most
    three rounds) until about 2 * n_undirected distinct directed edges exist."""
    g = torch.Generator(device=device).manual_seed(seed)
    perm = torch.randperm(n, generator=g, device=device)
    key = torch.empty(0, dtype=torch.int64, device=device)
    need = n_undirected
    for _ in range(4):
        src, dst = _rmat_edges(n, max(int(need), 1), g, device, a, b, c, chunk)
        src, dst = perm[src], perm[dst]
        keep = src != dst
        lo, hi = torch.minimum(src[keep], dst[keep]), torch.maximum(src[keep], dst[keep])
        key = torch.unique(torch.cat([key, lo * n + hi]))
        short = n_undirected - key.numel()
        if short <= 0.01 * n_undirected:
            break
        need = short * 1.5
    lo = torch.div(key, n, rounding_mode="floor")
    hi = key - lo * n
    return _symmetric_csr(lo, hi, n, self_loops)


# The benchmark configurations: nodes, sampled undirected edges, features, hidden, classes.
CONFIGS = {
    # 2-layer GCN on an Erdos-Renyi graph; runs on CPU (oracle) and GPU
    "cfg1": dict(model="gcn", nodes=4096, avg_degree=10, feats=128, hidden=64, classes=16, layers=2,
                 batch_norm=False, dropout=0.0, bits=2, kept_frac=1.0, graph="er", self_loops=True, gcn_norm=True),
    # 3-layer GCN, arxiv-shaped
    "cfg2": dict(model="gcn", nodes=169343, undirected=1_166_243, feats=128, hidden=256, classes=40, layers=3,
                 batch_norm=True, dropout=0.5, bits=2, kept_frac=1.0, graph="rmat", self_loops=True, gcn_norm=True),
    # 3-layer GraphSAGE-mean, reddit-shaped
    "cfg3": dict(model="sage", nodes=232965, undirected=11_600_000, feats=602, hidden=256, classes=41, layers=3,
                 batch_norm=False, dropout=0.5, bits=2, kept_frac=0.125, graph="rmat", self_loops=True,
                 gcn_norm=False),
    # 3-layer GraphSAGE-mean, products-shaped, row-partitioned across GPUs
    "cfg4": dict(model="sage", nodes=2449029, undirected=61_859_140, feats=100, hidden=256, classes=47, layers=3,
                 batch_norm=False, dropout=0.5, bits=2, kept_frac=0.125, graph="rmat", self_loops=False,
                 gcn_norm=False),
}


def build_graph(cfg, seed=0, device="cpu", nodes=None):
    """Adjacency of a benchmark configuration (optionally shrunk to `nodes` nodes at the same mean degree)."""
    c = CONFIGS[cfg] if isinstance(cfg, str) else cfg
    n = c["nodes"] if nodes is None else nodes
    if c["graph"] == "er":
        return erdos_renyi(n, c["avg_degree"], seed, device, c["self_loops"])
    m = c["undirected"] if nodes is None else int(c["undirected"] * (nodes / c["nodes"]))
    return rmat(n, m, seed, device, self_loops=c["self_loops"])
