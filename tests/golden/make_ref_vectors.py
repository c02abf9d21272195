"""Generate golden vectors from the reference's OWN unmodified CUDA kernels.

Run on a machine with a GPU after `python oracle/build_ref.py` has produced oracle/_ref/*.so (built
from the reference checkout).  For each case the input is regenerated from a numpy seed, the reference
kernels (pack_single_precision, unpack_single_precision, spmm) are run, and only the OUTPUTS plus
the seeds needed to regenerate the inputs and the cuRAND noise are stored.

usage: python tests/golden/make_ref_vectors.py [out_dir]   (default: tests/golden)
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))

# (N, D, bits, numpy seed, torch seed): odd and ragged shapes on purpose
PACK_CASES = [
    (64, 128, 1, 1, 11), (64, 128, 2, 2, 12), (64, 128, 4, 3, 13), (64, 128, 8, 4, 14),
    (37, 13, 2, 5, 15), (131, 76, 2, 6, 16), (50, 602, 2, 7, 17), (29, 40, 4, 8, 18),
    (23, 32, 1, 9, 19), (4096, 128, 2, 10, 20),
]
SPMM_CASES = [(300, 64, 2000, 21), (257, 40, 1500, 22)]  # (nodes, K, nnz, seed)


def digest(a):
    """sha256 of an array's bytes as uint8[32]: keeps the fixture small; comparisons are bit-exact anyway."""
    import hashlib
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def make_x(N, D, seed):
    rng = np.random.default_rng(seed)
    return np.maximum(rng.standard_normal((N, D)).astype(np.float32), 0)


def make_graph(n, nnz, seed):
    rng = np.random.default_rng(seed)
    key = np.unique(rng.integers(0, n * n, size=nnz, dtype=np.int64))
    row, col = key // n, key % n
    val = rng.standard_normal(key.size).astype(np.float32)
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    return rowptr, col, val


def main(out_dir):
    import ref_quantization as rq
    import ref_spmm as rs
    dev = "cuda"
    out = {}
    for i, (N, D, bits, nseed, tseed) in enumerate(PACK_CASES):
        x = torch.from_numpy(make_x(N, D, nseed)).to(dev)
        mn, mx = x.min(1)[0], x.max(1)[0]
        scale = (2 ** bits - 1) / (mx - mn)          # exact/exact/ops.py:39
        torch.manual_seed(tseed)
        offset = int(torch.cuda.default_generators[torch.cuda.current_device()].get_offset())
        packed = rq.pack_single_precision(x, mn, mx, scale, bits, True)   # ops.py:40
        torch.cuda.synchronize()
        sb, mb = scale.to(torch.bfloat16), mn.to(torch.bfloat16)           # ops.py:80-81
        unpacked = rq.unpack_single_precision(packed, bits, sb.float(), mb.float(), N, D)  # ops.py:94-97
        small = N * D <= 8192
        out[f"pack{i}_meta"] = np.array([N, D, bits, nseed, tseed, offset], np.int64)
        pk = packed.cpu().numpy().view(np.uint8)[:-1]
        out[f"pack{i}_packed"] = pk if small else digest(pk)
        out[f"pack{i}_scale"] = scale.cpu().numpy() if small else scale.cpu().numpy()[:64]
        out[f"pack{i}_min"] = mn.cpu().numpy() if small else mn.cpu().numpy()[:64]
        out[f"pack{i}_unpacked"] = digest(unpacked.cpu().numpy())
    for i, (n, K, nnz, seed) in enumerate(SPMM_CASES):
        rowptr, col, val = make_graph(n, nnz, seed)
        mat = np.random.default_rng(seed + 100).standard_normal((n, K)).astype(np.float32)
        t = lambda a: torch.from_numpy(a).to(dev)
        for red in ("sum", "mean"):
            for hv in (True, False):
                v = t(val) if hv else None
                if red == "sum":
                    o = rs.spmm_sum_fw(None, t(rowptr), t(col), v, None, None, t(mat))
                else:
                    o = rs.spmm_mean_fw(None, t(rowptr), t(col), v, None, None, None, t(mat))
                out[f"spmm{i}_{red}_{int(hv)}"] = digest(o.cpu().numpy())
        out[f"spmm{i}_meta"] = np.array([n, K, nnz, seed], np.int64)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


HALF_PACK_CASES = [(64, 128, 1, 31, 41), (64, 128, 2, 32, 42), (131, 76, 4, 33, 43), (37, 13, 8, 34, 44),
                   (1000, 256, 2, 35, 45)]
MORE_SPMM_CASES = [(300, 64, 2000, 51), (257, 40, 1500, 52)]


def make_half(N, D, seed):
    return (np.random.default_rng(seed).standard_normal((N, D)) * 2.5).astype(np.float16)


def main_more(out_dir):
    """Second fixture: the half instantiations of pack / unpack / SpMM, and on fp32 the max / min aggregation
    (values and winning-edge positions) and the edge-value gradient."""
    import ref_quantization as rq
    import ref_spmm as rs
    dev = "cuda"
    out = {}
    t = lambda a: torch.from_numpy(a).to(dev)
    for i, (N, D, bits, nseed, tseed) in enumerate(HALF_PACK_CASES):
        x = t(make_half(N, D, nseed))
        mn, mx = x.min(1)[0], x.max(1)[0]
        scale = (2 ** bits - 1) / (mx - mn)          # half tensor ops (exact/exact/ops.py:39 on an fp16 activation)
        torch.manual_seed(tseed)
        offset = int(torch.cuda.default_generators[torch.cuda.current_device()].get_offset())
        packed = rq.pack_single_precision(x, mn, mx, scale, bits, True)
        torch.cuda.synchronize()
        unpacked = rq.unpack_single_precision(packed, bits, scale, mn, N, D)   # fp16 statistics stay fp16 (ops.py:82-83)
        out[f"hpack{i}_meta"] = np.array([N, D, bits, nseed, tseed, offset], np.int64)
        out[f"hpack{i}_packed"] = digest(packed.cpu().numpy().view(np.uint8)[:-1])
        out[f"hpack{i}_scale"] = digest(scale.cpu().numpy().view(np.uint16))
        out[f"hpack{i}_min"] = digest(mn.cpu().numpy().view(np.uint16))
        out[f"hpack{i}_unpacked"] = digest(unpacked.cpu().numpy().view(np.uint16))
    for i, (n, K, nnz, seed) in enumerate(MORE_SPMM_CASES):
        rowptr, col, val = make_graph(n, nnz, seed)
        row = np.repeat(np.arange(n), np.diff(rowptr))
        mat = np.random.default_rng(seed + 100).standard_normal((n, K)).astype(np.float32)
        grad = np.random.default_rng(seed + 200).standard_normal((n, K)).astype(np.float32)
        math, valh = mat.astype(np.float16), (val * 0.5).astype(np.float16)
        for red in ("sum", "mean"):
            for hv in (True, False):
                v = t(valh) if hv else None
                if red == "sum":
                    o = rs.spmm_sum_fw(None, t(rowptr), t(col), v, None, None, t(math))
                else:
                    o = rs.spmm_mean_fw(None, t(rowptr), t(col), v, None, None, None, t(math))
                out[f"hspmm{i}_{red}_{int(hv)}"] = digest(o.cpu().numpy().view(np.uint16))
            # the edge-value gradient through spmm_{sum,mean}_bw (spmm.cc:57-79, 115-139 -> spmm_value_bw_kernel)
            perm = np.argsort(col * n + row, kind="stable")
            colptr = np.zeros(n + 1, np.int64)
            np.cumsum(np.bincount(col, minlength=n), out=colptr[1:])
            args = [t(row), t(rowptr), t(col), t(val)]
            if red == "mean":
                args.append(t(np.diff(rowptr)))
            args += [t(colptr), t(perm), t(mat), t(grad), True, True, False]
            gv = (rs.spmm_sum_bw if red == "sum" else rs.spmm_mean_bw)(*args)[0]
            out[f"valuebw{i}_{red}"] = digest(gv.cpu().numpy())
        for red, fn in (("max", rs.spmm_max_fw), ("min", rs.spmm_min_fw)):
            for hv in (True, False):
                o, arg = fn(t(rowptr), t(col), t(val) if hv else None, t(mat))
                out[f"minmax{i}_{red}_{int(hv)}_out"] = digest(o.cpu().numpy())
                out[f"minmax{i}_{red}_{int(hv)}_arg"] = digest(arg.cpu().numpy().astype(np.int64))
        out[f"more{i}_meta"] = np.array([n, K, nnz, seed], np.int64)
    path = os.path.join(out_dir, "ref_vectors_more.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    where = sys.argv[1] if len(sys.argv) > 1 else HERE
    main(where)
    main_more(where)
