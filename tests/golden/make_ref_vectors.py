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


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
