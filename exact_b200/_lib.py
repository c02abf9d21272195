"""ctypes binding of libexact_b200.so -- the only route from Python to the CUDA kernels.

There is no CPU or eager-PyTorch fallback: if the library is missing or a call fails, an exception
is raised.
"""
import ctypes
import os

from . import _build

_lib = None

c_i64 = ctypes.c_int64
c_u64 = ctypes.c_uint64
c_int = ctypes.c_int
c_f32 = ctypes.c_float
c_ptr = ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/exact_b200.h declaration by declaration.
SIGNATURES = {
    "exact_version": (c_int, []),
    "exact_last_error": (ctypes.c_char_p, []),
    "exact_packed_bytes": (c_i64, [c_i64, c_i64, c_int]),
    "exact_quantize_pack": (c_int, [c_ptr, c_int, c_i64, c_i64, c_int, c_ptr, c_u64, c_u64, c_i64,
                                    c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr]),
    "exact_pack_single_precision": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr,
                                            c_u64, c_u64, c_i64, c_ptr, c_ptr]),
    "exact_unpack_single_precision": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_int, c_i64, c_i64, c_ptr, c_ptr]),
    "exact_mask_words": (c_i64, [c_i64]),
    "exact_act_quantized_relu_forward": (c_int, [c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_act_quantized_relu_backward": (c_int, [c_ptr, c_ptr, c_i64, c_ptr, c_ptr]),
    "exact_act_quantized_dropout_forward": (c_int, [c_ptr, c_i64, c_f32, c_ptr, c_u64, c_u64, c_i64, c_ptr, c_ptr,
                                                    c_ptr]),
    "exact_act_quantized_dropout_backward": (c_int, [c_ptr, c_ptr, c_i64, c_f32, c_ptr, c_ptr]),
    "exact_act_quantized_relu_dropout_forward": (c_int, [c_ptr, c_i64, c_f32, c_ptr, c_u64, c_u64, c_i64, c_ptr, c_ptr,
                                                         c_ptr]),
    "exact_spmm_split": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_i64, c_ptr, c_ptr, c_ptr,
                                 c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_spmm_split_static": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_i64, c_ptr, c_ptr,
                                        c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr]),
    "exact_rp_workspace_bytes": (c_i64, [c_i64, c_i64]),
    "exact_rp_quantize_pack": (c_int, [c_ptr, c_i64, c_i64, c_ptr, c_i64, c_int, c_u64, c_u64, c_i64, c_ptr, c_ptr,
                                       c_ptr, c_ptr, c_ptr, c_ptr]),
    "exact_unpack_rp_workspace_bytes": (c_i64, [c_i64, c_i64]),
    "exact_unpack_dequant_rp": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_rademacher": (c_int, [c_u64, c_u64, c_i64, c_i64, c_ptr, c_ptr]),
    "exact_rows_mask_count": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_rows_compact_write": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_rows_expand": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_i64, c_i64, c_ptr, c_i64, c_ptr]),
    "exact_linear_workspace_bytes": (c_i64, [c_i64, c_i64, c_i64]),
    "exact_linear_forward": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_i64, c_ptr, c_i64, c_i64, c_ptr, c_i64,
                                     c_i64, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_ptr]),
    "exact_spmm": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr, c_ptr]),
}

DTYPE_F32 = 0
DTYPE_BF16 = 1
REDUCE = {"sum": 0, "add": 0, "mean": 1}


class ExactB200Error(RuntimeError):
    pass


def lib_path():
    """The in-tree library, or the file EXACT_B200_LIBRARY names."""
    return os.environ.get("EXACT_B200_LIBRARY") or _build.LIB


def load():
    """Load (once) and return the ctypes handle.  Raises if the library has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ExactB200Error(
                f"{path} not found: build it with `python -m exact_b200._build` (needs nvcc); "
                "exact_b200 has no fallback path")
        lib = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is missing: fail loudly
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc, what):
    if rc != 0:
        msg = load().exact_last_error()
        raise ExactB200Error(f"{what} failed (code {rc}): {msg.decode() if msg else ''}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr():
    import torch
    return torch.cuda.current_stream().cuda_stream


# ---- launch accounting and optional per-kernel CUDA-event timing ----------------------------------
LAUNCHES = 0      # kernels of this library launched so far (each kernel-launching entry point = 1)
TIMER = None      # a KernelTimer while a benchmark wants per-kernel device times


class KernelTimer:
    """Brackets every library call with CUDA events on the launching stream.  summary() synchronises
    and returns, per entry point: launches, total ms, algorithmic bytes."""

    def __init__(self):
        self.records = {}

    def bracket(self, name, nbytes, thunk):
        import torch
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        rc = thunk()
        b.record()
        self.records.setdefault(name, []).append((a, b, nbytes))
        return rc

    def summary(self):
        import torch
        torch.cuda.synchronize()
        out = {}
        for name, recs in self.records.items():
            ms = [a.elapsed_time(b) for a, b, _ in recs]
            out[name] = {"launches": len(recs), "ms": sum(ms), "bytes": sum(r[2] for r in recs)}
        return out


def invoke(name, nbytes, *args):
    """Call entry point `name`; count it as one kernel launch; raise on a non-zero return code."""
    global LAUNCHES
    fn = getattr(load(), name)
    LAUNCHES += 1
    if TIMER is not None:
        rc = TIMER.bracket(name, nbytes, lambda: fn(*args))
    else:
        rc = fn(*args)
    check(rc, name)
