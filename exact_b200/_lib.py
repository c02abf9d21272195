"""ctypes binding of libexact_b200.so -- the only route from Python to the CUDA kernels.

There is no CPU or eager-PyTorch fallback: if the library is missing or a call fails, an exception
is raised.
"""
import ctypes
import time
import os
import threading

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
    "exact_status": (c_int, [ctypes.POINTER(c_int), c_ptr]),
    "exact_status_async": (c_int, [c_ptr, c_ptr]),
    "exact_clear_status": (c_int, [c_ptr]),
    "exact_set_status": (c_int, [c_int, c_ptr]),
    "exact_packed_bytes": (c_i64, [c_i64, c_i64, c_int]),
    "exact_quantize_pack": (c_int, [c_ptr, c_int, c_i64, c_i64, c_int, c_ptr, c_u64, c_u64, c_i64,
                                    c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr]),
    "exact_pack_single_precision": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr,
                                            c_u64, c_u64, c_i64, c_ptr, c_ptr]),
    "exact_unpack_single_precision": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_int, c_i64, c_i64, c_ptr, c_ptr]),
    "exact_mask_words": (c_i64, [c_i64]),
    "exact_act_quantized_relu_forward": (c_int, [c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_act_quantized_relu_backward": (c_int, [c_ptr, c_ptr, c_i64, c_ptr, c_ptr]),
    "exact_act_quantized_leaky_relu_forward": (c_int, [c_ptr, c_i64, c_f32, c_ptr, c_ptr, c_ptr]),
    "exact_act_quantized_leaky_relu_backward": (c_int, [c_ptr, c_ptr, c_i64, c_f32, c_ptr, c_ptr]),
    "exact_act_quantized_dropout_forward": (c_int, [c_ptr, c_i64, c_f32, c_ptr, c_u64, c_u64, c_i64, c_ptr, c_ptr,
                                                    c_ptr]),
    "exact_act_quantized_dropout_backward": (c_int, [c_ptr, c_ptr, c_i64, c_f32, c_ptr, c_ptr]),
    "exact_act_quantized_relu_dropout_forward": (c_int, [c_ptr, c_i64, c_f32, c_ptr, c_u64, c_u64, c_i64, c_ptr, c_ptr,
                                                         c_ptr]),
    "exact_spmm_split": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_i64, c_ptr, c_ptr, c_ptr,
                                 c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_spmm_split_static": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_i64, c_ptr, c_ptr,
                                        c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr]),
    "exact_spmm_split_routed": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_i64, c_ptr, c_ptr,
                                        c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_i64, c_i64,
                                        ctypes.POINTER(c_ptr), c_int, c_ptr]),
    "exact_quantize_pack_f16": (c_int, [c_ptr, c_i64, c_i64, c_int, c_ptr, c_u64, c_u64, c_i64, c_ptr, c_ptr, c_ptr, c_ptr]),
    "exact_pack_single_precision_f16": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr, c_u64, c_u64, c_i64,
                                                c_ptr, c_ptr]),
    "exact_unpack_single_precision_f16": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_ptr]),
    "exact_act_quantized_forward_f16": (c_int, [c_int, c_ptr, c_i64, c_f32, c_ptr, c_u64, c_u64, c_i64, c_ptr, c_ptr,
                                                c_ptr]),
    "exact_act_quantized_backward_f16": (c_int, [c_int, c_ptr, c_ptr, c_i64, c_f32, c_ptr, c_ptr]),
    "exact_spmm_f16": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr, c_ptr]),
    "exact_rows_scale_colsum_workspace_bytes": (c_i64, [c_i64]),
    "exact_rows_scale_colsum": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_ptr]),
    "exact_bn_backward_workspace_bytes": (c_i64, [c_i64]),
    "exact_bn_backward_from_packed": (c_int, [c_ptr, c_i64, c_i64, c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int,
                                              c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr]),
    "exact_crows_slot_bytes": (c_i64, [c_i64]),
    "exact_crows_pack": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_i64, ctypes.POINTER(c_ptr), c_int, c_ptr, c_ptr]),
    "exact_crows_unpack": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_i64, c_ptr]),
    "exact_cols_scatter": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_i64, c_i64, ctypes.POINTER(c_ptr), c_int, c_ptr]),
    "exact_rows_scatter": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_i64, c_i64, ctypes.POINTER(c_ptr), c_int, c_ptr]),
    "exact_peer_alloc": (c_int, [c_i64, ctypes.POINTER(c_ptr)]),
    "exact_peer_free": (c_int, [c_ptr]),
    "exact_peer_export": (c_int, [c_ptr, c_ptr]),
    "exact_peer_import": (c_int, [c_ptr, ctypes.POINTER(c_ptr)]),
    "exact_peer_close": (c_int, [c_ptr]),
    "exact_rp_workspace_bytes": (c_i64, [c_i64, c_i64]),
    "exact_rp_quantize_pack": (c_int, [c_ptr, c_i64, c_i64, c_ptr, c_i64, c_int, c_u64, c_u64, c_i64, c_ptr, c_ptr,
                                       c_ptr, c_ptr, c_ptr, c_ptr]),
    "exact_unpack_rp_workspace_bytes": (c_i64, [c_i64, c_i64]),
    "exact_unpack_dequant_rp": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_rademacher": (c_int, [c_u64, c_u64, c_i64, c_i64, c_ptr, c_ptr]),
    "exact_grad_weight_workspace_bytes": (c_i64, [c_i64, c_i64, c_int]),
    "exact_grad_weight_from_packed": (c_int, [c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_i64,
                                              c_int, c_ptr, c_i64, c_ptr, c_i64, c_ptr]),
    "exact_rows_mask_count": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_rows_compact_write": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "exact_rows_expand": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_i64, c_i64, c_ptr, c_i64, c_ptr]),
    "exact_linear_workspace_bytes": (c_i64, [c_i64, c_i64, c_i64]),
    "exact_linear_forward": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_i64, c_ptr, c_i64, c_i64, c_ptr, c_i64,
                                     c_i64, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_ptr]),
    "exact_spmm_minmax": (c_int, [c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_int, c_ptr, c_ptr, c_ptr]),
    "exact_spmm_value_bw": (c_int, [c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr, c_ptr]),
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


_tls = threading.local()


def ptr(t):
    """Device pointer of a tensor (None -> NULL).  The tensor's device is noted for the next invoke(), which
    launches on that device and refuses arguments that live on different devices."""
    if t is None:
        return None
    if t.is_cuda:
        devs = getattr(_tls, "devices", None)
        if devs is None:
            devs = _tls.devices = set()
        devs.add(t.device.index)
    return t.data_ptr()


class _CurrentStream:
    """Placeholder for "the current stream of the device the call runs on"; invoke() resolves it."""


STREAM = _CurrentStream()


def stream_ptr():
    return STREAM


def resolve_device(noted, current):
    """The device a call runs on, given the devices of its tensor arguments and the current device."""
    if len(noted) > 1:
        raise ExactB200Error(f"arguments live on different CUDA devices: {sorted(noted)}")
    return next(iter(noted)) if noted else current


# ---- device-side status ------------------------------------------------------------------------------
# Entry points whose kernels wait on on-chip barriers (bounded): after one of them ran on a device, the next
# check_status() of that device reads the library's status word.
STATUS_CALLS = {"exact_rp_quantize_pack", "exact_unpack_dequant_rp", "exact_linear_forward",
                "exact_grad_weight_from_packed"}
STATUS_PENDING = {}   # device index -> True while unchecked launches exist
STATUS_NAMES = {1: "exact_rp_quantize_pack", 2: "exact_unpack_dequant_rp", 4: "exact_linear_forward",
                8: "exact_grad_weight_from_packed"}


def raise_for_status(word):
    """ExactB200Error naming the entry points whose bits are set in a non-zero status word."""
    if word:
        names = [n for bit, n in STATUS_NAMES.items() if word & bit] or ["an unknown kernel"]
        raise ExactB200Error(f"device status {word}: a bounded on-chip wait expired in {', '.join(names)}; "
                             "outputs since the last check are incomplete")


def check_status(device=None, force=False):
    """Raise ExactB200Error if a kernel of this library abandoned work on `device` (a bounded on-chip wait
    ran out) since the last check.  Synchronises the device's current stream, so it belongs where the
    caller synchronises anyway (reading the loss, the end of a step); without launches to check it is free."""
    import torch
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if not (force or STATUS_PENDING.get(dev)):
        return
    lib = load()
    word = c_int(0)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        check(lib.exact_status(ctypes.byref(word), stream), "exact_status")
        STATUS_PENDING[dev] = False
        if word.value != 0:
            check(lib.exact_clear_status(stream), "exact_clear_status")
    raise_for_status(word.value)


_POLLS = {}   # device index -> (pinned int32 tensor, event) of the status copy in flight


def poll_status(device=None):
    """check_status without a synchronisation: looks at the copy of the status word enqueued by the previous
    poll (if it has arrived) and enqueues the next one behind the work launched so far.  A training loop that
    polls once per step learns of an abandoned kernel one step late and never waits for the GPU."""
    import torch
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    lib = load()
    prev = _POLLS.get(dev)
    word = 0
    if prev is not None:
        pinned, event = prev
        if not event.query():
            return            # still in flight: look again at the next poll
        word = int(pinned[0])
    else:
        pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
    if word == 0 and not STATUS_PENDING.get(dev):
        _POLLS.pop(dev, None)
        return
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev)
        if word != 0:
            check(lib.exact_clear_status(stream.cuda_stream), "exact_clear_status")
        check(lib.exact_status_async(pinned.data_ptr(), stream.cuda_stream), "exact_status_async")
        event = torch.cuda.Event()
        event.record(stream)
    STATUS_PENDING[dev] = False
    _POLLS[dev] = (pinned, event)
    raise_for_status(word)


# ---- launch accounting and optional per-kernel CUDA-event timing ----------------------------------
LAUNCHES = 0      # kernels of this library launched so far (each kernel-launching entry point = 1)
TIMER = None      # a KernelTimer while a benchmark wants per-kernel device times
HOST_CLOCK = None  # [ns, calls] while a benchmark wants the host time spent inside invoke() (binding + C entry point)


LIBRARY_CALLS = {}   # name -> calls: dense work of the path handed to a library kernel (torch) instead of this library's


def note_library_call(name):
    """Counts a dense operation of the path that went to a library GEMM (shape or dtype outside this library's
    tensor-core kernels); bench.py reports the counts per step next to its own launches."""
    LIBRARY_CALLS[name] = LIBRARY_CALLS.get(name, 0) + 1


class KernelTimer:
    """Brackets every library call with CUDA events on the launching stream.  summary() synchronises
    and returns, per entry point: launches, total ms, algorithmic bytes (what must move at least once) and,
    for gathers, the bytes requested from L2 when nothing is reused (`l2_bytes`) and edges x columns; for the
    dense-layer GEMM the tensor-core flop (extra keyword arguments of invoke())."""

    def __init__(self):
        self.records = {}

    def bracket(self, name, nbytes, thunk, extra=None):
        import torch
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        rc = thunk()
        b.record()
        self.records.setdefault(name, []).append((a, b, nbytes, extra or {}))
        return rc

    def summary(self):
        import torch
        torch.cuda.synchronize()
        out = {}
        for name, recs in self.records.items():
            ms = [r[0].elapsed_time(r[1]) for r in recs]
            out[name] = {"launches": len(recs), "ms": sum(ms), "bytes": sum(r[2] for r in recs)}
            for key in ("l2_bytes", "flops", "edge_columns"):
                if any(key in r[3] for r in recs):
                    out[name][key] = sum(r[3].get(key, r[2] if key == "l2_bytes" else 0) for r in recs)
        return out


def invoke(name, nbytes, *args, device=None, **extra):
    """Call entry point `name` on the device its tensor arguments live on (made current for the call, with
    that device's current stream); count it as one kernel launch; raise on a non-zero return code."""
    global LAUNCHES
    import torch
    fn = getattr(load(), name)
    noted = getattr(_tls, "devices", None) or set()
    _tls.devices = set()
    if device is not None:
        noted = noted | {torch.device(device).index if torch.device(device).index is not None
                         else torch.cuda.current_device()}
    dev = resolve_device(noted, torch.cuda.current_device())
    LAUNCHES += 1
    t0 = time.perf_counter_ns() if HOST_CLOCK is not None else 0
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        args = tuple(stream if a is STREAM else a for a in args)
        if TIMER is not None:
            rc = TIMER.bracket(name, nbytes, lambda: fn(*args), extra)
        else:
            rc = fn(*args)
    if HOST_CLOCK is not None:
        HOST_CLOCK[0] += time.perf_counter_ns() - t0
        HOST_CLOCK[1] += 1
    check(rc, name)
    if name in STATUS_CALLS:
        STATUS_PENDING[dev] = True
