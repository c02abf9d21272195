"""Host-side helpers of the activation-compression path that the reference keeps in exact/exact/utils.py: index
narrowing, pinned-host parking of saved tensors, memory accounting."""
import torch

_INT32_MAX = 2 ** 31 - 1
_ITEMSIZE = {torch.int64: 8, torch.float64: 8, torch.float32: 4, torch.int32: 4, torch.bfloat16: 2,
             torch.float16: 2, torch.int16: 2, torch.int8: 1, torch.uint8: 1, torch.bool: 1}


def cast_low_bit_int(idx_vec):
    """Index vector narrowed to int32 when its values allow it (the reference also narrows to int16, utils.py:9-19;
    the SpMM here reads int32 or int64 indices only)."""
    if idx_vec is None:
        return None
    if idx_vec.dtype != torch.int64:
        raise TypeError("cast_low_bit_int expects int64 indices")
    fits = idx_vec.numel() == 0 or int(idx_vec.max()) < _INT32_MAX
    return idx_vec.to(torch.int32) if fits else idx_vec


def swap_to_cpu(tensor):
    """A pinned host copy of `tensor`, enqueued without waiting (config.swap; utils.py:31-34)."""
    host = torch.empty_like(tensor, device="cpu", pin_memory=True)
    return host.copy_(tensor, non_blocking=True)


def get_memory_usage(gpu, print_info=False):
    """Bytes torch has allocated on `gpu` (utils.py:37-44); optionally prints allocated and reserved MB."""
    used = torch.cuda.memory_allocated(gpu)
    if print_info:
        mb = 1.0 / (1024 * 1024)
        print(f"allocated: {used * mb:.2f} MB", flush=True)
        print(f"reserved:  {torch.cuda.memory_reserved(gpu) * mb:.2f} MB", flush=True)
    return used


def compute_tensor_bytes(tensors):
    """Total payload bytes of a tensor or a sequence of tensors (utils.py:47-66)."""
    seq = tensors if isinstance(tensors, (list, tuple)) else (tensors,)
    total = 0
    for t in seq:
        if t.dtype not in _ITEMSIZE:
            raise ValueError(f"unsupported dtype {t.dtype}")
        total += t.numel() * _ITEMSIZE[t.dtype]
    return total


def empty_cache(ratio):
    """torch.cuda.empty_cache() when less than `ratio` of the reserved memory is in use (utils.py:69-75)."""
    if ratio is None:
        return
    reserved = torch.cuda.memory_reserved()
    if reserved > 0 and torch.cuda.memory_allocated() < ratio * reserved:
        torch.cuda.empty_cache()
