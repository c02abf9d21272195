"""Small helpers kept from the reference's exact/exact/utils.py (memory accounting and index casts)."""
import json
from collections import OrderedDict

import numpy as np
import torch


def cast_low_bit_int(idx_vec):
    """utils.py:9-19.  The B200 SpMM reads int32 or int64 indices, so int16 is never produced."""
    if idx_vec is None:
        return idx_vec
    assert idx_vec.dtype == torch.int64
    if idx_vec.numel() == 0 or int(idx_vec.max()) < np.iinfo(np.int32).max:
        return idx_vec.to(torch.int32)
    return idx_vec


def cast_adj(data):
    """utils.py:22-28: narrow every index array of data.adj_t in place."""
    data.adj_t.to_int32_()


def swap_to_cpu(tensor):
    """utils.py:31-34."""
    tensor_cpu = torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu", pin_memory=True)
    tensor_cpu.copy_(tensor, non_blocking=True)
    return tensor_cpu


def get_memory_usage(gpu, print_info=False):
    """utils.py:37-44."""
    allocated = torch.cuda.memory_allocated(gpu)
    reserved = torch.cuda.memory_reserved(gpu)
    if print_info:
        print("allocated: %.2f MB" % (allocated / 1024 / 1024), flush=True)
        print("reserved:  %.2f MB" % (reserved / 1024 / 1024), flush=True)
    return allocated


_BYTES = {torch.int64: 8, torch.float64: 8, torch.float32: 4, torch.int32: 4, torch.bfloat16: 2,
          torch.float16: 2, torch.int16: 2, torch.int8: 1, torch.uint8: 1, torch.bool: 1}


def compute_tensor_bytes(tensors):
    """utils.py:47-66."""
    if not isinstance(tensors, (list, tuple)):
        tensors = [tensors]
    ret = 0
    for x in tensors:
        if x.dtype not in _BYTES:
            raise ValueError(x.dtype)
        ret += int(np.prod(x.size())) * _BYTES[x.dtype]
    return ret


def empty_cache(ratio):
    """utils.py:69-75."""
    if ratio is None:
        return
    allocated = torch.cuda.memory_allocated()
    reserved = torch.cuda.memory_reserved()
    if reserved > 0 and allocated / reserved < ratio:
        torch.cuda.empty_cache()


class GlobalExpRecorder:
    """utils.py:85-103."""

    def __init__(self):
        self.val_dict = OrderedDict()

    def record(self, key, value, float_round=6):
        if isinstance(value, (np.int32, np.int64)):
            value = int(value)
        if isinstance(value, (float, np.float32, np.float64)):
            value = round(float(value), float_round)
        self.val_dict[key] = value

    def dump(self, filename):
        with open(filename, "a") as fout:
            fout.write(json.dumps(self.val_dict) + "\n")

    def clear(self):
        pass


exp_recorder = GlobalExpRecorder()
