"""CPU checks of the C-ABI library: it loads, exports every symbol include/*.h declares, and its
argument validation works without touching a GPU."""
import ctypes
import glob
import os
import re

from exact_b200 import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        src = open(h).read()
        names += re.findall(r"EXACT_API\s+[\w\s\*]+?\b(exact_\w+)\s*\(", src)
    return sorted(set(names))


def test_header_symbols_are_exported():
    names = declared_symbols()
    assert len(names) >= 12
    lib = ctypes.CDLL(_build.LIB)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"


def test_bindings_cover_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.exact_version() >= 100
    assert lib.exact_packed_bytes(4096, 128, 2) == 131072
    assert lib.exact_packed_bytes(169343, 256, 2) == 42336 * 256
    assert lib.exact_packed_bytes(5, 3, 8) == 15
    assert lib.exact_packed_bytes(5, 3, 3) == -1
    assert lib.exact_mask_words(0) == 0 and lib.exact_mask_words(129) == 8


def test_bad_arguments_are_rejected_before_any_launch():
    lib = _lib.load()
    rc = lib.exact_quantize_pack(None, 0, 8, 8, 3, None, 0, 0, 0, None, None, None, None, None, None)
    assert rc == 1 and b"bits" in lib.exact_last_error()
    rc = lib.exact_quantize_pack(None, 0, 8, 8, 2, None, 0, 0, 4, None, None, None, None, None, None)
    assert rc == 1 and b"row_offset" in lib.exact_last_error()
    rc = lib.exact_quantize_pack(None, 0, 8, 8, 2, None, 0, 0, 0, None, None, None, None, None, None)
    assert rc == 1 and b"null" in lib.exact_last_error()
    rc = lib.exact_spmm(None, None, 2, None, None, 4, 4, 0, None, None)
    assert rc == 1 and b"idx_bytes" in lib.exact_last_error()
    # empty inputs are a no-op, as torch.empty-shaped calls are in the reference
    assert lib.exact_quantize_pack(None, 0, 0, 128, 2, None, 0, 0, 0, None, None, None, None, None, None) == 0
