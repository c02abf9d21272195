"""Python-visible operator modules with the names and signatures of the reference's compiled
extensions (exact/setup.py:5-22): quantization, spmm, backward_func.  Each function forwards to the
C ABI of libexact_b200.so."""
from . import backward_func, quantization, spmm  # noqa: F401
