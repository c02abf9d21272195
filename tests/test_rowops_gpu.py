"""exact_rows_scale_colsum: D^-1 g (zero-padded) and g.sum(0) in one pass over g, against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200.cpp_extension import backward_func as B
from helpers import normal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K", [(5000, 256), (3001, 47), (2000, 100), (1500, 13), (40000, 64), (1024, 1)])
@pytest.mark.parametrize("scaled", [True, False])
def test_rows_scale_colsum(N, K, scaled):
    g = normal(N, K, 61)
    rs = (1.0 / np.random.default_rng(62).integers(1, 50, N)).astype(np.float32)
    gt, rt = torch.from_numpy(g).cuda(), torch.from_numpy(rs).cuda()
    out, colsum = B.rows_scale_colsum(gt, rt if scaled else None, want_scaled=True, want_colsum=True)
    ref_out, ref_sum = oracle.rows_scale_colsum(g, rs if scaled else None)
    assert out.shape == ref_out.shape and np.array_equal(out.cpu().numpy(), ref_out)      # one fp32 multiply: exact
    err = np.abs(colsum.cpu().numpy() - ref_sum)
    assert np.all(err <= 4e-6 * np.sqrt(N) * np.abs(g).max() + 1e-6 * np.abs(ref_sum))
    # the column sums alone, a strided view (rows of a wider matrix), and run-to-run identity
    wide = torch.from_numpy(normal(N, K + 8, 63)).cuda()
    _, c1 = B.rows_scale_colsum(wide[:, :K])
    _, c2 = B.rows_scale_colsum(wide[:, :K])
    assert torch.equal(c1, c2)
    assert np.all(np.abs(c1.cpu().numpy() - wide[:, :K].double().sum(0).cpu().numpy())
                  <= 4e-6 * np.sqrt(N) * float(wide.abs().max()) + 1e-6)


def test_small_inputs_take_the_framework_ops():
    g = torch.randn(100, 12, device="cuda")
    out, colsum = B.rows_scale_colsum(g, torch.ones(100, device="cuda"), want_scaled=True)
    assert torch.equal(out, g) and torch.allclose(colsum, g.sum(0))
