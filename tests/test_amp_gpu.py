"""The AMP path (exact/exact/ops.py:130, 260, 313: custom_fwd(cast_inputs=torch.float16) on the quantised ops): under
torch.autocast the quantised layers run on fp16 tensors through the half kernels (fp16 pack / unpack with fp16
statistics, fp16 SpMM, fp16 masks) and train like the fp32 run."""
import pytest
import torch
import torch.nn.functional as F

from exact_b200 import QModule, _lib, config, graphs, models

pytestmark = pytest.mark.gpu


def _run(cfg_name, amp, seed=3, nodes=3000):
    c = dict(graphs.CONFIGS[cfg_name])
    config.fused_rp = True
    config.compress_activation = True
    config.simulate = False
    config.activation_compression_bits = [8]
    config.kept_frac = 1.0
    config.row_offset = 0
    adj = graphs.build_graph(c, seed=seed, device="cuda", nodes=nodes)
    if c["gcn_norm"]:
        from exact_b200 import gcn_norm
        adj = gcn_norm(adj, add_self_loops=False)
    n = adj.size(0)
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n, c["feats"], generator=gen).cuda()
    y = torch.randint(c["classes"], (n,), generator=gen).cuda()
    torch.manual_seed(seed)
    cls = models.GCN if c["model"] == "gcn" else models.SAGE
    net = QModule(cls(c["feats"], c["hidden"], c["classes"], c["layers"], dropout=c["dropout"],
                      batch_norm=c["batch_norm"])).cuda().train()
    config.manual_seed(seed)
    _lib.TIMER = _lib.KernelTimer()
    with torch.autocast("cuda", dtype=torch.float16, enabled=amp):
        out = net(x, adj)
        loss = F.cross_entropy(out.float(), y)
    loss.backward()
    calls = set(_lib.TIMER.summary())
    _lib.TIMER = None
    grads = {k: p.grad.detach().clone() for k, p in net.model.named_parameters()}
    return float(loss), out.detach().float(), grads, calls


@pytest.mark.parametrize("cfg_name", ["cfg4", "cfg2"])
def test_autocast_runs_the_half_kernels_and_matches_fp32(cfg_name):
    loss32, out32, g32, calls32 = _run(cfg_name, False)
    loss16, out16, g16, calls16 = _run(cfg_name, True)
    assert {"exact_quantize_pack_f16", "exact_spmm_f16", "exact_unpack_single_precision_f16"} <= calls16
    if cfg_name == "cfg4":   # in configuration 2 the activations follow a batch norm, which autocast keeps in fp32
        assert {"exact_act_quantized_forward_f16", "exact_act_quantized_backward_f16"} <= calls16
    assert not any(name.endswith("_f16") for name in calls32)
    assert abs(loss16 - loss32) < 2e-2 * abs(loss32)
    assert float((out16 - out32).norm() / out32.norm()) < 3e-2
    # a bias in front of a batch norm has a gradient of rounding noise only: compare against the layer's scale
    scale = max(float(v.norm()) for v in g32.values())
    for k, g in g16.items():
        assert g.dtype == torch.float32 and bool(torch.isfinite(g).all()), k
        err = float((g - g32[k]).norm())
        assert err < 0.1 * float(g32[k].norm()) + 2e-3 * scale, (k, err, float(g32[k].norm()))
