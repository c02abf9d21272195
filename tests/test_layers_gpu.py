"""GPU parity of the layer stack (QLinear, QBatchNorm1d, QGCNConv, QSAGEConv, QModule) against the
CPU restatement in oracle/gnn.py, which draws the same Philox noise in the same order."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from oracle import gnn as O
from exact_b200 import QModule, config, graphs, models
from exact_b200.layers import QLinear
from helpers import normal

pytestmark = pytest.mark.gpu


def relfro(a, b):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).norm() / (b.norm() + 1e-30))


def adj_numpy(adj):
    rowptr, col, val = adj.csr()
    return (rowptr.cpu().numpy().astype(np.int64), col.cpu().numpy().astype(np.int64),
            None if val is None else val.cpu().numpy())


def reset_config(bits=2, kept_frac=1.0, seed=0, fused_rp=False):
    config.fused_rp = fused_rp
    config.compress_activation = True
    config.simulate = False
    config.activation_compression_bits = [bits]
    config.kept_frac = kept_frac
    config.row_offset = 0
    config.manual_seed(seed)


@pytest.mark.parametrize("kept_frac", [1.0, 0.125])
@pytest.mark.parametrize("bits", [2, 8])
def test_qlinear_gradients(bits, kept_frac):
    reset_config(bits, kept_frac, seed=7)
    N, D, O_ = 1000, 128, 64
    x = torch.from_numpy(normal(N, D, 1))
    lin = QLinear(D, O_).cuda().train()
    g = torch.from_numpy(normal(N, O_, 2))
    xg = x.cuda().requires_grad_()
    out = lin(xg)
    out.backward(g.cuda())
    cfg = O.Cfg(bits, kept_frac, True, seed=7)
    w, b = lin.weight.detach().cpu().requires_grad_(), lin.bias.detach().cpu().requires_grad_()
    xc = x.clone().requires_grad_()
    ref = O.OQLinear.apply(cfg, xc, w, b, None)
    ref.backward(g)
    assert relfro(out, ref) < 1e-5
    assert relfro(xg.grad, xc.grad) < 1e-5
    assert relfro(lin.bias.grad, b.grad) < 1e-5
    # x_hat is identical on both sides (same noise, same R), so only GEMM rounding differs
    assert relfro(lin.weight.grad, w.grad) < 1e-4
    # and the compressed gradient is close to the exact one (the reference prints this, test_op.py:322-330)
    if bits == 8 and kept_frac == 1.0:
        assert relfro(lin.weight.grad, g.t() @ x) < 0.02


def run_model(cfg_name, nodes, seed, kept_frac=None, fused_rp=False):
    c = dict(graphs.CONFIGS[cfg_name])
    if kept_frac is not None:
        c["kept_frac"] = kept_frac
    reset_config(c["bits"], c["kept_frac"], seed, fused_rp)
    adj = graphs.build_graph(c, seed=seed, device="cpu", nodes=nodes)
    if c["gcn_norm"]:
        from exact_b200 import gcn_norm
        adj = gcn_norm(adj, add_self_loops=False)
    n = adj.size(0)
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n, c["feats"], generator=gen)
    y = torch.randint(c["classes"], (n,), generator=gen)
    torch.manual_seed(seed)
    cls = models.GCN if c["model"] == "gcn" else models.SAGE
    kw = dict(dropout=c["dropout"], batch_norm=c["batch_norm"])
    net = QModule(cls(c["feats"], c["hidden"], c["classes"], c["layers"], **kw)).cuda().train()
    params = {k: v.detach().cpu().clone() for k, v in net.state_dict().items()
              if "running" not in k and "num_batches" not in k}
    config.manual_seed(seed)
    out = net(x.cuda(), adj.cuda())
    loss = F.cross_entropy(out, y.cuda())
    loss.backward()
    grads = {k: p.grad for k, p in net.model.named_parameters()}
    ocfg = O.Cfg(c["bits"], c["kept_frac"], True, seed=seed, fused_rp=fused_rp)
    oloss, oout, ograds = O.train_step(ocfg, c["model"], params, x, adj_numpy(adj), y, c["layers"],
                                       c["batch_norm"], c["dropout"])
    return loss.item(), out, grads, oloss, oout, ograds


def test_config1_gcn_two_layers_forward_backward():
    """Benchmark configuration 1, second half: 2-layer GCN 128->64->16 on a 4,096-node Erdos-Renyi graph."""
    loss, out, grads, oloss, oout, ograds = run_model("cfg1", None, seed=3)
    assert abs(loss - oloss) < 1e-4 * abs(oloss)
    assert relfro(out, oout) < 1e-5
    for k, g in grads.items():
        assert relfro(g, ograds[k]) < 2e-2, k


def test_gcn_with_bn_dropout_small():
    loss, out, grads, oloss, oout, ograds = run_model("cfg2", 3000, seed=4)
    assert abs(loss - oloss) < 1e-4 * abs(oloss)
    assert relfro(out, oout) < 1e-4
    for k, g in grads.items():
        assert relfro(g, ograds[k]) < 5e-2, k


@pytest.mark.parametrize("fused_rp", [False, True])
@pytest.mark.parametrize("cfg_name,nodes", [("cfg3", 2000), ("cfg4", 3000)])
def test_sage_projection_small(cfg_name, nodes, fused_rp):
    """With the fused projection+pack kernel the projected values carry tf32 input rounding, so a small
    fraction of codes differs from the CPU model's; the gradients still agree to a few percent."""
    loss, out, grads, oloss, oout, ograds = run_model(cfg_name, nodes, seed=5, fused_rp=fused_rp)
    assert abs(loss - oloss) < 1e-4 * abs(oloss)
    assert relfro(out, oout) < 1e-4
    for k, g in grads.items():
        assert relfro(g, ograds[k]) < (0.15 if fused_rp else 5e-2), k


def test_fused_projection_flips_few_codes():
    """Why the fused-projection bound above is looser: the tensor core truncates x to tf32, the projected values
    move by about 1e-3 relative, and a value that sits next to a stochastic-rounding boundary then takes the
    neighbouring INT2 code.  Counted here against the oracle fed the fp32 product and the same noise: a few
    codes per thousand differ, and never by more than one step."""
    from exact_b200.cpp_extension import quantization as Q
    N, D, k, bits = 20000, 256, 32, 2
    x = normal(N, D, 31)
    seed, off_r, off_n = 5, 1, 2
    R = oracle.rademacher(seed, off_r, D, k)
    packed, sb, mb = Q.rp_quantize_pack(torch.from_numpy(x).cuda(), torch.from_numpy(R).cuda(), bits, seed=seed,
                                        offset=off_n, row_offset=0)
    noise = oracle.noise_b200_rows(seed, off_n, N, k)
    op, _, _, _, _ = oracle.quantize_activation(oracle.input2rp(x, R), noise, bits)
    got = packed.cpu().numpy().view(np.uint8)[:-1]
    shifts = np.arange(0, 8, bits, dtype=np.uint8)
    codes_got = ((got[:, None] >> shifts) & 3).astype(np.int16)
    codes_ref = ((op[:, None] >> shifts) & 3).astype(np.int16)
    diff = codes_got != codes_ref
    frac = diff.mean()
    print(f"fused projection: {frac:.5f} of the INT2 codes differ from the fp32-product oracle")
    assert frac < 0.01
    assert np.abs(codes_got - codes_ref)[diff].max() <= 1 if diff.any() else True


def test_grad_weight_in_projected_space_equals_reference_order():
    """(g^T Xq) R^T against the reference's g^T (Xq R^T) (ops.py:164-169): same noise, same R."""
    N, D, O_ = 3000, 256, 64
    x = torch.from_numpy(normal(N, D, 1)).cuda()
    g = torch.from_numpy(normal(N, O_, 2)).cuda()
    grads = []
    for flag, fused_bwd in ((True, True), (False, False), (False, True)):
        reset_config(2, 0.125, seed=9, fused_rp=True)
        config.grad_weight_in_projected_space = flag
        torch.manual_seed(0)
        lin = QLinear(D, O_).cuda().train()
        xg = x.clone().requires_grad_()
        out = lin(xg)
        config.fused_rp = fused_bwd      # backward only: fused unpack + transpose projection, or unpack then matmul
        out.backward(g)
        grads.append((lin.weight.grad.clone(), xg.grad.clone(), lin.bias.grad.clone()))
    config.grad_weight_in_projected_space = True
    config.fused_rp = True
    assert relfro(grads[0][0], grads[1][0]) < 1e-5          # reassociation only
    assert relfro(grads[2][0], grads[1][0]) < 5e-3          # tf32 inputs in the fused reconstruction
    for gset in grads[1:]:
        assert torch.equal(grads[0][1], gset[1]) and torch.equal(grads[0][2], gset[2])


@pytest.mark.parametrize("cfg_name,nodes", [("cfg3", 2000), ("cfg4", 3000)])
def test_one_node_sage_layer_is_a_reassociation(cfg_name, nodes):
    """QSAGEConv as one autograd node (one GEMM for lin_l + lin_r; (A^T g) W_l in the last layer) against
    the separate QMatmul / QLinear nodes: the same compressed tensors drawn in the same order, results
    equal up to fp32 summation order.  One stochastic-rounding code of a saved INT2 tensor that lands on
    the other side of its threshold moves a weight gradient of this 2000-row problem by about 0.5 %,
    hence the looser bound on the gradients."""
    runs = []
    for fuse, first in ((True, True), (True, False), (False, True)):
        config.fuse_sage_layer, config.aggregate_gradient_first = fuse, first
        # the separate nodes pack the last layer's aggregate with the fused projection kernel's noise stream
        config.aggregate_projected_first = False
        try:
            loss, out, grads, _, _, _ = run_model(cfg_name, nodes, seed=6, fused_rp=True)
        finally:
            config.fuse_sage_layer, config.aggregate_gradient_first = True, True
            config.aggregate_projected_first = True
        runs.append((loss, out, grads))
    # inside the node the order of the backward products does not touch the forward pass
    assert runs[0][0] == runs[1][0] and torch.equal(runs[0][1], runs[1][1])
    for k, g in runs[0][2].items():
        assert relfro(g, runs[1][2][k]) < 5e-5, (k, relfro(g, runs[1][2][k]))
    assert abs(runs[0][0] - runs[2][0]) < 1e-5 * abs(runs[2][0]) and relfro(runs[0][1], runs[2][1]) < 1e-5
    for k, g in runs[0][2].items():
        assert relfro(g, runs[2][2][k]) < 3e-2, (k, relfro(g, runs[2][2][k]))


@pytest.mark.parametrize("cfg_name,nodes", [("cfg3", 2000), ("cfg4", 3000)])
def test_last_layer_aggregates_projected_first(cfg_name, nodes):
    """A SAGE layer with few outputs aggregates [x R | x W_l^T] instead of x (aggregation is linear): the model's
    output and loss equal those of the plain order up to fp32 reassociation, and so do the gradients up to the
    different rounding noise of the one saved tensor that is packed by another kernel (the last layer's projected
    aggregate, which only lin_l's weight gradient reads)."""
    runs = []
    for flag in (True, False):
        config.aggregate_projected_first = flag
        try:
            loss, out, grads, oloss, oout, ograds = run_model(cfg_name, nodes, seed=9, fused_rp=True)
        finally:
            config.aggregate_projected_first = True
        runs.append((loss, out, grads))
        if flag:   # the CPU restatement (reference order) with the same noise
            assert abs(loss - oloss) < 1e-4 * abs(oloss) and relfro(out, oout) < 1e-4
            for k, g in grads.items():
                assert relfro(g, ograds[k]) < 0.15, k
    assert abs(runs[0][0] - runs[1][0]) < 1e-5 * abs(runs[1][0]) and relfro(runs[0][1], runs[1][1]) < 1e-5
    c = graphs.CONFIGS[cfg_name]
    pad4 = lambda v: (v + 3) // 4 * 4
    reordered = set()
    for i in range(c["layers"]):
        in_f = c["feats"] if i == 0 else c["hidden"]
        out_f = c["classes"] if i == c["layers"] - 1 else c["hidden"]
        if pad4(int(c["kept_frac"] * in_f + 0.999)) + pad4(out_f) < in_f:
            reordered.add(f"convs.{i}.lin_l.weight")
    assert reordered
    for k, g in runs[0][2].items():
        if k in reordered:
            continue    # read from the differently rounded saved tensor: equal within the quantisation noise only
        assert relfro(g, runs[1][2][k]) < 3e-2, (k, relfro(g, runs[1][2][k]))


@pytest.mark.parametrize("cfg_name,nodes", [("cfg2", 3000), ("cfg4", 3000)])
def test_relu_dropout_pair_as_one_module_changes_nothing(cfg_name, nodes):
    """QModule turns a model's ReLU + Dropout pair (ActDropout) into QReLUDropout: one pass, one mask, the
    same noise offset; outputs and gradients are bit-identical to QReLU followed by QDropout."""
    runs = []
    for fuse in (True, False):
        config.fuse_relu_dropout = fuse
        try:
            loss, out, grads, _, _, _ = run_model(cfg_name, nodes, seed=8, fused_rp=True)
        finally:
            config.fuse_relu_dropout = True
        runs.append((loss, out, grads))
    assert runs[0][0] == runs[1][0] and torch.equal(runs[0][1], runs[1][1])
    for k, g in runs[0][2].items():
        assert torch.equal(g, runs[1][2][k]), k


def test_eval_mode_bypasses_compression_and_state_dict_prefix():
    reset_config()
    net = QModule(models.GCN(16, 8, 4, 2, dropout=0.5, batch_norm=True)).cuda()
    assert all(not k.startswith("model.") for k in net.state_dict())
    net.load_state_dict(net.state_dict())
    adj = graphs.erdos_renyi(64, 4, 0).cuda()
    x = torch.randn(64, 16, device="cuda")
    net.eval()
    with torch.no_grad():
        a = net(x, adj)
        b = net(x, adj)
    assert torch.equal(a, b)
