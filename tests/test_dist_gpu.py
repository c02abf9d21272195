"""The row-sharded training path on a GPU, checked against the unsharded run.

2 and 8 ranks run as child processes that share the one device of the test box (tests/dist_worker.py:
backend gloo, collectives staged through the host; no kernel of one rank waits for a kernel of another).
Compared with the single-process run of the same model, seeds and graph:
  - the packed stream of the first compressed activation (INT2 codes of x R, k = 13): the concatenation of the
    shards' streams equals the unsharded stream bit for bit, and so do the bf16 row statistics;
  - the loss of every step and the first step's parameter gradients: equal up to the fp32 regrouping of the
    sums over ranks (gradients 2e-5 relative Frobenius at 2 ranks; at 8 ranks the shards are small enough to
    take the library GEMM for their dense layers and a few stochastic-rounding decisions flip: 5e-3; losses
    1e-5 relative at step 0, 1e-4 afterwards);
  - the peer-written compact rows against the collective exchange: same numbers."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world, out, name, **kw):
    port = _free_port()
    procs = []
    for r in range(world):
        cmd = [sys.executable, os.path.join(HERE, "dist_worker.py"), "--world", str(world), "--rank", str(r),
               "--port", str(port), "--out", str(out), "--name", name]
        for k, v in kw.items():
            cmd += [f"--{k}", str(v)]
        procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        logs.append(o)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} of {world} failed:\n{logs[r][-3000:]}"
    return [torch.load(os.path.join(out, f"w{world}_{name}_r{r}.pt")) for r in range(world)]


@pytest.fixture(scope="module")
def single(tmp_path_factory):
    out = tmp_path_factory.mktemp("dist1")
    return _run(1, out, "single")[0]


def _compare_with_single(parts, single, regrouped=False):
    world = len(parts)
    assert parts[0]["rows"][0] == 0 and all(parts[i]["rows"][1] == parts[i + 1]["rows"][0] for i in range(world - 1))
    assert all(p["rows"][0] % 8 == 0 for p in parts)
    packed = torch.cat([p["packed"] for p in parts])
    assert torch.equal(packed, single["packed"])            # bit-equal packed stream
    assert torch.equal(torch.cat([p["scale"] for p in parts]).view(torch.int16), single["scale"].view(torch.int16))
    assert torch.equal(torch.cat([p["min"] for p in parts]).view(torch.int16), single["min"].view(torch.int16))
    for p in parts:
        assert p["losses"] == parts[0]["losses"]
        assert abs(p["losses"][0] - single["losses"][0]) <= 1e-5 * abs(single["losses"][0])
        for a, b in zip(p["losses"], single["losses"]):
            assert abs(a - b) <= 1e-4 * abs(b)
        # Shards of fewer than 1,024 rows (8 ranks here) run their dense layers on the library's fp32 GEMM instead
        # of the tf32 head/tail tensor-core kernel: a 1e-6 relative difference in a layer's output, which flips
        # the stochastic rounding of a few INT2 codes of the next layer's saved activation; the gradients then
        # differ by a corresponding share of the quantisation noise.
        tol = 2e-5 if min(q["rows"][1] - q["rows"][0] for q in parts) >= 1024 and not regrouped else 5e-3
        for a, b in zip(p["grads0"], single["grads0"]):
            assert float((a - b).norm()) <= tol * float(b.norm()) + 1e-12
            assert float((a - b).abs().max()) <= 10 * tol * float(b.abs().max()) + 1e-9
        for a, b in zip(p["params"], parts[0]["params"]):
            assert torch.equal(a, b)                          # replicas stay in step


@pytest.mark.parametrize("routed", [0, 1])
@pytest.mark.parametrize("world", [2, 8])
def test_sharded_run_with_feature_parallel_aggregation(world, routed, single, tmp_path):
    """The default route: column slices of every row to every rank, the whole adjacency times the slice, row
    blocks of the result back to their owners, by a scatter kernel (default) or stored by the SpMM itself
    (routed).  The pieces of long rows are summed separately, so sums are regrouped."""
    parts = _run(world, tmp_path, "cols%d" % routed, peer=1, colsplit=1, routed=routed)
    assert all(p["peers_used"] for p in parts), "the ranks could not map each other's buffers"
    assert all(p["exchange"].startswith("feature-parallel") for p in parts)
    _compare_with_single(parts, single, regrouped=True)


@pytest.mark.parametrize("world,minslice,expect", [(8, 12, {"in/4", "in/8"}), (8, 20, {"in/2", "in/4", "in/8"}), (2, 64, {"in/1", "in/2"})])
def test_feature_parallel_aggregation_with_row_blocks(world, minslice, expect, single, tmp_path):
    """config.aggregation_min_slice_columns: narrow operands are cut into fewer column slices and the rows into
    blocks (rank (i, j) multiplies row block i with slice j).  Every row is still summed in the order of its
    edges, so the numbers equal those of one slice per rank bit for bit."""
    parts = _run(world, tmp_path, "blocks", peer=1, colsplit=1, minslice=minslice)
    assert all(p["exchange"].startswith("feature-parallel") for p in parts)
    assert {k[0] for k in parts[0]["col_keys"] if k[0].startswith("in/")} == expect
    _compare_with_single(parts, single, regrouped=True)
    plain = _run(world, tmp_path, "slices", peer=1, colsplit=1)
    assert parts[0]["losses"] == plain[0]["losses"]
    for p, q in zip(parts, plain):
        assert all(torch.equal(a, b) for a, b in zip(p["grads0"], q["grads0"]))


@pytest.mark.parametrize("world,minslice,chunks", [(8, 20, 2), (8, 0, 4), (2, 0, 2)])
def test_feature_parallel_aggregation_with_result_in_pieces(world, minslice, chunks, single, tmp_path):
    """config.aggregation_result_chunks: a rank's row block is summed in pieces of whole owners' rows and each
    piece's result is stored into its owners' buffers on a side stream while the next piece is summed.  The
    numbers are those of one piece."""
    parts = _run(world, tmp_path, "pieces", peer=1, colsplit=1, minslice=minslice, chunks=chunks)
    _compare_with_single(parts, single, regrouped=True)
    plain = _run(world, tmp_path, "onepiece", peer=1, colsplit=1)
    assert parts[0]["losses"] == plain[0]["losses"]
    for p, q in zip(parts, plain):
        assert all(torch.equal(a, b) for a, b in zip(p["grads0"], q["grads0"]))


def test_feature_parallel_aggregation_with_slice_major_result_buffers(single, tmp_path):
    """config.slice_major_result: the second exchange writes dense per-source slices into the owners' buffers,
    interleaved into rows locally."""
    parts = _run(2, tmp_path, "slicemajor", peer=1, colsplit=1, slicemajor=1)
    _compare_with_single(parts, single, regrouped=True)


def test_feature_parallel_aggregation_with_overlapped_first_exchange(single, tmp_path):
    """config.overlap_exchange: the first exchange on a side stream while the layer's independent work (compressing
    x, x W_r^T, the weight gradients) runs on the main stream; the GEMM of a layer is then split in two, so the
    numbers are a reassociation of the default order."""
    parts = _run(2, tmp_path, "ovl", peer=1, colsplit=1, overlap=1)
    assert all(p["exchange"].startswith("feature-parallel") for p in parts)
    _compare_with_single(parts, single, regrouped=True)


@pytest.mark.parametrize("world", [2, 8])
def test_sharded_run_with_peer_written_compact_rows(world, single, tmp_path):
    parts = _run(world, tmp_path, "peer", peer=1, colsplit=0)
    assert all(p["peers_used"] for p in parts), "the ranks could not map each other's buffers"
    assert parts[0]["forms"]["fw256"][0] == "compact" and parts[0]["forms"]["bw256"][0] == "compact"
    _compare_with_single(parts, single)


def test_sharded_run_with_collective_exchange(single, tmp_path):
    parts = _run(2, tmp_path, "coll", peer=0, colsplit=0)
    assert not any(p["peers_used"] for p in parts)
    _compare_with_single(parts, single)
