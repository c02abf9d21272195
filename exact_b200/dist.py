"""Row-partitioned full-batch training across the GPUs of one node.

The reference is single-GPU (no collective anywhere in it).  Here node rows are split into shards of
a multiple of 8 rows, one shard per rank.  Pack, unpack, masks, projections and the dense layers are
row-local; the only exchange on the activation path is the neighbour-feature all-gather that precedes
each SpMM (forward: features; backward: the incoming gradient, multiplied by the transposed local
structure).  Weight gradients are summed with one small all-reduce per step.

Every rank draws stochastic-rounding noise, dropout uniforms and projection signs keyed by global
row / element indices (config.row_offset), so an N-rank run reproduces the 1-rank packed streams."""
import torch
import torch.distributed as dist

from .conf import config
from .cpp_extension import spmm as ext_spmm
from .sparse import SparseTensor


def shard_rows(n, world):
    """Rows per shard: ceil(n / world) rounded up to a multiple of 8."""
    return ((n + world - 1) // world + 7) // 8 * 8


class ShardedSparseTensor:
    """Rows [row_start, row_end) of a square adjacency and the same rows of its transpose, with global
    column ids, plus the process group that holds the other shards."""

    def __init__(self, full: SparseTensor, reduce, rank, world, group=None, index_dtype=torch.int32):
        n = full.size(0)
        assert full.size(1) == n
        self.n_global, self.rank, self.world, self.group = n, rank, world, group
        self.reduce = "sum" if reduce in ("sum", "add") else reduce
        self.shard = shard_rows(n, world)
        self.row_start = min(rank * self.shard, n)
        self.row_end = min(self.row_start + self.shard, n)
        r0, r1 = self.row_start, self.row_end
        rowptr, col, val = full.csr()
        e0, e1 = int(rowptr[r0]), int(rowptr[r1])
        self.rowptr = (rowptr[r0:r1 + 1] - e0).to(index_dtype).contiguous()
        self.col = col[e0:e1].to(index_dtype).contiguous()
        self.value = None if val is None else val[e0:e1].contiguous()
        t_ptr, t_col, t_w = full.storage.transposed(self.reduce)
        f0, f1 = int(t_ptr[r0]), int(t_ptr[r1])
        self.t_rowptr = (t_ptr[r0:r1 + 1] - f0).to(index_dtype).contiguous()
        self.t_col = t_col[f0:f1].to(index_dtype).contiguous()
        self.t_w = None if t_w is None else t_w[f0:f1].contiguous()
        self._gather_buf = {}
        self._const_gather = None   # (tensor, version, gathered): input features do not change between epochs

    @property
    def local_rows(self):
        return self.row_end - self.row_start

    def size(self, dim):
        return self.local_rows if dim == 0 else self.n_global

    def gather(self, x_local, tag):
        """All-gather of the row shards of an [local_rows, K] matrix -> [n_global, K] in local HBM."""
        K = x_local.size(1)
        key = (tag, K, x_local.dtype)
        buf = self._gather_buf.get(key)
        if buf is None:
            buf = torch.empty((self.world * self.shard, K), dtype=x_local.dtype, device=x_local.device)
            self._gather_buf[key] = buf
        if self.world == 1:
            return x_local
        if x_local.size(0) != self.shard:   # the last shard is shorter: pad to the common size
            pad = buf[self.rank * self.shard:(self.rank + 1) * self.shard]
            pad[:x_local.size(0)].copy_(x_local)
            pad[x_local.size(0):].zero_()
            x_local = pad
        dist.all_gather_into_tensor(buf, x_local.contiguous(), group=self.group)
        return buf[:self.n_global]


class sharded_spmm(torch.autograd.Function):
    """out_local = A[rows] @ gather(x);  grad_x_local = (A^T)[rows] @ gather(grad_out) with the
    transposed weights of spmm.cc:70-77 / 128-137."""

    @staticmethod
    def gathered_operand(adj, x):
        """All rows of the dense operand in local HBM."""
        if x.requires_grad:
            return adj.gather(x.contiguous(), "fw")
        # a leaf that needs no gradient is the model's input features: in full-batch training the same
        # tensor comes back every epoch, so its gathered copy is kept until the tensor is modified
        c = adj._const_gather
        if c is not None and c[0] is x and c[1] == x._version:
            return c[2]
        x_full = adj.gather(x.contiguous(), "fw_const").clone() if adj.world > 1 else x
        adj._const_gather = (x, x._version, x_full)
        return x_full

    @staticmethod
    def forward(ctx, adj, x, reduce):
        ctx.adj = adj
        return ext_spmm._spmm(adj.rowptr, adj.col, adj.value, sharded_spmm.gathered_operand(adj, x), reduce)

    @staticmethod
    def backward(ctx, grad_out):
        adj = ctx.adj
        g_full = adj.gather(grad_out.contiguous(), "bw")
        return None, ext_spmm._spmm(adj.t_rowptr, adj.t_col, adj.t_w, g_full, "sum"), None


def init_process_group_from_env():
    """One process per GPU, launched by torchrun: NCCL over NVLink, device = LOCAL_RANK."""
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {"device_id": torch.device("cuda", local)} if backend == "nccl" else {}
        dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return rank, world, local


def shard_graph(full, reduce, rank, world, group=None):
    """Shard `full` for this rank and point the noise keys at the shard's global row offset."""
    adj = ShardedSparseTensor(full, reduce, rank, world, group)
    config.row_offset = adj.row_start
    return adj


def allreduce_gradients(params, group=None):
    """Sum the (small) parameter gradients over ranks with one flattened all-reduce."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, group=group)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()
