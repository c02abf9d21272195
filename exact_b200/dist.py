"""Row-partitioned full-batch training across the GPUs of one node.

The reference is single-GPU (no collective anywhere in it).  Here node rows are split into shards of
a multiple of 8 rows, one shard per rank.  Pack, unpack, masks, projections and the dense layers are
row-local; the only exchange on the activation path is the neighbour-feature all-gather that precedes
each SpMM (forward: features; backward: the incoming gradient, multiplied by the transposed local
structure).  Weight gradients are summed with one small all-reduce per step.

Every rank draws stochastic-rounding noise, dropout uniforms and projection signs keyed by global
row / element indices (config.row_offset), so an N-rank run reproduces the 1-rank packed streams."""
import ctypes
import warnings

import torch
import torch.distributed as dist

from . import _lib
from .conf import config
from .cpp_extension import rows as ext_rows
from .cpp_extension import spmm as ext_spmm
from .sparse import SparseTensor


def _host_staged(t, group):
    """CUDA tensors under the gloo backend (several ranks sharing one GPU in tests) go through the host."""
    return t.is_cuda and dist.get_backend(group) == "gloo"


def all_gather_into_tensor(out, inp, group=None):
    if _host_staged(inp, group):
        o = torch.empty(out.shape, dtype=out.dtype)
        dist.all_gather_into_tensor(o, inp.cpu(), group=group)
        out.copy_(o)
    else:
        dist.all_gather_into_tensor(out, inp, group=group)


def all_reduce(t, op=dist.ReduceOp.SUM, group=None):
    if _host_staged(t, group):
        h = t.cpu()
        dist.all_reduce(h, op=op, group=group)
        t.copy_(h)
    else:
        dist.all_reduce(t, op=op, group=group)


def column_split_active(world):
    """Whether a run of `world` ranks aggregates feature-parallel (config.column_split_aggregation; None: from 8
    ranks on)."""
    flag = config.column_split_aggregation
    return world >= 8 if flag is None else bool(flag)


def shard_rows(n, world):
    """Rows per shard: ceil(n / world) rounded up to a multiple of 8."""
    return ((n + world - 1) // world + 7) // 8 * 8


class PeerBuffers:
    """One device buffer per rank that every rank of the node can write: allocated by the library on its
    owner, exported as a CUDA IPC handle, opened by the other processes.  `ptrs[r]` is the address of rank
    r's buffer as seen from this process (this rank's own allocation at ptrs[rank])."""

    allocated_bytes = 0     # device memory held by live buffers of this process (outside torch's allocator)
    peak_allocated_bytes = 0

    def __init__(self, nbytes, rank, world, group, device):
        lib = _lib.load()
        self.rank, self.world, self.group, self.device, self.nbytes = rank, world, group, device, nbytes
        self.local = ctypes.c_void_p()
        self.ptrs = [None] * world
        self._imported = []
        with torch.cuda.device(device):
            _lib.check(lib.exact_peer_alloc(nbytes, ctypes.byref(self.local)), "exact_peer_alloc")
            PeerBuffers.allocated_bytes += nbytes
            PeerBuffers.peak_allocated_bytes = max(PeerBuffers.peak_allocated_bytes, PeerBuffers.allocated_bytes)
            handle = ctypes.create_string_buffer(64)
            _lib.check(lib.exact_peer_export(self.local, handle), "exact_peer_export")
            handles = [None] * world
            dist.all_gather_object(handles, (rank, handle.raw), group=group)
            for r, raw in handles:
                if r == rank:
                    self.ptrs[r] = self.local.value
                    continue
                p = ctypes.c_void_p()
                _lib.check(lib.exact_peer_import(ctypes.create_string_buffer(raw, 64), ctypes.byref(p)),
                           "exact_peer_import")
                self._imported.append(p)
                self.ptrs[r] = p.value

    def local_tensor(self):
        """This rank's buffer as a uint8 tensor (no copy; the memory stays owned by this object)."""
        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.local.value, False),
                                        "version": 2}
        t = torch.as_tensor(raw, device=self.device)
        t._exact_owner = self     # keep the allocation alive as long as the view
        return t

    def close(self):
        """Unmap the peers' buffers, wait for every rank to have done so, free this rank's own."""
        lib = _lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._imported:
                lib.exact_peer_close(p)
            self._imported = []
            if dist.is_initialized():
                dist.barrier(group=self.group)
            if self.local:
                lib.exact_peer_free(self.local)
                self.local = ctypes.c_void_p()
                PeerBuffers.allocated_bytes -= self.nbytes


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
        # the whole adjacency and its transpose (feature-parallel aggregation: every rank multiplies all rows
        # with its column slice)
        self.full_rowptr = rowptr.to(index_dtype).contiguous()
        self.full_col = col.to(index_dtype).contiguous()
        self.full_value = None if val is None else val.contiguous()
        self.full_t = {self.reduce: (t_ptr.to(index_dtype).contiguous(), t_col.to(index_dtype).contiguous(),
                                     None if t_w is None else t_w.contiguous())}
        if self.reduce != "sum" and val is None:
            # the transposed mean with pre-scaled rows needs no weights: same structure, no values
            self.full_t["sum"] = (self.full_t[self.reduce][0], self.full_t[self.reduce][1], None)
        self._col_bufs = {}         # (kind, width) -> [PeerBuffers, PeerBuffers] of the feature-parallel exchange
        self._col_turn = {}
        self._blocks = {}           # (matrix, first rank, ranks) -> CSR of those ranks' rows
        self._gather_buf = {}
        self._dense_streak = {}     # tag -> calls left before compaction is tried again after a dense operand
        self._const_gather = None   # (tensor, version, gathered): input features do not change between epochs
        self._operand_form = ext_rows.OperandForm()
        self._peers = {}            # K -> [PeerBuffers, PeerBuffers], used alternately
        self._peer_turn = {}        # K -> exchanges done
        self._peers_failed = False
        self._sync = None           # the small tensor whose all-reduce orders the peers' writes before the reads

    # ---- peer exchange ---------------------------------------------------------------------------------
    def _peer_buffers(self, K, device):
        """The two buffers of world * shard slots that compact rows of K columns alternate between, or None
        when they cannot be set up on every rank (the collective exchange is used then).  Two, because a rank
        may start writing the rows of the next exchange while a slower peer still reads those of this one;
        the all-reduce of the exchange in between separates the reuse of a buffer from its last readers."""
        if self._peers_failed or not (config.peer_exchange and device.type == "cuda" and dist.is_initialized()):
            return None
        pair = self._peers.get(K)
        if pair is None:
            ok, made = 1, []
            try:
                nbytes = self.world * self.shard * ext_rows.slot_bytes(K)
                for _ in range(2):
                    made.append(PeerBuffers(nbytes, self.rank, self.world, self.group, device))
            except Exception as e:   # every rank must learn of it: agree below
                ok = 0
                warnings.warn(f"peer buffers unavailable ({e}); using the collective exchange")
            flag = torch.tensor([ok], dtype=torch.int32, device=device)
            all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            if int(flag.item()) == 0:
                self._peers_failed = True
                return None
            pair = self._peers[K] = made
            self._peer_turn[K] = 0
        turn = self._peer_turn[K]
        self._peer_turn[K] = turn + 1
        return pair[turn & 1]

    def _column_buffers(self, kind, width, nbytes, device):
        """Double-buffered peer buffers of one exchange kind and width, or None when the ranks cannot map each
        other's memory (see _peer_buffers for why there are two)."""
        if self._peers_failed or not (config.peer_exchange and device.type == "cuda" and dist.is_initialized()):
            return None
        key = (kind, width)
        pair = self._col_bufs.get(key)
        if pair is None:
            ok, made = 1, []
            try:
                for _ in range(2):
                    made.append(PeerBuffers(nbytes, self.rank, self.world, self.group, device))
            except Exception as e:   # every rank must learn of it: agree below
                ok = 0
                warnings.warn(f"peer buffers unavailable ({e}); using the collective exchange")
            flag = torch.tensor([ok], dtype=torch.int32, device=device)
            all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            if int(flag.item()) == 0:
                self._peers_failed = True
                return None
            pair = self._col_bufs[key] = made
            self._col_turn[key] = 0
        turn = self._col_turn[key]
        self._col_turn[key] = turn + 1
        return pair[turn & 1]

    def _order_peer_stores(self, device):
        """All ranks' stores into each other's buffers, enqueued so far, happen before anything enqueued after."""
        if self._sync is None:
            self._sync = torch.zeros(1, dtype=torch.int32, device=device)
        all_reduce(self._sync, group=self.group)

    def aggregate(self, x_local, reduce, transposed=False, rowscale=None, unweighted=False, meanwhile=None):
        """reduce(A, x) (or A^T x when `transposed`: spmm.cc:70-77, 128-137) for this rank's rows, with x given
        by rows: [local_rows, K] on every rank.  Feature-parallel: every rank receives a slice of Kp = ceil(K / P)
        columns of ALL rows (each rank stores its rows' slices into the peers' buffers), multiplies the whole
        adjacency with it, and stores each row block of its result slice into the owner's output buffer.  Two
        all-to-all exchanges of N K / P elements per rank instead of an all-gather of N K (P - 1) / P, equal work
        on every rank whatever the degree distribution, and gathers over a P times narrower operand.  The
        sums of long rows are regrouped (their pieces are added separately).  Returns None when the
        ranks cannot write each other's memory (the caller takes the row-split route; `meanwhile` has then not
        been called).  `meanwhile`: work of the caller that does not depend on the result; it is enqueued on the
        current stream while the first exchange (NVLink-bound stores, issued on a side stream) is in flight."""
        n_loc, K = x_local.shape
        dev = x_local.device
        P, S, N = self.world, self.shard, self.n_global
        if not (column_split_active(self.world) and x_local.dtype == torch.float32 and K % 4 == 0):
            return None
        # Pc column slices times Pr = P / Pc row blocks.  Rank (i, j) = i * Pc + j receives slice j (Kp columns) of
        # ALL rows and multiplies row block i of the adjacency (the rows of ranks i * Pc .. i * Pc + Pc - 1) with
        # it.  Pc = P, one block: the plain column split.  A gather costs one L2 request per edge up to 128 bytes
        # of slice, so slices of 8 - 16 columns take as long as one of 32; fewer, wider slices over 1 / Pr of
        # the edges are faster as long as the wider first exchange (N K / Pc elements into every rank) allows.
        Pc = self.column_slices(K)
        Pr = P // Pc
        blk, sl = self.rank // Pc, self.rank % Pc
        Kp = ((K + Pc - 1) // Pc + 3) // 4 * 4
        inb = self._column_buffers("in/%d" % Pc, Kp, P * S * Kp * 4, dev)
        if inb is None:
            return None
        outb = self._column_buffers("out/%d" % Pc, Kp, S * Pc * Kp * 4, dev)
        if outb is None:
            return None
        x_local = x_local if (x_local.stride(1) == 1 and x_local.stride(0) % 4 == 0 and x_local.data_ptr() % 16 == 0) \
            else x_local.contiguous()

        def first_exchange():
            for b in range(Pr):      # slice q of this rank's rows to rank (b, q), every b
                ext_rows.cols_scatter(x_local, rowscale, self.row_start, Kp, inb.ptrs[b * Pc:(b + 1) * Pc])

        if meanwhile is not None and config.overlap_exchange:
            main = torch.cuda.current_stream(dev)
            side = self._side_stream(dev)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                first_exchange()
            meanwhile()
            main.wait_stream(side)      # x_local and rowscale stay alive in this frame until both streams have joined
        else:
            first_exchange()
            if meanwhile is not None:
                meanwhile()
        self._order_peer_stores(dev)
        slice_all = inb.local_tensor().view(torch.float32).view(P * S, Kp)[:N]
        first = blk * Pc                                  # this rank's row block: the rows of ranks first .. first + Pc - 1
        if transposed:
            # rows already scaled by 1 / deg (here or by the caller): A_mean^T g = A^T (D^-1 g), no edge weights
            unweighted = unweighted or rowscale is not None
            mkey = ("t", "sum" if (unweighted and "sum" in self.full_t) else self.reduce)

            def spmm_rows(o0, on, **kw):
                ptr, col, w = self._row_range(mkey, o0, on)
                if ptr.numel() <= 1:
                    return None
                return ext_spmm._spmm(ptr, col, None if unweighted else w, slice_all, "sum", regroup=True, **kw)
        else:
            def spmm_rows(o0, on, **kw):
                ptr, col, w = self._row_range(("a",), o0, on)
                if ptr.numel() <= 1:
                    return None
                return ext_spmm._spmm(ptr, col, w, slice_all, reduce, regroup=True, **kw)
        owners = outb.ptrs[first:first + Pc]              # the ranks whose rows this rank's block covers
        if Pr == 1 and config.slice_major_result:
            # the owner's buffer holds P dense [S, Kp] slices, one per source rank: every store of the second
            # exchange is contiguous whatever Kp (row-major, a rank's pieces are Kp * 4 bytes at a pitch of K * 4:
            # 32 - 128 bytes at 8 ranks); the owner interleaves the slices locally afterwards
            col0, ldd = 0, Kp
            ptrs = [p + self.rank * S * Kp * 4 for p in outb.ptrs]
        else:
            col0, ldd, ptrs = sl * Kp, Pc * Kp, owners
        chunks = min(max(int(config.aggregation_result_chunks), 1), Pc)
        while Pc % chunks:
            chunks -= 1
        if Pr == 1 and config.routed_aggregation_output and P <= 8:
            # every result row goes from the warp that summed it straight into its owner's buffer
            spmm_rows(first, Pc, route=(S, col0, ldd, ptrs))
        elif chunks == 1:
            y = spmm_rows(first, Pc)
            if y is not None:
                ext_rows.rows_scatter(y, S, col0, ldd, ptrs)
        else:
            # the block in `chunks` pieces of whole owners: the stores of a piece's result into its owners' buffers
            # (NVLink-bound, on a side stream) run while the next piece is summed (L2-bound)
            main = torch.cuda.current_stream(dev)
            side = self._side_stream(dev)
            per = Pc // chunks
            for c in range(chunks):
                y = spmm_rows(first + c * per, per)
                if y is None:
                    continue
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    ext_rows.rows_scatter(y, S, col0, ldd, ptrs[c * per:(c + 1) * per])
                y.record_stream(side)
            main.wait_stream(side)
        self._order_peer_stores(dev)
        if Pr == 1 and config.slice_major_result:
            out = outb.local_tensor().view(torch.float32).view(P, S, Kp)[:, :n_loc].permute(1, 0, 2).reshape(n_loc, P * Kp)
            return out if K == P * Kp else out[:, :K].contiguous()
        out = outb.local_tensor().view(torch.float32).view(S, Pc * Kp)[:n_loc]
        # the buffer is written again two aggregations of this width later: callers consume the result at once
        return out if K == Pc * Kp else out[:, :K].contiguous()

    def column_slices(self, K):
        """Number of column slices Pc (a divisor of the world size) the feature-parallel aggregation of a
        K-column operand uses: the world size halved until a slice has config.aggregation_min_slice_columns
        columns (0: always the world size)."""
        Pc = self.world
        m = config.aggregation_min_slice_columns
        while m > 0 and Pc > 1 and Pc % 2 == 0 and -(-K // Pc) < m:
            Pc //= 2
        return Pc

    def _row_range(self, key, first, count):
        """CSR (rowptr, col, weights) of the rows of ranks first .. first + count - 1 of the adjacency (key
        ("a",)) or its transpose (key ("t", reduce)): the whole matrix for all ranks, else a slice of the arrays
        (the rows are a contiguous range), copied once."""
        if key[0] == "t":
            full = self.full_t[key[1]]
        else:
            full = (self.full_rowptr, self.full_col, self.full_value)
        if first == 0 and count == self.world:
            return full
        got = self._blocks.get((key, first, count))
        if got is None:
            rowptr, col, w = full
            b0 = min(first * self.shard, self.n_global)
            b1 = min(b0 + count * self.shard, self.n_global)
            e0, e1 = int(rowptr[b0]), int(rowptr[b1])
            got = ((rowptr[b0:b1 + 1] - e0).contiguous(), col[e0:e1].clone(), None if w is None else w[e0:e1].clone())
            self._blocks[(key, first, count)] = got
        return got

    def _side_stream(self, dev):
        st = getattr(self, "_side", None)
        if st is None:
            st = self._side = torch.cuda.Stream(device=dev)
        return st

    def describe_exchange(self):
        if self._col_bufs:
            cuts = sorted({int(k[0].split("/")[1]) for k in self._col_bufs if "/" in str(k[0])}, reverse=True)
            grid = ", ".join("%dx%d" % (c, self.world // c) for c in cuts)
            return ("feature-parallel aggregation: two all-to-all exchanges written into the peers' buffers"
                    + (f" (column slices x row blocks: {grid})" if grid else ""))
        if self._peers:
            return "compact rows written into the peers' buffers"
        return "rows through the collective library" + (" (zero-compacted)" if config.compact_gather else "")

    def exchange(self, x_local, tag, rowscale=None):
        """Every row of the [local_rows, K] operand (times rowscale[:, None]) as a dense [n_global, K] matrix in
        local HBM.  When the operand is mostly zeros and the ranks can write each other's memory, each rank
        compacts its rows once and stores them into every rank's buffer (one kernel, plain stores over
        NVLink: a third of the dense bytes), an all-reduce of one word orders those stores before anyone's
        reads, and one kernel expands the slots into the dense rows the SpMM gathers: no sizes to agree on, no
        host synchronisation.  Otherwise the rows go through the collective library."""
        K = x_local.size(1)
        dev = x_local.device
        mode, density = self._operand_form.mode(tag, K, x_local.dtype)
        if mode == "probe":
            # share of non-zero entries over all ranks, from a local pack (one-off; every rank gets the same
            # number, so every rank takes the same route)
            kept = torch.zeros(1, dtype=torch.int64, device=dev)
            ext_rows.crows_pack(x_local.contiguous(), rowscale, kept_total=kept)
            all_reduce(kept, group=self.group)
            density = float(kept.item()) / max(self.n_global * K, 1)
            mode = self._operand_form.decide(tag, density)
        if mode == "compact":
            pb = self._peer_buffers(K, dev)
            if pb is not None:
                ext_rows.crows_pack(x_local.contiguous(), rowscale, row0=self.row_start, dst_ptrs=pb.ptrs)
                if self._sync is None:
                    self._sync = torch.zeros(1, dtype=torch.int32, device=dev)
                all_reduce(self._sync, group=self.group)
                cr = ext_rows.CompactRows(None, self.n_global, K, density, address=pb.ptrs[self.rank], device=dev)
                out = self._buffer((tag, K, torch.float32), (self.world * self.shard, K), torch.float32, dev)
                return ext_rows.crows_unpack(cr, self.n_global, out=out)
        if rowscale is not None:
            x_local = x_local * rowscale.unsqueeze(1)
        return self.gather(x_local.contiguous(), tag, try_compact=(mode == "compact"))

    def close(self):
        for pair in list(self._peers.values()) + list(self._col_bufs.values()):
            for pb in pair:
                pb.close()
        self._peers, self._col_bufs = {}, {}

    @property
    def local_rows(self):
        return self.row_end - self.row_start

    def size(self, dim):
        return self.local_rows if dim == 0 else self.n_global

    def _buffer(self, key, shape, dtype, device):
        buf = self._gather_buf.get(key)
        if buf is None or buf.shape != torch.Size(shape):
            buf = torch.empty(shape, dtype=dtype, device=device)
            self._gather_buf[key] = buf
        return buf

    def gather(self, x_local, tag, try_compact=True):
        """All rows of an [local_rows, K] matrix in local HBM: [n_global, K], through the collective library.
        Operands that are mostly exact zeros (ReLU + dropout outputs, gradients that passed their masks)
        cross NVLink zero-compacted and are expanded on arrival; others (and all with try_compact=False) go
        as they are."""
        if self.world == 1:
            return x_local
        K = x_local.size(1)
        if (try_compact and config.compact_gather and x_local.dtype == torch.float32 and K % 32 == 0 and K >= 64):
            left = self._dense_streak.get(tag, 0)
            if left > 0:
                self._dense_streak[tag] = left - 1
            else:
                out = self._gather_compacted(x_local, tag)
                if out is not None:
                    return out
                self._dense_streak[tag] = 16
        return self._gather_dense(x_local, tag)

    def _gather_dense(self, x_local, tag):
        K = x_local.size(1)
        buf = self._buffer((tag, K, x_local.dtype), (self.world * self.shard, K), x_local.dtype, x_local.device)
        if x_local.size(0) != self.shard:   # the last shard is shorter: pad to the common size
            pad = buf[self.rank * self.shard:(self.rank + 1) * self.shard]
            pad[:x_local.size(0)].copy_(x_local)
            pad[x_local.size(0):].zero_()
            x_local = pad
        all_gather_into_tensor(buf, x_local.contiguous(), group=self.group)
        return buf[:self.n_global]

    def _gather_compacted(self, x_local, tag):
        """mask + row offsets + kept values of every shard, then one expansion into dense rows.  Returns
        None (nothing sent yet beyond the counts) when some shard is too dense for this to pay."""
        dev, K, W, S, R = x_local.device, x_local.size(1), x_local.size(1) // 32, self.shard, self.world
        n_loc = x_local.size(0)
        x_local = x_local.contiguous()
        mask = self._buffer((tag, "mask_loc"), (S, W), torch.int32, dev)
        rowcnt = self._buffer((tag, "rowcnt"), (S,), torch.int32, dev)
        if n_loc < S:
            mask[n_loc:].zero_()
            rowcnt[n_loc:].zero_()
        ext_rows.mask_count(x_local, mask[:n_loc], rowcnt[:n_loc])
        rowoff = self._buffer((tag, "rowoff_loc"), (S + 1,), torch.int64, dev)
        rowoff[:1].zero_()
        torch.cumsum(rowcnt, 0, out=rowoff[1:])
        counts = self._buffer((tag, "counts"), (R,), torch.int64, dev)
        all_gather_into_tensor(counts, rowoff[S:S + 1], group=self.group)
        cap = int(counts.max().item())          # the one host synchronisation of the exchange
        if cap > config.compact_gather_max_density * S * K:
            return None
        cap = max((cap + 255) // 256 * 256, 256)
        vals = torch.empty(cap, dtype=torch.float32, device=dev)
        ext_rows.compact_write(x_local, rowoff, vals)
        vals_all = torch.empty(R * cap, dtype=torch.float32, device=dev)
        all_gather_into_tensor(vals_all, vals, group=self.group)
        rowoff_all = self._buffer((tag, "rowoff_all"), (R * (S + 1),), torch.int64, dev)
        all_gather_into_tensor(rowoff_all, rowoff, group=self.group)
        mask_all = self._buffer((tag, "mask_all"), (R * S, W), torch.int32, dev)
        all_gather_into_tensor(mask_all, mask, group=self.group)
        out = self._buffer((tag, K, x_local.dtype), (R * S, K), torch.float32, dev)
        ext_rows.expand(mask_all, rowoff_all, vals_all, R * S, K, S, S + 1, cap, out)
        return out[:self.n_global]


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
        if not config.cache_constant_gather:
            return adj.gather(x.contiguous(), "fw_const")
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
    all_reduce(flat, group=group)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()
