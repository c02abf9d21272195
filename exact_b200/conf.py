"""Global quantisation config: the same mutable singleton as the reference's exact/exact/conf.py:1-24,
plus the explicit noise key the B200 kernels use instead of torch's global CUDA generator."""


class QuantizationConfig:
    def __init__(self):
        # --- fields of the reference (conf.py:3-21) ---
        self.compress_activation = True
        self.activation_compression_bits = [2]
        self.initial_bits = 8
        self.stochastic = True
        self.use_gradient = False
        self.simulate = False
        self.enable_quantized_bn = True
        self.kept_frac = 1.0
        self.single_precision = True
        self.dropout2 = False
        self.empty_cache_threshold = None
        self.swap = False
        self.amp = False
        self.debug_memory_op_forward = False
        self.debug_memory_op_backward = False
        self.debug_remove_bn = False
        self.debug_remove_relu = False
        self.debug_remove_dropout = False
        # --- additions ---
        # Philox key and running offset for stochastic rounding, dropout and projection signs.  Every
        # call that draws noise takes the next offset, so a run is reproduced by (seed, call order).
        self.seed = 0
        self._offset = 0
        # Global index of this process's first node row (multiple of 8) when rows are sharded across
        # GPUs: keys the noise by global row so that shards reproduce the single-GPU stream.
        self.row_offset = 0
        # Fuse projection + quantise + pack into one kernel when the shape allows it.
        self.fused_rp = True
        # qlinear backward with a projected activation: form (g^T Xq) R^T instead of g^T (Xq R^T).  Same
        # result up to fp32 reassociation; the [N, D] reconstruction is never written.
        self.grad_weight_in_projected_space = True
        # Read back (synchronising) the status word of kernels with bounded on-chip waits after each call
        # (debugging).  Independently of it, QModule.forward polls the library-wide status word once per
        # training step without synchronising (poll_device_status) and raises one step late.
        self.check_device_status = False
        self.poll_device_status = True
        # SpMM: rows with more edges than this are cut into pieces that separate warps sum (0: never).
        self.spmm_long_row = 256
        # Do not produce compressed copies that no backward formula reads (the SpMM's dense operand
        # when edge values need no gradient).  Outputs and gradients are unaffected.
        self.skip_dead_saves = True
        # Dense-layer GEMMs over node rows on the tensor cores with operands split into tf32 head and tail
        # (fp32-equivalent accuracy); False: the library's fp32 GEMM.
        self.linear_tensor_core = True
        # Weight gradients of the quantised linear layers straight from the packed activation on the tensor
        # cores (tf32 inputs, fp32 accumulation: about 5e-4 relative, far below the quantisation noise of the
        # activation); False: unpack, then the library's fp32 GEMM.
        self.grad_weight_tensor_core = True
        # qbatch_norm.backward reads the saved input in its packed form (two passes over the packed bytes) instead
        # of dequantising it into an [N, D] tensor for ATen's backward.
        self.bn_backward_from_packed = True
        # Row-sharded aggregation inside the one-node GraphSAGE layer: exchange the dense operand as compact
        # rows (kept columns + values per row) when at most this share of its entries is non-zero, as outputs
        # of ReLU + dropout and gradients that passed their masks are.  Same dense rows bit for bit.
        self.compact_operand = True
        self.compact_operand_max_density = 0.5
        # Row-sharded runs: aggregate feature-parallel (every rank multiplies the whole adjacency with a column
        # slice of the operand; two all-to-all exchanges written into the peers' buffers) instead of gathering
        # all rows of the operand on every rank.  Needs peer_exchange; the pieces of long rows are then summed
        # separately.  None: from 8 ranks on (measured per epoch of the 2.45 M-node benchmark: 34.9 against 32.9 ms
        # at 2 ranks, 23.6 against 21.1 ms at 4, 15.2 against 15.4 ms at 8; the gathered volume of the row split
        # grows with the ranks, the two exchanges of the column split shrink).  True / False: always / never.
        self.column_split_aggregation = None
        # Columns a slice of the feature-parallel aggregation should at least have.  Operands with fewer than
        # world * this many columns are cut into fewer slices (the world size halved until a slice is wide enough)
        # and the rows into as many blocks: rank (i, j) multiplies row block i with column slice j.  0: always one
        # slice per rank.  A gather costs one L2 request per edge whatever its width up to 128 bytes, so eight
        # slices of 6 - 16 columns each take as long as eight of 32; wider slices over fewer rows cost less until
        # the first exchange (N K / slices elements into every rank) outweighs it.  Measured per epoch of the
        # 2.45 M-node benchmark at 8 ranks: 15.30 ms with 0, 14.45 ms with 12 (the operands of 48 and 80 columns in
        # 4 slices x 2 row blocks), 14.79 - 14.92 ms with 20 (48 columns in 2 x 4, 80 and 100 in 4 x 2), 15.41 ms with
        # 24, 17.42 ms with 32; same numbers bit for bit.
        self.aggregation_min_slice_columns = 12
        # Pieces (of whole owners' rows) a rank's row block of the feature-parallel aggregation is summed in: with
        # more than one, a piece's result is stored into its owners' buffers on a side stream while the next piece
        # is summed.  Same numbers.  Measured per epoch at 8 ranks: 14.9 ms with 1, 15.5 ms with 2, 16.5 ms with 4
        # (the gathers and the peer stores slow each other down, and every piece adds launches): 1.
        self.aggregation_result_chunks = 1
        # ... on: every rank's SpMM stores its result rows straight into their owners' buffers (the second exchange
        # folded into the kernel); off: a local result followed by a scatter kernel.  Off by default: the narrow
        # kernel takes the rows in length-sorted order, and rows of 48 - 256 bytes stored over NVLink in that order
        # moved at about 100 GB/s (26.6 ms of SpMM per epoch at 4 GPUs against 10.4 ms + 2 ms for result + scatter).
        self.routed_aggregation_output = False
        # On: the result slices of the feature-parallel aggregation arrive slice-major in their owner's buffer
        # (contiguous stores over NVLink whatever the slice width) and are interleaved into rows locally.  Measured at
        # 4 ranks: the scatter kernel drops from 3.2 to 2.4 ms per epoch, the local interleaving copies add 1.7 ms.
        self.slice_major_result = False
        # The first exchange of the feature-parallel aggregation runs on a side stream while the layer's work that
        # does not need the aggregate (compressing x, x W_r^T, the weight gradients) runs on the main stream.
        self.overlap_exchange = False   # measured at 4 ranks: 25.1 ms per epoch against 23.1 without (the overlapped
        #                                 kernels share SMs and HBM with the exchange and slow down by more than it hides)
        # Row shards write their compact rows straight into every peer's buffer (plain stores over NVLink,
        # buffers mapped with CUDA IPC) instead of going through a collective; off, or when the mapping
        # fails, the collective-library exchange is used.
        self.peer_exchange = True
        # Row-sharded aggregation: send operands that are mostly exact zeros (ReLU + dropout outputs and
        # gradients that passed their masks) zero-compacted; shards denser than the bound go as they are.
        self.compact_gather = True
        # Row-sharded aggregation of the model's input features (a leaf that needs no gradient): keep the
        # gathered copy while the same unmodified tensor keeps coming back, as it does in full-batch training.
        self.cache_constant_gather = True
        self.compact_gather_max_density = 0.6
        # A model's ReLU + Dropout pair held in an ActDropout child becomes one QReLUDropout (one pass over
        # the activation, one saved mask) instead of QReLU followed by QDropout; same outputs and gradients.
        self.fuse_relu_dropout = True
        # QSAGEConv as one autograd node: same compressed tensors, one GEMM for lin_l + lin_r, the two
        # input-gradient products accumulated in the GEMM epilogue.  Same result up to fp32 reassociation.
        self.fuse_sage_layer = True
        # Inside that node, when lin_l has no more outputs than inputs, back-propagate (A^T g) W_l instead
        # of A^T (g W_l): the transposed aggregation (and the gradient exchange of a row-sharded run)
        # works on g, which is narrower or sparser than g W_l.
        self.aggregate_gradient_first = True
        # Forward of a SAGE layer with few outputs (k + out_features < in_features, the last layer): aggregate
        # [x R | x W_l^T] instead of x; reduce(A, x) R = reduce(A, x R) up to fp32 reassociation.
        self.aggregate_projected_first = True

        # Called as hook(quantized, randmat) with every compressed activation the layers save (tests and the
        # benchmark use it to hash the packed streams); None: no call.
        self.quantized_hook = None

    def manual_seed(self, seed):
        self.seed = int(seed)
        self._offset = 0

    def next_offset(self):
        off = self._offset
        self._offset += 1
        return off


config = QuantizationConfig()
