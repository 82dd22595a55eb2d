"""Sampling across the GPUs of one box.

Two ways to spread a batch (neither exists in the reference, which runs one request on one
GPU; internal/api/engine_provider.go:66-71):

* rows sharded: every rank samples its own rows; nothing is exchanged (`row_shard`).
* vocabulary sharded: every rank holds a contiguous range of columns of every row.  Each rank
  takes its local shortlist (values already penalised and scaled, ids global), the shortlists
  are all-gathered -- k (value, id) pairs per row and rank, a few hundred bytes -- and every
  rank merges them and finishes its rows.  Because the ranges are contiguous and ties go to the
  lower global id, the merge of the local shortlists is exactly the global shortlist.

Two carriers for the all-gather: `NcclVocabShardedPlan` goes through the library's own entry point
(mantleCudaSampleVocabSharded: shortlist kernel, ncclAllGather and merge kernel queued by one C
call on one stream, the form a non-Python host uses); `VocabShardedPlan` and
`sample_vocab_sharded` let torch.distributed move the blocks (NCCL on GPUs, gloo in the CPU
tests).  Either way the gathered shortlists land in local memory before any kernel reads them.
"""
import torch
import torch.distributed as dist


def row_shard(rows, world_size, rank):
    """Contiguous block of rows for `rank`: (first, count)."""
    base, extra = divmod(rows, world_size)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def vocab_shard(vocab_total, world_size, rank):
    """Contiguous column range of `rank`: (offset, width).  Widths differ by at most one."""
    base, extra = divmod(vocab_total, world_size)
    offset = rank * base + min(rank, extra)
    return offset, base + (1 if rank < extra else 0)


def gather_parts(val, idx, cnt, group=None):
    """All-gathers the local shortlists.

    val, idx: [rows, cap]; cnt: [rows].  Returns ([G, rows, cap], [G, rows, cap], [G, rows]) in
    rank order, the layout the merge step reads (part p of row r at (p * rows + r) * cap).
    """
    world = dist.get_world_size(group)
    rows, cap = val.shape
    g_val = torch.empty((world, rows, cap), dtype=val.dtype, device=val.device)
    g_idx = torch.empty((world, rows, cap), dtype=idx.dtype, device=idx.device)
    g_cnt = torch.empty((world, rows), dtype=cnt.dtype, device=cnt.device)
    dist.all_gather_into_tensor(g_val.view(world * rows, cap), val.contiguous(), group=group)
    dist.all_gather_into_tensor(g_idx.view(world * rows, cap), idx.contiguous(), group=group)
    dist.all_gather_into_tensor(g_cnt.view(world * rows), cnt.contiguous(), group=group)
    return g_val, g_idx, g_cnt


def packed_part_bytes(rows, cap):
    """Bytes of one rank's block: [rows*cap float values][rows*cap int32 ids][rows int32 counts],
    padded to 256 (mantleCudaSamplePackedPartBytes)."""
    return ((rows * cap * 2 + rows) * 4 + 255) & ~255


def packed_part_views(block, rows, cap):
    """(val [rows, cap] float32, idx [rows, cap] int32, cnt [rows] int32) views into one block
    (a uint8 tensor of packed_part_bytes(rows, cap) bytes)."""
    words = block.view(torch.int32)
    n = rows * cap
    return words[:n].view(torch.float32).view(rows, cap), words[n:2 * n].view(rows, cap), words[2 * n:2 * n + rows]


class VocabShardedPlan:
    """A vocabulary-sharded batch bound to its buffers: build once, step many times.

    A step is the local shortlist kernel writing this rank's block, ONE all-gather of the blocks,
    and the merge kernel; nothing is allocated per step."""

    def __init__(self, local_logits, params_dev, max_top_k, vocab_total, history=None, hist_len=None, exclude=None,
                 cand_cap=0, group=None, world=None, rank=None):
        from . import native, sampler

        self.group = group
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        self.offset, width = vocab_shard(vocab_total, self.world, self.rank)
        if local_logits.shape[1] != width:
            raise ValueError("rank %d holds %d columns, its share of %d is %d"
                             % (self.rank, local_logits.shape[1], vocab_total, width))
        self.lib = native.load()
        self.sampler = sampler
        self.native = native
        dev = local_logits.device
        rows = local_logits.shape[0]
        self.rows, self.k, self.vocab_total = rows, max_top_k, vocab_total
        self.keep = [local_logits, params_dev, history, hist_len, exclude]
        nbytes = packed_part_bytes(rows, max_top_k)
        self.block = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self.gathered = torch.zeros(self.world * nbytes, dtype=torch.uint8, device=dev)
        self.val, self.idx, self.cnt = packed_part_views(self.block, rows, max_top_k)
        import ctypes as C

        b = native.SampleBatch()
        b.logits = local_logits.data_ptr()
        b.dtype = native.DTYPE_F32 if local_logits.dtype == torch.float32 else native.DTYPE_BF16
        b.rows, b.vocab, b.max_top_k, b.row_stride = rows, width, max_top_k, local_logits.stride(0)
        if history is not None and history.numel() > 0:
            b.history, b.hist_stride = history.data_ptr(), history.shape[1]
            if hist_len is not None:
                b.hist_len = hist_len.data_ptr()
        if exclude is not None and exclude.numel() > 0:
            b.exclude, b.n_exclude = exclude.data_ptr(), exclude.numel()
        b.params = params_dev.data_ptr()
        self.local = b
        out = sampler.SampleOutputs()
        out.next = torch.full((rows,), -2, dtype=torch.int32, device=dev)
        out.cand_idx = torch.full((rows, cand_cap), -1, dtype=torch.int32, device=dev) if cand_cap else None
        out.cand_prob = torch.zeros((rows, cand_cap), dtype=torch.float64, device=dev) if cand_cap else None
        out.n_kept = torch.zeros(rows, dtype=torch.int32, device=dev)
        out.cut = torch.zeros(rows, dtype=torch.int32, device=dev)
        out.status = torch.zeros(1, dtype=torch.int32, device=dev)
        out.token_prob = torch.zeros(rows, dtype=torch.float64, device=dev)
        out.softmax_sum = torch.zeros(rows, dtype=torch.float64, device=dev)
        self.out = out
        m = native.SampleBatch()
        m.rows, m.vocab, m.max_top_k = rows, vocab_total, max_top_k
        m.params, m.next = params_dev.data_ptr(), out.next.data_ptr()
        if cand_cap:
            m.cand_idx, m.cand_prob, m.cand_stride = out.cand_idx.data_ptr(), out.cand_prob.data_ptr(), cand_cap
        m.n_kept, m.cut, m.status = out.n_kept.data_ptr(), out.cut.data_ptr(), out.status.data_ptr()
        m.token_prob, m.softmax_sum = out.token_prob.data_ptr(), out.softmax_sum.data_ptr()
        self.merge = m
        self.C = C

    def step(self):
        """Queues one sampling step on torch's current stream; every rank gets the same tokens."""
        C, native = self.C, self.native
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: C.c_void_p(t.data_ptr())
        rc = self.lib.mantleCudaSampleLocalTopK(C.byref(self.local), self.offset, self.vocab_total, p(self.val),
                                                p(self.idx), p(self.cnt), self.k, stream)
        native.check(rc, "mantleCudaSampleLocalTopK")
        dist.all_gather_into_tensor(self.gathered, self.block, group=self.group)
        rc = self.lib.mantleCudaSampleMergePacked(C.byref(self.merge), self.world, p(self.gathered), self.k, stream)
        native.check(rc, "mantleCudaSampleMergePacked")
        return self.out


class NcclVocabShardedPlan(VocabShardedPlan):
    """The same step through mantleCudaSampleVocabSharded: one C call per step queues the local
    shortlist kernel, ncclAllGather on the given communicator and the merge, all on the caller's
    stream.  `comm` is an mantle_b200.nccl.Communicator whose ranks are the shards in column order."""

    def __init__(self, comm, local_logits, params_dev, max_top_k, vocab_total, **kw):
        from . import nccl

        self.comm = comm
        self.nccl_lib = nccl.load()
        super().__init__(local_logits, params_dev, max_top_k, vocab_total, world=comm.world_size, rank=comm.rank, **kw)
        # one descriptor serves both kernels: the shard's logits and width, the merge's outputs
        b = self.local
        m = self.merge
        b.next, b.cand_idx, b.cand_prob, b.cand_stride = m.next, m.cand_idx, m.cand_prob, m.cand_stride
        b.n_kept, b.cut, b.status, b.token_prob, b.softmax_sum = m.n_kept, m.cut, m.status, m.token_prob, m.softmax_sum

    def step(self):
        C = self.C
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        nccl_rc = C.c_int(0)
        rc = self.nccl_lib.mantleCudaSampleVocabSharded(
            C.byref(self.local), self.offset, self.vocab_total, self.comm.handle, C.c_void_p(self.block.data_ptr()),
            C.c_void_p(self.gathered.data_ptr()), stream, C.byref(nccl_rc))
        if rc != 0:
            raise self.native.CudaError(rc, "mantleCudaSampleVocabSharded (ncclResult %d)" % nccl_rc.value)
        return self.out


def sample_vocab_sharded(local_logits, params_dev, max_top_k, vocab_total, history=None, hist_len=None,
                         exclude=None, cand_cap=0, group=None):
    """One sampling step over vocabulary-sharded logits.  Every rank returns the same tokens.

    local_logits: this rank's [rows, width] columns (vocab_shard(vocab_total, world, rank));
    history / exclude hold GLOBAL token ids and are the same on every rank.
    """
    from . import sampler

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    offset, width = vocab_shard(vocab_total, world, rank)
    if local_logits.shape[1] != width:
        raise ValueError("rank %d holds %d columns, its share of %d is %d" % (rank, local_logits.shape[1], vocab_total, width))
    val, idx, cnt = sampler.local_topk(local_logits, params_dev, max_top_k, offset, vocab_total, history=history,
                                       hist_len=hist_len, exclude=exclude)
    g_val, g_idx, g_cnt = gather_parts(val, idx, cnt, group)
    return sampler.merge_parts(params_dev, max_top_k, vocab_total, g_val, g_idx, g_cnt, cand_cap=cand_cap)
