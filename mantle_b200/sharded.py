"""Sampling across the GPUs of one box.

Two ways to spread a batch (neither exists in the reference, which runs one request on one
GPU; internal/api/engine_provider.go:66-71):

* rows sharded: every rank samples its own rows; nothing is exchanged (`row_shard`).
* vocabulary sharded: every rank holds a contiguous range of columns of every row.  Each rank
  takes its local shortlist (values already penalised and scaled, ids global), the shortlists
  are all-gathered -- k (value, id) pairs per row and rank, a few hundred bytes -- and every
  rank merges them and finishes its rows.  Because the ranges are contiguous and ties go to the
  lower global id, the merge of the local shortlists is exactly the global shortlist.

torch.distributed (NCCL on GPUs, gloo in the CPU tests) carries the all-gather; the gathered
shortlists land in local memory before any kernel reads them.
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
