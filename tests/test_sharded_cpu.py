"""The multi-rank host logic on CPU: two gloo ranks, no GPU.

Rows sharded: the blocks partition the batch.  Vocabulary sharded: each rank's local shortlist
(taken here by the oracle, the kernels need a GPU) is all-gathered by the product code, and the
merge of the gathered shortlists in the order (value descending, global id ascending) must be
the oracle's shortlist on the whole row.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as O
from mantle_b200 import sharded


def test_row_shards_partition_the_batch():
    for rows in (1, 7, 64, 4096, 4097):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                first, n = sharded.row_shard(rows, world, r)
                seen += list(range(first, first + n))
            assert seen == list(range(rows))
    for V in (10, 262144, 151936):
        for world in (1, 2, 8):
            cols = []
            for r in range(world):
                off, w = sharded.vocab_shard(V, world, r)
                cols.append((off, w))
            assert cols[0][0] == 0 and sum(w for _, w in cols) == V
            assert all(cols[i][0] + cols[i][1] == cols[i + 1][0] for i in range(world - 1))


def _rank_main(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(3)  # the same data on both ranks
        rows, V, k = 12, 1001, 7
        logits = (np.round(rng.standard_normal((rows, V)) * 4) / 2).astype(np.float32)  # many ties
        inv_temp = np.float32(1.0) / np.float32(0.7)
        off, width = sharded.vocab_shard(V, world, rank)
        val = np.zeros((rows, k), dtype=np.float32)
        idx = np.full((rows, k), -1, dtype=np.int32)
        cnt = np.zeros(rows, dtype=np.int32)
        for r in range(rows):
            i, v = O.topk(logits[r, off:off + width], k, inv_temp)
            cnt[r] = len(i)
            val[r, : len(i)] = v
            idx[r, : len(i)] = i + off
        g_val, g_idx, g_cnt = sharded.gather_parts(torch.from_numpy(val), torch.from_numpy(idx), torch.from_numpy(cnt))
        assert g_val.shape == (world, rows, k) and g_cnt.shape == (world, rows)
        assert torch.equal(g_val[rank], torch.from_numpy(val)) and torch.equal(g_idx[rank], torch.from_numpy(idx))
        for r in range(rows):
            cand = [(float(g_val[p, r, j]), int(g_idx[p, r, j])) for p in range(world) for j in range(int(g_cnt[p, r]))]
            cand.sort(key=lambda t: (-t[0], t[1]))
            want_i, want_v = O.topk(logits[r], k, inv_temp)
            assert [c[1] for c in cand[:k]] == want_i.tolist(), (rank, r)
            assert [np.float32(c[0]) for c in cand[:k]] == want_v.tolist()
        # the same through one block per rank and ONE all-gather (the layout the packed merge reads)
        nbytes = sharded.packed_part_bytes(rows, k)
        assert nbytes % 256 == 0 and nbytes >= (2 * rows * k + rows) * 4
        block = torch.zeros(nbytes, dtype=torch.uint8)
        b_val, b_idx, b_cnt = sharded.packed_part_views(block, rows, k)
        b_val.copy_(torch.from_numpy(val)); b_idx.copy_(torch.from_numpy(idx)); b_cnt.copy_(torch.from_numpy(cnt))
        gathered = torch.zeros(world * nbytes, dtype=torch.uint8)
        dist.all_gather_into_tensor(gathered, block)
        for p in range(world):
            pv, pi, pc = sharded.packed_part_views(gathered[p * nbytes:(p + 1) * nbytes], rows, k)
            assert torch.equal(pv, g_val[p]) and torch.equal(pi, g_idx[p]) and torch.equal(pc, g_cnt[p])
        open(os.path.join(tmp, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_vocab_sharded_gather_two_ranks(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), "ok%d" % r)) for r in range(world))
