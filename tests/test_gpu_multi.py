"""Vocabulary-sharded sampling over NCCL on two GPUs against the oracle on the whole row.
Needs two CUDA devices; skipped on a single-GPU box."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import oracle_lib as O
        from gpu_util import compare
        from mantle_b200 import sampler, sharded, workloads

        dev = "cuda:%d" % rank
        w = workloads.make("vocab_sharded", rows=96, device="cpu")  # identical on both ranks
        V = w.vocab
        off, width = sharded.vocab_shard(V, world, rank)
        local = w.logits[:, off:off + width].contiguous().to(dev)
        p_dev = sampler.params_to_device(w.params, dev)
        out = sharded.sample_vocab_sharded(local, p_dev, w.max_top_k, V, history=w.history.to(dev), cand_cap=50)
        torch.cuda.synchronize()
        gpu = dict(next=out.next.cpu().numpy(), n_kept=out.n_kept.cpu().numpy(), cut=out.cut.cpu().numpy(),
                   cand_idx=out.cand_idx.cpu().numpy(), cand_prob=out.cand_prob.cpu().numpy())
        ref = O.sample_rows(w.logits.numpy().copy(), w.params, history=w.history.numpy(), cand_cap=50)
        compare(gpu, ref, 50, where="rank %d" % rank)
        assert int(out.status.item()) == 0
        # the same step through one packed all-gather, twice in a row on the same buffers
        plan = sharded.VocabShardedPlan(local, p_dev, w.max_top_k, V, history=w.history.to(dev), cand_cap=50)
        for _ in range(2):
            o2 = plan.step()
            torch.cuda.synchronize()
            gpu2 = dict(next=o2.next.cpu().numpy(), n_kept=o2.n_kept.cpu().numpy(), cut=o2.cut.cpu().numpy(),
                        cand_idx=o2.cand_idx.cpu().numpy(), cand_prob=o2.cand_prob.cpu().numpy())
            compare(gpu2, ref, 50, where="packed, rank %d" % rank)
        # the same step through the library's own entry point: shortlist kernel, ncclAllGather on a
        # communicator made with ncclCommInitRank, and merge, queued by one C call
        from mantle_b200 import nccl

        comm = nccl.communicator_from_torch()
        plan3 = sharded.NcclVocabShardedPlan(comm, local, p_dev, w.max_top_k, V, history=w.history.to(dev), cand_cap=50)
        for _ in range(2):
            o3 = plan3.step()
            torch.cuda.synchronize()
            gpu3 = dict(next=o3.next.cpu().numpy(), n_kept=o3.n_kept.cpu().numpy(), cut=o3.cut.cpu().numpy(),
                        cand_idx=o3.cand_idx.cpu().numpy(), cand_prob=o3.cand_prob.cpu().numpy(),
                        token_prob=o3.token_prob.cpu().numpy(), softmax_sum=o3.softmax_sum.cpu().numpy())
            compare(gpu3, ref, 50, where="C entry point, rank %d" % rank)
            assert int(o3.status.item()) == 0
        torch.cuda.synchronize()
        dist.barrier()
        comm.close()
        open(os.path.join(tmp, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_vocab_sharded_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), "ok%d" % r)) for r in range(world))
