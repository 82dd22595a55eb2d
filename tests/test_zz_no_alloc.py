"""The entry point that allocates nothing, mantleCudaSampleRowsNoAlloc, against
mantleCudaSampleRows on the same batches, through the C-ABI.

Some hosts cannot give the sampler a workspace because they may not allocate device memory
at the point where they sample; for them the split-row scratch is a fixed array inside the
library.  The two entry points run the same kernels, so every output must be identical: token
ids, shortlist ids and lengths exactly, probabilities bit for bit.  Two calls in a row check
that nothing left in the shared array by one call leaks into the next.  This file sorts last
on purpose, so that a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from mantle_b200 import native, sampler, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def outputs(o):
    torch.cuda.synchronize()
    return {k: getattr(o, k).cpu().numpy().copy() for k in ("next", "n_kept", "cut", "cand_idx", "cand_prob", "status")}


def test_no_alloc_matches_workspace_entry_point_twice():
    for call, (rows, seed) in enumerate([(48, 11), (7, 12)]):
        w = workloads.make("mixed_batch", rows=rows, seed=seed, device=DEV)
        p_dev = sampler.params_to_device(w.params, DEV)
        plan = sampler.BatchPlan(w.logits, p_dev, w.max_top_k, history=w.history, cand_cap=32)
        assert plan.splits > 1 and plan.workspace_bytes > 0, "the batch must be one that needs scratch"
        assert plan.workspace_bytes <= plan.lib.mantleCudaSamplerStaticScratchBytes()
        want = outputs(plan.launch())
        # back to the state before the first launch: the second entry point must write everything itself
        # (shortlist slots past n_kept are never written by either)
        plan.out.next.fill_(-2)
        plan.out.cand_idx.fill_(-1)
        plan.out.cand_prob.fill_(0)
        plan.out.n_kept.fill_(0)
        plan.out.cut.fill_(0)
        got = outputs(sampler.launch_no_alloc(plan))
        for key in want:
            assert np.array_equal(got[key], want[key]), (call, key)
        assert np.all(got["next"] >= 0) and got["status"][0] == 0


def test_no_alloc_refuses_what_does_not_fit():
    rows, V = 280, 40000  # 280 rows run split (fewer than one wave); at top_k 1024 their scratch exceeds 4 MiB
    logits = torch.randn(rows, V, device=DEV)
    params = np.array([sampler.new_sampler_params(sampler.SamplerConfig(temperature=0.8, top_k=1024, top_p=0.9), 0.5)] * rows)
    plan = sampler.BatchPlan(logits, sampler.params_to_device(params, DEV), 1024, splits=4)
    assert plan.workspace_bytes > plan.lib.mantleCudaSamplerStaticScratchBytes()
    with pytest.raises(native.CudaError) as e:
        sampler.launch_no_alloc(plan)
    assert e.value.code == native.CUDA_ERROR_INVALID_VALUE and "static scratch" in str(e.value)
    plan.launch()  # the workspace entry point still takes it
    torch.cuda.synchronize()
    assert int(plan.out.status.item()) == 0
