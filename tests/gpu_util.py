"""Shared helpers of the GPU parity tests: run a batch through the CUDA C-ABI and through
the CPU oracle on identical bytes and compare everything the two report."""
import numpy as np
import torch

import oracle_lib as O
from mantle_b200 import native, sampler


def to_bf16_bits(t):
    """bfloat16 torch tensor -> numpy uint16 bit patterns."""
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def run_gpu(logits, params, max_top_k, history=None, hist_len=None, exclude=None, cand_cap=0, flags=0, splits=0,
            vocab=None, logit_scale=0.0, logit_softcap=0.0):
    """logits: CUDA tensor.  Returns dict of numpy arrays plus the plan."""
    dev = logits.device
    p_dev = sampler.params_to_device(params, dev)
    h_dev = None if history is None else torch.as_tensor(np.ascontiguousarray(history, dtype=np.int32)).to(dev)
    hl_dev = None if hist_len is None else torch.as_tensor(np.ascontiguousarray(hist_len, dtype=np.int32)).to(dev)
    ex_dev = None if exclude is None else torch.as_tensor(np.ascontiguousarray(exclude, dtype=np.int32)).to(dev)
    with torch.cuda.device(dev):
        plan = sampler.BatchPlan(logits, p_dev, max_top_k, history=h_dev, hist_len=hl_dev, exclude=ex_dev,
                                 cand_cap=cand_cap, flags=flags, splits=splits, vocab=vocab,
                                 logit_scale=logit_scale, logit_softcap=logit_softcap)
        out = plan.launch()
        torch.cuda.synchronize(dev)
    res = dict(
        next=out.next.cpu().numpy(),
        n_kept=out.n_kept.cpu().numpy(),
        cut=out.cut.cpu().numpy(),
        status=int(out.status.item()),
        cand_idx=None if out.cand_idx is None else out.cand_idx.cpu().numpy(),
        cand_prob=None if out.cand_prob is None else out.cand_prob.cpu().numpy(),
        token_prob=out.token_prob.cpu().numpy(),
        softmax_sum=out.softmax_sum.cpu().numpy(),
        splits=plan.splits,
    )
    return res


def compare(gpu, ref, cand_cap=0, exact_prob=True, where=""):
    """Token ids, shortlist lengths, nucleus lengths and shortlist ids are integers: exact.
    Probabilities: bit-equal doubles where both sides sum in shortlist order; always within
    1e-5 relative after rounding to float32 (the tolerance the sampling contract states)."""
    assert np.array_equal(gpu["next"], ref["next"]), (where, np.nonzero(gpu["next"] != ref["next"])[0][:8],
                                                      gpu["next"][:8], ref["next"][:8])
    assert np.array_equal(gpu["n_kept"], ref["n_kept"]), where
    assert np.array_equal(gpu["cut"], ref["cut"]), where
    # the sampled token's probability and the softmax normaliser: bit-equal where the sums run in
    # shortlist order, within 1e-5 relative (the contract's tolerance) everywhere
    for name in ("token_prob", "softmax_sum"):
        if gpu.get(name) is not None and ref.get(name) is not None:
            if exact_prob:
                assert np.array_equal(gpu[name], ref[name]), (where, name)
            assert np.all(np.abs(gpu[name] - ref[name]) <= 1e-5 * np.abs(ref[name])), (where, name)
    if cand_cap:
        rows = len(ref["next"])
        for r in range(rows):
            n = min(int(ref["n_kept"][r]), cand_cap)
            assert np.array_equal(gpu["cand_idx"][r, :n], ref["cand_idx"][r, :n]), (where, r)
            a, b = gpu["cand_prob"][r, :n], ref["cand_prob"][r, :n]
            if exact_prob:
                assert np.array_equal(a, b), (where, r)
            a32, b32 = a.astype(np.float32), b.astype(np.float32)
            assert np.all(np.abs(a32 - b32) <= 1e-5 * np.abs(b32)), (where, r)


def widen_bf16(bits):
    """uint16 bfloat16 bit patterns -> the float32 values they stand for (exact)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def check_against_oracle(logits_np, params, max_top_k, history=None, hist_len=None, exclude=None, cand_cap=0,
                         flags=0, splits=0, device="cuda:0", where="", bf16=False, logit_scale=0.0,
                         logit_softcap=0.0, exact_prob=True):
    """logits_np: float32 [rows, V] host array (or uint16 bf16 bits when bf16=True).  With a
    multiplier or soft cap the oracle rewrites its copy of the logits first, as the reference's
    model head does, and the GPU applies the same arithmetic on the fly."""
    if bf16:
        dev_logits = torch.from_numpy(logits_np.view(np.int16).copy()).to(device).view(torch.bfloat16)
    else:
        dev_logits = torch.from_numpy(logits_np.copy()).to(device)
    gpu = run_gpu(dev_logits, params, max_top_k, history, hist_len, exclude, cand_cap, flags, splits,
                  logit_scale=logit_scale, logit_softcap=logit_softcap)
    ref_logits = logits_np.copy()
    if logit_scale or logit_softcap:
        if bf16:
            ref_logits = np.ascontiguousarray(widen_bf16(ref_logits))
        O.postprocess(ref_logits, logit_scale, logit_softcap)
    ref = O.sample_rows(ref_logits, params, history=history, hist_len=hist_len, exclude=exclude, cand_cap=cand_cap)
    # long shortlists are summed in a different association than the reference's: 1e-5, not bit-equal
    compare(gpu, ref, cand_cap, exact_prob=exact_prob and max_top_k <= native.MAX_TOP_K, where=where)
    assert gpu["status"] == 0, where
    if flags & native.FLAG_WRITE_BACK_PENALTY:
        assert np.array_equal(dev_logits.cpu().numpy(), ref_logits), where  # the in-place side effect
    elif not bf16:
        assert np.array_equal(dev_logits.cpu().numpy(), logits_np), where   # read-only otherwise
    return gpu, ref
