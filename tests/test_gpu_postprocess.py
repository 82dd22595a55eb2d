"""The model head's multiplier and soft cap (simd/runtime.go:258-272): the in-place kernel
against the oracle bit for bit, and the sampler applying them on the fly against the oracle
that rewrites its logits first."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import check_against_oracle, compare, run_gpu
from mantle_b200 import native, sampler, workloads
from test_gpu_parity import random_params

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = [(0.0, 30.0), (0.5, 0.0), (2.25, 30.0), (1.0, 5.0), (0.0625, 0.75)]


def special_values():
    v = [0.0, -0.0, 1e-30, -1e-30, 1e-10, 0.1733593, 1.0, -1.0, 29.9, 30.0, 150.0, 299.9, 300.0, 300.1, -300.1, 1e6,
         -1e6, 3e38, -3e38, float("inf"), float("-inf")]
    return np.array(v, dtype=np.float32)


@pytest.mark.parametrize("scale,cap", CASES)
def test_in_place_kernel_is_bit_exact(scale, cap):
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((7, 4099)) * 12).astype(np.float32)
    x[0, : len(special_values())] = special_values()
    x[1] = np.linspace(-11 * max(cap, 1.0), 11 * max(cap, 1.0), x.shape[1], dtype=np.float32)
    pad = np.full((7, 4104), 777.0, dtype=np.float32)  # a row stride wider than the row
    pad[:, : x.shape[1]] = x
    d = torch.from_numpy(pad).to(DEV)
    sampler.logit_postprocess_rows_(d[:, : x.shape[1]], scale, cap)
    torch.cuda.synchronize()
    ref = O.postprocess(x.copy(), scale, cap)
    got = d.cpu().numpy()
    assert np.array_equal(got[:, : x.shape[1]].view(np.uint32), ref.view(np.uint32))
    assert np.all(got[:, x.shape[1]:] == 777.0)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("scale,cap", CASES)
def test_fused_random_small(seed, scale, cap):
    rng = np.random.default_rng(900 + seed)
    rows = 40
    V = int(rng.choice([1, 3, 33, 257, 1000, 5000, 9001]))
    logits = (rng.standard_normal((rows, V)) * 8).astype(np.float32)
    if seed % 2:
        logits = (np.round(logits) * 2).astype(np.float32)  # heavy ties, many saturated by a small cap
    logits[rng.random((rows, V)) < 0.03] = 0.0
    H = 40
    hist = rng.integers(-2, V + 2, size=(rows, H)).astype(np.int32)
    hist_len = rng.integers(0, H + 1, size=rows).astype(np.int32)
    exclude = rng.integers(0, V, size=3).astype(np.int32)
    params = random_params(rng, rows)
    check_against_oracle(logits, params, 300, history=hist, hist_len=hist_len, exclude=exclude,
                         cand_cap=min(V, 300), logit_scale=scale, logit_softcap=cap,
                         where="seed %d V %d scale %g cap %g" % (seed, V, scale, cap))


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("scale,cap", [(0.0, 30.0), (0.75, 30.0), (3.0, 0.0)])
def test_fused_wide_rows(bf16, scale, cap):
    """Rows as wide as a real vocabulary: one CTA per row and rows split over several CTAs."""
    w = workloads.make("mixed_batch", rows=24, seed=5)
    logits = w.logits.numpy()
    if bf16:
        logits = w.logits.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    hist = w.history.numpy()
    for splits in (1, 0):
        check_against_oracle(logits, w.params, w.max_top_k, history=hist, cand_cap=64, splits=splits, bf16=bf16,
                             logit_scale=scale, logit_softcap=cap, where="bf16 %s splits %d" % (bf16, splits))


def test_fused_saturating_cap():
    """A cap so small that most of the row lands on +-cap exactly: ties by the thousand, resolved
    by index, and a raw-logit filter that can exclude nothing above atanh(1 - margin)."""
    rng = np.random.default_rng(77)
    rows, V = 16, 40000
    logits = (rng.standard_normal((rows, V)) * 20).astype(np.float32)
    params = random_params(rng, rows, ks=(1, 5, 40, 200))
    hist = rng.integers(0, V, size=(rows, 64)).astype(np.int32)
    check_against_oracle(logits, params, 200, history=hist, cand_cap=200, logit_softcap=0.5, where="saturating")


def test_fused_long_shortlists():
    """top_k 257..1024 (the 512-thread shape of the plain-load kernel) and top_k above 1024 (the
    long-shortlist kernel) with post-processing."""
    rng = np.random.default_rng(78)
    rows, V = 12, 30011
    logits = (rng.standard_normal((rows, V)) * 6).astype(np.float32)
    hist = rng.integers(0, V, size=(rows, 32)).astype(np.int32)
    params = random_params(rng, rows, ks=(300, 511, 513, 700, 1024))
    check_against_oracle(logits, params, 1024, history=hist, cand_cap=1024, logit_scale=1.5, logit_softcap=30.0,
                         where="k<=1024")
    params = random_params(rng, rows, ks=(2000, 30011))
    check_against_oracle(logits, params, V, history=hist, cand_cap=0, logit_scale=1.5, logit_softcap=30.0,
                         exact_prob=False, where="k>1024")


def test_fused_equals_rewrite_then_sample_with_tanhf():
    """The tanhf flavour of the cap (the reference's device kernel) has no CPU twin; the fused
    path must pick the tokens the unfused device path picks: rewrite in place, then sample."""
    rng = np.random.default_rng(79)
    rows, V = 64, 50000
    logits = (rng.standard_normal((rows, V)) * 9).astype(np.float32)
    hist = rng.integers(0, V, size=(rows, 48)).astype(np.int32)
    params = random_params(rng, rows)
    d = torch.from_numpy(logits).to(DEV)
    fused = run_gpu(d, params, 300, history=hist, cand_cap=300, flags=native.FLAG_SOFTCAP_TANHF, logit_scale=0.5,
                    logit_softcap=20.0)
    assert np.array_equal(d.cpu().numpy(), logits)  # the fused path reads only
    sampler.logit_postprocess_rows_(d, 0.5, 20.0, flags=native.FLAG_SOFTCAP_TANHF)
    plain = run_gpu(d, params, 300, history=hist, cand_cap=300)
    for key in ("next", "n_kept", "cut", "cand_idx", "cand_prob"):
        assert np.array_equal(fused[key], plain[key]), key
    assert fused["status"] == 0


def test_fused_vocabulary_shards():
    """Local shortlists of vocabulary shards with post-processing, merged: the whole-row answer."""
    rng = np.random.default_rng(80)
    rows, V, G, k = 32, 8192, 4, 50
    logits = (rng.standard_normal((rows, V)) * 7).astype(np.float32)
    hist = rng.integers(0, V, size=(rows, 64)).astype(np.int32)
    params = np.array([O.normalize(temperature=0.7, top_k=k, top_p=0.95, repeat_penalty=1.15, repeat_last_n=64,
                                   uniform=float(rng.random())) for _ in range(rows)])
    ref_logits = O.postprocess(logits.copy(), 2.0, 30.0)
    ref = O.sample_rows(ref_logits, params, history=hist)
    d = torch.from_numpy(logits).to(DEV)
    p_dev = sampler.params_to_device(params, d.device)
    h_dev = torch.from_numpy(hist).to(DEV)
    shard = V // G
    parts = []
    for g in range(G):
        parts.append(sampler.local_topk(d[:, g * shard:(g + 1) * shard], p_dev, k, g * shard, V, history=h_dev,
                                        logit_scale=2.0, logit_softcap=30.0))
    val = torch.stack([p[0] for p in parts]).contiguous()
    idx = torch.stack([p[1] for p in parts]).contiguous()
    cnt = torch.stack([p[2] for p in parts]).contiguous()
    out = sampler.merge_parts(p_dev, k, V, val, idx, cnt)
    torch.cuda.synchronize()
    assert np.array_equal(out.next.cpu().numpy(), ref["next"])


def test_fused_unaligned_rows_and_forced_splits():
    """Rows that start off a 16-byte boundary, a padded stride whose padding must never be read,
    and rows forced over several CTAs, all with post-processing."""
    rng = np.random.default_rng(81)
    for V, stride in [(9999, 9999), (10001, 10003), (151937, 151937)]:
        rows = 7
        full = (rng.standard_normal((rows, stride)) * 6).astype(np.float32)
        full[:, V:] = 1e30
        params = random_params(rng, rows, ks=(1, 20, 200))
        hist = rng.integers(0, V, size=(rows, 64)).astype(np.int32)
        ref_logits = O.postprocess(full[:, :V].copy(), 0.75, 12.0)  # a copy: the device gets the raw logits
        ref = O.sample_rows(ref_logits, params, history=hist, cand_cap=200)
        for splits in (1, 3, 0):
            dev = torch.from_numpy(full).to(DEV)
            gpu = run_gpu(dev, params, 200, history=hist, cand_cap=200, vocab=V, splits=splits, logit_scale=0.75,
                          logit_softcap=12.0)
            compare(gpu, ref, 200, where="V %d stride %d splits %d" % (V, stride, splits))
            assert gpu["status"] == 0
