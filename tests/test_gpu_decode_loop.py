"""A batched decode loop with histories that never leave the device, against the reference's
loop restated on the CPU (inference/engine.go:233-300: sample, leave on a stop token, append the
token to the context, next step) with the oracle as its sampler."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from mantle_b200 import native, sampler

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def reference_loop(logits_steps, params_steps, prompts, stop):
    """One python list of context tokens per row; returns tokens per step (-9 once a row is done)."""
    rows = len(prompts)
    toks = [list(p) for p in prompts]
    done = [False] * rows
    out = []
    for lg, ps in zip(logits_steps, params_steps):
        step = np.full(rows, -9, dtype=np.int64)
        for r in range(rows):
            if done[r]:
                continue
            hist = np.array([toks[r]], dtype=np.int32) if toks[r] else None
            res = O.sample_rows(lg[r:r + 1].copy(), ps[r:r + 1], history=hist, exclude=np.array(stop, dtype=np.int32))
            nxt = int(res["next"][0])
            step[r] = nxt
            if nxt in stop:
                done[r] = True
            else:
                toks[r].append(nxt)
        out.append(step)
    return out, toks, done


@pytest.mark.parametrize("stride,keep", [(64, 32), (512, 24)])
def test_decode_loop_with_device_histories(stride, keep):
    rng = np.random.default_rng(2024 + stride)
    rows, V, steps, last_n = 24, 3001, 90, 24
    stop = [1500, 2500]
    prompts = [rng.integers(0, V, size=int(rng.integers(0, 20))).tolist() for _ in range(rows)]
    base = np.zeros(rows, dtype=O.PARAMS_DTYPE)
    for r in range(rows):
        base[r] = O.normalize(temperature=float(rng.choice([0.0, 0.7, 1.0])), top_k=int(rng.choice([1, 8, 40])),
                              top_p=float(rng.choice([0.9, 1.0])), repeat_penalty=float(rng.choice([1.0, 1.2, 1.5])),
                              repeat_last_n=last_n)
    logits_steps, params_steps = [], []
    for t in range(steps):
        lg = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
        lg[:, :40] += 4.0          # a small hot set, so that repeats (and the penalty) actually occur
        lg[:, stop] = -30.0
        for r in range(0, rows, 3):  # every third row meets a stop token at a step of its own
            if t == 20 + 2 * r:
                lg[r, stop[r % 2]] = 60.0
        p = base.copy()
        p["uniform"] = rng.random(rows)
        logits_steps.append(lg)
        params_steps.append(p)
    ref_steps, ref_toks, ref_done = reference_loop(logits_steps, params_steps, prompts, stop)

    hist = torch.zeros((rows, stride), dtype=torch.int32, device=DEV)
    hist_len = torch.zeros(rows, dtype=torch.int32, device=DEV)
    for r, p in enumerate(prompts):
        hist[r, : len(p)] = torch.tensor(p, dtype=torch.int32)
        hist_len[r] = len(p)
    done = torch.zeros(rows, dtype=torch.int32, device=DEV)
    stop_dev = torch.tensor(stop, dtype=torch.int32, device=DEV)
    for t in range(steps):
        d = torch.from_numpy(logits_steps[t]).to(DEV)
        p_dev = sampler.params_to_device(params_steps[t], d.device)
        out = sampler.sample_rows(d, p_dev, 40, history=hist, hist_len=hist_len, exclude=stop_dev)
        was_done = done.cpu().numpy().astype(bool)
        sampler.history_append_rows_(hist, hist_len, out.next, keep, stop=stop_dev, done=done)
        torch.cuda.synchronize()
        got = out.next.cpu().numpy()
        live = ~was_done
        assert np.array_equal(got[live], ref_steps[t][live]), (t, got, ref_steps[t])
    assert np.array_equal(done.cpu().numpy().astype(bool), np.array(ref_done))
    assert any(ref_done) and not all(ref_done)
    h, n = hist.cpu().numpy(), hist_len.cpu().numpy()
    for r in range(rows):
        m = min(int(n[r]), last_n, len(ref_toks[r]))
        assert m == min(last_n, len(ref_toks[r]))
        assert h[r, n[r] - m:n[r]].tolist() == ref_toks[r][len(ref_toks[r]) - m:], r  # the penalty window
    if stride == 64:
        assert max(len(t) for t in ref_toks) > stride  # at least one buffer wrapped
