"""The batched decode loop (MantleBatchSampler: per-row configurations, histories and "has ended"
flags on the device) against the reference's loop restated on the CPU (inference/engine.go:189,
233-300: sample, leave on a stop token, append the token to the context, next step) with the
oracle as its sampler and one random generator per request, drawn from exactly when the
reference's Sampler draws (sampler.go:140-142, 224)."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from mantle_b200 import sampler

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def argmax_shortcut(p):
    return bool(p["greedy"]) or (p["top_k"] == 1 and p["top_p"] >= 1 and p["temperature"] == 1)


class Request:
    """What the reference keeps per request: toks, the normalised sampler, its generator."""

    def __init__(self, params, prompt, seed):
        self.params = params
        self.toks = list(prompt)
        self.rng = np.random.default_rng(seed).random
        self.done = False

    def sample(self, logits_row, stop):
        p = np.array([self.params], dtype=O.PARAMS_DTYPE)
        if not argmax_shortcut(self.params):
            p["uniform"] = self.rng()  # one draw per stochastic Sample, none otherwise
        hist = np.array([self.toks], dtype=np.int32) if self.toks else None
        res = O.sample_rows(logits_row[None, :].copy(), p, history=hist, exclude=np.array(stop, dtype=np.int32))
        return int(res["next"][0])


def make_logits(rng, rows, V, stop, t, stop_rows):
    lg = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
    lg[:, :40] += 4.0          # a small hot set, so that repeats (and the penalty) actually occur
    lg[:, stop] = -30.0
    for r in stop_rows:        # these rows meet a stop token at a step of their own
        if t == 20 + 2 * r:
            lg[r, stop[r % 2]] = 60.0
    return lg


@pytest.mark.parametrize("capacity,V,ks", [(64, 3001, (1, 8, 40)), (512, 3001, (1, 8, 40)),
                                           (64, 60001, (1, 40, 100))])  # the last: whole rows of the histogram kernel
def test_decode_loop_through_the_batch_sampler(capacity, V, ks):
    rng = np.random.default_rng(2024 + capacity + V)
    rows, steps, last_n = (24 if V < 10000 else 12), 90, 24
    stop = [1500, V - 501]
    cfgs, reqs = [], []
    for r in range(rows):
        cfg = sampler.SamplerConfig(seed=100 + r, temperature=float(rng.choice([0.0, 0.7, 1.0])),
                                    top_k=int(rng.choice(ks)), top_p=float(rng.choice([0.9, 1.0])),
                                    repeat_penalty=float(rng.choice([1.0, 1.2, 1.5])), repeat_last_n=last_n)
        prompt = rng.integers(0, V, size=int(rng.integers(0, 20))).tolist()
        cfgs.append(cfg)
        reqs.append(Request(sampler.new_sampler_params(cfg), prompt, 100 + r))

    bs = sampler.BatchSampler(rows, V, capacity, stop, device=DEV)
    gpu_rngs = [np.random.default_rng(100 + r).random for r in range(rows)]
    for r in range(rows):
        assert not bs.needs_uniform(r)  # not started yet
        bs.set_row(r, cfgs[r], reqs[r].toks)
        assert bs.needs_uniform(r) == (not argmax_shortcut(reqs[r].params))
        assert bs.can_use_device_greedy(r) == sampler.can_use_device_greedy(reqs[r].params)

    stop_rows = range(0, rows, 3)
    for t in range(steps):
        lg = make_logits(rng, rows, V, stop, t, stop_rows)
        was_done = [q.done for q in reqs]
        nxt, ended = bs.step(torch.from_numpy(lg).to(DEV), gpu_rngs)
        for r, q in enumerate(reqs):
            if q.done:
                assert nxt[r] == -1 and ended[r] == 1
                continue
            tok = q.sample(lg[r], stop)
            assert nxt[r] == tok, (t, r, nxt[r], tok)
            if tok in stop:
                q.done = True           # the reference leaves its loop before the append
            else:
                q.toks.append(tok)
            assert bool(ended[r]) == q.done
        assert not any(was_done[r] and not reqs[r].done for r in range(rows))
    done = [q.done for q in reqs]
    assert any(done) and not all(done)
    assert max(len(q.toks) for q in reqs) > 64  # with capacity 64 at least one history buffer wrapped
    _, _, status = bs.results()
    assert status == 0

    # a finished slot takes a new request; a live one is ended by the host
    r_new = done.index(True)
    r_end = done.index(False)
    cfg = sampler.SamplerConfig(seed=7, temperature=0.8, top_k=20, top_p=0.95, repeat_penalty=1.3, repeat_last_n=last_n)
    prompt = rng.integers(0, V, size=100).tolist()  # longer than capacity 64: the most recent ids are kept
    reqs[r_new] = Request(sampler.new_sampler_params(cfg), prompt, 7)
    gpu_rngs[r_new] = np.random.default_rng(7).random
    bs.set_row(r_new, cfg, prompt)
    bs.end_row(r_end)
    reqs[r_end].done = True
    for t in range(10):
        lg = make_logits(rng, rows, V, stop, -1, ())
        nxt, ended = bs.step(torch.from_numpy(lg).to(DEV), gpu_rngs)
        for r, q in enumerate(reqs):
            if q.done:
                assert nxt[r] == -1 and ended[r] == 1
                continue
            tok = q.sample(lg[r], stop)
            assert nxt[r] == tok, ("restart", t, r)
            q.toks.append(tok)
    bs.close()


def test_batch_sampler_rejects_a_window_the_history_cannot_hold():
    bs = sampler.BatchSampler(4, 1000, 64, [], device=DEV)
    from mantle_b200 import native

    with pytest.raises(native.CudaError):
        bs.set_row(0, sampler.SamplerConfig(temperature=1.0, repeat_penalty=1.1, repeat_last_n=33))
    bs.set_row(0, sampler.SamplerConfig(temperature=1.0, repeat_penalty=1.1, repeat_last_n=32))
    bs.close()
