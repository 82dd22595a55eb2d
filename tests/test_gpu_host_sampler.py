"""The host-side Sampler object (the mirror of logits.Sampler) on a GPU.  The first four tests
are the reference's own tests (internal/logits/sampler_test.go) restated against it."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from mantle_b200.sampler import Sampler, SamplerConfig

pytestmark = pytest.mark.gpu


def f32(x):
    return np.array(x, dtype=np.float32)


def test_sampler_determinism():  # sampler_test.go:7-16
    cfg = SamplerConfig(seed=42, temperature=0.9, top_k=4, top_p=0.95)
    s1, s2 = Sampler(cfg, 64), Sampler(cfg, 64)
    assert s1.sample(f32([0, 1, 2, 3, 4, 5])) == s2.sample(f32([0, 1, 2, 3, 4, 5]))


def test_sampler_greedy():  # sampler_test.go:20-27
    s = Sampler(SamplerConfig(seed=99, temperature=1.0, top_k=1, top_p=1.0), 64)
    assert s.sample(f32([-1, 5, 3, 7, 2])) == 3


def test_sampler_temp_zero_is_greedy():  # sampler_test.go:29-41
    s = Sampler(SamplerConfig(seed=99, temperature=0.0, top_k=40, top_p=0.95), 64)
    assert s.sample(f32([-1, 5, 3, 7, 2])) == 3
    assert s.can_use_device_greedy()


def test_sampler_top_p():  # sampler_test.go:47-58
    s = Sampler(SamplerConfig(seed=7, temperature=1.0, top_k=5, top_p=0.5), 64)
    for _ in range(10):
        assert s.sample(f32([10, 0, 0, 0, 0])) == 0


def test_uniform_is_consumed_only_on_the_stochastic_path():  # sampler.go:140-142, 224
    draws = []

    def rng():
        draws.append(1)
        return 0.5

    Sampler(SamplerConfig(temperature=0.0), 64, rng=rng).sample(f32([1, 2, 3]))
    Sampler(SamplerConfig(temperature=1.0, top_k=1, top_p=1.0), 64, rng=rng).sample(f32([1, 2, 3]))
    assert draws == []
    Sampler(SamplerConfig(temperature=0.5, top_k=1, top_p=1.0), 64, rng=rng).sample(f32([1, 2, 3]))
    assert draws == [1]


def test_sample_matches_oracle_and_patches_the_slice_in_place():
    rng = np.random.default_rng(4)
    V = 151936
    for trial in range(6):
        cfg = dict(temperature=float(rng.choice([0.0, 0.6, 1.0])), top_k=int(rng.choice([0, 1, 20, 200])),
                   top_p=float(rng.choice([0.9, 1.0])), min_p=float(rng.choice([0.0, 0.05])),
                   repeat_penalty=float(rng.choice([1.0, 1.1, 1.3])), repeat_last_n=int(rng.choice([0, 64, 512])))
        u = float(rng.random())
        s = Sampler(SamplerConfig(**cfg), V, rng=lambda: u)
        logits = (rng.standard_normal(V) * 3).astype(np.float32)
        recent = rng.integers(-5, V + 5, size=int(rng.integers(0, 700))).astype(np.int64)
        exclude = rng.integers(0, V, size=2).astype(np.int64)
        p = O.normalize(uniform=u, **cfg)
        got_p = s.params()
        for field in ("temperature", "top_k", "top_p", "min_p", "repeat_penalty", "repeat_last_n", "greedy"):
            assert got_p[field] == p[field], field
        want_logits = logits.copy()[None, :]
        ref = O.sample_rows(want_logits, np.array([p]), history=recent.astype(np.int32)[None, :] if recent.size else None,
                            exclude=exclude.astype(np.int32))
        dev = torch.from_numpy(logits.copy()).cuda()
        got = s.sample(logits, recent, exclude)
        assert got == ref["next"][0], (trial, cfg)
        assert np.array_equal(logits, want_logits[0])  # the in-place penalty side effect (sampler.go:132-136)
        assert s.sample_device(dev, recent, exclude) == ref["next"][0]
        s.close()
