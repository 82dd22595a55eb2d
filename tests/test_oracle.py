"""The CPU oracle against the reference's own known answers and a second restatement.

No GPU needed.  The expected values are the ones internal/logits/sampler_test.go holds.
"""
import numpy as np
import pytest

import oracle_lib as O
import pyref


def run1(logits, uniform=0.5, recent=None, exclude=None, cand_cap=16, **cfg):
    p = O.normalize(uniform=uniform, **cfg)
    lg = np.array([logits], dtype=np.float32)
    hist = None if recent is None else np.array([recent], dtype=np.int32)
    out = O.sample_rows(lg, np.array([p]), history=hist, exclude=exclude, cand_cap=cand_cap, use_sort=0)
    return out, lg[0]


# ---- golden vectors: internal/logits/sampler_test.go -------------------------------------------

def test_reference_greedy_topk1():  # sampler_test.go:20-27
    out, _ = run1([-1, 5, 3, 7, 2], seed=99, temperature=1.0, top_k=1, top_p=1.0)
    assert out["next"][0] == 3


def test_reference_temp_zero_is_greedy():  # sampler_test.go:29-41
    out, _ = run1([-1, 5, 3, 7, 2], seed=99, temperature=0.0, top_k=40, top_p=0.95)
    assert out["next"][0] == 3


def test_reference_top_p_prefix():  # sampler_test.go:47-58: index 0 on every draw
    for r in [0.0, 1e-9, 0.25, 0.5, 0.75, 0.999, 1.0 - 2.0 ** -53]:
        out, _ = run1([10, 0, 0, 0, 0], uniform=r, seed=7, temperature=1.0, top_k=5, top_p=0.5)
        assert out["next"][0] == 0
        assert out["cut"][0] == 1


def test_reference_determinism():  # sampler_test.go:7-16 (pins equality only)
    a, _ = run1([0, 1, 2, 3, 4, 5], uniform=0.37, seed=42, temperature=0.9, top_k=4, top_p=0.95)
    b, _ = run1([0, 1, 2, 3, 4, 5], uniform=0.37, seed=42, temperature=0.9, top_k=4, top_p=0.95)
    assert a["next"][0] == b["next"][0]
    assert a["n_kept"][0] == 4


def test_reference_greedy_pair():  # inference/engine_panic_test.go:29-35 uses greedy on {1,0}
    out, _ = run1([1, 0], temperature=0.0)
    assert out["next"][0] == 0


# ---- constructor normalisation: sampler.go:61-83 ---------------------------------------------

def test_normalize_defaults():
    p = O.normalize()
    assert p["greedy"] == 1 and p["temperature"] == 1.0
    assert p["top_k"] == 40 and p["top_p"] == 1.0
    assert p["repeat_penalty"] == 1.0 and p["repeat_last_n"] == 64
    p = O.normalize(temperature=0.7, top_k=-3, top_p=1.5, repeat_penalty=-1, repeat_last_n=-5, min_p=0.05)
    assert p["greedy"] == 0 and p["temperature"] == np.float32(0.7)
    assert p["top_k"] == 40 and p["top_p"] == 1.0 and p["min_p"] == np.float32(0.05)
    assert p["repeat_penalty"] == 1.0 and p["repeat_last_n"] == 64
    p = O.normalize(temperature=0.7, top_k=20, top_p=0.95, repeat_penalty=1.1, repeat_last_n=256)
    assert p["top_k"] == 20 and p["top_p"] == np.float32(0.95)
    assert p["repeat_penalty"] == np.float32(1.1) and p["repeat_last_n"] == 256


def test_can_use_device_greedy():  # sampler.go:56-58
    assert O.can_use_device_greedy(O.normalize(temperature=0.0, repeat_penalty=1.0))
    assert not O.can_use_device_greedy(O.normalize(temperature=0.0, repeat_penalty=1.1))
    assert not O.can_use_device_greedy(O.normalize(temperature=0.5, repeat_penalty=1.0))


# ---- fast_exp: sampler.go:10-31 -----------------------------------------------------------------

def test_fast_exp_known_points():
    assert O.fast_exp(0.0) == 1.0
    assert O.fast_exp(89.0) == float(np.float32(3.4028235e38))
    assert O.fast_exp(-89.0) == 0.0
    assert O.fast_exp(-88.0) == 0.0  # k = -127: the scale factor's bits are zero
    assert abs(O.fast_exp(-10.0) - 4.539988e-05) < 1e-11


def test_fast_exp_matches_second_restatement_and_libm():
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.uniform(-90, 90, 4000), rng.uniform(-1, 1, 1000), [-0.0, 0.34657359, -0.34657359]])
    for x in xs.astype(np.float32):
        a, b = O.fast_exp(x), float(pyref.fast_exp(x))
        assert a == b, (x, a, b)
        if -80 < x < 80:
            assert abs(a - np.exp(np.float64(x))) <= 1e-3 * np.exp(np.float64(x))


# ---- hand-derived branch cases ------------------------------------------------------------------

def test_penalty_sign_rule_dedupe_and_exclude():
    logits = [2.0, -2.0, 0.0, 4.0, 1.0, 3.0]
    out, lg = run1(logits, recent=[0, 1, 0, 2, 5, 99, -1], exclude=[5], temperature=0.0,
                   repeat_penalty=2.0, repeat_last_n=64)
    # 0: positive, divided once although seen twice; 1: negative, multiplied; 2: zero stays;
    # 5: excluded; 99 and -1: out of range, ignored
    assert lg.tolist() == [1.0, -4.0, 0.0, 4.0, 1.0, 3.0]
    assert out["next"][0] == 3


def test_penalty_window_and_inactive():
    logits = [5.0, 4.0, 3.0]
    _, lg = run1(logits, recent=[0, 1, 2], temperature=0.0, repeat_penalty=2.0, repeat_last_n=2)
    assert lg.tolist() == [5.0, 2.0, 1.5]
    _, lg = run1(logits, recent=[0, 1, 2], temperature=0.0, repeat_penalty=1.0)
    assert lg.tolist() == logits
    _, lg = run1(logits, recent=[0, 1, 2], temperature=0.0, repeat_penalty=0.5)
    assert lg.tolist() == logits  # penalties in (0,1] never run (sampler.go:99)


def test_penalty_changes_greedy_choice():
    out, _ = run1([5.0, 4.9], recent=[0], temperature=0.0, repeat_penalty=1.1)
    assert out["next"][0] == 1
    assert not O.can_use_device_greedy(O.normalize(temperature=0.0, repeat_penalty=1.1))


def test_argmax_ties_take_lowest_index():
    out, _ = run1([1.0, 7.0, 7.0, -0.0, 7.0], temperature=0.0)
    assert out["next"][0] == 1
    out, _ = run1([-0.0, 0.0, -1.0], temperature=0.0)
    assert out["next"][0] == 0  # -0.0 == +0.0: the first one wins


def test_topk_order_and_ties():
    idx, val = O.topk([1, 3, 3, 2, 3, 0], 3, 1.0)
    assert idx.tolist() == [1, 2, 4]
    idx, val = O.topk([1, 3, 3, 2, 3, 0], 2, 1.0)
    assert idx.tolist() == [1, 2]  # the equal value arriving later is rejected
    idx, val = O.topk([0.0, -0.0, 0.0], 2, 1.0)
    assert idx.tolist() == [0, 1]
    idx, val = O.topk([1, 2, 3], 10, 0.5)
    assert idx.tolist() == [2, 1, 0] and val.tolist() == [1.5, 1.0, 0.5]


def test_nan_is_admitted_while_the_shortlist_has_room():
    """The reference's topK on NaN (sampler.go:268-275): `topVal[pos-1] < v` is false on either
    side of a NaN, so a NaN is appended while the list has room and then shields everything
    before it from later, larger values.  The answer depends on where the NaN sits, which is why
    NaN logits are outside the sampling contract; the oracle restates the behaviour as it is."""
    idx, val = O.topk([np.nan, 1.0, 2.0], 2, 1.0)
    assert idx.tolist() == [0, 2] and np.isnan(val[0]) and val[1] == 2.0
    idx, val = O.topk([1.0, 2.0, np.nan], 2, 1.0)  # the list is full when the NaN arrives: dropped
    assert idx.tolist() == [1, 0]


def test_topk1_with_temperature_takes_full_path():
    out, _ = run1([1.0, 2.0, 0.5], uniform=0.99, temperature=0.5, top_k=1, top_p=1.0)
    assert out["next"][0] == 1 and out["n_kept"][0] == 1 and out["cut"][0] == 1
    assert out["cand_prob"][0, 0] == 1.0


def test_top_p_one_means_no_cut_and_tail_mass_falls_on_last():
    out, _ = run1([0.0, 0.0, 0.0, 0.0], uniform=1.0 - 2.0 ** -53, temperature=1.0, top_k=4, top_p=1.0)
    assert out["cut"][0] == 4 and out["next"][0] == 3
    # r beyond the (un-renormalised) nucleus mass falls on the last nucleus entry
    out, _ = run1([0.0, 0.0, 0.0, 0.0], uniform=0.9, temperature=1.0, top_k=4, top_p=0.5)
    assert out["cut"][0] == 2 and out["next"][0] == 1


def test_min_p_filters_and_renormalises():
    logits = [4.0, 3.9, 0.0, -3.0]
    out, _ = run1(logits, uniform=0.999, temperature=1.0, top_k=4, top_p=1.0, min_p=0.5)
    assert out["n_kept"][0] == 2
    assert abs(out["cand_prob"][0, :2].sum() - 1.0) < 1e-12
    assert out["next"][0] == 1
    out, _ = run1(logits, uniform=0.999, temperature=1.0, top_k=4, top_p=1.0, min_p=0.0)
    assert out["n_kept"][0] == 4 and out["next"][0] in (2, 3)


def test_k_larger_than_vocab():
    out, _ = run1([0.5, 1.5], uniform=0.0, temperature=1.0, top_k=40, top_p=1.0)
    assert out["n_kept"][0] == 2 and out["next"][0] == 1


# ---- C oracle == numpy restatement on seeded random small cases ----------------------------------

@pytest.mark.parametrize("seed", range(6))
def test_oracle_equals_second_restatement(seed):
    rng = np.random.default_rng(100 + seed)
    rows = 40
    V = int(rng.integers(1, 300))
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    logits[rng.random((rows, V)) < 0.1] = 0.0
    logits = np.round(logits * 4) / 4 if seed % 2 else logits  # force ties on odd seeds
    logits = logits.astype(np.float32)
    H = 24
    hist = rng.integers(-2, V + 2, size=(rows, H)).astype(np.int32)
    hist_len = rng.integers(0, H + 1, size=rows).astype(np.int32)
    exclude = rng.integers(0, V, size=3).astype(np.int32)
    params = np.zeros(rows, dtype=O.PARAMS_DTYPE)
    for r in range(rows):
        params[r] = O.normalize(
            temperature=float(rng.choice([0.0, 0.3, 0.8, 1.0, 1.5])),
            top_k=int(rng.choice([0, 1, 2, 5, 40, 500])),
            top_p=float(rng.choice([0.0, 0.5, 0.9, 0.95, 1.0])),
            min_p=float(rng.choice([0.0, 0.05, 0.3])),
            repeat_penalty=float(rng.choice([0.0, 1.0, 1.1, 1.3])),
            repeat_last_n=int(rng.choice([0, 4, 64])),
            uniform=float(rng.random()),
        )
    ref_logits = logits.copy()
    out = O.sample_rows(logits, params, history=hist, hist_len=hist_len, exclude=exclude, cand_cap=V, use_sort=0)
    out_sorted = O.sample_rows(ref_logits.copy(), params, history=hist, hist_len=hist_len, exclude=exclude,
                               cand_cap=V, use_sort=1)
    for r in range(rows):
        row = ref_logits[r].copy()
        tok, idx, prob, cut = pyref.sample(row, hist[r, : hist_len[r]], exclude, params[r])
        assert tok == out["next"][r], (seed, r)
        assert np.array_equal(row, logits[r])  # in-place penalty side effect
        assert cut == out["cut"][r]
        n = out["n_kept"][r]
        assert n == len(idx) or (cut == 0 and n == 0)
        if n:
            assert out["cand_idx"][r, :n].tolist() == idx
            assert out["cand_prob"][r, :n].tolist() == [float(x) for x in prob]
    # insertion shortlist == full ordering (the large-k stand-in)
    for key in ("next", "n_kept", "cut", "cand_idx", "cand_prob"):
        assert np.array_equal(out[key], out_sorted[key]), key


def test_bf16_rows_are_widened_exactly():
    rng = np.random.default_rng(5)
    f = (rng.standard_normal((8, 64)) * 2).astype(np.float32)
    bits = (f.view(np.uint32) >> 16).astype(np.uint16)  # truncation is fine here: any bf16 pattern will do
    wide = (bits.astype(np.uint32) << 16).view(np.float32).copy()
    params = np.array([O.normalize(temperature=0.9, top_k=10, top_p=0.9, uniform=0.1 * i) for i in range(8)])
    a = O.sample_rows(bits, params, cand_cap=10)
    b = O.sample_rows(wide, params, cand_cap=10)
    for key in ("next", "n_kept", "cut", "cand_idx", "cand_prob"):
        assert np.array_equal(a[key], b[key])


def test_batch_driver_threads_agree():
    rng = np.random.default_rng(9)
    logits = (rng.standard_normal((33, 500)) * 3).astype(np.float32)
    params = np.array([O.normalize(temperature=0.8, top_k=20, top_p=0.95, uniform=float(rng.random()))
                       for _ in range(33)])
    a = O.sample_rows(logits.copy(), params, threads=1)
    b = O.sample_rows(logits.copy(), params, threads=4)
    assert a["threads"] == 1 and b["threads"] == 4
    assert np.array_equal(a["next"], b["next"])


# ---- the model head's post-processing (simd/runtime.go:258-272, simd/ops.go:165-175) --------------

def test_postprocess_properties_the_reference_tests_hold():
    """internal/backend/cuda/graph_test.go:255-263: a cap that is not positive is the identity;
    a large logit is damped to something positive below itself.  Plus the gates of the
    multiplier (0 and 1 leave the logits alone) and the saturation points of fastTanh."""
    x = np.array([1.0, 100.0, -3.0, 0.0], dtype=np.float32)
    assert np.array_equal(O.postprocess(x.copy(), 0.0, 0.0), x)
    assert np.array_equal(O.postprocess(x.copy(), 1.0, -5.0), x)
    y = O.postprocess(x.copy(), 0.0, 30.0)
    assert 0.0 < y[1] < 30.0 and abs(y[1] - 30.0 * np.tanh(100.0 / 30.0)) < 1e-3
    assert np.array_equal(O.postprocess(x.copy(), 2.0, 0.0), x * np.float32(2.0))
    assert O.fast_tanh(10.5) == 1.0 and O.fast_tanh(-10.5) == -1.0 and O.fast_tanh(0.0) == 0.0
    # fastTanh built on fastExp: (e - 1) / (e + 1) in float32
    for v in (0.3, -0.3, 2.5, 9.99):
        e = np.float32(O.fast_exp(float(np.float32(2.0) * np.float32(v))))
        assert O.fast_tanh(v) == float((e - np.float32(1.0)) / (e + np.float32(1.0)))


def test_fast_tanh_error_bound():
    """The streaming kernel's raw-logit filter relies on |fastTanh - tanh| < 1e-5 (it allows for
    several times that); sampled here, the exhaustive figure over [-10, 10] is 1.7e-6."""
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.uniform(-10, 10, 200000), rng.uniform(-0.5, 0.5, 100000)]).astype(np.float32)
    got = O.postprocess(xs.copy(), 0.0, 1.0)
    assert np.max(np.abs(got.astype(np.float64) - np.tanh(xs.astype(np.float64)))) < 3e-6


# ---- committed fixtures (tests/golden) ------------------------------------------------------------

def load_golden():
    import json
    import os

    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    with open(os.path.join(here, "reference_vectors.json")) as f:
        ref = json.load(f)["cases"]
    z = np.load(os.path.join(here, "oracle_cases.npz"))
    return ref, z


def test_reference_vectors_file():
    """Every expected value the reference's tests hold, from the committed transcription."""
    ref, _ = load_golden()
    assert len(ref) == 5
    for case in ref:
        toks = []
        for u in case["uniforms"]:
            out, _ = run1(case["logits"], uniform=u, **case["config"])
            toks.append(int(out["next"][0]))
            if "expect_next" in case:
                assert toks[-1] == case["expect_next"], case["source"]
            if "expect_cut" in case:
                assert int(out["cut"][0]) == case["expect_cut"], case["source"]
            if "expect_n_kept" in case:
                assert int(out["n_kept"][0]) == case["expect_n_kept"], case["source"]
        if case.get("expect_same_token_for_equal_uniforms"):
            assert len(set(toks)) == 1, case["source"]


def test_oracle_reproduces_the_committed_cases():
    """The oracle has not drifted from the answers committed with its inputs, with and without the
    model head's post-processing; make_fixtures.py wrote them."""
    _, z = load_golden()
    params = z["params"].view(O.PARAMS_DTYPE)
    for prefix, scale, cap in (("", 0.0, 0.0), ("post_", float(z["post_scale"]), float(z["post_cap"]))):
        lg = z["logits"].copy()
        if prefix:
            O.postprocess(lg, scale, cap)
        out = O.sample_rows(lg, params, history=z["history"], hist_len=z["hist_len"], exclude=z["exclude"],
                            cand_cap=z["cand_idx"].shape[1])
        assert np.array_equal(out["next"], z[prefix + "next"])
        assert np.array_equal(out["n_kept"], z[prefix + "n_kept"])
        assert np.array_equal(out["cut"], z[prefix + "cut"])
        assert np.array_equal(out["cand_idx"], z[prefix + "cand_idx"])
        assert np.array_equal(out["cand_prob"], z[prefix + "cand_prob"])
    assert len(set(z["next"].tolist())) > 10  # the batch is not degenerate


def test_second_restatement_reproduces_the_committed_cases():
    """The numpy restatement (written independently of the C oracle) gives the committed tokens."""
    _, z = load_golden()
    params = z["params"].view(O.PARAMS_DTYPE)
    for r in range(0, z["logits"].shape[0], 3):
        hl = int(z["hist_len"][r])
        tok, idx, prob, cut = pyref.sample(z["logits"][r].copy(), z["history"][r, :hl].tolist(),
                                           z["exclude"].tolist(), params[r])
        assert tok == int(z["next"][r]), r
        assert cut == int(z["cut"][r]), r
