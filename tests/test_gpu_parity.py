"""Parity of the CUDA sampler with the CPU oracle, through the C-ABI, on a B200."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import check_against_oracle, compare, run_gpu, to_bf16_bits
from mantle_b200 import native, sampler, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def P(uniform=0.5, **cfg):
    return O.normalize(uniform=uniform, **cfg)


def one(logits, uniform=0.5, recent=None, exclude=None, cand_cap=8, flags=0, **cfg):
    p = np.array([P(uniform, **cfg)])
    lg = np.array([logits], dtype=np.float32)
    hist = None if recent is None else np.array([recent], dtype=np.int32)
    return check_against_oracle(lg, p, max(1, min(int(p[0]["top_k"]), 1024)), history=hist, exclude=exclude,
                                cand_cap=cand_cap, flags=flags)


# ---- the reference's own test vectors (internal/logits/sampler_test.go) through the C-ABI --------

def test_reference_vectors():
    g, _ = one([-1, 5, 3, 7, 2], seed=99, temperature=1.0, top_k=1, top_p=1.0)  # :20-27
    assert g["next"][0] == 3
    g, _ = one([-1, 5, 3, 7, 2], seed=99, temperature=0.0, top_k=40, top_p=0.95)  # :29-41
    assert g["next"][0] == 3
    for r in [0.0, 0.3, 0.999999, 1.0 - 2.0 ** -53]:  # :47-58
        g, _ = one([10, 0, 0, 0, 0], uniform=r, seed=7, temperature=1.0, top_k=5, top_p=0.5)
        assert g["next"][0] == 0 and g["cut"][0] == 1
    a, _ = one([0, 1, 2, 3, 4, 5], uniform=0.37, seed=42, temperature=0.9, top_k=4, top_p=0.95)  # :7-16
    b, _ = one([0, 1, 2, 3, 4, 5], uniform=0.37, seed=42, temperature=0.9, top_k=4, top_p=0.95)
    assert a["next"][0] == b["next"][0]
    g, _ = one([1, 0], temperature=0.0)  # inference/engine_panic_test.go:29-35
    assert g["next"][0] == 0


# ---- hand-derived branch cases ---------------------------------------------------------------------

def test_penalty_rules():
    for flags in (0, native.FLAG_WRITE_BACK_PENALTY):
        g, _ = one([2.0, -2.0, 0.0, 4.0, 1.0, 3.0], recent=[0, 1, 0, 2, 5, 99, -1], exclude=[5], temperature=0.0,
                   repeat_penalty=2.0, repeat_last_n=64, flags=flags)
        assert g["next"][0] == 3
        g, _ = one([5.0, 4.0, 3.0], recent=[0, 1, 2], temperature=0.0, repeat_penalty=2.0, repeat_last_n=2, flags=flags)
        assert g["next"][0] == 0
        g, _ = one([5.0, 4.9], recent=[0], temperature=0.0, repeat_penalty=1.1, flags=flags)
        assert g["next"][0] == 1
        one([5.0, 4.0, 3.0], recent=[0, 1, 2], temperature=0.7, top_k=3, repeat_penalty=0.5, flags=flags)
        one([5.0, 4.0, 3.0], recent=[0, 1, 2], temperature=0.7, top_k=3, repeat_penalty=1.0, flags=flags)


def test_ties_and_signed_zero():
    g, _ = one([1.0, 7.0, 7.0, -0.0, 7.0], temperature=0.0)
    assert g["next"][0] == 1
    g, _ = one([-0.0, 0.0, -1.0], temperature=0.0)
    assert g["next"][0] == 0
    g, _ = one([0.0, -0.0, 0.0, -5.0], uniform=0.5, temperature=1.0, top_k=2, top_p=1.0)
    assert g["cand_idx"][0, :2].tolist() == [0, 1]
    g, _ = one([1, 3, 3, 2, 3, 0], uniform=0.9, temperature=1.0, top_k=2, top_p=1.0)
    assert g["cand_idx"][0, :2].tolist() == [1, 2]


def test_tail_branches():
    g, _ = one([1.0, 2.0, 0.5], uniform=0.99, temperature=0.5, top_k=1, top_p=1.0)
    assert g["next"][0] == 1 and g["n_kept"][0] == 1
    g, _ = one([0.0, 0.0, 0.0, 0.0], uniform=1.0 - 2.0 ** -53, temperature=1.0, top_k=4, top_p=1.0)
    assert g["cut"][0] == 4 and g["next"][0] == 3
    g, _ = one([0.0, 0.0, 0.0, 0.0], uniform=0.9, temperature=1.0, top_k=4, top_p=0.5)
    assert g["cut"][0] == 2 and g["next"][0] == 1
    g, _ = one([4.0, 3.9, 0.0, -3.0], uniform=0.999, temperature=1.0, top_k=4, top_p=1.0, min_p=0.5)
    assert g["n_kept"][0] == 2 and g["next"][0] == 1
    g, _ = one([0.5, 1.5], uniform=0.0, temperature=1.0, top_k=40, top_p=1.0)
    assert g["n_kept"][0] == 2 and g["next"][0] == 1
    one([100.0, -100.0, 0.0], uniform=0.5, temperature=0.3, top_k=3, top_p=0.9)  # fast_exp below -88


# ---- seeded random small cases, every parameter combination -----------------------------------------

def random_params(rng, rows, ks=(0, 1, 2, 5, 40, 300)):
    params = np.zeros(rows, dtype=O.PARAMS_DTYPE)
    for r in range(rows):
        params[r] = O.normalize(
            temperature=float(rng.choice([0.0, 0.3, 0.8, 1.0, 1.5])),
            top_k=int(rng.choice(ks)),
            top_p=float(rng.choice([0.0, 0.5, 0.9, 0.95, 1.0])),
            min_p=float(rng.choice([0.0, 0.05, 0.3])),
            repeat_penalty=float(rng.choice([0.0, 1.0, 1.1, 1.3])),
            repeat_last_n=int(rng.choice([0, 4, 64])),
            uniform=float(rng.random()),
        )
    return params


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("flags", [0, native.FLAG_WRITE_BACK_PENALTY])
def test_random_small(seed, flags):
    rng = np.random.default_rng(500 + seed)
    rows = 48
    V = int(rng.choice([1, 2, 3, 7, 33, 64, 257, 1000, 5000, 9001]))
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    if seed % 2:
        logits = (np.round(logits * 2) / 2).astype(np.float32)  # heavy ties
    logits[rng.random((rows, V)) < 0.05] = 0.0
    logits[rng.random((rows, V)) < 0.02] = -0.0
    H = 40
    hist = rng.integers(-2, V + 2, size=(rows, H)).astype(np.int32)
    hist_len = rng.integers(0, H + 1, size=rows).astype(np.int32)
    exclude = rng.integers(0, V, size=3).astype(np.int32)
    params = random_params(rng, rows)
    check_against_oracle(logits, params, 300, history=hist, hist_len=hist_len, exclude=exclude, cand_cap=min(V, 300),
                         flags=flags, where="seed %d V %d" % (seed, V))


@pytest.mark.parametrize("V", [4096 * 2 + 5, 40000, 151936])
@pytest.mark.parametrize("splits", [1, 3])
def test_random_wide(V, splits):
    rng = np.random.default_rng(V + splits)
    rows = 24
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    hist = rng.integers(0, V, size=(rows, 300)).astype(np.int32)
    params = random_params(rng, rows, ks=(0, 1, 20, 50, 200, 512))
    g, _ = check_against_oracle(logits, params, 512, history=hist, cand_cap=512, splits=splits,
                                where="V %d splits %d" % (V, splits))
    assert g["splits"] == splits


def test_unaligned_rows_and_stride():
    # rows that start off a 16-byte boundary: odd vocabulary with a dense layout, and a padded stride
    rng = np.random.default_rng(77)
    for V, stride in [(9999, 9999), (10001, 10003), (151937, 151937)]:
        rows = 9
        full = (rng.standard_normal((rows, stride)) * 3).astype(np.float32)
        full[:, V:] = 1e30  # padding beyond the vocabulary must never be read as a candidate
        params = random_params(rng, rows, ks=(1, 20, 200))
        hist = rng.integers(0, V, size=(rows, 64)).astype(np.int32)
        dev = torch.from_numpy(full).to(DEV)
        gpu = run_gpu(dev, params, 200, history=hist, cand_cap=200, vocab=V)
        ref = O.sample_rows(np.ascontiguousarray(full[:, :V]), params, history=hist, cand_cap=200)
        compare(gpu, ref, 200, where="V %d stride %d" % (V, stride))


def test_bf16_rows():
    rng = np.random.default_rng(5)
    rows, V = 16, 128256
    t = (torch.from_numpy(rng.standard_normal((rows, V)).astype(np.float32)) * 2).to(torch.bfloat16)
    bits = to_bf16_bits(t)
    params = random_params(rng, rows, ks=(1, 20, 50, 400))
    hist = rng.integers(0, V, size=(rows, 128)).astype(np.int32)
    check_against_oracle(bits, params, 400, history=hist, cand_cap=400, bf16=True)
    check_against_oracle(bits[:, :1001].copy(), params, 400, history=hist, cand_cap=400, bf16=True, splits=1)


# ---- inputs built to break a streaming selection -----------------------------------------------------

@pytest.mark.parametrize("kind", ["ascending", "descending", "all_equal", "mostly_neg_inf", "two_values", "huge_k"])
def test_adversarial_rows(kind):
    rng = np.random.default_rng(11)
    rows, V = 6, 60000
    if kind == "ascending":
        logits = np.tile(np.linspace(-20, 20, V, dtype=np.float32), (rows, 1))
    elif kind == "descending":
        logits = np.tile(np.linspace(20, -20, V, dtype=np.float32), (rows, 1))
    elif kind == "all_equal":
        logits = np.full((rows, V), 1.25, dtype=np.float32)
    elif kind == "mostly_neg_inf":
        logits = np.full((rows, V), -np.inf, dtype=np.float32)
        for r in range(rows):
            logits[r, rng.integers(0, V, size=7)] = rng.standard_normal(7).astype(np.float32)
    elif kind == "two_values":
        logits = rng.choice(np.array([0.5, 2.0], dtype=np.float32), size=(rows, V))
    else:
        logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    ks = (600, 1024) if kind == "huge_k" else (1, 20, 200)
    params = random_params(rng, rows, ks=ks)
    hist = rng.integers(0, V, size=(rows, 64)).astype(np.int32)
    for splits in (1, 2):
        check_against_oracle(logits, params, 1024 if kind == "huge_k" else 200, history=hist,
                             cand_cap=1024 if kind == "huge_k" else 200, splits=splits, where=kind)


@pytest.mark.parametrize("max_k", [64, 224, 1024])
@pytest.mark.parametrize("kind", ["step_up", "outlier", "plateau", "slow_ramp", "few_levels", "masked"])
def test_histogram_kernel_hazards(kind, max_k):
    """Rows built against the kernel whose threshold comes from a running histogram of the candidate
    buffer (shortlists above 28 entries): a first region far below the rest of the row, an outlier
    that stretches the bins, the k-th value repeated thousands of times, a slow upward trend that
    keeps the buffer filling, a handful of distinct values, most of the row masked to -inf."""
    rng = np.random.default_rng(4242 + max_k)
    rows, V = 5, 70001
    base = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
    if kind == "step_up":
        logits = base.copy()
        logits[:, :13000] -= 40.0
    elif kind == "outlier":
        logits = base.copy()
        logits[:, 17] = 3.0e30
        logits[:, 50000] = 1.0e6
    elif kind == "plateau":
        logits = base.copy()
        for r in range(rows):
            v = np.sort(logits[r])[-(max_k // 2 + 3)]  # a value inside every shortlist
            logits[r, rng.choice(V, size=6000, replace=False)] = v
    elif kind == "slow_ramp":
        logits = base * 0.05 + np.linspace(-8, 8, V, dtype=np.float32)[None, :]
    elif kind == "few_levels":
        logits = rng.choice(np.array([-1.0, 0.0, 0.5, 0.75, 3.0], dtype=np.float32), size=(rows, V),
                            p=[0.3, 0.3, 0.2, 0.19, 0.01])
    else:
        logits = np.full((rows, V), -np.inf, dtype=np.float32)
        keep = rng.choice(V, size=max_k + 40, replace=False)
        logits[:, keep] = base[:, keep]
    ks = (33, max_k // 2, max_k)
    params = random_params(rng, rows, ks=ks)
    hist = rng.integers(0, V, size=(rows, 200)).astype(np.int32)
    for splits in (1, 2):
        check_against_oracle(logits.astype(np.float32), params, max_k, history=hist, cand_cap=max_k, splits=splits,
                             where="%s max_k %d splits %d" % (kind, max_k, splits))


@pytest.mark.parametrize("seed", range(4))
@pytest.mark.parametrize("max_k", [224, 1024])
def test_histogram_kernel_random_rows(seed, max_k):
    """Random rows of random texture (value granularity from float32 noise down to a few levels, a
    random share masked to -inf, a random trend along the row) at every shortlist length the
    histogram kernel serves, in both of its shapes."""
    rng = np.random.default_rng(9000 + 10 * seed + max_k)
    rows = 20
    V = int(rng.choice([50000, 151936, 262144]))
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    for r in range(rows):
        step = float(rng.choice([0.0, 0.0, 1.0 / 64, 0.25, 1.0]))
        if step:
            logits[r] = np.round(logits[r] / step) * step
        logits[r] += np.linspace(0, float(rng.choice([0.0, 0.0, 6.0, -6.0])), V, dtype=np.float32)
        share = float(rng.choice([0.0, 0.0, 0.3, 0.9]))
        if share:
            logits[r, rng.random(V) < share] = -np.inf
    ks = (33, 40, 64, 100, 200, 224) if max_k == 224 else (225, 256, 400, 512, 1000, 1024)
    params = random_params(rng, rows, ks=ks)
    hist = rng.integers(0, V, size=(rows, 300)).astype(np.int32)
    check_against_oracle(logits, params, max_k, history=hist, cand_cap=max_k,
                         where="seed %d V %d max_k %d" % (seed, V, max_k))


# ---- the benchmark configurations ---------------------------------------------------------------------

def test_config_single_row():
    w = workloads.make("single_row", device=DEV)
    check_against_oracle(w.logits.cpu().numpy(), w.params, w.max_top_k, history=w.history.cpu().numpy(), cand_cap=20)


def test_config_mixed_batch():
    w = workloads.make("mixed_batch", device=DEV)
    assert set(np.unique(w.params["top_k"])) <= {1, 20, 40, 50, 200}  # 0 became 40
    for splits in (0, 1):
        check_against_oracle(w.logits.cpu().numpy(), w.params, w.max_top_k, history=w.history.cpu().numpy(),
                             cand_cap=200, splits=splits)


def test_config_throughput_slice():
    w = workloads.make("throughput", rows=512, device=DEV)
    for splits in (1, 0):
        check_against_oracle(w.logits.cpu().numpy(), w.params, w.max_top_k, history=w.history.cpu().numpy(),
                             cand_cap=20, splits=splits)


def test_full_size_properties():
    """4096 x 151936, the benchmark's batch: every row against the oracle (tokens, shortlists,
    probabilities), and size-independent properties: the launch is idempotent (logits are
    read-only), permuting the rows permutes the tokens, a greedy pass over the same rows equals
    torch's argmax, every token lies inside its row's nucleus."""
    w = workloads.make("throughput", device=DEV)
    rows = w.rows
    a = run_gpu(w.logits, w.params, w.max_top_k, history=w.history.cpu().numpy(), cand_cap=20)
    b = run_gpu(w.logits, w.params, w.max_top_k, history=w.history.cpu().numpy(), cand_cap=20)
    for key in ("next", "n_kept", "cut", "cand_idx", "cand_prob"):
        assert np.array_equal(a[key], b[key])
    assert a["status"] == 0 and np.all(a["n_kept"] == 20) and np.all(a["cut"] >= 1)
    # the oracle on every row of the full batch
    ref = O.sample_rows(w.logits.cpu().numpy(), w.params, history=w.history.cpu().numpy(), cand_cap=20)
    compare(a, ref, 20)
    # row permutation
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(3))
    c = run_gpu(w.logits[perm.to(DEV)].contiguous(), w.params[perm.numpy()], w.max_top_k,
                history=w.history.cpu().numpy()[perm.numpy()], cand_cap=0)
    assert np.array_equal(c["next"], a["next"][perm.numpy()])
    # greedy == torch argmax (no penalty)
    g = sampler.argmax_rows(w.logits).cpu().numpy()
    assert np.array_equal(g, torch.argmax(w.logits, dim=1).cpu().numpy())
    # the token is one of the shortlist ids, inside the nucleus
    pos = (a["cand_idx"] == a["next"][:, None]).argmax(axis=1)
    assert np.all(a["cand_idx"][np.arange(rows), pos] == a["next"]) and np.all(pos < a["cut"])


@pytest.mark.parametrize("top_k", [100, 600])
def test_full_size_properties_long_shortlists(top_k):
    """The same 4096 x 151936 batch with longer shortlists (the kernel with the running histogram,
    in both of its shapes): idempotence, the oracle on the rows (all of them at top_k 100), row permutation, and
    every row's shortlist ids equal to torch's top-k ids as a set wherever the k-th value is unique."""
    w = workloads.make("throughput", device=DEV)
    rows = w.rows
    params = w.params.copy()
    params["top_k"] = top_k
    hist = w.history.cpu().numpy()
    a = run_gpu(w.logits, params, top_k, history=hist, cand_cap=top_k)
    b = run_gpu(w.logits, params, top_k, history=hist, cand_cap=top_k)
    for key in ("next", "n_kept", "cut", "cand_idx", "cand_prob"):
        assert np.array_equal(a[key], b[key])
    assert a["status"] == 0 and np.all(a["n_kept"] == top_k) and np.all(a["cut"] >= 1)
    sel = np.arange(0, rows, 1 if top_k == 100 else 97)  # every row at top_k 100, a strided sample at 600
    ref = O.sample_rows(w.logits[sel].cpu().numpy(), params[sel], history=hist[sel], cand_cap=top_k)
    sub = {k: (v[sel] if isinstance(v, np.ndarray) else v) for k, v in a.items()}
    compare(sub, ref, top_k)
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(5))
    c = run_gpu(w.logits[perm.to(DEV)].contiguous(), params[perm.numpy()], top_k, history=hist[perm.numpy()], cand_cap=0)
    assert np.array_equal(c["next"], a["next"][perm.numpy()])
    # shortlist ids against torch on rows without a penalty window (the first 64 have their history cleared)
    p2 = params[:64].copy()
    p2["repeat_penalty"] = 1.0
    d = run_gpu(w.logits[:64].contiguous(), p2, top_k, cand_cap=top_k)
    vals, ids = torch.topk(w.logits[:64], top_k + 1, dim=1)
    unique_kth = (vals[:, top_k - 1] > vals[:, top_k]).cpu().numpy()
    got = np.sort(d["cand_idx"][:, :top_k], axis=1)
    want = np.sort(ids[:, :top_k].cpu().numpy(), axis=1)
    assert unique_kth.any() and np.array_equal(got[unique_kth], want[unique_kth])


# ---- stand-alone entry points ---------------------------------------------------------------------------

def test_argmax_rows():
    rng = np.random.default_rng(2)
    for rows, V in [(1, 1), (3, 5), (7, 4097), (300, 151936), (5, 200001)]:
        x = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
        x = (np.round(x * 4) / 4).astype(np.float32)
        want = np.array([O.lib().mantle_oracle_argmax(x[r].ctypes.data_as(C.c_void_p), V) for r in range(rows)])
        got = sampler.argmax_rows(torch.from_numpy(x).to(DEV)).cpu().numpy()
        assert np.array_equal(got, want), (rows, V)
    x = np.array([[-0.0, 0.0, -1.0], [1.0, 7.0, 7.0]], dtype=np.float32)
    assert sampler.argmax_rows(torch.from_numpy(x).to(DEV)).cpu().numpy().tolist() == [0, 1]


def test_repeat_penalty_rows_in_place_then_preapplied():
    rng = np.random.default_rng(3)
    rows, V = 20, 30000
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    hist = rng.integers(-3, V + 3, size=(rows, 500)).astype(np.int32)
    hist_len = rng.integers(0, 501, size=rows).astype(np.int32)
    exclude = hist[:, 0].copy()[:5]
    params = random_params(rng, rows, ks=(1, 20, 50))
    dev = torch.from_numpy(logits.copy()).to(DEV)
    p_dev = sampler.params_to_device(params, DEV)
    sampler.repeat_penalty_rows_(dev, p_dev, torch.from_numpy(hist).to(DEV), torch.from_numpy(hist_len).to(DEV),
                                 torch.from_numpy(exclude).to(DEV))
    ref_logits = logits.copy()
    ref = O.sample_rows(ref_logits, params, history=hist, hist_len=hist_len, exclude=exclude, cand_cap=50)
    assert np.array_equal(dev.cpu().numpy(), ref_logits)
    gpu = run_gpu(dev, params, 50, history=hist, hist_len=hist_len, exclude=exclude, cand_cap=50,
                  flags=native.FLAG_PENALTY_PREAPPLIED)
    compare(gpu, ref, 50)


def test_vocab_sharded_on_one_gpu():
    """Eight column shards of one row set, each run as its own local top-k, then merged:
    equal to the oracle on the whole row (the all-gather is the caller's and moves bytes only)."""
    w = workloads.make("vocab_sharded", rows=64, device=DEV)
    V, G = w.vocab, 8
    p_dev = sampler.params_to_device(w.params, DEV)
    vals, idxs, cnts = [], [], []
    for g in range(G):
        lo = g * (V // G)
        shard = w.logits[:, lo:lo + V // G].contiguous()
        v, i, c = sampler.local_topk(shard, p_dev, w.max_top_k, lo, V, history=w.history)
        vals.append(v), idxs.append(i), cnts.append(c)
    out = sampler.merge_parts(p_dev, w.max_top_k, V, torch.stack(vals), torch.stack(idxs), torch.stack(cnts),
                              cand_cap=50)
    torch.cuda.synchronize()
    gpu = dict(next=out.next.cpu().numpy(), n_kept=out.n_kept.cpu().numpy(), cut=out.cut.cpu().numpy(),
               cand_idx=out.cand_idx.cpu().numpy(), cand_prob=out.cand_prob.cpu().numpy())
    ref = O.sample_rows(w.logits.cpu().numpy(), w.params, history=w.history.cpu().numpy(), cand_cap=50)
    compare(gpu, ref, 50)


def test_vocab_sharded_packed_blocks_on_one_gpu():
    """The same eight shards written into one packed block each (what a single all-gather moves)
    and merged by mantleCudaSampleMergePacked."""
    from mantle_b200 import sharded

    w = workloads.make("vocab_sharded", rows=64, device=DEV)
    V, G, k, rows = w.vocab, 8, w.max_top_k, 64
    p_dev = sampler.params_to_device(w.params, DEV)
    lib = native.load()
    nbytes = C.c_size_t(0)
    assert lib.mantleCudaSamplePackedPartBytes(rows, k, C.byref(nbytes)) == 0
    assert nbytes.value == sharded.packed_part_bytes(rows, k)
    gathered = torch.zeros(G * nbytes.value, dtype=torch.uint8, device=DEV)
    for g in range(G):
        lo = g * (V // G)
        shard = w.logits[:, lo:lo + V // G].contiguous()
        v, i, c = sampler.local_topk(shard, p_dev, k, lo, V, history=w.history)
        bv, bi, bc = sharded.packed_part_views(gathered[g * nbytes.value:(g + 1) * nbytes.value], rows, k)
        bv.copy_(v), bi.copy_(i), bc.copy_(c)
    nxt = torch.full((rows,), -2, dtype=torch.int32, device=DEV)
    n_kept = torch.zeros(rows, dtype=torch.int32, device=DEV)
    cut = torch.zeros(rows, dtype=torch.int32, device=DEV)
    b = native.SampleBatch()
    b.rows, b.vocab, b.max_top_k = rows, V, k
    b.params, b.next, b.n_kept, b.cut = p_dev.data_ptr(), nxt.data_ptr(), n_kept.data_ptr(), cut.data_ptr()
    rc = lib.mantleCudaSampleMergePacked(C.byref(b), G, C.c_void_p(gathered.data_ptr()), k,
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    ref = O.sample_rows(w.logits.cpu().numpy(), w.params, history=w.history.cpu().numpy())
    assert np.array_equal(nxt.cpu().numpy(), ref["next"])
    assert np.array_equal(n_kept.cpu().numpy(), ref["n_kept"]) and np.array_equal(cut.cpu().numpy(), ref["cut"])


# ---- errors -------------------------------------------------------------------------------------------------

def test_top_k_beyond_bound_sets_status():
    params = np.array([P(0.5, temperature=1.0, top_k=50, top_p=1.0), P(0.5, temperature=1.0, top_k=5, top_p=1.0)])
    logits = torch.randn(2, 1000, device=DEV)
    g = run_gpu(logits, params, 10, cand_cap=10)
    assert g["status"] & native.STATUS_TOPK_RANGE
    assert g["next"][0] == -1 and 0 <= g["next"][1] < 1000


def test_nan_logits_are_never_admitted_and_an_all_nan_row_is_flagged():
    """NaN is outside the sampling contract (the reference's own answer depends on where in the row
    the NaN sits, sampler.go:268-275).  What the library documents instead: a NaN never enters a
    shortlist -- so a row with a few of them samples like the same row with those columns far below
    everything else -- and a row holding nothing else returns token 0 with MANTLE_SAMPLE_STATUS_NAN."""
    rng = np.random.default_rng(12)
    rows, V = 6, 5000
    lg = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    holes = rng.integers(0, V, size=(rows, 7))
    with_nan, lowered = lg.copy(), lg.copy()
    for r in range(rows):
        with_nan[r, holes[r]] = np.nan
        lowered[r, holes[r]] = -1e30
    params = np.array([P(float(rng.random()), temperature=0.8, top_k=int(k), top_p=0.9, repeat_penalty=1.0)
                       for k in (1, 5, 40, 40, 200, 1000)])
    params[0]["greedy"] = 1
    for max_k, splits in ((1000, 0), (1000, 3), (2000, 0)):  # streaming, split rows, long-shortlist kernel
        g = run_gpu(torch.from_numpy(with_nan).to(DEV), params, max_k, splits=splits)
        ref = O.sample_rows(lowered.copy(), params)
        assert np.array_equal(g["next"], ref["next"]), (max_k, splits)
        assert np.array_equal(g["cut"], ref["cut"]) and g["status"] == 0
    allnan = np.full((2, 3000), np.nan, dtype=np.float32)
    allnan[1] = lg[1, :3000]
    for max_k in (40, 2000):
        g = run_gpu(torch.from_numpy(allnan).to(DEV), params[2:4], max_k)
        assert g["next"][0] == 0 and g["status"] == native.STATUS_NAN
        assert g["next"][1] == O.sample_rows(allnan[1:2].copy(), params[3:4])["next"][0]


def test_skipped_rows_are_not_sampled():
    """`skip`: rows of a batched decode loop that have ended cost nothing and report token -1."""
    rng = np.random.default_rng(13)
    rows, V = 9, 40000
    lg = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    params = np.array([P(float(rng.random()), temperature=0.8, top_k=30, top_p=0.9) for _ in range(rows)])
    skip = (np.arange(rows) % 3 == 1).astype(np.int32)
    ref = O.sample_rows(lg.copy(), params)
    d = torch.from_numpy(lg).to(DEV)
    p_dev = sampler.params_to_device(params, DEV)
    skip_dev = torch.from_numpy(skip).to(DEV)
    for max_k, splits in ((30, 1), (30, 0), (2000, 0)):
        plan = sampler.BatchPlan(d, p_dev, max_k, splits=splits)
        plan.batch.skip = skip_dev.data_ptr()
        out = plan.launch()
        torch.cuda.synchronize()
        got = out.next.cpu().numpy()
        assert np.array_equal(got[skip == 0], ref["next"][skip == 0]), (max_k, splits)
        assert np.all(got[skip == 1] == -1) and np.all(out.n_kept.cpu().numpy()[skip == 1] == 0)
        assert int(out.status.item()) == 0


def test_outputs_do_not_overrun():
    rng = np.random.default_rng(8)
    rows, V = 5, 3000
    logits = torch.from_numpy((rng.standard_normal((rows, V)) * 3).astype(np.float32)).to(DEV)
    params = np.array([P(float(rng.random()), temperature=0.9, top_k=40, top_p=1.0) for _ in range(rows)])
    g = run_gpu(logits, params, 40, cand_cap=8)  # fewer candidate slots than the shortlist: truncated, not overrun
    ref = O.sample_rows(logits.cpu().numpy(), params, cand_cap=8)
    assert np.array_equal(g["next"], ref["next"]) and np.array_equal(g["cand_idx"], ref["cand_idx"])


def test_host_buffer_entry_point():
    """The host-slice form: pinned host inputs in, token ids out, copies inside the call."""
    rng = np.random.default_rng(21)
    rows, V = 40, 50000
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    hist = rng.integers(0, V, size=(rows, 100)).astype(np.int32)
    hist_len = rng.integers(0, 101, size=rows).astype(np.int32)
    exclude = np.array([hist[0, 0], 7], dtype=np.int32)
    params = random_params(rng, rows, ks=(1, 20, 50))
    for flags in (0, native.FLAG_WRITE_BACK_PENALTY):
        for splits in (0, 1):
            host_logits = torch.from_numpy(logits.copy())
            plan = sampler.HostBatchPlan(host_logits, params, 50, history=torch.from_numpy(hist),
                                         hist_len=torch.from_numpy(hist_len), exclude=torch.from_numpy(exclude),
                                         cand_cap=50, flags=flags, splits=splits, device=DEV)
            out = plan.launch()
            torch.cuda.synchronize()
            ref_logits = logits.copy()
            ref = O.sample_rows(ref_logits, params, history=hist, hist_len=hist_len, exclude=exclude, cand_cap=50)
            gpu = dict(next=out.next.numpy(), n_kept=out.n_kept.numpy(), cut=out.cut.numpy(),
                       cand_idx=out.cand_idx.numpy(), cand_prob=out.cand_prob.numpy())
            compare(gpu, ref, 50)
            assert int(out.status.item()) == 0
            want = ref_logits if flags else logits
            assert np.array_equal(plan.logits.numpy(), want)


# ---- long shortlists: top_k above 1024, up to the whole vocabulary ---------------------------------------

def wide_check(logits_np, params, history=None, exclude=None, bf16=False, where=""):
    """Long shortlists are never materialised: token, shortlist length and nucleus length are what
    both sides report.  The oracle orders the whole row (the stand-in for the reference's O(V*k)
    insertion loop, proven equal to it on small cases)."""
    if bf16:
        dev = torch.from_numpy(logits_np.view(np.int16).copy()).to(DEV).view(torch.bfloat16)
    else:
        dev = torch.from_numpy(logits_np.copy()).to(DEV)
    max_k = int(max(params["top_k"].max(), 1025))
    gpu = run_gpu(dev, params, max_k, history, None, exclude, 0)
    ref = O.sample_rows(logits_np.copy(), params, history=history, exclude=exclude, cand_cap=0)
    # sums in a different association than the reference's: the sampled token's probability and the
    # normaliser are held to the contract's 1e-5 relative, integers to equality
    compare(gpu, ref, 0, exact_prob=False, where=where)
    assert gpu["status"] == 0
    return gpu, ref


@pytest.mark.parametrize("seed", range(4))
def test_long_shortlists_small_vocab(seed):
    rng = np.random.default_rng(900 + seed)
    rows, V = 40, int(rng.choice([1500, 4097, 9000]))
    logits = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
    if seed % 2:
        logits = (np.round(logits * 8) / 8).astype(np.float32)  # tie groups of dozens of columns
    params = np.zeros(rows, dtype=O.PARAMS_DTYPE)
    for r in range(rows):
        params[r] = O.normalize(
            temperature=float(rng.choice([0.0, 0.7, 1.0, 1.3])),
            top_k=int(rng.choice([1100, V // 2 + 600, V, 2 * V])),
            top_p=float(rng.choice([0.3, 0.9, 0.97, 1.0])),
            min_p=float(rng.choice([0.0, 0.0, 0.02, 0.3])),
            repeat_penalty=float(rng.choice([1.0, 1.2])),
            repeat_last_n=64,
            uniform=float(rng.choice([0.0, rng.random(), rng.random(), 1.0 - 2.0 ** -53])),
        )
    hist = rng.integers(0, V, size=(rows, 64)).astype(np.int32)
    exclude = rng.integers(0, V, size=2).astype(np.int32)
    wide_check(logits, params, history=hist, exclude=exclude, where="seed %d V %d" % (seed, V))


def test_long_shortlist_degenerate_rows():
    V = 3000
    logits = np.zeros((4, V), dtype=np.float32)           # one tie group holds everything
    logits[1] = np.where(np.arange(V) % 2 == 0, 1.0, -1.0)  # two tie groups
    logits[2, 7] = 50.0                                    # one column takes all the mass
    logits[3] = np.linspace(-3, 3, V, dtype=np.float32)
    params = np.array([O.normalize(temperature=1.0, top_k=V, top_p=0.9, uniform=u) for u in (0.5, 0.7, 0.99, 0.123)])
    wide_check(logits, params)
    params = np.array([O.normalize(temperature=1.0, top_k=1500, top_p=1.0, uniform=u) for u in (0.999999, 0.7, 0.99, 0.123)])
    wide_check(logits, params)


def test_config_full_vocab_nucleus():
    """BASELINE config 2: 256 bf16 rows, vocab 128 256, top_k = V, top_p 0.9, temperature 1."""
    w = workloads.make("full_vocab_nucleus", device=DEV)
    bits = to_bf16_bits(w.logits)
    gpu, ref = wide_check(bits, w.params, bf16=True)
    assert np.all(ref["n_kept"] == w.vocab) and ref["cut"].min() > 1000  # tens of thousands of nucleus entries


@pytest.mark.parametrize("H", [1501, 3000, 1024])
def test_history_layouts(H):
    """History rows that cannot be staged by a bulk copy (odd stride), that exceed the staged
    window, and that fit it exactly; shortlists of 20 (plain-load kernel) and 400 (ring kernel)."""
    rng = np.random.default_rng(H)
    rows, V = 12, 70001
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    hist = rng.integers(-1, V + 1, size=(rows, H)).astype(np.int32)
    hist_len = rng.integers(H // 2, H + 1, size=rows).astype(np.int32)
    exclude = hist[0, :3].copy()
    for k, last_n in [(20, 64), (20, 5000), (400, 5000), (400, 700)]:
        params = np.array([O.normalize(temperature=0.8, top_k=k, top_p=0.95, repeat_penalty=1.3, repeat_last_n=last_n,
                                       uniform=float(rng.random())) for _ in range(rows)])
        check_against_oracle(logits, params, k, history=hist, hist_len=hist_len, exclude=exclude, cand_cap=k,
                             where="H %d k %d window %d" % (H, k, last_n))


def test_bounded_wait_gives_up_and_reports():
    """Failure detection without a fault: a wait on a barrier nothing completes runs out after
    its limit, the kernel reports it in the status word, and the context keeps working."""
    import time

    lib = native.load()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = time.perf_counter()
    rc = lib.mantleCudaSamplerSelfTestBoundedWait(20_000_000, C.c_void_p(status.data_ptr()),  # 20 ms
                                                  C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert int(status.item()) == native.STATUS_TIMEOUT
    assert 0.015 < dt < 1.0, dt
    assert lib.mantleCudaSamplerSelfTestBoundedWait(0, C.c_void_p(status.data_ptr()), None) == native.CUDA_ERROR_INVALID_VALUE
    # the context is still good: sample something
    g, _ = one([-1, 5, 3, 7, 2], temperature=0.0)
    assert g["next"][0] == 3


def test_committed_fixtures():
    """The CUDA path against tests/golden/oracle_cases.npz: inputs and oracle answers committed
    together, without and with the model head's multiplier and soft cap."""
    import os

    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_cases.npz"))
    params = z["params"].view(O.PARAMS_DTYPE)
    cap = z["cand_idx"].shape[1]
    for prefix, kw in (("", {}), ("post_", dict(logit_scale=float(z["post_scale"]), logit_softcap=float(z["post_cap"])))):
        d = torch.from_numpy(z["logits"].copy()).to(DEV)
        g = run_gpu(d, params, 300, history=z["history"], hist_len=z["hist_len"], exclude=z["exclude"], cand_cap=cap,
                    **kw)
        ref = dict(next=z[prefix + "next"], n_kept=z[prefix + "n_kept"], cut=z[prefix + "cut"],
                   cand_idx=z[prefix + "cand_idx"], cand_prob=z[prefix + "cand_prob"])
        compare(g, ref, cap, where="fixture " + (prefix or "plain"))
        assert g["status"] == 0
