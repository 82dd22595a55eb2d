"""Writes tests/golden/oracle_cases.npz: seeded inputs and what the CPU oracle answers for them.

The reference is Go and cannot run where this is built, so its own expected values are in
reference_vectors.json (transcribed from its test files) and the oracle is pinned to those by
tests/test_oracle.py.  This file adds regression fixtures on top: a batch that walks every branch
of the sampler (penalty on and off, window shorter than the history, an exclude list, greedy rows,
top_k 1 with a temperature, min-p, top_p 1, ties, signed zeros), with the oracle's tokens,
shortlist lengths, nucleus lengths and leading shortlist entries, and the same batch with the
model head's multiplier and soft cap applied first.  The inputs are stored, not regenerated, so
the fixture does not depend on a random generator's stream.

    python tests/golden/make_fixtures.py        # from the repository root; needs no GPU
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as O  # noqa: E402

ROWS, V, H, CAND = 48, 777, 48, 12


def build_inputs():
    rng = np.random.default_rng(20261125)
    logits = (rng.standard_normal((ROWS, V)) * 3).astype(np.float32)
    logits[::2] = np.round(logits[::2] * 2) / 2           # every other row: heavy ties
    logits[rng.random((ROWS, V)) < 0.03] = 0.0
    logits[rng.random((ROWS, V)) < 0.02] = -0.0
    history = rng.integers(-2, V + 2, size=(ROWS, H)).astype(np.int32)
    hist_len = rng.integers(0, H + 1, size=ROWS).astype(np.int32)
    exclude = np.array([3, 500, 776], dtype=np.int32)
    params = np.zeros(ROWS, dtype=O.PARAMS_DTYPE)
    temps = [0.0, 0.3, 0.8, 1.0, 1.5]
    ks = [0, 1, 2, 5, 40, 300]
    ps = [0.0, 0.5, 0.9, 0.95, 1.0]
    mins = [0.0, 0.05, 0.3]
    pens = [0.0, 1.0, 1.1, 1.3]
    lasts = [0, 4, 64]
    for r in range(ROWS):
        params[r] = O.normalize(temperature=temps[r % 5], top_k=ks[(r // 5) % 6], top_p=ps[(r // 3) % 5],
                                min_p=mins[(r // 7) % 3], repeat_penalty=pens[(r // 2) % 4],
                                repeat_last_n=lasts[r % 3], uniform=float(rng.random()))
    return logits, history, hist_len, exclude, params


def answers(logits, history, hist_len, exclude, params, scale=0.0, cap=0.0):
    lg = logits.copy()
    if scale or cap:
        O.postprocess(lg, scale, cap)
    out = O.sample_rows(lg, params, history=history, hist_len=hist_len, exclude=exclude, cand_cap=CAND)
    return out["next"], out["n_kept"], out["cut"], out["cand_idx"], out["cand_prob"]


def main():
    logits, history, hist_len, exclude, params = build_inputs()
    nxt, n_kept, cut, cand_idx, cand_prob = answers(logits, history, hist_len, exclude, params)
    p_next, p_kept, p_cut, p_idx, p_prob = answers(logits, history, hist_len, exclude, params, scale=0.5, cap=6.0)
    np.savez_compressed(
        os.path.join(HERE, "oracle_cases.npz"),
        logits=logits, history=history, hist_len=hist_len, exclude=exclude, params=params.view(np.uint8),
        next=nxt, n_kept=n_kept, cut=cut, cand_idx=cand_idx, cand_prob=cand_prob,
        post_scale=np.float32(0.5), post_cap=np.float32(6.0),
        post_next=p_next, post_n_kept=p_kept, post_cut=p_cut, post_cand_idx=p_idx, post_cand_prob=p_prob,
    )
    print("wrote oracle_cases.npz:", ROWS, "rows x", V, "columns")


if __name__ == "__main__":
    main()
