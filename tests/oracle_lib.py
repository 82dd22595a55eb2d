"""ctypes binding of the CPU oracle (oracle/sampler_oracle.c).  Test infrastructure only."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "build", "liboracle_sampler.so")

PARAMS_DTYPE = np.dtype(
    [
        ("temperature", "<f4"),
        ("top_p", "<f4"),
        ("min_p", "<f4"),
        ("repeat_penalty", "<f4"),
        ("top_k", "<i4"),
        ("repeat_last_n", "<i4"),
        ("greedy", "<i4"),
        ("reserved", "<i4"),
        ("uniform", "<f8"),
    ],
    align=True,
)
assert PARAMS_DTYPE.itemsize == 40


class SamplerConfig(C.Structure):
    _fields_ = [
        ("seed", C.c_int64),
        ("temperature", C.c_float),
        ("top_k", C.c_int32),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repeat_penalty", C.c_float),
        ("repeat_last_n", C.c_int32),
    ]


_lib = None


def build():
    src = os.path.join(ORACLE_DIR, "sampler_oracle.c")
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR], stdout=subprocess.DEVNULL)


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(ORACLE_SO)
        L.mantle_oracle_fast_exp.restype = C.c_float
        L.mantle_oracle_fast_exp.argtypes = [C.c_float]
        L.mantle_oracle_fast_tanh.restype = C.c_float
        L.mantle_oracle_fast_tanh.argtypes = [C.c_float]
        L.mantle_oracle_postprocess.restype = None
        L.mantle_oracle_postprocess.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_float]
        L.mantle_oracle_normalize_config.restype = None
        L.mantle_oracle_normalize_config.argtypes = [C.c_void_p, C.c_void_p]
        L.mantle_oracle_can_use_device_greedy.restype = C.c_int
        L.mantle_oracle_can_use_device_greedy.argtypes = [C.c_void_p]
        L.mantle_oracle_argmax.restype = C.c_int
        L.mantle_oracle_argmax.argtypes = [C.c_void_p, C.c_int]
        for name in ("mantle_oracle_topk_insertion", "mantle_oracle_topk_sorted"):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        L.mantle_oracle_sample_rows.restype = C.c_int
        L.mantle_oracle_sample_rows.argtypes = [
            C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64,
            C.c_void_p, C.c_int, C.c_void_p,
            C.c_void_p, C.c_int,
            C.c_void_p, C.c_void_p,
            C.c_void_p, C.c_void_p, C.c_int,
            C.c_void_p, C.c_void_p, C.c_int, C.c_int,
            C.c_void_p, C.c_void_p,
        ]
        L.mantle_oracle_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def fast_exp(x):
    return float(np.float32(lib().mantle_oracle_fast_exp(C.c_float(float(np.float32(x))))))


def fast_tanh(x):
    return float(lib().mantle_oracle_fast_tanh(C.c_float(x)))


def postprocess(logits, scale=0.0, softcap=0.0):
    """The model head's multiplier and soft cap, in place on a contiguous float32 array."""
    assert logits.dtype == np.float32 and logits.flags.c_contiguous
    lib().mantle_oracle_postprocess(_ptr(logits), logits.size, C.c_float(scale), C.c_float(softcap))
    return logits


def normalize(seed=0, temperature=0.0, top_k=0, top_p=0.0, min_p=0.0, repeat_penalty=0.0, repeat_last_n=0,
              uniform=0.0):
    """NewSampler's normalisation -> one PARAMS_DTYPE record."""
    cfg = SamplerConfig(seed, temperature, top_k, top_p, min_p, repeat_penalty, repeat_last_n)
    out = np.zeros(1, dtype=PARAMS_DTYPE)
    lib().mantle_oracle_normalize_config(C.byref(cfg), _ptr(out))
    out["uniform"] = uniform
    return out[0]


def can_use_device_greedy(p):
    a = np.array([p], dtype=PARAMS_DTYPE)
    return bool(lib().mantle_oracle_can_use_device_greedy(_ptr(a)))


def topk(logits, k, inv_temp, sorted_variant=False):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    idx = np.zeros(max(k, 1) + 1, dtype=np.int32)
    val = np.zeros(max(k, 1) + 1, dtype=np.float32)
    f = lib().mantle_oracle_topk_sorted if sorted_variant else lib().mantle_oracle_topk_insertion
    n = f(_ptr(logits), logits.size, k, C.c_float(float(np.float32(inv_temp))), _ptr(idx), _ptr(val))
    return idx[:n].copy(), val[:n].copy()


def sample_rows(logits, params, history=None, hist_len=None, exclude=None, cand_cap=0, use_sort=-1,
                threads=0, vocab=None):
    """Runs the oracle over a batch.

    logits: [rows, stride] float32 (patched in place, as the reference does) or uint16
    holding bfloat16 bit patterns (left untouched).  Returns a dict with next, n_kept,
    cut, softmax_sum, token_prob and, when cand_cap > 0, cand_idx / cand_prob.
    """
    assert logits.ndim == 2 and logits.flags.c_contiguous
    rows, stride = logits.shape
    V = stride if vocab is None else vocab
    dtype = {np.dtype(np.float32): 0, np.dtype(np.uint16): 1}[logits.dtype]
    params = np.ascontiguousarray(params, dtype=PARAMS_DTYPE)
    assert params.shape == (rows,)
    hs = 0
    if history is not None:
        history = np.ascontiguousarray(history, dtype=np.int32)
        assert history.ndim == 2 and history.shape[0] == rows
        hs = history.shape[1]
        if hs == 0:
            history = None
    if hist_len is not None:
        hist_len = np.ascontiguousarray(hist_len, dtype=np.int32)
    if exclude is not None:
        exclude = np.ascontiguousarray(exclude, dtype=np.int32)
    nxt = np.full(rows, -1, dtype=np.int32)
    n_kept = np.zeros(rows, dtype=np.int32)
    cut = np.zeros(rows, dtype=np.int32)
    cand_idx = np.full((rows, cand_cap), -1, dtype=np.int32) if cand_cap else None
    cand_prob = np.zeros((rows, cand_cap), dtype=np.float64) if cand_cap else None
    softmax_sum = np.zeros(rows, dtype=np.float64)
    token_prob = np.zeros(rows, dtype=np.float64)
    used = lib().mantle_oracle_sample_rows(
        _ptr(logits), dtype, rows, V, stride,
        _ptr(history), hs, _ptr(hist_len),
        _ptr(exclude), 0 if exclude is None else exclude.size,
        _ptr(params), _ptr(nxt),
        _ptr(cand_idx), _ptr(cand_prob), cand_cap,
        _ptr(n_kept), _ptr(cut), use_sort, threads,
        _ptr(softmax_sum), _ptr(token_prob),
    )
    return dict(next=nxt, n_kept=n_kept, cut=cut, cand_idx=cand_idx, cand_prob=cand_prob, threads=used,
                softmax_sum=softmax_sum, token_prob=token_prob)
