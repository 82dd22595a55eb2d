"""Seeded synthetic sampling batches with the shapes, sizes and value distributions of
the five benchmark configurations.  They stand in for real model logits (a 151 936-wide
Qwen3 head, a 128 256-wide Llama-3-class head, a 262 144-wide Gemma-class head): no model
weights or datasets are needed, and none are read.

Every generator is a pure function of (name, rows, seed, device).  Logits are produced
with torch on the requested device (CPU and CUDA generators give different streams; the
tests copy whichever was generated to the other side, so the CUDA path and the CPU
checker always see identical bytes).
"""
import numpy as np
import torch

from .native import PARAMS_DTYPE
from .sampler import SamplerConfig, new_sampler_params

BASE_SEED = 20261125

SPECS = {
    # name: rows, vocab, dtype, sigma, hist, description
    "single_row": dict(rows=1, vocab=151936, dtype="f32", sigma=3.0, hist=64),
    "mixed_batch": dict(rows=64, vocab=151936, dtype="f32", sigma=3.0, hist=256),
    "full_vocab_nucleus": dict(rows=256, vocab=128256, dtype="bf16", sigma=2.0, hist=0),
    "throughput": dict(rows=4096, vocab=151936, dtype="f32", sigma=3.0, hist=1024),
    "vocab_sharded": dict(rows=1024, vocab=262144, dtype="f32", sigma=3.0, hist=512),
}


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & np.uint64(0xFFFFFFFFFFFFFFFF)
    z = x
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def uniforms(seed, rows):
    """rows doubles in [0,1) on the 2^-53 lattice, the lattice of Go's rand.Float64."""
    with np.errstate(over="ignore"):
        x = _splitmix64(np.uint64(seed) * np.uint64(0x100000001B3) + np.arange(rows, dtype=np.uint64))
    return (x >> np.uint64(11)).astype(np.float64) * (2.0 ** -53)


class Workload:
    """logits [rows, vocab] (torch, on `device`), history [rows, H] int32 or None,
    params (numpy PARAMS_DTYPE, host), max_top_k, and the byte count one pass must read."""

    def __init__(self, name, logits, history, params, max_top_k, vocab):
        self.name = name
        self.logits = logits
        self.history = history
        self.hist_len = None
        self.exclude = None
        self.params = params
        self.max_top_k = max_top_k
        self.vocab = vocab
        self.rows = logits.shape[0]

    @property
    def bytes_per_row(self):
        """Algorithmic bytes per row: one read of the logits row plus the history ids."""
        h = 0 if self.history is None else self.history.shape[1]
        return self.vocab * self.logits.element_size() + 4 * h


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _boost_(logits, g, n_ids, amount):
    """Adds `amount` (a scalar or a [n_ids] tensor) to n_ids distinct seeded columns of every row."""
    rows, V = logits.shape
    # distinct ids per row: n_ids of a random permutation prefix, built from sorted random keys
    keys = torch.rand((rows, 4 * n_ids), generator=g, device=logits.device)
    ids = (keys * V).long().clamp_(max=V - 1)
    out = torch.empty((rows, n_ids), dtype=torch.long, device=logits.device)
    ids_cpu = ids.cpu().numpy()
    for r in range(rows):
        _, first = np.unique(ids_cpu[r], return_index=True)
        first.sort()
        out[r] = torch.from_numpy(ids_cpu[r][first[:n_ids]]).to(logits.device)
    amt = amount if torch.is_tensor(amount) else torch.full((n_ids,), float(amount))
    amt = amt.to(logits.device, torch.float32).expand(rows, n_ids)
    logits.scatter_add_(1, out, amt)
    return out


def make(name, rows=None, seed=None, device="cpu", vocab=None):
    spec = dict(SPECS[name])
    rows = spec["rows"] if rows is None else rows
    V = spec["vocab"] if vocab is None else vocab
    cfg_index = list(SPECS).index(name)
    seed = BASE_SEED + 1000 * cfg_index if seed is None else seed
    device = torch.device(device)
    g = _gen(device, seed)
    logits = torch.randn((rows, V), generator=g, device=device, dtype=torch.float32) * spec["sigma"]
    H = spec["hist"]
    history = None
    if H:
        history = torch.randint(0, V, (rows, H), generator=g, device=device, dtype=torch.int32)
    u = uniforms(seed, rows)
    params = np.zeros(rows, dtype=PARAMS_DTYPE)
    rng = np.random.default_rng(seed)

    if name in ("single_row", "throughput"):
        _boost_(logits, g, 16, 8.0)
        cfg = SamplerConfig(temperature=0.6, top_k=20, top_p=0.95, repeat_penalty=1.1, repeat_last_n=H)
        for r in range(rows):
            params[r] = new_sampler_params(cfg, u[r])
        max_k = 20
    elif name == "mixed_batch":
        ranks = torch.arange(1, 65, dtype=torch.float32)
        _boost_(logits, g, 64, 10.0 * ranks.pow(-1.1))
        ks = rng.choice([0, 1, 20, 50, 200], size=rows)
        for r in range(rows):
            cfg = SamplerConfig(
                temperature=float(rng.uniform(0.2, 1.5)),
                top_k=int(ks[r]),  # 0 means 40 through the reference's constructor (sampler.go:66-68)
                top_p=float(rng.uniform(0.8, 1.0)),
                repeat_penalty=float(rng.uniform(1.0, 1.3)),
                repeat_last_n=H,
            )
            params[r] = new_sampler_params(cfg, u[r])
        max_k = 200
    elif name == "full_vocab_nucleus":
        logits = logits.to(torch.bfloat16)  # round-to-nearest-even; widened exactly on the device
        # "top_k = 0 means the whole vocabulary" is expressed as top_k = V: the reference's
        # constructor maps 0 to 40, and only TopK >= V reaches every candidate (sampler.go:147)
        cfg = SamplerConfig(temperature=1.0, top_k=V, top_p=0.9, repeat_penalty=1.0)
        for r in range(rows):
            params[r] = new_sampler_params(cfg, u[r])
        max_k = V
    elif name == "vocab_sharded":
        _boost_(logits, g, 32, 8.0)
        cfg = SamplerConfig(temperature=0.7, top_k=50, top_p=0.95, repeat_penalty=1.15, repeat_last_n=H)
        for r in range(rows):
            params[r] = new_sampler_params(cfg, u[r])
        max_k = 50
    else:
        raise KeyError(name)
    return Workload(name, logits, history, params, max_k, V)
