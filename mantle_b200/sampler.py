"""Host-side mirror of the reference's sampler interface over the CUDA C-ABI.

Names follow internal/logits/sampler.go: SamplerConfig (:34-42), new_sampler_params =
NewSampler's normalisation (:61-83), can_use_device_greedy (:56-58).  `sample_rows`
is Sampler.Sample (:98-234) for a batch whose logits already live on the GPU, the
hand-off point the reference's device-greedy path uses
(internal/backend/cuda/ops.go:1289-1346).  torch supplies device memory and streams;
all arithmetic happens in the CUDA library.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import native
from .native import PARAMS_DTYPE


@dataclass
class SamplerConfig:
    """logits.SamplerConfig, field for field."""

    seed: int = 0
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    min_p: float = 0.0
    repeat_penalty: float = 0.0
    repeat_last_n: int = 0


def new_sampler_params(cfg, uniform=0.0):
    """NewSampler's normalisation (sampler.go:61-83) -> one PARAMS_DTYPE record."""
    p = np.zeros((), dtype=PARAMS_DTYPE)
    t = np.float32(cfg.temperature)
    p["greedy"] = 1 if t <= 0 else 0
    p["temperature"] = np.float32(1.0) if t <= 0 else t
    p["top_k"] = 40 if cfg.top_k <= 0 else cfg.top_k
    tp = np.float32(cfg.top_p)
    p["top_p"] = np.float32(1.0) if (tp <= 0 or tp > 1) else tp
    p["min_p"] = np.float32(cfg.min_p)
    rp = np.float32(cfg.repeat_penalty)
    p["repeat_penalty"] = np.float32(1.0) if rp <= 0 else rp
    p["repeat_last_n"] = 64 if cfg.repeat_last_n <= 0 else cfg.repeat_last_n
    p["uniform"] = uniform
    return p


def can_use_device_greedy(p):
    """Sampler.CanUseDeviceGreedy (sampler.go:56-58)."""
    return bool(p["greedy"]) and bool(p["repeat_penalty"] <= np.float32(1.0))


def params_to_device(params, device):
    """numpy PARAMS_DTYPE array -> uint8 device tensor holding the same bytes."""
    params = np.ascontiguousarray(params, dtype=PARAMS_DTYPE)
    return torch.from_numpy(params.view(np.uint8).reshape(-1).copy()).to(device)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_ptr(stream):
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


class SampleOutputs:
    __slots__ = ("next", "cand_idx", "cand_prob", "n_kept", "cut", "status", "token_prob", "softmax_sum")

    def __init__(self):
        for name in self.__slots__:
            setattr(self, name, None)


class BatchPlan:
    """A batch descriptor bound to device tensors: build once, launch many times.

    logits   [rows, >=vocab] float32 or bfloat16 CUDA tensor, rows contiguous in memory
    params   uint8 CUDA tensor of rows*40 bytes (params_to_device)
    history  optional [rows, H] int32 CUDA tensor, oldest id first; hist_len optional [rows] int32
    exclude  optional [E] int32 CUDA tensor (stop tokens)
    logit_scale, logit_softcap   the model head's multiplier and soft cap (simd/runtime.go:258-272),
             applied on the fly; 0 switches either off
    """

    def __init__(self, logits, params, max_top_k, history=None, hist_len=None, exclude=None, vocab=None,
                 cand_cap=0, want_counts=True, flags=0, splits=0, logit_scale=0.0, logit_softcap=0.0):
        self.lib = native.load()
        if not logits.is_cuda or logits.dim() != 2 or logits.stride(1) != 1:
            raise ValueError("logits must be a 2-D CUDA tensor with unit column stride")
        if logits.dtype == torch.float32:
            dtype = native.DTYPE_F32
        elif logits.dtype == torch.bfloat16:
            dtype = native.DTYPE_BF16
        else:
            raise ValueError("logits must be float32 or bfloat16")
        dev = logits.device
        rows = logits.shape[0]
        self.device = dev
        self.rows = rows
        self.keep = [logits, params, history, hist_len, exclude]
        out = SampleOutputs()
        out.next = torch.full((rows,), -2, dtype=torch.int32, device=dev)
        out.cand_idx = torch.full((rows, cand_cap), -1, dtype=torch.int32, device=dev) if cand_cap else None
        out.cand_prob = torch.zeros((rows, cand_cap), dtype=torch.float64, device=dev) if cand_cap else None
        out.n_kept = torch.zeros(rows, dtype=torch.int32, device=dev) if want_counts else None
        out.cut = torch.zeros(rows, dtype=torch.int32, device=dev) if want_counts else None
        out.status = torch.zeros(1, dtype=torch.int32, device=dev)
        out.token_prob = torch.zeros(rows, dtype=torch.float64, device=dev) if want_counts else None
        out.softmax_sum = torch.zeros(rows, dtype=torch.float64, device=dev) if want_counts else None
        self.out = out
        b = native.SampleBatch()
        b.logits = logits.data_ptr()
        b.dtype = dtype
        b.rows = rows
        b.vocab = logits.shape[1] if vocab is None else vocab
        b.max_top_k = max_top_k
        b.row_stride = logits.stride(0)
        if history is not None and history.numel() > 0:
            if history.dtype != torch.int32 or history.dim() != 2 or not history.is_contiguous():
                raise ValueError("history must be a contiguous [rows, H] int32 tensor")
            b.history = history.data_ptr()
            b.hist_stride = history.shape[1]
            if hist_len is not None:
                b.hist_len = hist_len.data_ptr()
        if exclude is not None and exclude.numel() > 0:
            b.exclude = exclude.data_ptr()
            b.n_exclude = exclude.numel()
        b.params = params.data_ptr()
        b.next = out.next.data_ptr()
        if cand_cap:
            b.cand_idx = out.cand_idx.data_ptr()
            b.cand_prob = out.cand_prob.data_ptr()
            b.cand_stride = cand_cap
        if want_counts:
            b.n_kept = out.n_kept.data_ptr()
            b.cut = out.cut.data_ptr()
            b.token_prob = out.token_prob.data_ptr()
            b.softmax_sum = out.softmax_sum.data_ptr()
        b.status = out.status.data_ptr()
        b.splits = splits
        b.flags = flags
        b.logit_scale = logit_scale
        b.logit_softcap = logit_softcap
        self.batch = b
        nbytes = C.c_size_t(0)
        native.check(self.lib.mantleCudaSamplerWorkspaceBytes(C.byref(b), C.byref(nbytes)), "WorkspaceBytes")
        self.workspace_bytes = nbytes.value
        self.workspace = torch.empty(max(nbytes.value, 16), dtype=torch.uint8, device=dev) if nbytes.value else None
        s = C.c_int(0)
        native.check(self.lib.mantleCudaSamplerSplits(C.byref(b), C.byref(s)), "Splits")
        self.splits = s.value
        # kernels one launch() queues: the streaming kernel, plus the merge when a row is split
        self.kernels_per_launch = 2 if (self.splits > 1 or max_top_k > native.MAX_TOP_K) else 1
        self.kernel_name = self.lib.mantleCudaSamplerKernelName(C.byref(b)).decode()

    def launch(self, stream=None):
        """Queues the batch on `stream` (default: torch's current stream).  Does not synchronise."""
        rc = self.lib.mantleCudaSampleRows(C.byref(self.batch), _ptr(self.workspace), self.workspace_bytes,
                                           _stream_ptr(stream))
        native.check(rc, "mantleCudaSampleRows")
        return self.out


def sample_rows(logits, params, max_top_k, **kw):
    """One-shot form of BatchPlan: sample every row, return the outputs (device tensors)."""
    with torch.cuda.device(logits.device):
        return BatchPlan(logits, params, max_top_k, **kw).launch()


def logit_postprocess_rows_(logits, logit_scale=0.0, logit_softcap=0.0, flags=0, stream=None):
    """The model head's multiplier and soft cap alone, in place on float32 rows
    (simd/runtime.go:258-272; device form native/softmax.cu:963-970)."""
    lib = native.load()
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("logits must be a 2-D float32 CUDA tensor with unit column stride")
    with torch.cuda.device(logits.device):
        rc = lib.mantleCudaLogitPostprocessRowsF32(logits.data_ptr(), logits.shape[0], logits.shape[1],
                                                   logits.stride(0), logit_scale, logit_softcap, flags,
                                                   _stream_ptr(stream))
    native.check(rc, "mantleCudaLogitPostprocessRowsF32")
    return logits


def history_append_rows_(history, hist_len, next_tokens, keep, stop=None, done=None, stream=None):
    """`toks = append(toks, next)` of the reference's decode loop (inference/engine.go:244-250) for
    device-resident histories: [rows, stride] int32 ids, [rows] int32 lengths, both updated in place."""
    lib = native.load()
    with torch.cuda.device(history.device):
        rc = lib.mantleCudaHistoryAppendRows(history.data_ptr(), hist_len.data_ptr(), history.shape[1],
                                             history.shape[0], next_tokens.data_ptr(), keep, _ptr(stop),
                                             0 if stop is None else stop.numel(), _ptr(done), _stream_ptr(stream))
    native.check(rc, "mantleCudaHistoryAppendRows")


def repeat_penalty_rows_(logits, params, history, hist_len=None, exclude=None, stream=None):
    """The reference's in-place repeat penalty alone (sampler.go:99-138) on float32 rows."""
    lib = native.load()
    b = native.SampleBatch()
    b.logits = logits.data_ptr()
    b.dtype = native.DTYPE_F32
    b.rows = logits.shape[0]
    b.vocab = logits.shape[1]
    b.row_stride = logits.stride(0)
    b.history = history.data_ptr()
    b.hist_stride = history.shape[1]
    if hist_len is not None:
        b.hist_len = hist_len.data_ptr()
    if exclude is not None and exclude.numel() > 0:
        b.exclude = exclude.data_ptr()
        b.n_exclude = exclude.numel()
    b.params = params.data_ptr()
    with torch.cuda.device(logits.device):
        native.check(lib.mantleCudaRepeatPenaltyRowsF32(C.byref(b), _stream_ptr(stream)), "RepeatPenaltyRowsF32")
    return logits


def argmax_rows(x, stream=None):
    """Lowest-index argmax of every row of a float32 CUDA matrix (sampler.go:237-250)."""
    lib = native.load()
    out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.mantleCudaArgMaxRowsF32(_ptr(x), x.shape[0], x.shape[1], x.stride(0), _ptr(out), _stream_ptr(stream))
    native.check(rc, "mantleCudaArgMaxRowsF32")
    return out


def local_topk(logits, params, max_top_k, vocab_offset, vocab_total, history=None, hist_len=None, exclude=None,
               part_cap=None, stream=None, logit_scale=0.0, logit_softcap=0.0, flags=0):
    """Vocabulary-sharded step 1: this GPU's shortlist with global ids.  Returns (val, idx, cnt)."""
    lib = native.load()
    rows = logits.shape[0]
    cap = max_top_k if part_cap is None else part_cap
    dev = logits.device
    val = torch.zeros((rows, cap), dtype=torch.float32, device=dev)
    idx = torch.full((rows, cap), -1, dtype=torch.int32, device=dev)
    cnt = torch.zeros(rows, dtype=torch.int32, device=dev)
    b = native.SampleBatch()
    b.logits = logits.data_ptr()
    b.dtype = native.DTYPE_F32 if logits.dtype == torch.float32 else native.DTYPE_BF16
    b.rows = rows
    b.vocab = logits.shape[1]
    b.max_top_k = max_top_k
    b.row_stride = logits.stride(0)
    if history is not None and history.numel() > 0:
        b.history = history.data_ptr()
        b.hist_stride = history.shape[1]
        if hist_len is not None:
            b.hist_len = hist_len.data_ptr()
    if exclude is not None and exclude.numel() > 0:
        b.exclude = exclude.data_ptr()
        b.n_exclude = exclude.numel()
    b.params = params.data_ptr()
    b.flags = flags
    b.logit_scale = logit_scale
    b.logit_softcap = logit_softcap
    with torch.cuda.device(dev):
        rc = lib.mantleCudaSampleLocalTopK(C.byref(b), vocab_offset, vocab_total, _ptr(val), _ptr(idx), _ptr(cnt), cap,
                                           _stream_ptr(stream))
    native.check(rc, "mantleCudaSampleLocalTopK")
    return val, idx, cnt


def merge_parts(params, max_top_k, vocab_total, part_val, part_idx, part_cnt, cand_cap=0, stream=None):
    """Vocabulary-sharded step 2: merge [parts, rows, cap] shortlists and finish every row."""
    lib = native.load()
    parts, rows, cap = part_val.shape
    dev = part_val.device
    out = SampleOutputs()
    out.next = torch.full((rows,), -2, dtype=torch.int32, device=dev)
    out.cand_idx = torch.full((rows, cand_cap), -1, dtype=torch.int32, device=dev) if cand_cap else None
    out.cand_prob = torch.zeros((rows, cand_cap), dtype=torch.float64, device=dev) if cand_cap else None
    out.n_kept = torch.zeros(rows, dtype=torch.int32, device=dev)
    out.cut = torch.zeros(rows, dtype=torch.int32, device=dev)
    out.status = torch.zeros(1, dtype=torch.int32, device=dev)
    out.token_prob = torch.zeros(rows, dtype=torch.float64, device=dev)
    out.softmax_sum = torch.zeros(rows, dtype=torch.float64, device=dev)
    b = native.SampleBatch()
    b.rows = rows
    b.vocab = vocab_total
    b.max_top_k = max_top_k
    b.params = params.data_ptr()
    b.next = out.next.data_ptr()
    if cand_cap:
        b.cand_idx = out.cand_idx.data_ptr()
        b.cand_prob = out.cand_prob.data_ptr()
        b.cand_stride = cand_cap
    b.n_kept = out.n_kept.data_ptr()
    b.cut = out.cut.data_ptr()
    b.status = out.status.data_ptr()
    b.token_prob = out.token_prob.data_ptr()
    b.softmax_sum = out.softmax_sum.data_ptr()
    with torch.cuda.device(dev):
        rc = lib.mantleCudaSampleMergeParts(C.byref(b), parts, _ptr(part_val), _ptr(part_idx), _ptr(part_cnt), cap,
                                            _stream_ptr(stream))
    native.check(rc, "mantleCudaSampleMergeParts")
    return out


class HostBatchPlan:
    """The host-buffer form, mantleCudaSampleRowsHost: inputs and outputs are pinned host
    tensors, every copy happens inside the call.  This is the shape of the reference's call
    site, where the logits reach Sample as a host slice (internal/inference/engine.go:233)."""

    def __init__(self, logits, params, max_top_k, history=None, hist_len=None, exclude=None, cand_cap=0, flags=0,
                 splits=0, device="cuda:0"):
        self.lib = native.load()
        self.device = torch.device(device)
        if logits.is_cuda or logits.dim() != 2 or logits.stride(1) != 1:
            raise ValueError("logits must be a 2-D host tensor with unit column stride")
        rows = logits.shape[0]
        pin = lambda t: t if t is None or t.is_pinned() else t.pin_memory()
        self.logits = pin(logits)
        self.params = pin(torch.from_numpy(np.ascontiguousarray(params, dtype=PARAMS_DTYPE).view(np.uint8).reshape(-1).copy()))
        self.history = pin(history)
        self.hist_len = pin(hist_len)
        self.exclude = pin(exclude)
        out = SampleOutputs()
        out.next = torch.full((rows,), -2, dtype=torch.int32).pin_memory()
        out.cand_idx = torch.full((rows, cand_cap), -1, dtype=torch.int32).pin_memory() if cand_cap else None
        out.cand_prob = torch.zeros((rows, cand_cap), dtype=torch.float64).pin_memory() if cand_cap else None
        out.n_kept = torch.zeros(rows, dtype=torch.int32).pin_memory()
        out.cut = torch.zeros(rows, dtype=torch.int32).pin_memory()
        out.status = torch.zeros(1, dtype=torch.int32).pin_memory()
        out.token_prob = torch.zeros(rows, dtype=torch.float64).pin_memory()
        out.softmax_sum = torch.zeros(rows, dtype=torch.float64).pin_memory()
        self.out = out
        b = native.SampleBatch()
        b.logits = self.logits.data_ptr()
        b.dtype = native.DTYPE_F32 if logits.dtype == torch.float32 else native.DTYPE_BF16
        b.rows = rows
        b.vocab = logits.shape[1]
        b.max_top_k = max_top_k
        b.row_stride = logits.stride(0)
        if self.history is not None and self.history.numel() > 0:
            b.history = self.history.data_ptr()
            b.hist_stride = self.history.shape[1]
            if self.hist_len is not None:
                b.hist_len = self.hist_len.data_ptr()
        if self.exclude is not None and self.exclude.numel() > 0:
            b.exclude = self.exclude.data_ptr()
            b.n_exclude = self.exclude.numel()
        b.params = self.params.data_ptr()
        b.next = out.next.data_ptr()
        if cand_cap:
            b.cand_idx = out.cand_idx.data_ptr()
            b.cand_prob = out.cand_prob.data_ptr()
            b.cand_stride = cand_cap
        b.n_kept = out.n_kept.data_ptr()
        b.cut = out.cut.data_ptr()
        b.status = out.status.data_ptr()
        b.token_prob = out.token_prob.data_ptr()
        b.softmax_sum = out.softmax_sum.data_ptr()
        b.splits = splits
        b.flags = flags
        self.batch = b
        n = C.c_size_t(0)
        native.check(self.lib.mantleCudaSamplerHostWorkspaceBytes(C.byref(b), C.byref(n)), "HostWorkspaceBytes")
        self.workspace_bytes = n.value
        with torch.cuda.device(self.device):
            self.workspace = torch.empty(n.value + 256, dtype=torch.uint8, device=self.device)
        base = self.workspace.data_ptr()
        self._ws_ptr = (base + 255) // 256 * 256
        s = C.c_int(0)
        native.check(self.lib.mantleCudaSamplerSplits(C.byref(b), C.byref(s)), "Splits")
        self.kernels_per_launch = 1 if s.value == 1 else 2
        self.h2d_bytes = (self.logits.numel() * self.logits.element_size() + self.params.numel()
                          + sum(t.numel() * t.element_size() for t in (self.history, self.hist_len, self.exclude)
                                if t is not None))
        self.d2h_bytes = sum(t.numel() * t.element_size()
                             for t in (out.next, out.cand_idx, out.cand_prob, out.n_kept, out.cut, out.status, out.token_prob,
                                       out.softmax_sum)
                             if t is not None)

    def launch(self, stream=None):
        """Queues copies-in, kernels and copies-out on `stream`; the caller synchronises."""
        with torch.cuda.device(self.device):
            rc = self.lib.mantleCudaSampleRowsHost(C.byref(self.batch), C.c_void_p(self._ws_ptr), self.workspace_bytes,
                                                   _stream_ptr(stream))
        native.check(rc, "mantleCudaSampleRowsHost")
        return self.out


def launch_no_alloc(plan, stream=None):
    """Queues `plan`'s batch through mantleCudaSampleRowsNoAlloc: the same sampling, with the
    split-row scratch taken from the library's fixed device array instead of the plan's
    workspace.  For callers that cannot allocate device memory where they sample.  Raises
    CudaError carrying the library's message when the batch does not fit the fixed array."""
    rc = plan.lib.mantleCudaSampleRowsNoAlloc(C.byref(plan.batch), _stream_ptr(stream))
    if rc != 0:
        msg = plan.lib.mantleCudaSamplerLastError()
        err = native.CudaError(rc, "mantleCudaSampleRowsNoAlloc")
        err.args = (err.args[0] + (": " + msg.decode() if msg else ""),)
        raise err
    return plan.out


class Sampler:
    """logits.Sampler (internal/logits/sampler.go:44-98) over the C++ host object of
    include/mantle_host_sampler.h: NewSampler -> Sampler(cfg), Sample -> sample(), and
    CanUseDeviceGreedy.  The uniform draw is the caller's (the reference draws rng.Float64()
    once per non-greedy Sample; `rng` here is any callable returning a float in [0,1))."""

    def __init__(self, cfg, max_vocab, rng=None, device="cuda:0"):
        self.lib = native.load()
        self.device = torch.device(device)
        c = native.SamplerConfigC(cfg.seed, cfg.temperature, cfg.top_k, cfg.top_p, cfg.min_p, cfg.repeat_penalty,
                                  cfg.repeat_last_n)
        with torch.cuda.device(self.device):
            self.handle = self.lib.mantleSamplerNew(C.byref(c), max_vocab)
        if not self.handle:
            raise RuntimeError("mantleSamplerNew failed")
        if rng is None:
            gen = np.random.default_rng(cfg.seed if cfg.seed >= 0 else None)
            rng = gen.random
        self.rng = rng

    def close(self):
        if self.handle:
            with torch.cuda.device(self.device):
                self.lib.mantleSamplerFree(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def params(self):
        p = np.zeros(1, dtype=PARAMS_DTYPE)
        native.check(self.lib.mantleSamplerParams(self.handle, p.ctypes.data_as(C.c_void_p)), "mantleSamplerParams")
        return p[0]

    def can_use_device_greedy(self):
        return bool(self.lib.mantleSamplerCanUseDeviceGreedy(self.handle))

    def _draw(self):
        # one draw per call that takes the stochastic path, none otherwise (sampler.go:140-142, 224)
        return float(self.rng()) if self.lib.mantleSamplerNeedsUniform(self.handle) else 0.0

    @staticmethod
    def _ids(ids):
        a = np.ascontiguousarray([] if ids is None else ids, dtype=np.int64)
        return a, (a.ctypes.data_as(C.c_void_p) if a.size else None)

    def sample(self, logits, recent=None, exclude_penalty=None):
        """Sample(logits, recent, excludePenalty): `logits` is a float32 numpy vector, patched in
        place by the repeat penalty as the reference patches its slice.  Returns the token id."""
        if logits.dtype != np.float32 or logits.ndim != 1 or not logits.flags.c_contiguous:
            raise ValueError("logits must be a contiguous float32 vector")
        if logits.size == 0:
            raise ValueError("argmax: empty slice")  # the reference panics (sampler.go:239)
        r, rp = self._ids(recent)
        x, xp = self._ids(exclude_penalty)
        tok = C.c_int(-1)
        with torch.cuda.device(self.device):
            rc = self.lib.mantleSamplerSample(self.handle, logits.ctypes.data_as(C.c_void_p), logits.size, rp, r.size,
                                              xp, x.size, self._draw(), C.byref(tok))
        native.check(rc, "mantleSamplerSample")
        return tok.value

    def sample_device(self, logits, recent=None, exclude_penalty=None):
        """The same on a float32 CUDA vector that stays on the GPU (and is left untouched)."""
        r, rp = self._ids(recent)
        x, xp = self._ids(exclude_penalty)
        tok = C.c_int(-1)
        with torch.cuda.device(self.device):
            rc = self.lib.mantleSamplerSampleDevice(self.handle, _ptr(logits), logits.numel(), rp, r.size, xp, x.size,
                                                    self._draw(), _stream_ptr(None), C.byref(tok))
        native.check(rc, "mantleSamplerSampleDevice")
        return tok.value


class BatchSampler:
    """The decode loop's sampling state for `rows` requests at once (include/mantle_batch_sampler.h):
    what Generator.RunWithContext keeps per request -- toks, the Sampler, the stop tokens
    (internal/inference/engine.go:189, 233-300) -- held on the device for the whole batch.

        bs = BatchSampler(rows, vocab, hist_capacity, stop_tokens)
        bs.set_row(r, SamplerConfig(...), context_tokens)      # a request starts
        while ...:
            logits = model(...)                                 # [rows, >= vocab] CUDA tensor
            next_tokens, ended = bs.step(logits, rngs)          # one uniform per live stochastic row

    `rngs[r]` is any callable returning a float in [0, 1): row r's own generator, drawn from exactly
    when the reference's Sampler of that request would draw (sampler.go:140-142, 224)."""

    def __init__(self, rows, vocab, hist_capacity, stop_tokens=(), device="cuda:0"):
        self.lib = native.load()
        self.device = torch.device(device)
        self.rows, self.vocab = rows, vocab
        stop = np.ascontiguousarray(list(stop_tokens), dtype=np.int64)
        with torch.cuda.device(self.device):
            self.handle = self.lib.mantleBatchSamplerNew(rows, vocab, hist_capacity,
                                                         stop.ctypes.data_as(C.c_void_p) if stop.size else None, stop.size)
        if not self.handle:
            raise RuntimeError("mantleBatchSamplerNew failed")
        self._uniforms = np.zeros(rows, dtype=np.float64)

    def close(self):
        if self.handle:
            with torch.cuda.device(self.device):
                self.lib.mantleBatchSamplerFree(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_row(self, row, cfg, context=(), stream=None):
        """A request starts on `row`: NewSampler(cfg) and toks := copy(context)."""
        c = native.SamplerConfigC(cfg.seed, cfg.temperature, cfg.top_k, cfg.top_p, cfg.min_p, cfg.repeat_penalty,
                                  cfg.repeat_last_n)
        ctx = np.ascontiguousarray(list(context), dtype=np.int64)
        with torch.cuda.device(self.device):
            rc = self.lib.mantleBatchSamplerSetRow(self.handle, row, C.byref(c),
                                                   ctx.ctypes.data_as(C.c_void_p) if ctx.size else None, ctx.size,
                                                   _stream_ptr(stream))
        native.check(rc, "mantleBatchSamplerSetRow")

    def end_row(self, row, stream=None):
        with torch.cuda.device(self.device):
            native.check(self.lib.mantleBatchSamplerEndRow(self.handle, row, _stream_ptr(stream)), "mantleBatchSamplerEndRow")

    def needs_uniform(self, row):
        return bool(self.lib.mantleBatchSamplerNeedsUniform(self.handle, row))

    def can_use_device_greedy(self, row):
        return bool(self.lib.mantleBatchSamplerCanUseDeviceGreedy(self.handle, row))

    def draw(self, rngs):
        """This step's uniforms: one draw from rngs[r] for every row that consumes one."""
        u = self._uniforms
        for r in range(self.rows):
            u[r] = float(rngs[r]()) if self.needs_uniform(r) else 0.0
        return u

    def step_async(self, logits, uniforms, stream=None, logit_scale=0.0, logit_softcap=0.0):
        """Queues one step on `stream`; results() after the stream has been synchronised."""
        if not logits.is_cuda or logits.dim() != 2 or logits.stride(1) != 1 or logits.shape[0] != self.rows:
            raise ValueError("logits must be a [rows, >= vocab] CUDA tensor with unit column stride")
        dtype = {torch.float32: native.DTYPE_F32, torch.bfloat16: native.DTYPE_BF16}[logits.dtype]
        u = np.ascontiguousarray(uniforms, dtype=np.float64)
        if u.shape != (self.rows,):
            raise ValueError("one uniform per row")
        with torch.cuda.device(self.device):
            rc = self.lib.mantleBatchSamplerStep(self.handle, _ptr(logits), dtype, logits.stride(0),
                                                 u.ctypes.data_as(C.c_void_p), logit_scale, logit_softcap,
                                                 _stream_ptr(stream))
        native.check(rc, "mantleBatchSamplerStep")

    def results(self):
        """(next tokens, ended flags, status word) of the last step, as numpy arrays (copies)."""
        nxt, end, dev = C.c_void_p(), C.c_void_p(), C.c_void_p()
        status = C.c_int32(0)
        native.check(self.lib.mantleBatchSamplerResults(self.handle, C.byref(nxt), C.byref(end), C.byref(status),
                                                        C.byref(dev)), "mantleBatchSamplerResults")
        n = np.ctypeslib.as_array(C.cast(nxt, C.POINTER(C.c_int32)), shape=(self.rows,)).copy()
        e = np.ctypeslib.as_array(C.cast(end, C.POINTER(C.c_int32)), shape=(self.rows,)).copy()
        return n, e, status.value

    def step(self, logits, rngs, **kw):
        """draw + step_async + synchronise + results: one iteration of the reference's loop for the batch."""
        self.step_async(logits, self.draw(rngs), **kw)
        torch.cuda.current_stream(self.device).synchronize()
        n, e, status = self.results()
        return n, e
