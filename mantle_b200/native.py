"""ctypes binding of the CUDA sampler library (include/mantle_cuda_sampler.h).

There is no CPU implementation behind this module: if the library is missing it raises,
it does not fall back.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

DTYPE_F32 = 0
DTYPE_BF16 = 1
MAX_TOP_K = 1024
MAX_VOCAB = 1 << 20
FLAG_WRITE_BACK_PENALTY = 1
FLAG_PENALTY_PREAPPLIED = 2
FLAG_SOFTCAP_TANHF = 4
STATUS_TOPK_RANGE = 1
STATUS_EMPTY = 2
STATUS_TIMEOUT = 4
STATUS_NAN = 8
CUDA_ERROR_INVALID_VALUE = 1

# MantleSampleParams, include/mantle_sample_params.h
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


class SampleBatch(C.Structure):
    """MantleSampleBatch, include/mantle_cuda_sampler.h."""

    _fields_ = [
        ("logits", C.c_void_p),
        ("dtype", C.c_int32),
        ("rows", C.c_int32),
        ("vocab", C.c_int32),
        ("max_top_k", C.c_int32),
        ("row_stride", C.c_int64),
        ("history", C.c_void_p),
        ("hist_len", C.c_void_p),
        ("hist_stride", C.c_int32),
        ("n_exclude", C.c_int32),
        ("exclude", C.c_void_p),
        ("params", C.c_void_p),
        ("next", C.c_void_p),
        ("cand_idx", C.c_void_p),
        ("cand_prob", C.c_void_p),
        ("n_kept", C.c_void_p),
        ("cut", C.c_void_p),
        ("status", C.c_void_p),
        ("cand_stride", C.c_int32),
        ("splits", C.c_int32),
        ("flags", C.c_uint32),
        ("reserved", C.c_uint32),
        ("logit_scale", C.c_float),
        ("logit_softcap", C.c_float),
        ("token_prob", C.c_void_p),
        ("softmax_sum", C.c_void_p),
        ("skip", C.c_void_p),
    ]


EXPORTS = {
    "mantleCudaSamplerAbiVersion": (C.c_int, []),
    "mantleCudaSampleRows": (C.c_int, [C.POINTER(SampleBatch), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mantleCudaSamplerWorkspaceBytes": (C.c_int, [C.POINTER(SampleBatch), C.POINTER(C.c_size_t)]),
    "mantleCudaSamplerSplits": (C.c_int, [C.POINTER(SampleBatch), C.POINTER(C.c_int)]),
    "mantleCudaSamplerKernelName": (C.c_char_p, [C.POINTER(SampleBatch)]),
    "mantleCudaRepeatPenaltyRowsF32": (C.c_int, [C.POINTER(SampleBatch), C.c_void_p]),
    "mantleCudaLogitPostprocessRowsF32": (
        C.c_int,
        [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_float, C.c_float, C.c_uint32, C.c_void_p],
    ),
    "mantleCudaHistoryAppendRows": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p],
    ),
    "mantleCudaArgMaxRowsF32": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_void_p]),
    "mantleCudaSampleLocalTopK": (
        C.c_int,
        [C.POINTER(SampleBatch), C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p],
    ),
    "mantleCudaSamplePackedPartBytes": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_size_t)]),
    "mantleCudaSampleMergePacked": (C.c_int, [C.POINTER(SampleBatch), C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "mantleCudaSampleRowsHost": (C.c_int, [C.POINTER(SampleBatch), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mantleCudaSamplerHostWorkspaceBytes": (C.c_int, [C.POINTER(SampleBatch), C.POINTER(C.c_size_t)]),
    "mantleCudaSampleRowsNoAlloc": (C.c_int, [C.POINTER(SampleBatch), C.c_void_p]),
    "mantleCudaSamplerStaticScratchBytes": (C.c_size_t, []),
    "mantleCudaSamplerLastError": (C.c_char_p, []),
    "mantleCudaSamplerSelfTestBoundedWait": (C.c_int, [C.c_ulonglong, C.c_void_p, C.c_void_p]),
    "mantleCudaSampleMergeParts": (
        C.c_int,
        [C.POINTER(SampleBatch), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p],
    ),
}



class SamplerConfigC(C.Structure):
    """MantleSamplerConfig, include/mantle_sample_params.h: logits.SamplerConfig field for field."""

    _fields_ = [
        ("seed", C.c_int64),
        ("temperature", C.c_float),
        ("top_k", C.c_int32),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repeat_penalty", C.c_float),
        ("repeat_last_n", C.c_int32),
    ]


# include/mantle_host_sampler.h
HOST_EXPORTS = {
    "mantleSamplerNew": (C.c_void_p, [C.POINTER(SamplerConfigC), C.c_int]),
    "mantleSamplerFree": (None, [C.c_void_p]),
    "mantleSamplerParams": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mantleSamplerCanUseDeviceGreedy": (C.c_int, [C.c_void_p]),
    "mantleSamplerNeedsUniform": (C.c_int, [C.c_void_p]),
    "mantleSamplerSample": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_double, C.POINTER(C.c_int)],
    ),
    "mantleSamplerSampleDevice": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p,
         C.POINTER(C.c_int)],
    ),
}

# include/mantle_batch_sampler.h
BATCH_EXPORTS = {
    "mantleBatchSamplerNew": (C.c_void_p, [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "mantleBatchSamplerFree": (None, [C.c_void_p]),
    "mantleBatchSamplerSetRow": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(SamplerConfigC), C.c_void_p, C.c_int, C.c_void_p]),
    "mantleBatchSamplerEndRow": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "mantleBatchSamplerNeedsUniform": (C.c_int, [C.c_void_p, C.c_int]),
    "mantleBatchSamplerCanUseDeviceGreedy": (C.c_int, [C.c_void_p, C.c_int]),
    "mantleBatchSamplerStep": (
        C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_float, C.c_float, C.c_void_p]),
    "mantleBatchSamplerResults": (
        C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.POINTER(C.c_void_p)]),
}

_lib = None


class CudaError(RuntimeError):
    """A non-zero cudaError_t from the library (native/runtime.go:443-455 wraps codes the same way)."""

    def __init__(self, code, where):
        self.code = int(code)
        super().__init__("%s failed: cudaError %d" % (where, self.code))


def lib_path():
    return _build.LIB_PATH


def load():
    """Loads the library (building it first when nvcc is present and it is stale)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    try:
        _build.build_native()
    except Exception:
        if not os.path.exists(path):
            raise
    if not os.path.exists(path):
        raise RuntimeError("CUDA sampler library missing: %s (run python -m mantle_b200.build)" % path)
    L = C.CDLL(path)
    for name, (res, args) in list(EXPORTS.items()) + list(HOST_EXPORTS.items()) + list(BATCH_EXPORTS.items()):
        f = getattr(L, name)  # AttributeError here means the build is broken: do not hide it
        f.restype = res
        f.argtypes = args
    if L.mantleCudaSamplerAbiVersion() != 3:
        raise RuntimeError("CUDA sampler library ABI mismatch")
    _lib = L
    return L


def check(code, where):
    if code != 0:
        raise CudaError(code, where)
