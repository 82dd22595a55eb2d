"""The C-ABI library without a GPU: it loads, exports every symbol the header declares,
and rejects bad arguments with cudaErrorInvalidValue before touching the device."""
import ctypes as C
import os
import re

import numpy as np

from mantle_b200 import native, sampler

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mantle_cuda_sampler.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(mantleCuda\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = native.load()
    names = declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), n
        assert n in native.EXPORTS, "binding missing for " + n
    assert lib.mantleCudaSamplerAbiVersion() == 3


def test_struct_layout_matches_header():
    assert native.PARAMS_DTYPE.itemsize == 40
    assert native.PARAMS_DTYPE.fields["uniform"][1] == 32
    assert C.sizeof(native.SampleBatch) == 168
    assert native.SampleBatch.row_stride.offset == 24
    assert native.SampleBatch.cand_stride.offset == 120


def good_batch():
    b = native.SampleBatch()
    b.logits = 0x1000
    b.dtype = native.DTYPE_F32
    b.rows = 4
    b.vocab = 1000
    b.max_top_k = 40
    b.row_stride = 1000
    b.params = 0x2000
    b.next = 0x3000
    return b


def test_invalid_arguments_are_rejected_on_the_host():
    lib = native.load()
    inv = native.CUDA_ERROR_INVALID_VALUE
    n = C.c_size_t(123)
    assert lib.mantleCudaSamplerWorkspaceBytes(C.byref(good_batch()), C.byref(n)) == 0
    mutations = [
        ("logits", 0), ("rows", 0), ("vocab", 0), ("vocab", native.MAX_VOCAB + 1), ("dtype", 7),
        ("row_stride", 999), ("max_top_k", 0), ("max_top_k", native.MAX_VOCAB + 1), ("params", 0), ("next", 0),
        ("n_exclude", 3), ("hist_stride", -1), ("flags", 8), ("reserved", 1), ("splits", -1), ("logits", 0x1001),
        ("logit_scale", -2.0), ("logit_scale", float("nan")), ("logit_scale", float("inf")),
        ("logit_softcap", float("inf")),
    ]
    for field, value in mutations:
        b = good_batch()
        setattr(b, field, value)
        assert lib.mantleCudaSampleRows(C.byref(b), None, 0, None) == inv, field
        assert lib.mantleCudaSamplerWorkspaceBytes(C.byref(b), C.byref(n)) == inv, field
    b = good_batch()
    b.cand_idx = 0x4000  # candidates wanted but no room per row
    assert lib.mantleCudaSampleRows(C.byref(b), None, 0, None) == inv
    b = good_batch()
    b.max_top_k, b.cand_idx, b.cand_prob, b.cand_stride = native.MAX_TOP_K + 1, 0x4000, 0x5000, 8
    assert lib.mantleCudaSampleRows(C.byref(b), None, 0, None) == inv  # long shortlists are never materialised
    b = good_batch()
    b.dtype = native.DTYPE_BF16
    b.flags = native.FLAG_WRITE_BACK_PENALTY  # bf16 rows cannot hold the penalised value
    assert lib.mantleCudaSampleRows(C.byref(b), None, 0, None) == inv
    for flag in (native.FLAG_WRITE_BACK_PENALTY, native.FLAG_PENALTY_PREAPPLIED):
        b = good_batch()
        b.logit_softcap, b.flags = 30.0, flag  # fused post-processing never rewrites the logits
        assert lib.mantleCudaSampleRows(C.byref(b), None, 0, None) == inv
    assert lib.mantleCudaLogitPostprocessRowsF32(None, 1, 10, 10, 1.0, 30.0, 0, None) == inv
    assert lib.mantleCudaLogitPostprocessRowsF32(0x10, 1, 10, 5, 1.0, 30.0, 0, None) == inv
    assert lib.mantleCudaLogitPostprocessRowsF32(0x10, 1, 10, 10, -1.0, 30.0, 0, None) == inv
    assert lib.mantleCudaLogitPostprocessRowsF32(0x10, 1, 10, 10, 1.0, 30.0, 1, None) == inv
    b = good_batch()
    b.rows, b.splits = 1, 4  # split rows need a workspace
    assert lib.mantleCudaSampleRows(C.byref(b), None, 0, None) == inv
    assert lib.mantleCudaArgMaxRowsF32(None, 1, 10, 10, 0x10, None) == inv
    assert lib.mantleCudaArgMaxRowsF32(0x10, 1, 0, 10, 0x10, None) == inv
    assert lib.mantleCudaArgMaxRowsF32(0x10, 1, 10, 5, 0x10, None) == inv
    assert lib.mantleCudaSampleLocalTopK(C.byref(good_batch()), 0, 1000, None, 0x10, 0x10, 40, None) == inv
    assert lib.mantleCudaSampleLocalTopK(C.byref(good_batch()), 500, 1000, 0x10, 0x10, 0x10, 40, None) == inv
    assert lib.mantleCudaSampleMergeParts(C.byref(good_batch()), 200, 0x10, 0x10, 0x10, 40, None) == inv
    assert lib.mantleCudaRepeatPenaltyRowsF32(None, None) == inv
    assert lib.mantleCudaHistoryAppendRows(None, 0x10, 64, 4, 0x10, 32, None, 0, None, None) == inv
    assert lib.mantleCudaHistoryAppendRows(0x10, 0x10, 64, 4, 0x10, 33, None, 0, None, None) == inv  # keep > stride/2
    assert lib.mantleCudaHistoryAppendRows(0x10, 0x10, 64, 0, 0x10, 32, None, 0, None, None) == inv
    assert lib.mantleCudaHistoryAppendRows(0x10, 0x10, 64, 4, 0x10, 32, None, 2, None, None) == inv  # stop list missing


def test_constructor_normalisation_matches_the_oracle():
    import oracle_lib as O

    rng = np.random.default_rng(0)
    for _ in range(200):
        cfg = dict(
            temperature=float(rng.choice([-1.0, 0.0, 0.3, 1.0, 2.0])),
            top_k=int(rng.choice([-1, 0, 1, 40, 100000])),
            top_p=float(rng.choice([-0.5, 0.0, 0.5, 1.0, 1.5])),
            min_p=float(rng.choice([0.0, 0.05])),
            repeat_penalty=float(rng.choice([-1.0, 0.0, 1.0, 1.3])),
            repeat_last_n=int(rng.choice([-1, 0, 64, 1024])),
        )
        a = sampler.new_sampler_params(sampler.SamplerConfig(**cfg), uniform=0.25)
        b = O.normalize(uniform=0.25, **cfg)
        assert a.tobytes() == np.array(b).tobytes(), cfg
        assert sampler.can_use_device_greedy(a) == O.can_use_device_greedy(b)


def test_batch_sampler_argument_checks_need_no_gpu():
    """mantleBatchSampler*: bad arguments are refused before any device call."""
    lib = native.load()
    inv = native.CUDA_ERROR_INVALID_VALUE
    assert not lib.mantleBatchSamplerNew(0, 1000, 64, None, 0)
    assert not lib.mantleBatchSamplerNew(4, 0, 64, None, 0)
    assert not lib.mantleBatchSamplerNew(4, native.MAX_VOCAB + 1, 64, None, 0)
    assert not lib.mantleBatchSamplerNew(4, 1000, 1, None, 0)
    assert not lib.mantleBatchSamplerNew(4, 1000, 64, None, 2)  # two stop tokens, no list
    cfg = native.SamplerConfigC(0, 1.0, 40, 0.9, 0.0, 1.1, 64)
    assert lib.mantleBatchSamplerSetRow(None, 0, C.byref(cfg), None, 0, None) == inv
    assert lib.mantleBatchSamplerEndRow(None, 0, None) == inv
    assert lib.mantleBatchSamplerStep(None, None, 0, 0, None, 0.0, 0.0, None) == inv
    assert lib.mantleBatchSamplerResults(None, None, None, None, None) == inv
    assert lib.mantleBatchSamplerNeedsUniform(None, 0) == 0
    assert lib.mantleBatchSamplerCanUseDeviceGreedy(None, 0) == 0
    lib.mantleBatchSamplerFree(None)  # a no-op


def test_nccl_entry_point_is_exported_and_checks_its_arguments():
    """libmantle_cuda_sampler_nccl loads, exports what its header declares and refuses a call
    without a communicator before touching NCCL or the device."""
    from mantle_b200 import nccl

    text = open(os.path.join(ROOT, "include", "mantle_cuda_sampler_nccl.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\bint\s+(mantleCuda\w+)\s*\(", text)
    assert names == ["mantleCudaSampleVocabSharded"]
    lib = nccl.load()
    for n in names:
        assert hasattr(lib, n)
    rc = C.c_int(-1)
    b = good_batch()
    assert lib.mantleCudaSampleVocabSharded(C.byref(b), 0, 1000, None, 0x1000, 0x2000, None, C.byref(rc)) == native.CUDA_ERROR_INVALID_VALUE
    assert rc.value == 0
