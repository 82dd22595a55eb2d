// Vocabulary-sharded sampling in one call: local shortlist -> ncclAllGather -> merge.
// See include/mantle_cuda_sampler_nccl.h.  Built into libmantle_cuda_sampler_nccl, which links
// the sampler library and NCCL; the kernels themselves live in the sampler library.

#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>

#include "../../include/mantle_cuda_sampler_nccl.h"

extern "C" int mantleCudaSampleVocabSharded(const MantleSampleBatch* batch, int vocab_offset, int vocab_total,
                                            void* nccl_comm, void* packed_local, void* packed_all,
                                            mantleCudaStream_t stream, int* nccl_result) {
    if (nccl_result) *nccl_result = (int)ncclSuccess;
    if (!batch || !nccl_comm || !packed_local || !packed_all) return (int)cudaErrorInvalidValue;
    if (batch->rows <= 0 || batch->max_top_k < 1) return (int)cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(packed_local) % 16 || reinterpret_cast<uintptr_t>(packed_all) % 16)
        return (int)cudaErrorInvalidValue;
    ncclComm_t comm = static_cast<ncclComm_t>(nccl_comm);
    int ranks = 0;
    ncclResult_t nr = ncclCommCount(comm, &ranks);
    if (nr != ncclSuccess || ranks < 1) {
        if (nccl_result) *nccl_result = (int)nr;
        return (int)cudaErrorUnknown;
    }
    const int k = batch->max_top_k;
    if ((long long)ranks * k > 4096) return (int)cudaErrorInvalidValue;
    size_t block = 0;
    int rc = mantleCudaSamplePackedPartBytes(batch->rows, k, &block);
    if (rc) return rc;

    // 1. this rank's shortlists into its packed block: [values][ids][counts]
    const size_t n = (size_t)batch->rows * (size_t)k;
    float* val = static_cast<float*>(packed_local);
    int32_t* idx = reinterpret_cast<int32_t*>(val + n);
    int32_t* cnt = idx + n;
    rc = mantleCudaSampleLocalTopK(batch, vocab_offset, vocab_total, val, idx, cnt, k, stream);
    if (rc) return rc;

    // 2. one all-gather moves every rank's block; the gathered blocks land in this GPU's own
    //    memory before the merge reads them
    nr = ncclAllGather(packed_local, packed_all, block, ncclChar, comm, static_cast<cudaStream_t>(stream));
    if (nr != ncclSuccess) {
        if (nccl_result) *nccl_result = (int)nr;
        return (int)cudaErrorUnknown;
    }

    // 3. merge and finish every row: the descriptor's outputs and parameters, the whole row's width
    MantleSampleBatch m = *batch;
    m.vocab = vocab_total;
    m.row_stride = vocab_total;
    return mantleCudaSampleMergePacked(&m, ranks, packed_all, k, stream);
}
