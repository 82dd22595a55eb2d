/*
 * Vocabulary-sharded sampling across the GPUs of one box, in one call per rank.
 *
 * The reference has no multi-GPU path at all (its link line, internal/backend/cuda/native/
 * runtime.go:6, names no collective library; one request runs on one GPU,
 * internal/api/engine_provider.go:66-71), so this entry point replaces nothing: it is what
 * Sampler.Sample (internal/logits/sampler.go:98-234) becomes when the LM head's output is
 * split by columns over several GPUs.  It lives in a library of its own,
 * libmantle_cuda_sampler_nccl, so that hosts without NCCL can still load the sampler; a cgo
 * host adds `-lmantle_cuda_sampler_nccl -lnccl` to its link line.
 */
#ifndef MANTLE_CUDA_SAMPLER_NCCL_H
#define MANTLE_CUDA_SAMPLER_NCCL_H

#include "mantle_cuda_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * One sampling step over logits split by columns: this rank holds columns
 * [vocab_offset, vocab_offset + batch->vocab) of rows that are vocab_total wide.  Queues, on
 * `stream`:
 *   1. mantleCudaSampleLocalTopK: this rank's shortlist of every row (penalty applied to the ids
 *      it owns, values scaled, global ids) into `packed_local`, one packed block of
 *      mantleCudaSamplePackedPartBytes(rows, max_top_k) bytes;
 *   2. ncclAllGather of the blocks over `nccl_comm` (an ncclComm_t whose ranks are the shards in
 *      column order) into `packed_all`, ranks * that many bytes;
 *   3. mantleCudaSampleMergePacked: the merge of the ranks' shortlists -- exactly the global
 *      shortlist, because the shards are contiguous and ties go to the lower global id -- and
 *      the rest of Sample (softmax, min-p, top-p, draw).
 * Every rank ends with the same tokens in batch->next (and the same optional outputs).
 * history / exclude hold global ids and are the same on every rank; params likewise.
 * batch->max_top_k * ranks must not exceed 4096.  Nothing is allocated and nothing
 * synchronises; both buffers are the caller's, 16-byte aligned, on the current device.
 * Returns a cudaError_t as int; an NCCL failure is reported as cudaErrorUnknown with the
 * ncclResult_t in *nccl_result when that pointer is given.
 */
int mantleCudaSampleVocabSharded(const MantleSampleBatch* batch, int vocab_offset, int vocab_total,
                                 void* nccl_comm, void* packed_local, void* packed_all,
                                 mantleCudaStream_t stream, int* nccl_result);

#ifdef __cplusplus
}
#endif

#endif /* MANTLE_CUDA_SAMPLER_NCCL_H */
