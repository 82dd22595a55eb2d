//go:build cuda && nccl

package native

// cgo binding of libmantle_cuda_sampler_nccl: vocabulary-sharded sampling in one call per rank.
// Behind its own build tag because it adds NCCL to the link line; add
// `-lmantle_cuda_sampler_nccl -lnccl` to #cgo LDFLAGS when building with `-tags "cuda nccl"`.
// The reference links no collective library (runtime.go:6) and has no multi-GPU path; this is
// what Sampler.Sample becomes when the LM head's output is split by columns over several GPUs.
// Not compiled here (no Go toolchain).

/*
#include <stdint.h>
#include <stddef.h>
typedef void* cudaStream_t;
struct MantleSampleBatch;

extern int mantleCudaSampleVocabSharded(const struct MantleSampleBatch* b, int vocabOffset, int vocabTotal,
	void* ncclComm, void* packedLocal, void* packedAll, cudaStream_t s, int* ncclResult);

static int sampleVocabShardedW(const void* b, int off, int total, void* comm, void* local, void* all, cudaStream_t s, int* nr) {
	return mantleCudaSampleVocabSharded((const struct MantleSampleBatch*)b, off, total, comm, local, all, s, nr);
}
*/
import "C"

import (
	"fmt"
	"unsafe"
)

// NcclComm is an ncclComm_t the host made with ncclCommInitRank (rank r holds the r-th range of
// columns); the sampler only borrows it.
type NcclComm struct{ Ptr unsafe.Pointer }

// SampleVocabSharded queues, on stream: this rank's shortlist of every row into packedLocal
// (SamplePackedPartBytes(rows, MaxTopK) bytes), ncclAllGather of the blocks into packedAll
// (ranks times that), and the merge with the rest of Sample.  b.Logits holds this rank's columns
// [vocabOffset, vocabOffset+b.Vocab) of rows vocabTotal wide; History, Exclude and Params are the
// same on every rank and hold global ids.  Every rank ends with the same tokens in b.Next.
func SampleVocabSharded(b *SampleBatch, vocabOffset, vocabTotal int, comm NcclComm, packedLocal, packedAll DeviceBuffer,
	stream Stream) error {
	cb, err := b.c()
	if err != nil {
		return err
	}
	if comm.Ptr == nil || packedLocal.ptr == nil || packedAll.ptr == nil {
		return fmt.Errorf("vocabulary-sharded sampling needs a communicator and both packed buffers")
	}
	var ncclResult C.int
	code := C.sampleVocabShardedW(unsafe.Pointer(&cb), C.int(vocabOffset), C.int(vocabTotal), comm.Ptr, packedLocal.ptr,
		packedAll.ptr, stream.ptr, &ncclResult)
	if code != 0 && ncclResult != 0 {
		return fmt.Errorf("%w (ncclResult %d)", cudaErr(code), int(ncclResult))
	}
	return cudaErr(code)
}
