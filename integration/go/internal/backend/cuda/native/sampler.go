//go:build cuda

// Package native: cgo binding of the device-side logits sampler.
//
// This file sits next to argmax.go and follows its conventions (file-local preamble that
// forward-declares the C symbols, a static wrapper per symbol, Go functions that validate and
// return cudaErr(code)).  It was written against the reference tree without a Go toolchain at
// hand and has not been compiled; the same C symbols are exercised from C++ and Python.
//
// Link: add libmantle_cuda_sampler (built by `python -m mantle_b200.build`, or sampler_kernels.cu
// and host_sampler.cu added to scripts/build_cuda.sh with
// -gencode arch=compute_100a,code=sm_100a -fmad=false) to the #cgo LDFLAGS line of runtime.go.
package native

/*
#include <stdint.h>
#include <stddef.h>
typedef void* cudaStream_t;

typedef struct MantleSampleParams {
	float temperature, top_p, min_p, repeat_penalty;
	int32_t top_k, repeat_last_n, greedy, reserved;
	double uniform;
} MantleSampleParams;

typedef struct MantleSampleBatch {
	const void* logits;
	int32_t dtype, rows, vocab, max_top_k;
	int64_t row_stride;
	const int32_t* history;
	const int32_t* hist_len;
	int32_t hist_stride, n_exclude;
	const int32_t* exclude;
	const MantleSampleParams* params;
	int32_t* next;
	int32_t* cand_idx;
	double* cand_prob;
	int32_t* n_kept;
	int32_t* cut;
	int32_t* status;
	int32_t cand_stride, splits;
	uint32_t flags, reserved;
	float logit_scale, logit_softcap;
} MantleSampleBatch;

extern int mantleCudaSampleRows(const MantleSampleBatch* b, void* ws, size_t wsBytes, cudaStream_t s);
extern int mantleCudaSamplerWorkspaceBytes(const MantleSampleBatch* b, size_t* bytes);
extern int mantleCudaSampleRowsNoAlloc(const MantleSampleBatch* b, cudaStream_t s);
extern int mantleCudaArgMaxRowsF32(const float* x, int rows, int n, int64_t stride, int* out, cudaStream_t s);
extern int mantleCudaLogitPostprocessRowsF32(float* x, int rows, int n, int64_t stride, float scale, float softcap,
	uint32_t flags, cudaStream_t s);

static int mantleCudaSampleRowsWrapper(const MantleSampleBatch* b, void* ws, size_t n, cudaStream_t s) {
	return mantleCudaSampleRows(b, ws, n, s);
}
static int mantleCudaSamplerWorkspaceBytesWrapper(const MantleSampleBatch* b, size_t* n) {
	return mantleCudaSamplerWorkspaceBytes(b, n);
}
static int mantleCudaSampleRowsNoAllocWrapper(const MantleSampleBatch* b, cudaStream_t s) {
	return mantleCudaSampleRowsNoAlloc(b, s);
}
static int mantleCudaArgMaxRowsF32Wrapper(const float* x, int rows, int n, int64_t stride, int* out, cudaStream_t s) {
	return mantleCudaArgMaxRowsF32(x, rows, n, stride, out, s);
}
static int mantleCudaLogitPostprocessRowsF32Wrapper(float* x, int rows, int n, int64_t stride, float scale,
	float softcap, uint32_t flags, cudaStream_t s) {
	return mantleCudaLogitPostprocessRowsF32(x, rows, n, stride, scale, softcap, flags, s);
}
*/
import "C"

import (
	"fmt"
	"unsafe"
)

// SampleParams is one row's normalised sampling parameters (what logits.NewSampler leaves in
// the Sampler, plus the uniform draw of this step).
type SampleParams struct {
	Temperature   float32
	TopP          float32
	MinP          float32
	RepeatPenalty float32
	TopK          int32
	RepeatLastN   int32
	Greedy        int32
	reserved      int32
	Uniform       float64
}

// HeadPost is what the model head does to the logits before sampling (LMHeadMultiplier and
// FinalLogitSoftcap, simd/runtime.go:258-272).  The zero value means neither.
type HeadPost struct {
	Scale   float32 // applied when neither 0 nor 1
	Softcap float32 // applied when > 0
	Tanhf   bool    // tanhf as mantleCudaLogitSoftcapF32 has it, instead of the host path's fastTanh
}

// SampleRowsF32 samples `rows` rows of device-resident float32 logits.  params, history,
// exclude and next are device buffers laid out as include/mantle_cuda_sampler.h describes;
// workspace may be the zero DeviceBuffer when SamplerWorkspaceBytes reports 0.  post is
// applied to the logits on the fly; they are not rewritten.
func SampleRowsF32(logits DeviceBuffer, rows, vocab int, rowStride int64, params, history DeviceBuffer,
	histStride int, exclude DeviceBuffer, nExclude int, maxTopK int, post HeadPost, next, workspace DeviceBuffer,
	workspaceBytes int64, stream Stream) error {
	if logits.ptr == nil || params.ptr == nil || next.ptr == nil {
		return fmt.Errorf("sample buffer is nil")
	}
	if rows <= 0 || vocab <= 0 {
		return fmt.Errorf("sample rows and vocab must be > 0")
	}
	var b C.MantleSampleBatch
	b.logits = logits.ptr
	b.dtype = 0
	b.rows = C.int32_t(rows)
	b.vocab = C.int32_t(vocab)
	b.max_top_k = C.int32_t(maxTopK)
	b.row_stride = C.int64_t(rowStride)
	b.history = (*C.int32_t)(history.ptr)
	b.hist_stride = C.int32_t(histStride)
	b.exclude = (*C.int32_t)(exclude.ptr)
	b.n_exclude = C.int32_t(nExclude)
	b.params = (*C.MantleSampleParams)(params.ptr)
	b.next = (*C.int32_t)(next.ptr)
	b.logit_scale = C.float(post.Scale)
	b.logit_softcap = C.float(post.Softcap)
	if post.Tanhf {
		b.flags |= 4 // MANTLE_SAMPLE_SOFTCAP_TANHF
	}
	return cudaErr(C.mantleCudaSampleRowsWrapper(&b, workspace.ptr, C.size_t(workspaceBytes), stream.ptr))
}

// ArgMaxRowsF32To is the batched, lowest-index replacement of ArgMaxF32To.
func ArgMaxRowsF32To(x DeviceBuffer, rows, n int, stride int64, outIdx DeviceBuffer, stream Stream) error {
	if x.ptr == nil || outIdx.ptr == nil {
		return fmt.Errorf("argmax buffer is nil")
	}
	if rows <= 0 || n <= 0 {
		return fmt.Errorf("argmax rows and n must be > 0")
	}
	return cudaErr(C.mantleCudaArgMaxRowsF32Wrapper((*C.float)(x.ptr), C.int(rows), C.int(n), C.int64_t(stride),
		(*C.int)(outIdx.ptr), stream.ptr))
}

// LogitPostprocessF32 rewrites device-resident logits in place: the multiplier loop and the soft
// cap of the model head in one kernel.  It takes the place of LogitSoftcapF32 (softmax.go:62-77).
func LogitPostprocessF32(data DeviceBuffer, rows, n int, stride int64, post HeadPost, stream Stream) error {
	if data.ptr == nil {
		return fmt.Errorf("logit postprocess buffer is nil")
	}
	if rows <= 0 || n <= 0 {
		return fmt.Errorf("logit postprocess rows and n must be > 0")
	}
	var flags C.uint32_t
	if post.Tanhf {
		flags = 4
	}
	return cudaErr(C.mantleCudaLogitPostprocessRowsF32Wrapper((*C.float)(data.ptr), C.int(rows), C.int(n),
		C.int64_t(stride), C.float(post.Scale), C.float(post.Softcap), flags, stream.ptr))
}

var _ = unsafe.Pointer(nil)
