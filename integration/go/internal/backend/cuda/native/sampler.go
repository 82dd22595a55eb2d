//go:build cuda

// Package native: cgo binding of the device-side logits sampler (libmantle_cuda_sampler).
//
// This file sits next to argmax.go and follows its conventions: a file-local preamble that
// forward-declares the C symbols, a static wrapper per symbol, Go functions that validate their
// arguments and return cudaErr(code).  Every symbol of mantle_cuda_sampler.h,
// mantle_host_sampler.h and mantle_batch_sampler.h is declared and wrapped here.  It was written
// against the reference tree without a Go toolchain at hand and has not been compiled; the same
// C symbols are exercised from C++ and Python.
//
// Link: add `-lmantle_cuda_sampler` to the #cgo LDFLAGS line of runtime.go (the library is built
// by `python -m mantle_b200.build`; or add sampler_kernels.cu, host_sampler.cu and
// host_batch_sampler.cu to scripts/build_cuda.sh with
// `-gencode arch=compute_100a,code=sm_100a -fmad=false`).
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

typedef struct MantleSamplerConfig {
	int64_t seed;
	float temperature;
	int32_t top_k;
	float top_p, min_p, repeat_penalty;
	int32_t repeat_last_n;
} MantleSamplerConfig;

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
	double* token_prob;
	double* softmax_sum;
	const int32_t* skip;
} MantleSampleBatch;

typedef struct MantleHostSampler MantleHostSampler;
typedef struct MantleBatchSampler MantleBatchSampler;

// mantle_cuda_sampler.h
extern int mantleCudaSamplerAbiVersion(void);
extern int mantleCudaSampleRows(const MantleSampleBatch* b, void* ws, size_t wsBytes, cudaStream_t s);
extern int mantleCudaSamplerWorkspaceBytes(const MantleSampleBatch* b, size_t* bytes);
extern int mantleCudaSamplerSplits(const MantleSampleBatch* b, int* splits);
extern const char* mantleCudaSamplerKernelName(const MantleSampleBatch* b);
extern int mantleCudaRepeatPenaltyRowsF32(const MantleSampleBatch* b, cudaStream_t s);
extern int mantleCudaLogitPostprocessRowsF32(float* x, int rows, int n, int64_t stride, float scale, float softcap,
	uint32_t flags, cudaStream_t s);
extern int mantleCudaHistoryAppendRows(int32_t* history, int32_t* histLen, int histStride, int rows,
	const int32_t* next, int keep, const int32_t* stop, int nStop, int32_t* done, cudaStream_t s);
extern int mantleCudaArgMaxRowsF32(const float* x, int rows, int n, int64_t stride, int* out, cudaStream_t s);
extern int mantleCudaSampleLocalTopK(const MantleSampleBatch* b, int vocabOffset, int vocabTotal, float* partVal,
	int32_t* partIdx, int32_t* partCnt, int partCap, cudaStream_t s);
extern int mantleCudaSampleMergeParts(const MantleSampleBatch* b, int parts, const float* partVal,
	const int32_t* partIdx, const int32_t* partCnt, int partCap, cudaStream_t s);
extern int mantleCudaSamplePackedPartBytes(int rows, int partCap, size_t* bytes);
extern int mantleCudaSampleMergePacked(const MantleSampleBatch* b, int parts, const void* packed, int partCap,
	cudaStream_t s);
extern int mantleCudaSampleRowsHost(const MantleSampleBatch* hb, void* ws, size_t wsBytes, cudaStream_t s);
extern int mantleCudaSamplerHostWorkspaceBytes(const MantleSampleBatch* hb, size_t* bytes);
extern int mantleCudaSampleRowsNoAlloc(const MantleSampleBatch* b, cudaStream_t s);
extern size_t mantleCudaSamplerStaticScratchBytes(void);
extern const char* mantleCudaSamplerLastError(void);
extern int mantleCudaSamplerSelfTestBoundedWait(unsigned long long limitNs, int32_t* status, cudaStream_t s);

// mantle_host_sampler.h
extern MantleHostSampler* mantleSamplerNew(const MantleSamplerConfig* cfg, int maxVocab);
extern void mantleSamplerFree(MantleHostSampler* s);
extern int mantleSamplerParams(const MantleHostSampler* s, MantleSampleParams* out);
extern int mantleSamplerCanUseDeviceGreedy(const MantleHostSampler* s);
extern int mantleSamplerNeedsUniform(const MantleHostSampler* s);
extern int mantleSamplerSample(MantleHostSampler* s, float* logits, int n, const int64_t* recent, int nRecent,
	const int64_t* exclude, int nExclude, double uniform, int* token);
extern int mantleSamplerSampleDevice(MantleHostSampler* s, const float* devLogits, int n, const int64_t* recent,
	int nRecent, const int64_t* exclude, int nExclude, double uniform, cudaStream_t wait, int* token);

// mantle_batch_sampler.h
extern MantleBatchSampler* mantleBatchSamplerNew(int rows, int vocab, int histCapacity, const int64_t* stop, int nStop);
extern void mantleBatchSamplerFree(MantleBatchSampler* s);
extern int mantleBatchSamplerSetRow(MantleBatchSampler* s, int row, const MantleSamplerConfig* cfg,
	const int64_t* context, int nContext, cudaStream_t stream);
extern int mantleBatchSamplerEndRow(MantleBatchSampler* s, int row, cudaStream_t stream);
extern int mantleBatchSamplerNeedsUniform(const MantleBatchSampler* s, int row);
extern int mantleBatchSamplerCanUseDeviceGreedy(const MantleBatchSampler* s, int row);
extern int mantleBatchSamplerStep(MantleBatchSampler* s, const void* devLogits, int dtype, int64_t rowStride,
	const double* uniforms, float logitScale, float logitSoftcap, cudaStream_t stream);
extern int mantleBatchSamplerResults(MantleBatchSampler* s, const int32_t** next, const int32_t** ended,
	int32_t* status, const int32_t** devNext);

// One static wrapper per symbol, as argmax.go has them: cgo calls these.
static int sampleRowsW(const MantleSampleBatch* b, void* ws, size_t n, cudaStream_t s) { return mantleCudaSampleRows(b, ws, n, s); }
static int workspaceBytesW(const MantleSampleBatch* b, size_t* n) { return mantleCudaSamplerWorkspaceBytes(b, n); }
static int splitsW(const MantleSampleBatch* b, int* n) { return mantleCudaSamplerSplits(b, n); }
static int repeatPenaltyW(const MantleSampleBatch* b, cudaStream_t s) { return mantleCudaRepeatPenaltyRowsF32(b, s); }
static int postprocessW(float* x, int rows, int n, int64_t stride, float scale, float softcap, uint32_t flags, cudaStream_t s) {
	return mantleCudaLogitPostprocessRowsF32(x, rows, n, stride, scale, softcap, flags, s);
}
static int historyAppendW(int32_t* h, int32_t* hl, int stride, int rows, const int32_t* next, int keep,
	const int32_t* stop, int nStop, int32_t* done, cudaStream_t s) {
	return mantleCudaHistoryAppendRows(h, hl, stride, rows, next, keep, stop, nStop, done, s);
}
static int argMaxRowsW(const float* x, int rows, int n, int64_t stride, int* out, cudaStream_t s) {
	return mantleCudaArgMaxRowsF32(x, rows, n, stride, out, s);
}
static int localTopKW(const MantleSampleBatch* b, int off, int total, float* v, int32_t* i, int32_t* c, int cap, cudaStream_t s) {
	return mantleCudaSampleLocalTopK(b, off, total, v, i, c, cap, s);
}
static int mergePartsW(const MantleSampleBatch* b, int parts, const float* v, const int32_t* i, const int32_t* c, int cap, cudaStream_t s) {
	return mantleCudaSampleMergeParts(b, parts, v, i, c, cap, s);
}
static int packedPartBytesW(int rows, int cap, size_t* n) { return mantleCudaSamplePackedPartBytes(rows, cap, n); }
static int mergePackedW(const MantleSampleBatch* b, int parts, const void* p, int cap, cudaStream_t s) {
	return mantleCudaSampleMergePacked(b, parts, p, cap, s);
}
static int sampleRowsHostW(const MantleSampleBatch* b, void* ws, size_t n, cudaStream_t s) { return mantleCudaSampleRowsHost(b, ws, n, s); }
static int hostWorkspaceBytesW(const MantleSampleBatch* b, size_t* n) { return mantleCudaSamplerHostWorkspaceBytes(b, n); }
static int sampleRowsNoAllocW(const MantleSampleBatch* b, cudaStream_t s) { return mantleCudaSampleRowsNoAlloc(b, s); }
static int selfTestBoundedWaitW(unsigned long long ns, int32_t* st, cudaStream_t s) { return mantleCudaSamplerSelfTestBoundedWait(ns, st, s); }
static int samplerSampleW(MantleHostSampler* s, float* l, int n, const int64_t* r, int nr, const int64_t* x, int nx, double u, int* t) {
	return mantleSamplerSample(s, l, n, r, nr, x, nx, u, t);
}
static int samplerSampleDeviceW(MantleHostSampler* s, const float* l, int n, const int64_t* r, int nr, const int64_t* x, int nx,
	double u, cudaStream_t w, int* t) {
	return mantleSamplerSampleDevice(s, l, n, r, nr, x, nx, u, w, t);
}
static int batchSetRowW(MantleBatchSampler* s, int row, const MantleSamplerConfig* c, const int64_t* ctx, int n, cudaStream_t st) {
	return mantleBatchSamplerSetRow(s, row, c, ctx, n, st);
}
static int batchStepW(MantleBatchSampler* s, const void* l, int dtype, int64_t stride, const double* u, float scale, float cap, cudaStream_t st) {
	return mantleBatchSamplerStep(s, l, dtype, stride, u, scale, cap, st);
}
static int batchResultsW(MantleBatchSampler* s, const int32_t** next, const int32_t** ended, int32_t* status, const int32_t** devNext) {
	return mantleBatchSamplerResults(s, next, ended, status, devNext);
}
*/
import "C"

import (
	"fmt"
	"unsafe"
)

// SamplerABIVersion is what this binding was written against.
const SamplerABIVersion = 3

// Flags and status bits of mantle_cuda_sampler.h.
const (
	SampleWriteBackPenalty  = 1
	SamplePenaltyPreapplied = 2
	SampleSoftcapTanhf      = 4

	SampleStatusTopKRange = 1
	SampleStatusEmpty     = 2
	SampleStatusTimeout   = 4
	SampleStatusNaN       = 8

	SampleMaxTopK = 1024
)

// CheckSamplerABI fails when the linked library is not the one this file describes.
func CheckSamplerABI() error {
	if v := int(C.mantleCudaSamplerAbiVersion()); v != SamplerABIVersion {
		return fmt.Errorf("mantle_cuda_sampler ABI %d, binding expects %d", v, SamplerABIVersion)
	}
	return nil
}

// SampleParams is one row's normalised sampling parameters (what logits.NewSampler leaves in
// the Sampler, plus the uniform draw of this step).  Layout = MantleSampleParams, 40 bytes.
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

// SamplerConfig is logits.SamplerConfig field for field (MantleSamplerConfig).
type SamplerConfig struct {
	Seed          int64
	Temperature   float32
	TopK          int32
	TopP          float32
	MinP          float32
	RepeatPenalty float32
	RepeatLastN   int32
}

func (c SamplerConfig) c() C.MantleSamplerConfig {
	return C.MantleSamplerConfig{
		seed: C.int64_t(c.Seed), temperature: C.float(c.Temperature), top_k: C.int32_t(c.TopK),
		top_p: C.float(c.TopP), min_p: C.float(c.MinP), repeat_penalty: C.float(c.RepeatPenalty),
		repeat_last_n: C.int32_t(c.RepeatLastN),
	}
}

// HeadPost is what the model head does to the logits before sampling (LMHeadMultiplier and
// FinalLogitSoftcap, simd/runtime.go:258-272).  The zero value means neither.
type HeadPost struct {
	Scale   float32 // applied when neither 0 nor 1
	Softcap float32 // applied when > 0
	Tanhf   bool    // tanhf as mantleCudaLogitSoftcapF32 has it, instead of the host path's fastTanh
}

func (p HeadPost) flags() C.uint32_t {
	if p.Tanhf {
		return SampleSoftcapTanhf
	}
	return 0
}

// SampleBatch describes one batch of rows; every DeviceBuffer is on the current device.  The zero
// DeviceBuffer stands for "not given" wherever mantle_cuda_sampler.h allows NULL.
type SampleBatch struct {
	Logits      DeviceBuffer // [Rows][RowStride] float32 (BF16: bfloat16)
	BF16        bool
	Rows, Vocab int
	RowStride   int64
	MaxTopK     int
	History     DeviceBuffer // [Rows][HistStride] int32, oldest first
	HistLen     DeviceBuffer // [Rows] int32 valid ids per row; zero: HistStride for every row
	HistStride  int
	Exclude     DeviceBuffer // NExclude int32 ids never penalised (the stop tokens)
	NExclude    int
	Params      DeviceBuffer // [Rows] SampleParams
	Next        DeviceBuffer // out [Rows] int32
	CandIdx     DeviceBuffer // optional out [Rows][CandStride] int32
	CandProb    DeviceBuffer // optional out [Rows][CandStride] float64
	CandStride  int
	NKept, Cut  DeviceBuffer // optional out [Rows] int32
	Status      DeviceBuffer // optional out: one int32 of status bits
	TokenProb   DeviceBuffer // optional out [Rows] float64
	SoftmaxSum  DeviceBuffer // optional out [Rows] float64
	Skip        DeviceBuffer // optional [Rows] int32: rows that are not sampled
	Splits      int          // CTAs per row; 0: the library's choice
	Flags       uint32
	Post        HeadPost
}

func (b *SampleBatch) c() (C.MantleSampleBatch, error) {
	var cb C.MantleSampleBatch
	if b.Logits.ptr == nil || b.Params.ptr == nil || b.Next.ptr == nil {
		return cb, fmt.Errorf("sample buffer is nil")
	}
	if b.Rows <= 0 || b.Vocab <= 0 {
		return cb, fmt.Errorf("sample rows and vocab must be > 0")
	}
	cb.logits = b.Logits.ptr
	if b.BF16 {
		cb.dtype = 1
	}
	cb.rows = C.int32_t(b.Rows)
	cb.vocab = C.int32_t(b.Vocab)
	cb.max_top_k = C.int32_t(b.MaxTopK)
	cb.row_stride = C.int64_t(b.RowStride)
	cb.history = (*C.int32_t)(b.History.ptr)
	cb.hist_len = (*C.int32_t)(b.HistLen.ptr)
	cb.hist_stride = C.int32_t(b.HistStride)
	cb.exclude = (*C.int32_t)(b.Exclude.ptr)
	cb.n_exclude = C.int32_t(b.NExclude)
	cb.params = (*C.MantleSampleParams)(b.Params.ptr)
	cb.next = (*C.int32_t)(b.Next.ptr)
	cb.cand_idx = (*C.int32_t)(b.CandIdx.ptr)
	cb.cand_prob = (*C.double)(b.CandProb.ptr)
	cb.cand_stride = C.int32_t(b.CandStride)
	cb.n_kept = (*C.int32_t)(b.NKept.ptr)
	cb.cut = (*C.int32_t)(b.Cut.ptr)
	cb.status = (*C.int32_t)(b.Status.ptr)
	cb.token_prob = (*C.double)(b.TokenProb.ptr)
	cb.softmax_sum = (*C.double)(b.SoftmaxSum.ptr)
	cb.skip = (*C.int32_t)(b.Skip.ptr)
	cb.splits = C.int32_t(b.Splits)
	cb.flags = C.uint32_t(b.Flags) | b.Post.flags()
	cb.logit_scale = C.float(b.Post.Scale)
	cb.logit_softcap = C.float(b.Post.Softcap)
	return cb, nil
}

// SampleRows is Sampler.Sample for every row of a device-resident batch.  workspace may be the
// zero DeviceBuffer when SamplerWorkspaceBytes reports 0.  Queued on stream; no synchronisation.
func SampleRows(b *SampleBatch, workspace DeviceBuffer, stream Stream) error {
	cb, err := b.c()
	if err != nil {
		return err
	}
	return cudaErr(C.sampleRowsW(&cb, workspace.ptr, C.size_t(workspace.nbytes), stream.ptr))
}

// SamplerWorkspaceBytes is what SampleRows needs for this batch (0 when rows are not split).
func SamplerWorkspaceBytes(b *SampleBatch) (int64, error) {
	cb, err := b.c()
	if err != nil {
		return 0, err
	}
	var n C.size_t
	if err := cudaErr(C.workspaceBytesW(&cb, &n)); err != nil {
		return 0, err
	}
	return int64(n), nil
}

// SamplerSplits is the number of CTAs per row SampleRows will use.
func SamplerSplits(b *SampleBatch) (int, error) {
	cb, err := b.c()
	if err != nil {
		return 0, err
	}
	var n C.int
	if err := cudaErr(C.splitsW(&cb, &n)); err != nil {
		return 0, err
	}
	return int(n), nil
}

// SamplerKernelName names the kernel that reads this batch's logits (for trace output).
func SamplerKernelName(b *SampleBatch) string {
	cb, err := b.c()
	if err != nil {
		return ""
	}
	return C.GoString(C.mantleCudaSamplerKernelName(&cb))
}

// SampleRowsNoAlloc is SampleRows with the split-row scratch taken from the library's fixed
// device array; refusals carry the library's message.
func SampleRowsNoAlloc(b *SampleBatch, stream Stream) error {
	cb, err := b.c()
	if err != nil {
		return err
	}
	if code := C.sampleRowsNoAllocW(&cb, stream.ptr); code != 0 {
		if msg := C.GoString(C.mantleCudaSamplerLastError()); msg != "" {
			return fmt.Errorf("%w: %s", cudaErr(code), msg)
		}
		return cudaErr(code)
	}
	return nil
}

// SamplerStaticScratchBytes is the size of the array behind SampleRowsNoAlloc.
func SamplerStaticScratchBytes() int64 { return int64(C.mantleCudaSamplerStaticScratchBytes()) }

// SamplerLastError is the text of the last refusal or status report on this OS thread.
func SamplerLastError() string { return C.GoString(C.mantleCudaSamplerLastError()) }

// RepeatPenaltyRowsF32 applies the repeat penalty alone, in place (sampler.go:99-138).
func RepeatPenaltyRowsF32(b *SampleBatch, stream Stream) error {
	cb, err := b.c()
	if err != nil {
		return err
	}
	return cudaErr(C.repeatPenaltyW(&cb, stream.ptr))
}

// SampleRowsHost is SampleRows for a batch in pinned host memory: every pointer of hb is a host
// pointer (wrapped as DeviceBuffer only for its ptr field); copies in, kernels and copies out are
// queued on stream and the caller synchronises it.
func SampleRowsHost(hb *SampleBatch, workspace DeviceBuffer, stream Stream) error {
	cb, err := hb.c()
	if err != nil {
		return err
	}
	return cudaErr(C.sampleRowsHostW(&cb, workspace.ptr, C.size_t(workspace.nbytes), stream.ptr))
}

// SamplerHostWorkspaceBytes is the device workspace SampleRowsHost needs.
func SamplerHostWorkspaceBytes(hb *SampleBatch) (int64, error) {
	cb, err := hb.c()
	if err != nil {
		return 0, err
	}
	var n C.size_t
	if err := cudaErr(C.hostWorkspaceBytesW(&cb, &n)); err != nil {
		return 0, err
	}
	return int64(n), nil
}

// ArgMaxRowsF32To is the batched, lowest-index replacement of ArgMaxF32To.
func ArgMaxRowsF32To(x DeviceBuffer, rows, n int, stride int64, outIdx DeviceBuffer, stream Stream) error {
	if x.ptr == nil || outIdx.ptr == nil {
		return fmt.Errorf("argmax buffer is nil")
	}
	if rows <= 0 || n <= 0 {
		return fmt.Errorf("argmax rows and n must be > 0")
	}
	return cudaErr(C.argMaxRowsW((*C.float)(x.ptr), C.int(rows), C.int(n), C.int64_t(stride), (*C.int)(outIdx.ptr), stream.ptr))
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
	return cudaErr(C.postprocessW((*C.float)(data.ptr), C.int(rows), C.int(n), C.int64_t(stride), C.float(post.Scale),
		C.float(post.Softcap), post.flags(), stream.ptr))
}

// HistoryAppendRows is `toks = append(toks, next)` (engine.go:244-250) for device-resident
// histories; stop and done may be zero buffers.
func HistoryAppendRows(history, histLen DeviceBuffer, histStride, rows int, next DeviceBuffer, keep int,
	stop DeviceBuffer, nStop int, done DeviceBuffer, stream Stream) error {
	if history.ptr == nil || histLen.ptr == nil || next.ptr == nil {
		return fmt.Errorf("history buffer is nil")
	}
	return cudaErr(C.historyAppendW((*C.int32_t)(history.ptr), (*C.int32_t)(histLen.ptr), C.int(histStride), C.int(rows),
		(*C.int32_t)(next.ptr), C.int(keep), (*C.int32_t)(stop.ptr), C.int(nStop), (*C.int32_t)(done.ptr), stream.ptr))
}

// SampleLocalTopK is step 1 of vocabulary-sharded sampling: this GPU's shortlist with global ids.
func SampleLocalTopK(b *SampleBatch, vocabOffset, vocabTotal int, partVal, partIdx, partCnt DeviceBuffer, partCap int,
	stream Stream) error {
	cb, err := b.cParts()
	if err != nil {
		return err
	}
	return cudaErr(C.localTopKW(&cb, C.int(vocabOffset), C.int(vocabTotal), (*C.float)(partVal.ptr),
		(*C.int32_t)(partIdx.ptr), (*C.int32_t)(partCnt.ptr), C.int(partCap), stream.ptr))
}

// cParts is c() for the shortlist step, which needs no Next.
func (b *SampleBatch) cParts() (C.MantleSampleBatch, error) {
	saved := b.Next
	if b.Next.ptr == nil {
		b.Next = b.Params // any non-nil pointer passes the check; the shortlist step never writes next
	}
	cb, err := b.c()
	b.Next = saved
	cb.next = (*C.int32_t)(saved.ptr)
	return cb, err
}

// SampleMergeParts is step 2 after the caller's all-gather: merge `parts` shortlists per row.
func SampleMergeParts(b *SampleBatch, parts int, partVal, partIdx, partCnt DeviceBuffer, partCap int, stream Stream) error {
	cb, err := b.cMerge()
	if err != nil {
		return err
	}
	return cudaErr(C.mergePartsW(&cb, C.int(parts), (*C.float)(partVal.ptr), (*C.int32_t)(partIdx.ptr),
		(*C.int32_t)(partCnt.ptr), C.int(partCap), stream.ptr))
}

// SamplePackedPartBytes is the size of one rank's packed block of shortlists.
func SamplePackedPartBytes(rows, partCap int) (int64, error) {
	var n C.size_t
	if err := cudaErr(C.packedPartBytesW(C.int(rows), C.int(partCap), &n)); err != nil {
		return 0, err
	}
	return int64(n), nil
}

// SampleMergePacked merges `parts` packed blocks (what one all-gather delivered).
func SampleMergePacked(b *SampleBatch, parts int, packed DeviceBuffer, partCap int, stream Stream) error {
	cb, err := b.cMerge()
	if err != nil {
		return err
	}
	return cudaErr(C.mergePackedW(&cb, C.int(parts), packed.ptr, C.int(partCap), stream.ptr))
}

// cMerge is c() for the merge steps, which read no logits.
func (b *SampleBatch) cMerge() (C.MantleSampleBatch, error) {
	saved := b.Logits
	if b.Logits.ptr == nil {
		b.Logits = b.Params
	}
	cb, err := b.c()
	b.Logits = saved
	cb.logits = saved.ptr
	return cb, err
}

// SamplerSelfTestBoundedWait runs the library's bounded wait on a barrier nothing completes; the
// kernel must return with SampleStatusTimeout in *status after limitNs.
func SamplerSelfTestBoundedWait(limitNs uint64, status DeviceBuffer, stream Stream) error {
	return cudaErr(C.selfTestBoundedWaitW(C.ulonglong(limitNs), (*C.int32_t)(status.ptr), stream.ptr))
}

// ---------------------------------------------------------------------------------------------
// mantle_host_sampler.h: the C++ mirror of logits.Sampler for one request.

// HostSampler wraps MantleHostSampler.
type HostSampler struct{ p *C.MantleHostSampler }

// NewHostSampler is logits.NewSampler for logits of at most maxVocab columns.
func NewHostSampler(cfg SamplerConfig, maxVocab int) (*HostSampler, error) {
	c := cfg.c()
	p := C.mantleSamplerNew(&c, C.int(maxVocab))
	if p == nil {
		return nil, fmt.Errorf("mantleSamplerNew failed")
	}
	return &HostSampler{p: p}, nil
}

func (s *HostSampler) Free() {
	if s != nil && s.p != nil {
		C.mantleSamplerFree(s.p)
		s.p = nil
	}
}

// Params is the configuration after NewSampler's normalisation.
func (s *HostSampler) Params() (SampleParams, error) {
	var out SampleParams
	err := cudaErr(C.mantleSamplerParams(s.p, (*C.MantleSampleParams)(unsafe.Pointer(&out))))
	return out, err
}

func (s *HostSampler) CanUseDeviceGreedy() bool { return C.mantleSamplerCanUseDeviceGreedy(s.p) != 0 }

// NeedsUniform: the next Sample consumes a draw (the caller calls rng.Float64() exactly then).
func (s *HostSampler) NeedsUniform() bool { return C.mantleSamplerNeedsUniform(s.p) != 0 }

func int64s(ids []int) (*C.int64_t, C.int) {
	if len(ids) == 0 {
		return nil, 0
	}
	return (*C.int64_t)(unsafe.Pointer(&ids[0])), C.int(len(ids)) // Go int is 64-bit on the supported targets
}

// Sample is Sampler.Sample on a host slice, patched in place by the penalty like the reference's.
func (s *HostSampler) Sample(logits []float32, recent, exclude []int, uniform float64) (int, error) {
	if len(logits) == 0 {
		return 0, fmt.Errorf("argmax: empty slice")
	}
	r, nr := int64s(recent)
	x, nx := int64s(exclude)
	var tok C.int
	code := C.samplerSampleW(s.p, (*C.float)(unsafe.Pointer(&logits[0])), C.int(len(logits)), r, nr, x, nx,
		C.double(uniform), &tok)
	return int(tok), samplerErr(code)
}

// SampleDevice is the same on device-resident float32 logits, which stay untouched.
func (s *HostSampler) SampleDevice(logits DeviceBuffer, n int, recent, exclude []int, uniform float64, wait Stream) (int, error) {
	if logits.ptr == nil || n <= 0 {
		return 0, fmt.Errorf("sample device buffer is nil or empty")
	}
	r, nr := int64s(recent)
	x, nx := int64s(exclude)
	var tok C.int
	code := C.samplerSampleDeviceW(s.p, (*C.float)(logits.ptr), C.int(n), r, nr, x, nx, C.double(uniform), wait.ptr, &tok)
	return int(tok), samplerErr(code)
}

// samplerErr adds the library's own words to a status failure (the reference's engine reports
// "panic in Sample: ..." there, engine.go:339-346).
func samplerErr(code C.int) error {
	err := cudaErr(code)
	if err == nil {
		return nil
	}
	if msg := C.GoString(C.mantleCudaSamplerLastError()); msg != "" {
		return fmt.Errorf("%w: %s", err, msg)
	}
	return err
}

// ---------------------------------------------------------------------------------------------
// mantle_batch_sampler.h: the decode loop's sampling state for a batch of requests.

// BatchSampler wraps MantleBatchSampler.
type BatchSampler struct {
	p    *C.MantleBatchSampler
	rows int
}

func NewBatchSampler(rows, vocab, histCapacity int, stop []int) (*BatchSampler, error) {
	sp, ns := int64s(stop)
	p := C.mantleBatchSamplerNew(C.int(rows), C.int(vocab), C.int(histCapacity), sp, ns)
	if p == nil {
		return nil, fmt.Errorf("mantleBatchSamplerNew failed")
	}
	return &BatchSampler{p: p, rows: rows}, nil
}

func (s *BatchSampler) Free() {
	if s != nil && s.p != nil {
		C.mantleBatchSamplerFree(s.p)
		s.p = nil
	}
}

// SetRow starts request `row`: NewSampler(cfg) and toks := copy(context).
func (s *BatchSampler) SetRow(row int, cfg SamplerConfig, context []int, stream Stream) error {
	c := cfg.c()
	cp, n := int64s(context)
	return samplerErr(C.batchSetRowW(s.p, C.int(row), &c, cp, n, stream.ptr))
}

func (s *BatchSampler) EndRow(row int, stream Stream) error {
	return cudaErr(C.mantleBatchSamplerEndRow(s.p, C.int(row), stream.ptr))
}

func (s *BatchSampler) NeedsUniform(row int) bool { return C.mantleBatchSamplerNeedsUniform(s.p, C.int(row)) != 0 }

func (s *BatchSampler) CanUseDeviceGreedy(row int) bool {
	return C.mantleBatchSamplerCanUseDeviceGreedy(s.p, C.int(row)) != 0
}

// Step queues one step for every live row; uniforms holds one draw per row.
func (s *BatchSampler) Step(logits DeviceBuffer, bf16 bool, rowStride int64, uniforms []float64, post HeadPost, stream Stream) error {
	if logits.ptr == nil || len(uniforms) != s.rows {
		return fmt.Errorf("batch sampler step: nil logits or %d uniforms for %d rows", len(uniforms), s.rows)
	}
	dtype := C.int(0)
	if bf16 {
		dtype = 1
	}
	return cudaErr(C.batchStepW(s.p, logits.ptr, dtype, C.int64_t(rowStride), (*C.double)(unsafe.Pointer(&uniforms[0])),
		C.float(post.Scale), C.float(post.Softcap), stream.ptr))
}

// Results returns the last step's tokens and "has ended" flags (views of pinned memory owned by
// the sampler, valid until the next Step), the status word, and the device copy of the tokens.
func (s *BatchSampler) Results() (next, ended []int32, status int32, devNext DeviceBuffer, err error) {
	var np, ep, dp *C.int32_t
	var st C.int32_t
	if err = cudaErr(C.batchResultsW(s.p, &np, &ep, &st, &dp)); err != nil {
		return
	}
	next = unsafe.Slice((*int32)(unsafe.Pointer(np)), s.rows)
	ended = unsafe.Slice((*int32)(unsafe.Pointer(ep)), s.rows)
	devNext = DeviceBuffer{ptr: unsafe.Pointer(dp), nbytes: int64(s.rows) * 4}
	return next, ended, int32(st), devNext, nil
}
