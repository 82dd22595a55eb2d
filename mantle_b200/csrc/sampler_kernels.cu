// Device-side logits sampler for sm_100a: the per-row work of Sampler.Sample
// (internal/logits/sampler.go:98-234) for a whole batch of rows.
//
// One CTA (or `splits` CTAs) streams one row of logits from HBM exactly once, 16 bytes
// per thread per load, keeps every element that can still reach the top-k shortlist in a
// shared-memory candidate buffer, cuts that buffer to exactly k entries with a
// shared-memory radix select, orders the k survivors, and runs the reference's tail
// (fastExp softmax in float32 with double sums, min-p, top-p cut, inverse-CDF draw) on
// them.  The repeat penalty is folded into the same pass through a V-bit bitmap of the
// de-duplicated history window in shared memory, so the logits stay read-only unless the
// caller asks for the reference's in-place side effect.
//
// Nothing here is a dense contraction, so no tensor-core instruction is used; the bound
// is HBM bandwidth and the design goal is one read of every logit and nothing else.
//
// Ordering contract (sampler.go:255-296): the shortlist is ordered by scaled value
// descending, ties by ascending index, and an equal value arriving later never displaces
// an earlier one.  With value keys that map -0.0 and +0.0 to the same key this is the
// total order (key descending, index ascending), which makes every selection below exact.
//
// Arithmetic contract: every float32 and float64 operation the reference performs is
// issued as a round-to-nearest intrinsic so nothing is contracted into an FMA.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <mutex>

#include "../../include/mantle_cuda_sampler.h"
#include "sampler_internal.h"

// Development aid, compiled out of the shipped library: with -DMANTLE_DEBUG_SWITCHES the
// environment variable MANTLE_SAMPLER_DEBUG switches pieces of the kernel off to cost them.
#ifdef MANTLE_DEBUG_SWITCHES
#define DEBUG_OFF(a, bit) (((a).debug >> (bit)) & 1)
#else
#define DEBUG_OFF(a, bit) 0
#endif

#include "sampler_common.cuh"
#include "sampler_select.cuh"
#include "sampler_tail.cuh"
#include "sampler_async.cuh"
#include "sampler_rows.cuh"
#include "scan_rows_ldg.cuh"
#include "scan_rows_hist.cuh"
#include "wide_rows.cuh"
#include "wide_rows_fast.cuh"
#include "merge_parts.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// host side

constexpr int kInvalid = (int)cudaErrorInvalidValue;

// The model head's post-processing as the reference gates it (simd/runtime.go:258,264): the
// multiplier when it is neither 0 nor 1, the soft cap when it is positive.  A negative or
// non-finite multiplier and an infinite cap are refused.
bool post_ok(float scale, float cap) {
    if (!(scale == scale) || std::isinf(scale) || scale < 0.0f) return false;
    if (std::isinf(cap)) return false;
    return true;
}
int post_mode_of(float scale, float cap, uint32_t flags) {
    int m = 0;
    if (scale != 0.0f && scale != 1.0f) m |= POST_SCALE;
    if (cap > 0.0f) m |= POST_CAP | ((flags & MANTLE_SAMPLE_SOFTCAP_TANHF) ? POST_TANHF : 0);
    return m;
}

bool batch_ok(const MantleSampleBatch* b, bool need_outputs) {
    if (!b || !b->logits || b->rows <= 0 || b->vocab <= 0) return false;
    if (b->vocab > MANTLE_SAMPLE_MAX_VOCAB) return false;
    if (b->dtype != MANTLE_DTYPE_F32 && b->dtype != MANTLE_DTYPE_BF16) return false;
    if (b->row_stride < b->vocab) return false;
    if (b->hist_stride < 0 || b->n_exclude < 0) return false;
    if (b->n_exclude > 0 && !b->exclude) return false;
    if (b->splits < 0 || b->reserved != 0) return false;
    if (b->flags & ~(MANTLE_SAMPLE_WRITE_BACK_PENALTY | MANTLE_SAMPLE_PENALTY_PREAPPLIED | MANTLE_SAMPLE_SOFTCAP_TANHF))
        return false;
    if (!post_ok(b->logit_scale, b->logit_softcap)) return false;
    // the fused post-processing leaves the logits as they are: nothing to write back, nothing pre-applied
    if (post_mode_of(b->logit_scale, b->logit_softcap, b->flags) &&
        (b->flags & (MANTLE_SAMPLE_WRITE_BACK_PENALTY | MANTLE_SAMPLE_PENALTY_PREAPPLIED)))
        return false;
    if ((b->flags & MANTLE_SAMPLE_WRITE_BACK_PENALTY) && b->dtype != MANTLE_DTYPE_F32) return false;
    const size_t esz = b->dtype == MANTLE_DTYPE_F32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(b->logits) % esz) return false;
    if (b->params && reinterpret_cast<uintptr_t>(b->params) % 8) return false;
    if (need_outputs) {
        if (!b->params || !b->next) return false;
        if (b->max_top_k < 1 || b->max_top_k > MANTLE_SAMPLE_MAX_VOCAB) return false;
        if (b->max_top_k > KMAX && (b->cand_idx || b->cand_prob)) return false;  // long shortlists are never materialised
        if ((b->cand_idx || b->cand_prob) && b->cand_stride <= 0) return false;
    }
    return true;
}

// What the library asks a device once and then remembers: the driver calls behind these
// figures cost microseconds, which shows on a single-row launch of under twenty.
constexpr int kMaxDevices = 64;
struct DeviceInfo {
    int per_sm;     // shared memory of one SM
    int per_block;  // largest opt-in dynamic shared memory of one CTA
    int sms;
};
DeviceInfo g_device_info[kMaxDevices];
std::atomic<int> g_device_known[kMaxDevices];
std::mutex g_device_mutex;

// Current device ordinal and its figures.  Without a usable device (argument checks run on
// hosts that have none) the B200's own figures stand in and the ordinal is -1.
DeviceInfo device_info(int* dev_out = nullptr) {
    const DeviceInfo b200 = {233472, 232448, 148};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        if (dev_out) *dev_out = -1;
        return b200;
    }
    if (dev_out) *dev_out = dev;
    if (g_device_known[dev].load(std::memory_order_acquire)) return g_device_info[dev];
    std::lock_guard<std::mutex> lock(g_device_mutex);
    DeviceInfo d = b200;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess && v > 0) d.per_sm = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess && v > 0) d.per_block = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) d.sms = v;
    g_device_info[dev] = d;
    g_device_known[dev].store(1, std::memory_order_release);
    return d;
}

// Raises a kernel's dynamic shared-memory limit on the current device when `smem` exceeds what
// an earlier launch already asked for; `granted` is the kernel's own per-device record.
template <class K>
int ensure_smem(K kern, size_t smem, std::atomic<int>* granted) {
    int dev = -1;
    (void)device_info(&dev);
    if (dev >= 0 && (size_t)granted[dev].load(std::memory_order_relaxed) >= smem) return 0;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0) granted[dev].store((int)smem, std::memory_order_relaxed);
    return 0;
}

// (from 225 entries on the seed of the small shape -- one value per thread -- admits a third of region 0)
bool small_shape(int max_top_k) { return max_top_k <= 224; }

int choose_splits(const MantleSampleBatch* b) {
    if (b->max_top_k > KMAX) return 1;  // long shortlists: one CTA per row, no merge
    const int vec = b->dtype == MANTLE_DTYPE_F32 ? 4 : 8;
    const int nvec = (b->vocab + vec - 1) / vec + 1;
    const bool small = small_shape(b->max_top_k);
    const int region = small ? ShapeK256::NT * ShapeK256::U : ShapeK1024::NT * ShapeK1024::U;
    const int per_sm = small ? ShapeK256::MINB : ShapeK1024::MINB;
    const int max_by_k = MERGE_CAP / b->max_top_k;  // the merge holds splits * k candidates
    if (b->splits > 0) return std::max(1, std::min(std::min(b->splits, max_by_k), std::min(nvec, 64)));
    // at least one full region per CTA (measured on one 151 936-column row: 9 CTAs 21.8 us, 18 19.0 us,
    // 37 17.7 us, 64 18.7 us)
    const int max_by_work = nvec / region;
    const int cap = std::max(1, std::min(std::min(max_by_k, max_by_work), 64));
    const int target = per_sm * device_info().sms;  // one full wave
    if (b->rows >= target) return 1;
    return std::max(1, std::min(cap, target / b->rows));  // rounded down: all the CTAs in one wave
}

void fill_args(KArgs& a, const MantleSampleBatch* b) {
    a.logits = b->logits;
    a.row_stride = b->row_stride;
    a.rows = b->rows;
    a.vocab = b->vocab;
    a.vocab_offset = 0;
    a.vocab_total = b->vocab;
    a.history = b->hist_stride > 0 ? b->history : nullptr;
    a.hist_len = b->hist_len;
    a.hist_stride = b->hist_stride;
    a.n_exclude = b->n_exclude;
    a.exclude = b->exclude;
    a.params = b->params;
    a.splits = 1;
    a.max_top_k = b->max_top_k;
    a.flags = b->flags;
    a.next = b->next;
    a.cand_idx = b->cand_idx;
    a.cand_prob = b->cand_prob;
    a.n_kept = b->n_kept;
    a.cut = b->cut;
    a.status = b->status;
    a.token_prob = b->token_prob;
    a.softmax_sum = b->softmax_sum;
    a.skip = b->skip;
    a.cand_stride = b->cand_stride;
    a.part_val = nullptr;
    a.part_idx = nullptr;
    a.part_cnt = nullptr;
    a.part_cap = 0;
    a.part_stride = 0;
    a.cnt_stride = 0;
    a.parts = 0;
    a.post.mode = post_mode_of(b->logit_scale, b->logit_softcap, b->flags);
    a.post.scale = b->logit_scale;
    a.post.cap = b->logit_softcap;
#ifdef MANTLE_DEBUG_SWITCHES
    const char* dbg = getenv("MANTLE_SAMPLER_DEBUG");
    a.debug = dbg ? atoi(dbg) : 0;
#endif
}

// CUT: the kernel that cuts its buffer exactly (short shortlists); else the one with the running histogram.
template <class S, typename T, int MODE, bool POST, bool CUT>
int launch_scan_as(const KArgs& a, cudaStream_t stream) {
    static std::atomic<int> granted[kMaxDevices];
    const size_t smem = S::SMEM_FIXED + bitmap_words(a.vocab) * sizeof(uint32_t);
    const long long items = (long long)a.rows * a.splits;
    if (items > 0x7fffffffLL) return kInvalid;
    void (*kern)(const KArgs);
    if constexpr (CUT) kern = scan_rows_ldg_kernel<S, T, MODE, POST>;
    else kern = scan_rows_hist_kernel<S, T, MODE, POST>;
    const int rc = ensure_smem(kern, smem, granted);
    if (rc) return rc;
    kern<<<(int)items, S::NT, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

template <class S, int MODE, bool CUT>
int launch_scan_shape(const KArgs& a, int dtype, cudaStream_t stream) {
    if (a.post.mode)
        return dtype == MANTLE_DTYPE_F32 ? launch_scan_as<S, float, MODE, true, CUT>(a, stream)
                                         : launch_scan_as<S, bf16_t, MODE, true, CUT>(a, stream);
    return dtype == MANTLE_DTYPE_F32 ? launch_scan_as<S, float, MODE, false, CUT>(a, stream)
                                     : launch_scan_as<S, bf16_t, MODE, false, CUT>(a, stream);
}

// The streaming kernel, and its shape, that serve the batch's longest shortlist: exact cuts for short
// shortlists, the running histogram for everything else.  With the head's post-processing a survivor's exact
// value is a few hundred instructions, and the histogram kernel computes them 32 at a time: it then wins at
// every shortlist length (top_k 20: 0.492 against 0.544 ms).  (Short items -- split rows, narrow vocabulary
// shards -- used to take the cut kernel at any length; measured again with the histogram kernel as it is now,
// 1024 rows of 32 768 columns at top_k 50 take 60 against 78 us, 64 rows of 16 882 at top_k 200 31 against 38.)
// Items of about one region (a single row split over the whole GPU) are over before the histogram has paid for
// its set-up: they keep the exact cuts at every shortlist length the small shape serves (one row at top_k 40: 19.1
// against 20.8 us; from two regions per item on the histogram kernel is ahead: 16 mixed rows 45.3 against 47.2 us).
bool cut_kernel(const KArgs& a, int dtype) {
    if (a.post.mode != 0) return false;
    if (a.max_top_k <= CUT_KMAX) return true;
    const int per_region = ShapeK256::NT * ShapeK256::U * (dtype == MANTLE_DTYPE_F32 ? 4 : 8);
    return a.max_top_k <= ShapeK256::KCAP && a.vocab / a.splits <= per_region * 3 / 2;
}

template <int MODE>
int launch_scan(const KArgs& a, int dtype, cudaStream_t stream) {
    if (cut_kernel(a, dtype)) return launch_scan_shape<ShapeK256, MODE, true>(a, dtype, stream);
    if (small_shape(a.max_top_k)) return launch_scan_shape<ShapeK256, MODE, false>(a, dtype, stream);
    return launch_scan_shape<ShapeK1024, MODE, false>(a, dtype, stream);
}

// `dependent`: the merge directly follows, on the same stream, the kernel that writes its parts;
// it is then launched programmatically dependent on that kernel, so that its start-up overlaps
// the other's end (the merge waits with griddepcontrol.wait before it reads a part).
template <class S>
int launch_merge_as(const KArgs& a, cudaStream_t stream, bool dependent) {
    static std::atomic<int> granted[kMaxDevices];
    const size_t smem = S::SMEM_FIXED;
    const int rc = ensure_smem(merge_parts_kernel<S>, smem, granted);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.rows);
    cfg.blockDim = dim3((unsigned)S::NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, merge_parts_kernel<S>, a);
}

int launch_merge(KArgs& a, cudaStream_t stream, bool dependent = false) {
    if (a.part_stride == 0) a.part_stride = (long long)a.rows * a.part_cap;
    if (a.cnt_stride == 0) a.cnt_stride = a.rows;
    const long long held = (long long)a.parts * std::min(a.part_cap, a.max_top_k);
    if (a.max_top_k <= ShapeK256::KCAP && held <= ShapeK256::CAP / 2)
        return launch_merge_as<ShapeK256>(a, stream, dependent);
    return launch_merge_as<ShapeMerge>(a, stream, dependent);
}

// Long shortlists: wide_hist_kernel settles the rows, wide_rows_kernel behind it takes the few it
// marks as unsettled (and returns at once for all others).
template <typename T>
int launch_wide_as(const KArgs& a, cudaStream_t stream) {
    static std::atomic<int> granted[2][kMaxDevices];
    const size_t bitmap = bitmap_words(a.vocab) * sizeof(uint32_t);
    const size_t smem_hist = WF_CTL_BYTES + 2 * (size_t)WF_BINS * (8 + 4) + (size_t)WF_BINS * 4 + (size_t)WF_CAND * 8 + bitmap;
    const size_t smem_rows = ((sizeof(WideCtl) + 127) / 128) * 128 + bitmap;
    int rc = ensure_smem(wide_hist_kernel<T>, smem_hist, granted[0]);
    if (rc) return rc;
    rc = ensure_smem(wide_rows_kernel<T>, smem_rows, granted[1]);
    if (rc) return rc;
    wide_hist_kernel<T><<<a.rows, WF_NT, smem_hist, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    wide_rows_kernel<T><<<a.rows, WIDE_NT, smem_rows, stream>>>(a);
    return (int)cudaGetLastError();
}

int launch_wide(const KArgs& a, int dtype, cudaStream_t stream) {
    return dtype == MANTLE_DTYPE_F32 ? launch_wide_as<float>(a, stream) : launch_wide_as<bf16_t>(a, stream);
}

int launch_penalty(const KArgs& a, cudaStream_t stream) {
    static std::atomic<int> granted[kMaxDevices];
    const size_t smem = bitmap_words(a.vocab) * sizeof(uint32_t);
    const int rc = ensure_smem(penalty_rows_kernel, smem, granted);
    if (rc) return rc;
    penalty_rows_kernel<<<a.rows, PENALTY_NT, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

// The reference's in-place side effect: rewrite the logits first, then sample them as they are.
int apply_write_back(KArgs& a, cudaStream_t stream) {
    if (!(a.flags & MANTLE_SAMPLE_WRITE_BACK_PENALTY)) return 0;
    int rc = 0;
    if (a.history && !(a.flags & MANTLE_SAMPLE_PENALTY_PREAPPLIED)) rc = launch_penalty(a, stream);
    a.flags |= MANTLE_SAMPLE_PENALTY_PREAPPLIED;
    return rc;
}

size_t parts_bytes(int rows, int parts, int cap) {
    size_t n = (size_t)rows * parts;
    size_t bytes = n * cap * (sizeof(float) + sizeof(int32_t)) + n * sizeof(int32_t);
    return (bytes + 255) & ~(size_t)255;
}

}  // namespace

extern "C" int mantleCudaSamplerAbiVersion(void) { return 3; }

extern "C" int mantleCudaSamplerSplits(const MantleSampleBatch* batch, int* splits) {
    if (!splits || !batch_ok(batch, true)) return kInvalid;
    *splits = choose_splits(batch);
    return 0;
}

extern "C" const char* mantleCudaSamplerKernelName(const MantleSampleBatch* batch) {
    if (!batch_ok(batch, true)) return "";
    if (batch->max_top_k > KMAX) return "wide_hist_kernel";
    KArgs a;
    fill_args(a, batch);
    a.splits = choose_splits(batch);
    return cut_kernel(a, batch->dtype) ? "scan_rows_ldg_kernel" : "scan_rows_hist_kernel";
}

extern "C" int mantleCudaSamplerWorkspaceBytes(const MantleSampleBatch* batch, size_t* bytes) {
    if (!bytes || !batch_ok(batch, true)) return kInvalid;
    const int s = choose_splits(batch);
    *bytes = s > 1 ? parts_bytes(batch->rows, s, batch->max_top_k) : 0;
    return 0;
}

extern "C" int mantleCudaSampleRows(const MantleSampleBatch* batch, void* workspace, size_t workspace_bytes,
                                    mantleCudaStream_t stream_) {
    if (!batch_ok(batch, true)) return kInvalid;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    KArgs a;
    fill_args(a, batch);
    const int s = choose_splits(batch);
    int rc = apply_write_back(a, stream);
    if (rc) return rc;
    if (batch->max_top_k > KMAX) return launch_wide(a, batch->dtype, stream);
    if (s == 1) return launch_scan<MODE_FUSED>(a, batch->dtype, stream);

    const size_t need = parts_bytes(batch->rows, s, batch->max_top_k);
    if (!workspace || workspace_bytes < need) return kInvalid;
    if (reinterpret_cast<uintptr_t>(workspace) % 16) return kInvalid;
    const size_t n = (size_t)batch->rows * s;
    a.splits = s;
    a.parts = s;
    a.part_cap = batch->max_top_k;
    a.part_val = static_cast<float*>(workspace);
    a.part_idx = reinterpret_cast<int32_t*>(a.part_val + n * a.part_cap);
    a.part_cnt = a.part_idx + n * a.part_cap;
    rc = launch_scan<MODE_PARTS>(a, batch->dtype, stream);
    if (rc) return rc;
    return launch_merge(a, stream, true);
}

extern "C" int mantleCudaRepeatPenaltyRowsF32(const MantleSampleBatch* batch, mantleCudaStream_t stream_) {
    if (!batch_ok(batch, false) || batch->dtype != MANTLE_DTYPE_F32 || !batch->params) return kInvalid;
    if (batch->flags & MANTLE_SAMPLE_PENALTY_PREAPPLIED) return kInvalid;
    KArgs a;
    fill_args(a, batch);
    return launch_penalty(a, static_cast<cudaStream_t>(stream_));
}

extern "C" int mantleCudaLogitPostprocessRowsF32(float* logits, int rows, int vocab, int64_t row_stride,
                                                float logit_scale, float logit_softcap, uint32_t flags,
                                                mantleCudaStream_t stream_) {
    if (!logits || rows <= 0 || vocab <= 0 || row_stride < vocab) return kInvalid;
    if (reinterpret_cast<uintptr_t>(logits) % 4 || (flags & ~MANTLE_SAMPLE_SOFTCAP_TANHF)) return kInvalid;
    if (!post_ok(logit_scale, logit_softcap)) return kInvalid;
    Post post = {post_mode_of(logit_scale, logit_softcap, flags), logit_scale, logit_softcap};
    if (!post.mode) return 0;
    const long long n = (long long)rows * vocab;
    const int grid = (int)std::min<long long>((n + 255) / 256, (long long)device_info().sms * 32);
    postprocess_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_)>>>(logits, rows, vocab, row_stride, post);
    return (int)cudaGetLastError();
}

extern "C" int mantleCudaHistoryAppendRows(int32_t* history, int32_t* hist_len, int hist_stride, int rows,
                                          const int32_t* next, int keep, const int32_t* stop, int n_stop,
                                          int32_t* done, mantleCudaStream_t stream_) {
    if (!history || !hist_len || !next || rows <= 0 || hist_stride < 2) return kInvalid;
    if (keep < 0 || keep > hist_stride / 2 || n_stop < 0 || (n_stop > 0 && !stop)) return kInvalid;
    const long long threads = (long long)rows * 32;
    if ((threads + 255) / 256 > 0x7fffffffLL) return kInvalid;
    history_append_rows_kernel<<<(int)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        history, hist_len, hist_stride, rows, next, keep, stop, n_stop, done);
    return (int)cudaGetLastError();
}

extern "C" int mantleCudaArgMaxRowsF32(const float* x, int rows, int n, int64_t row_stride, int* out_idx,
                                       mantleCudaStream_t stream_) {
    if (!x || !out_idx || rows <= 0 || n <= 0 || n > MANTLE_SAMPLE_MAX_VOCAB || row_stride < n) return kInvalid;
    if (reinterpret_cast<uintptr_t>(x) % 4) return kInvalid;
    MantleSampleBatch b = {};
    b.logits = x;
    b.dtype = MANTLE_DTYPE_F32;
    b.rows = rows;
    b.vocab = n;
    b.max_top_k = 1;
    b.row_stride = row_stride;
    b.next = out_idx;
    KArgs a;
    fill_args(a, &b);
    return launch_scan<MODE_FUSED>(a, MANTLE_DTYPE_F32, static_cast<cudaStream_t>(stream_));
}

extern "C" int mantleCudaSampleLocalTopK(const MantleSampleBatch* batch, int vocab_offset, int vocab_total,
                                         float* part_val, int32_t* part_idx, int32_t* part_cnt, int part_cap,
                                         mantleCudaStream_t stream_) {
    if (!batch_ok(batch, false) || !batch->params) return kInvalid;
    if (batch->max_top_k < 1 || batch->max_top_k > KMAX) return kInvalid;
    if (!part_val || !part_idx || !part_cnt || part_cap < batch->max_top_k) return kInvalid;
    if (vocab_offset < 0 || vocab_total < vocab_offset + batch->vocab) return kInvalid;
    KArgs a;
    fill_args(a, batch);
    a.vocab_offset = vocab_offset;
    a.vocab_total = vocab_total;
    a.parts = 1;
    a.part_cap = part_cap;
    a.part_val = part_val;
    a.part_idx = part_idx;
    a.part_cnt = part_cnt;
    int rc = apply_write_back(a, static_cast<cudaStream_t>(stream_));
    if (rc) return rc;
    return launch_scan<MODE_PARTS>(a, batch->dtype, static_cast<cudaStream_t>(stream_));
}

// One rank's shortlists as one block, so that a single all-gather moves everything:
// [rows * cap float values][rows * cap int32 ids][rows int32 counts], padded to 256 bytes.
static size_t packed_part_bytes(int rows, int cap) {
    const size_t b = ((size_t)rows * cap * 2 + (size_t)rows) * 4;
    return (b + 255) & ~(size_t)255;
}

extern "C" int mantleCudaSamplePackedPartBytes(int rows, int part_cap, size_t* bytes) {
    if (!bytes || rows <= 0 || part_cap <= 0) return kInvalid;
    *bytes = packed_part_bytes(rows, part_cap);
    return 0;
}

extern "C" int mantleCudaSampleMergePacked(const MantleSampleBatch* batch, int parts, const void* packed, int part_cap,
                                           mantleCudaStream_t stream_) {
    if (!batch || batch->rows <= 0 || !batch->params || !batch->next || batch->vocab <= 0) return kInvalid;
    if (batch->max_top_k < 1 || batch->max_top_k > KMAX) return kInvalid;
    if ((batch->cand_idx || batch->cand_prob) && batch->cand_stride <= 0) return kInvalid;
    if (parts < 1 || !packed || part_cap < 1 || reinterpret_cast<uintptr_t>(packed) % 16) return kInvalid;
    if ((long long)parts * (part_cap < batch->max_top_k ? part_cap : batch->max_top_k) > MERGE_CAP) return kInvalid;
    KArgs a;
    fill_args(a, batch);
    const size_t n = (size_t)batch->rows * part_cap;
    a.parts = parts;
    a.part_cap = part_cap;
    a.part_val = const_cast<float*>(static_cast<const float*>(packed));
    a.part_idx = reinterpret_cast<int32_t*>(a.part_val + n);
    a.part_cnt = a.part_idx + n;
    a.part_stride = (long long)(packed_part_bytes(batch->rows, part_cap) / 4);
    a.cnt_stride = a.part_stride;
    return launch_merge(a, static_cast<cudaStream_t>(stream_));
}

extern "C" int mantleCudaSampleMergeParts(const MantleSampleBatch* batch, int parts, const float* part_val,
                                          const int32_t* part_idx, const int32_t* part_cnt, int part_cap,
                                          mantleCudaStream_t stream_) {
    if (!batch || batch->rows <= 0 || !batch->params || !batch->next) return kInvalid;
    if (batch->max_top_k < 1 || batch->max_top_k > KMAX) return kInvalid;
    if ((batch->cand_idx || batch->cand_prob) && batch->cand_stride <= 0) return kInvalid;
    if (parts < 1 || !part_val || !part_idx || !part_cnt || part_cap < 1) return kInvalid;
    if ((long long)parts * (part_cap < batch->max_top_k ? part_cap : batch->max_top_k) > MERGE_CAP) return kInvalid;
    if (batch->vocab <= 0) return kInvalid;
    KArgs a;
    fill_args(a, batch);
    a.parts = parts;
    a.part_cap = part_cap;
    a.part_val = const_cast<float*>(part_val);
    a.part_idx = const_cast<int32_t*>(part_idx);
    a.part_cnt = const_cast<int32_t*>(part_cnt);
    return launch_merge(a, static_cast<cudaStream_t>(stream_));
}

// ---------------------------------------------------------------------------------------
// host-buffer entry point

namespace {

inline size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

// Carves the device workspace for a host batch.  Returns the total size.
struct HostPlan {
    size_t logits, history, hist_len, exclude, params, next, cand_idx, cand_prob, n_kept, cut, status, token_prob,
        softmax_sum, skip, split, total;
    size_t logits_bytes, history_bytes, split_bytes;
};

HostPlan plan_host(const MantleSampleBatch* b) {
    HostPlan p = {};
    const size_t esz = b->dtype == MANTLE_DTYPE_F32 ? 4 : 2;
    const size_t rows = (size_t)b->rows;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t at = off;
        off += align256(bytes);
        return at;
    };
    p.logits_bytes = ((rows - 1) * (size_t)b->row_stride + (size_t)b->vocab) * esz;
    p.logits = take(p.logits_bytes);
    p.history_bytes = (b->history && b->hist_stride > 0) ? rows * (size_t)b->hist_stride * 4 : 0;
    p.history = take(p.history_bytes);
    p.hist_len = take(b->hist_len ? rows * 4 : 0);
    p.exclude = take((size_t)b->n_exclude * 4);
    p.params = take(rows * sizeof(MantleSampleParams));
    p.next = take(rows * 4);
    p.cand_idx = take(b->cand_idx ? rows * (size_t)b->cand_stride * 4 : 0);
    p.cand_prob = take(b->cand_prob ? rows * (size_t)b->cand_stride * 8 : 0);
    p.n_kept = take(b->n_kept ? rows * 4 : 0);
    p.cut = take(b->cut ? rows * 4 : 0);
    p.status = take(b->status ? 4 : 0);
    p.token_prob = take(b->token_prob ? rows * 8 : 0);
    p.softmax_sum = take(b->softmax_sum ? rows * 8 : 0);
    p.skip = take(b->skip ? rows * 4 : 0);
    const int s = choose_splits(b);
    p.split_bytes = s > 1 ? parts_bytes(b->rows, s, b->max_top_k) : 0;
    p.split = take(p.split_bytes);
    p.total = off;
    return p;
}

}  // namespace

extern "C" int mantleCudaSamplerHostWorkspaceBytes(const MantleSampleBatch* host_batch, size_t* bytes) {
    if (!bytes || !batch_ok(host_batch, true)) return kInvalid;
    *bytes = plan_host(host_batch).total;
    return 0;
}

extern "C" int mantleCudaSampleRowsHost(const MantleSampleBatch* hb, void* device_workspace, size_t workspace_bytes,
                                        mantleCudaStream_t stream_) {
    if (!batch_ok(hb, true)) return kInvalid;
    const HostPlan p = plan_host(hb);
    if (!device_workspace || workspace_bytes < p.total) return kInvalid;
    if (reinterpret_cast<uintptr_t>(device_workspace) % 256) return kInvalid;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    char* ws = static_cast<char*>(device_workspace);
    const size_t rows = (size_t)hb->rows;
    cudaError_t e;
#define MANTLE_TRY(call)                  \
    do {                                  \
        e = (call);                       \
        if (e != cudaSuccess) return (int)e; \
    } while (0)
    MANTLE_TRY(cudaMemcpyAsync(ws + p.logits, hb->logits, p.logits_bytes, cudaMemcpyHostToDevice, stream));
    if (p.history_bytes)
        MANTLE_TRY(cudaMemcpyAsync(ws + p.history, hb->history, p.history_bytes, cudaMemcpyHostToDevice, stream));
    if (hb->hist_len)
        MANTLE_TRY(cudaMemcpyAsync(ws + p.hist_len, hb->hist_len, rows * 4, cudaMemcpyHostToDevice, stream));
    if (hb->n_exclude)
        MANTLE_TRY(cudaMemcpyAsync(ws + p.exclude, hb->exclude, (size_t)hb->n_exclude * 4, cudaMemcpyHostToDevice, stream));
    MANTLE_TRY(cudaMemcpyAsync(ws + p.params, hb->params, rows * sizeof(MantleSampleParams), cudaMemcpyHostToDevice, stream));
    if (hb->skip) MANTLE_TRY(cudaMemcpyAsync(ws + p.skip, hb->skip, rows * 4, cudaMemcpyHostToDevice, stream));
    if (hb->status) MANTLE_TRY(cudaMemsetAsync(ws + p.status, 0, 4, stream));

    MantleSampleBatch d = *hb;
    d.logits = ws + p.logits;
    d.history = p.history_bytes ? reinterpret_cast<const int32_t*>(ws + p.history) : nullptr;
    d.hist_len = hb->hist_len ? reinterpret_cast<const int32_t*>(ws + p.hist_len) : nullptr;
    d.exclude = hb->n_exclude ? reinterpret_cast<const int32_t*>(ws + p.exclude) : nullptr;
    d.params = reinterpret_cast<const MantleSampleParams*>(ws + p.params);
    d.next = reinterpret_cast<int32_t*>(ws + p.next);
    d.cand_idx = hb->cand_idx ? reinterpret_cast<int32_t*>(ws + p.cand_idx) : nullptr;
    d.cand_prob = hb->cand_prob ? reinterpret_cast<double*>(ws + p.cand_prob) : nullptr;
    d.n_kept = hb->n_kept ? reinterpret_cast<int32_t*>(ws + p.n_kept) : nullptr;
    d.cut = hb->cut ? reinterpret_cast<int32_t*>(ws + p.cut) : nullptr;
    d.status = hb->status ? reinterpret_cast<int32_t*>(ws + p.status) : nullptr;
    d.token_prob = hb->token_prob ? reinterpret_cast<double*>(ws + p.token_prob) : nullptr;
    d.softmax_sum = hb->softmax_sum ? reinterpret_cast<double*>(ws + p.softmax_sum) : nullptr;
    d.skip = hb->skip ? reinterpret_cast<const int32_t*>(ws + p.skip) : nullptr;
    int rc = mantleCudaSampleRows(&d, p.split_bytes ? ws + p.split : nullptr, p.split_bytes, stream_);
    if (rc) return rc;

    MANTLE_TRY(cudaMemcpyAsync(hb->next, ws + p.next, rows * 4, cudaMemcpyDeviceToHost, stream));
    if (hb->cand_idx)
        MANTLE_TRY(cudaMemcpyAsync(hb->cand_idx, ws + p.cand_idx, rows * (size_t)hb->cand_stride * 4, cudaMemcpyDeviceToHost, stream));
    if (hb->cand_prob)
        MANTLE_TRY(cudaMemcpyAsync(hb->cand_prob, ws + p.cand_prob, rows * (size_t)hb->cand_stride * 8, cudaMemcpyDeviceToHost, stream));
    if (hb->n_kept) MANTLE_TRY(cudaMemcpyAsync(hb->n_kept, ws + p.n_kept, rows * 4, cudaMemcpyDeviceToHost, stream));
    if (hb->cut) MANTLE_TRY(cudaMemcpyAsync(hb->cut, ws + p.cut, rows * 4, cudaMemcpyDeviceToHost, stream));
    if (hb->status) MANTLE_TRY(cudaMemcpyAsync(hb->status, ws + p.status, 4, cudaMemcpyDeviceToHost, stream));
    if (hb->token_prob)
        MANTLE_TRY(cudaMemcpyAsync(hb->token_prob, ws + p.token_prob, rows * 8, cudaMemcpyDeviceToHost, stream));
    if (hb->softmax_sum)
        MANTLE_TRY(cudaMemcpyAsync(hb->softmax_sum, ws + p.softmax_sum, rows * 8, cudaMemcpyDeviceToHost, stream));
    if (hb->flags & MANTLE_SAMPLE_WRITE_BACK_PENALTY)
        MANTLE_TRY(cudaMemcpyAsync(const_cast<void*>(hb->logits), ws + p.logits, p.logits_bytes, cudaMemcpyDeviceToHost, stream));
#undef MANTLE_TRY
    return 0;
}

// ---------------------------------------------------------------------------------------
// An entry point that allocates nothing.
//
// Some hosts cannot hand the sampler a workspace: a runtime that froze its device-memory
// plan before sampling was wired in, an embedding whose allocator is off limits inside the
// decode loop, a caller that may not call cudaMalloc at all at that point.  For them the
// scratch that split rows need (the per-CTA shortlists between the streaming kernel and the
// merge) lives in a fixed array inside the library image.  Every GPU that loads the library
// carries the array until the process exits, which is why it is kept small.

namespace {

constexpr size_t kStaticScratchBytes = (size_t)4 << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_split_scratch[kStaticScratchBytes];

void* g_scratch_addr[kMaxDevices];    // device address of g_split_scratch, per device ordinal
std::atomic<int> g_scratch_known[kMaxDevices];
std::mutex g_scratch_mutex;
thread_local char g_last_error[256];

void set_last_error(const char* fmt, unsigned long long a = 0, unsigned long long b = 0) {
    snprintf(g_last_error, sizeof g_last_error, fmt, a, b);
}

// In host code the array's name is only a handle: the address kernels can use has to be asked
// for, per device, with that device current.
int static_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) {
        set_last_error("device ordinal %llu is beyond the %llu devices the static scratch tracks",
                       (unsigned long long)dev, (unsigned long long)kMaxDevices);
        return kInvalid;
    }
    // The address is looked up once per device and lives as long as the device's primary context:
    // a cudaDeviceReset in this process invalidates it, and the library must not be used across one.
    if (!g_scratch_known[dev].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_scratch_mutex);
        if (!g_scratch_known[dev].load(std::memory_order_relaxed)) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_split_scratch);
            if (e != cudaSuccess) {
                set_last_error("cudaGetSymbolAddress failed with cudaError %llu", (unsigned long long)e);
                return (int)e;
            }
            g_scratch_addr[dev] = p;
            g_scratch_known[dev].store(1, std::memory_order_release);
        }
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" const char* mantleCudaSamplerLastError(void) { return g_last_error; }

void mantle_internal_set_last_error(const char* msg) { snprintf(g_last_error, sizeof g_last_error, "%s", msg); }

extern "C" size_t mantleCudaSamplerStaticScratchBytes(void) { return kStaticScratchBytes; }

extern "C" int mantleCudaSampleRowsNoAlloc(const MantleSampleBatch* batch, mantleCudaStream_t stream_) {
    g_last_error[0] = 0;
    if (!batch_ok(batch, true)) {
        set_last_error("invalid batch descriptor");
        return kInvalid;
    }
    const int s = choose_splits(batch);
    const size_t need = s > 1 ? parts_bytes(batch->rows, s, batch->max_top_k) : 0;
    if (need > kStaticScratchBytes) {
        set_last_error("batch needs %llu bytes of scratch, the static scratch holds %llu: pass a workspace to "
                       "mantleCudaSampleRows instead, or lower rows * splits * max_top_k",
                       (unsigned long long)need, (unsigned long long)kStaticScratchBytes);
        return kInvalid;
    }
    void* scratch = nullptr;
    const int rc = static_scratch(&scratch);
    if (rc) return rc;
    return mantleCudaSampleRows(batch, scratch, kStaticScratchBytes, stream_);
}

// Runs the bounded wait of the bulk-copy ring on a barrier that is never completed: after
// limit_ns the kernel must return with MANTLE_SAMPLE_STATUS_TIMEOUT in *status_dev.
extern "C" int mantleCudaSamplerSelfTestBoundedWait(unsigned long long limit_ns, int32_t* status_dev,
                                                    mantleCudaStream_t stream_) {
    if (!status_dev || limit_ns == 0 || limit_ns > 1000000000ull) return kInvalid;
    bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream_)>>>(limit_ns, status_dev);
    return (int)cudaGetLastError();
}
