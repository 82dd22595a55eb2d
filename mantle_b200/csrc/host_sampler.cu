// Host-side sampler object: see include/mantle_host_sampler.h.  Mirrors logits.Sampler
// (internal/logits/sampler.go:44-98) above the CUDA C-ABI.  All arithmetic of the sampling path
// runs in the kernels; this file normalises the configuration, stages the call's small inputs
// and moves bytes.

#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "../../include/mantle_host_sampler.h"
#include "sampler_internal.h"

struct MantleHostSampler {
    MantleSampleParams params;  // normalised; `uniform` filled per call
    int max_vocab;
    int device;
    cudaStream_t stream;
    cudaEvent_t event;
    // pinned staging: history window, exclude list, parameters, outputs
    int32_t* h_hist;
    int32_t* h_excl;
    MantleSampleParams* h_params;
    int32_t* h_next;
    int32_t* h_status;
    float* h_gather;  // penalised values of the window's columns, on their way back to the caller's slice
    int excl_cap;
    // device
    float* d_logits;  // the device copy of a host slice (max_vocab floats)
    void* d_ws;
    size_t d_ws_bytes;
};

namespace {

constexpr int kExcludeCap = 256;

// Fills the batch descriptor for one row; history and exclude are staged into pinned memory.
int stage(MantleHostSampler* s, MantleSampleBatch* b, int n, const int64_t* recent, int n_recent,
          const int64_t* exclude, int n_exclude, double uniform) {
    if (!s || n <= 0 || n > s->max_vocab || n_recent < 0 || n_exclude < 0 || n_exclude > s->excl_cap)
        return (int)cudaErrorInvalidValue;
    if ((n_recent > 0 && !recent) || (n_exclude > 0 && !exclude)) return (int)cudaErrorInvalidValue;
    const int window = n_recent < s->params.repeat_last_n ? n_recent : s->params.repeat_last_n;  // sampler.go:100-101
    for (int i = 0; i < window; i++) s->h_hist[i] = mantle_internal_narrow_id(recent[n_recent - window + i]);
    for (int i = 0; i < n_exclude; i++) s->h_excl[i] = mantle_internal_narrow_id(exclude[i]);
    *s->h_params = s->params;
    s->h_params->uniform = uniform;
    memset(b, 0, sizeof *b);
    b->dtype = MANTLE_DTYPE_F32;
    b->rows = 1;
    b->vocab = n;
    b->row_stride = n;
    b->max_top_k = s->params.top_k < n ? s->params.top_k : n;  // sampler.go:147
    b->history = window > 0 ? s->h_hist : nullptr;
    b->hist_stride = window;
    b->exclude = n_exclude > 0 ? s->h_excl : nullptr;
    b->n_exclude = n_exclude;
    b->params = s->h_params;
    b->next = s->h_next;
    b->status = s->h_status;
    return 0;
}

}  // namespace

extern "C" MantleHostSampler* mantleSamplerNew(const MantleSamplerConfig* cfg, int max_vocab) {
    if (!cfg || max_vocab <= 0 || max_vocab > MANTLE_SAMPLE_MAX_VOCAB) return nullptr;
    MantleHostSampler* s = new (std::nothrow) MantleHostSampler();
    if (!s) return nullptr;
    memset(s, 0, sizeof *s);
    mantle_internal_normalise(*cfg, &s->params);
    s->max_vocab = max_vocab;
    s->excl_cap = kExcludeCap;
    bool ok = cudaGetDevice(&s->device) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&s->event, cudaEventDisableTiming) == cudaSuccess;
    const size_t hist_bytes = sizeof(int32_t) * (size_t)(s->params.repeat_last_n + 4);
    ok = ok && cudaMallocHost(&s->h_hist, hist_bytes) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_excl, sizeof(int32_t) * kExcludeCap) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_params, sizeof(MantleSampleParams)) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_next, sizeof(int32_t)) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_status, sizeof(int32_t)) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_gather, hist_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&s->d_logits, sizeof(float) * (size_t)max_vocab) == cudaSuccess;
    if (ok) {
        // the largest workspace any later call can need: one row of max_vocab floats, split over CTAs
        MantleSampleBatch b;
        memset(&b, 0, sizeof b);
        static float dummy;
        b.logits = &dummy;
        b.dtype = MANTLE_DTYPE_F32;
        b.rows = 1;
        b.vocab = max_vocab;
        b.row_stride = max_vocab;
        b.max_top_k = MANTLE_SAMPLE_MAX_TOP_K < max_vocab ? MANTLE_SAMPLE_MAX_TOP_K : max_vocab;
        b.history = s->h_hist;
        b.hist_stride = s->params.repeat_last_n;
        b.exclude = s->h_excl;
        b.n_exclude = kExcludeCap;
        b.params = s->h_params;
        b.next = s->h_next;
        b.status = s->h_status;
        size_t a = 0, c = 0;
        ok = mantleCudaSamplerWorkspaceBytes(&b, &a) == 0;
        b.max_top_k = 1;  // few candidates allow more CTAs per row and a larger split buffer
        ok = ok && mantleCudaSamplerWorkspaceBytes(&b, &c) == 0;
        // the split scratch of the larger of the two, behind the small inputs' slots
        s->d_ws_bytes = (a > c ? a : c) + 2 * hist_bytes + sizeof(int32_t) * kExcludeCap + 8192;
        ok = ok && cudaMalloc(&s->d_ws, s->d_ws_bytes) == cudaSuccess;
    }
    if (!ok) {
        mantleSamplerFree(s);
        return nullptr;
    }
    return s;
}

extern "C" void mantleSamplerFree(MantleHostSampler* s) {
    if (!s) return;
    if (s->d_ws) cudaFree(s->d_ws);
    if (s->d_logits) cudaFree(s->d_logits);
    if (s->h_gather) cudaFreeHost(s->h_gather);
    if (s->h_hist) cudaFreeHost(s->h_hist);
    if (s->h_excl) cudaFreeHost(s->h_excl);
    if (s->h_params) cudaFreeHost(s->h_params);
    if (s->h_next) cudaFreeHost(s->h_next);
    if (s->h_status) cudaFreeHost(s->h_status);
    if (s->event) cudaEventDestroy(s->event);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

extern "C" int mantleSamplerParams(const MantleHostSampler* s, MantleSampleParams* out) {
    if (!s || !out) return (int)cudaErrorInvalidValue;
    *out = s->params;
    return 0;
}

extern "C" int mantleSamplerCanUseDeviceGreedy(const MantleHostSampler* s) {  // sampler.go:56-58
    return s && s->params.greedy && s->params.repeat_penalty <= 1.0f;
}

extern "C" int mantleSamplerNeedsUniform(const MantleHostSampler* s) { return s && !mantle_internal_argmax_shortcut(s->params); }

namespace {

// After the in-place penalty: the value of every window id's column, so that the host can patch
// its slice without the whole row coming back.  Ids out of range read nothing (sampler.go:116).
__global__ void gather_window_kernel(const float* logits, const int32_t* ids, int n_ids, int vocab, float* out) {
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n_ids; j += gridDim.x * blockDim.x) {
        const int id = ids[j];
        if (id >= 0 && id < vocab) out[j] = logits[id];
    }
}

// What a status word means, for mantleCudaSamplerLastError.
void report_status(int status) {
    if (status & MANTLE_SAMPLE_STATUS_EMPTY)
        mantle_internal_set_last_error("the shortlist was empty after min-p (min_p > 1): the reference panics in Sample here");
    else if (status & MANTLE_SAMPLE_STATUS_TOPK_RANGE)
        mantle_internal_set_last_error("top_k exceeded the bound the call was sized for");
    else if (status & MANTLE_SAMPLE_STATUS_NAN)
        mantle_internal_set_last_error("the logits held nothing but NaN");
    else
        mantle_internal_set_last_error("the sampling kernel reported an unknown status");
}

// Sample on logits that are on the device.  `d_logits` is patched in place when `write_back` is
// set.  Queues everything on the sampler's stream and synchronises it.
int sample_on_device(MantleHostSampler* s, const MantleSampleBatch& hb, const float* d_logits, bool write_back,
                     int* token) {
    // small inputs into the workspace, 256-byte slots: history | exclude | params | next | status | gathered | split scratch
    char* ws = static_cast<char*>(s->d_ws);
    const size_t hist_bytes = (((size_t)hb.hist_stride * 4 + 255) / 256 + 1) * 256;
    char* d_hist = ws;
    char* d_excl = d_hist + hist_bytes;
    char* d_params = d_excl + (((size_t)kExcludeCap * 4 + 255) / 256) * 256;
    char* d_next = d_params + 256;
    char* d_status = d_next + 256;
    char* d_gather = d_status + 256;
    char* d_split = d_gather + hist_bytes;
    MantleSampleBatch d = hb;
    d.logits = d_logits;
    d.flags = write_back ? MANTLE_SAMPLE_WRITE_BACK_PENALTY : 0u;
    cudaError_t e;
    if (hb.hist_stride > 0) {
        e = cudaMemcpyAsync(d_hist, hb.history, (size_t)hb.hist_stride * 4, cudaMemcpyHostToDevice, s->stream);
        if (e != cudaSuccess) return (int)e;
        d.history = reinterpret_cast<const int32_t*>(d_hist);
    }
    if (hb.n_exclude > 0) {
        e = cudaMemcpyAsync(d_excl, hb.exclude, (size_t)hb.n_exclude * 4, cudaMemcpyHostToDevice, s->stream);
        if (e != cudaSuccess) return (int)e;
        d.exclude = reinterpret_cast<const int32_t*>(d_excl);
    }
    e = cudaMemcpyAsync(d_params, hb.params, sizeof(MantleSampleParams), cudaMemcpyHostToDevice, s->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_status, 0, 4, s->stream);
    if (e != cudaSuccess) return (int)e;
    d.params = reinterpret_cast<const MantleSampleParams*>(d_params);
    d.next = reinterpret_cast<int32_t*>(d_next);
    d.status = reinterpret_cast<int32_t*>(d_status);
    size_t need = 0;
    int rc = mantleCudaSamplerWorkspaceBytes(&d, &need);
    if (rc) return rc;
    if ((size_t)(d_split - ws) + need > s->d_ws_bytes) return (int)cudaErrorInvalidValue;
    rc = mantleCudaSampleRows(&d, need ? d_split : nullptr, need, s->stream);
    if (rc) return rc;
    if (write_back) {
        gather_window_kernel<<<1, 256, 0, s->stream>>>(d_logits, d.history, hb.hist_stride, hb.vocab,
                                                       reinterpret_cast<float*>(d_gather));
        e = cudaGetLastError();
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(s->h_gather, d_gather, (size_t)hb.hist_stride * 4, cudaMemcpyDeviceToHost, s->stream);
        if (e != cudaSuccess) return (int)e;
    }
    e = cudaMemcpyAsync(s->h_next, d_next, 4, cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s->h_status, d_status, 4, cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return (int)e;
    *token = *s->h_next;
    if (*s->h_status) {
        report_status(*s->h_status);
        return (int)cudaErrorUnknown;
    }
    return 0;
}

}  // namespace

extern "C" int mantleSamplerSample(MantleHostSampler* s, float* logits, int n, const int64_t* recent, int n_recent,
                                   const int64_t* exclude, int n_exclude, double uniform, int* token) {
    if (!logits || !token) return (int)cudaErrorInvalidValue;
    MantleSampleBatch b;
    int rc = stage(s, &b, n, recent, n_recent, exclude, n_exclude, uniform);
    if (rc) return rc;
    cudaError_t e = cudaMemcpyAsync(s->d_logits, logits, (size_t)n * 4, cudaMemcpyHostToDevice, s->stream);
    if (e != cudaSuccess) return (int)e;
    // The reference patches the caller's slice (sampler.go:132-136), and only where the penalty
    // ran (sampler.go:99): the device rewrites its copy, the changed columns alone come back.
    const bool penalty = s->params.repeat_penalty > 1.0f && b.hist_stride > 0;
    rc = sample_on_device(s, b, s->d_logits, penalty, token);
    if (rc) return rc;
    if (penalty)
        for (int j = 0; j < b.hist_stride; j++) {
            const int32_t id = s->h_hist[j];
            if (id >= 0 && id < n) logits[id] = s->h_gather[j];
        }
    return 0;
}

extern "C" int mantleSamplerSampleDevice(MantleHostSampler* s, const float* dev_logits, int n, const int64_t* recent,
                                         int n_recent, const int64_t* exclude, int n_exclude, double uniform,
                                         mantleCudaStream_t wait_stream, int* token) {
    if (!dev_logits || !token) return (int)cudaErrorInvalidValue;
    MantleSampleBatch hb;
    int rc = stage(s, &hb, n, recent, n_recent, exclude, n_exclude, uniform);
    if (rc) return rc;
    // order after the producer of the logits
    cudaError_t e = cudaEventRecord(s->event, static_cast<cudaStream_t>(wait_stream));
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s->stream, s->event, 0);
    if (e != cudaSuccess) return (int)e;
    return sample_on_device(s, hb, dev_logits, false, token);
}
