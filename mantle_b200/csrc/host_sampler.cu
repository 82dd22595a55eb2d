// Host-side sampler object: see include/mantle_host_sampler.h.  Mirrors logits.Sampler
// (internal/logits/sampler.go:44-98) above the CUDA C-ABI.  All arithmetic of the sampling path
// runs in the kernels; this file normalises the configuration, stages the call's small inputs
// and moves bytes.

#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "../../include/mantle_host_sampler.h"

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
    int excl_cap;
    // device
    void* d_ws;
    size_t d_ws_bytes;
};

namespace {

constexpr int kExcludeCap = 256;

// NewSampler's normalisation, sampler.go:61-83.
void normalise(const MantleSamplerConfig& cfg, MantleSampleParams* p) {
    memset(p, 0, sizeof *p);
    p->greedy = cfg.temperature <= 0 ? 1 : 0;
    p->temperature = cfg.temperature <= 0 ? 1.0f : cfg.temperature;
    p->top_k = cfg.top_k <= 0 ? 40 : cfg.top_k;
    p->top_p = (cfg.top_p <= 0 || cfg.top_p > 1) ? 1.0f : cfg.top_p;
    p->min_p = cfg.min_p;
    p->repeat_penalty = cfg.repeat_penalty <= 0 ? 1.0f : cfg.repeat_penalty;
    p->repeat_last_n = cfg.repeat_last_n <= 0 ? 64 : cfg.repeat_last_n;
}

bool argmax_shortcut(const MantleSampleParams& p) {  // sampler.go:140
    return p.greedy || (p.top_k == 1 && p.top_p >= 1.0f && p.temperature == 1.0f);
}

int32_t narrow(int64_t id) { return (id < 0 || id > 0x7fffffffLL) ? -1 : (int32_t)id; }  // out of range: ignored anyway

// Fills the batch descriptor for one row; history and exclude are staged into pinned memory.
int stage(MantleHostSampler* s, MantleSampleBatch* b, int n, const int64_t* recent, int n_recent,
          const int64_t* exclude, int n_exclude, double uniform) {
    if (!s || n <= 0 || n > s->max_vocab || n_recent < 0 || n_exclude < 0 || n_exclude > s->excl_cap)
        return (int)cudaErrorInvalidValue;
    if ((n_recent > 0 && !recent) || (n_exclude > 0 && !exclude)) return (int)cudaErrorInvalidValue;
    const int window = n_recent < s->params.repeat_last_n ? n_recent : s->params.repeat_last_n;  // sampler.go:100-101
    for (int i = 0; i < window; i++) s->h_hist[i] = narrow(recent[n_recent - window + i]);
    for (int i = 0; i < n_exclude; i++) s->h_excl[i] = narrow(exclude[i]);
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
    normalise(*cfg, &s->params);
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
        ok = mantleCudaSamplerHostWorkspaceBytes(&b, &a) == 0;
        b.max_top_k = 1;  // few candidates allow more CTAs per row and a larger split buffer
        ok = ok && mantleCudaSamplerHostWorkspaceBytes(&b, &c) == 0;
        s->d_ws_bytes = (a > c ? a : c) + 4096;
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

extern "C" int mantleSamplerNeedsUniform(const MantleHostSampler* s) { return s && !argmax_shortcut(s->params); }

extern "C" int mantleSamplerSample(MantleHostSampler* s, float* logits, int n, const int64_t* recent, int n_recent,
                                   const int64_t* exclude, int n_exclude, double uniform, int* token) {
    if (!logits || !token) return (int)cudaErrorInvalidValue;
    MantleSampleBatch b;
    int rc = stage(s, &b, n, recent, n_recent, exclude, n_exclude, uniform);
    if (rc) return rc;
    b.logits = logits;
    b.flags = MANTLE_SAMPLE_WRITE_BACK_PENALTY;  // the reference patches the caller's slice (sampler.go:132-136)
    rc = mantleCudaSampleRowsHost(&b, s->d_ws, s->d_ws_bytes, s->stream);
    if (rc) return rc;
    cudaError_t e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return (int)e;
    *token = *s->h_next;
    return *s->h_status ? (int)cudaErrorUnknown : 0;
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
    // small inputs into the workspace, 256-byte slots: history | exclude | params | next | status | split scratch
    char* ws = static_cast<char*>(s->d_ws);
    const size_t hist_bytes = (((size_t)hb.hist_stride * 4 + 255) / 256 + 1) * 256;
    char* d_hist = ws;
    char* d_excl = d_hist + hist_bytes;
    char* d_params = d_excl + (((size_t)kExcludeCap * 4 + 255) / 256) * 256;
    char* d_next = d_params + 256;
    char* d_status = d_next + 256;
    char* d_split = d_status + 256;
    MantleSampleBatch d = hb;
    d.logits = dev_logits;
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
    rc = mantleCudaSamplerWorkspaceBytes(&d, &need);
    if (rc) return rc;
    if ((size_t)(d_split - ws) + need > s->d_ws_bytes) return (int)cudaErrorInvalidValue;
    rc = mantleCudaSampleRows(&d, need ? d_split : nullptr, need, s->stream);
    if (rc) return rc;
    e = cudaMemcpyAsync(s->h_next, d_next, 4, cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s->h_status, d_status, 4, cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    if (e != cudaSuccess) return (int)e;
    *token = *s->h_next;
    return *s->h_status ? (int)cudaErrorUnknown : 0;
}
