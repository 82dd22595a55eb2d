// The decode loop's sampling state for a batch of requests: see include/mantle_batch_sampler.h.
// Mirrors what Generator.RunWithContext keeps per request (internal/inference/engine.go:189,
// 233-300: toks, the Sampler, the stop tokens) for `rows` requests at once.  All arithmetic of
// the sampling path runs in the kernels; this file keeps the per-row configuration, moves the
// small per-step inputs and outputs and queues the kernels.

#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "../../include/mantle_batch_sampler.h"
#include "sampler_internal.h"

struct MantleBatchSampler {
    int rows, vocab, cap, keep, n_stop;
    // host
    MantleSampleParams* h_params[2];  // pinned, double-buffered: a step's upload may still be in flight
    cudaEvent_t params_free[2];       // recorded after the upload that reads h_params[i]
    int turn;
    int32_t* h_next;                  // pinned results
    int32_t* h_ended;
    int32_t* h_status;
    int32_t* h_stage;                 // pinned: one row's context on its way to the device, then three ints
    uint8_t* ended;                   // what the host knows: rows that have ended
    // device
    MantleSampleParams* d_params;
    int32_t* d_history;
    int32_t* d_hist_len;
    int32_t* d_ended;
    int32_t* d_next;
    int32_t* d_status;
    int32_t* d_stop;
    void* d_ws;
    size_t d_ws_bytes;
};

namespace {

constexpr int kInvalid = (int)cudaErrorInvalidValue;

// Upper bound of mantleCudaSamplerWorkspaceBytes over every batch this sampler can queue: rows are
// split only while rows * splits fits one wave of CTAs, and splits * top_k never exceeds 4096.
size_t workspace_bound(int rows) {
    const size_t split_rows = rows < 1024 ? (size_t)rows : 1024;
    return split_rows * (4096 * 8 + 64 * 4) + 4096;
}

}  // namespace

extern "C" MantleBatchSampler* mantleBatchSamplerNew(int rows, int vocab, int hist_capacity, const int64_t* stop,
                                                     int n_stop) {
    if (rows <= 0 || vocab <= 0 || vocab > MANTLE_SAMPLE_MAX_VOCAB || hist_capacity < 2 || n_stop < 0) return nullptr;
    if (n_stop > 0 && !stop) return nullptr;
    if ((long long)rows * hist_capacity > 0x7fffffffLL) return nullptr;
    MantleBatchSampler* s = new (std::nothrow) MantleBatchSampler();
    if (!s) return nullptr;
    memset(s, 0, sizeof *s);
    s->rows = rows;
    s->vocab = vocab;
    s->cap = hist_capacity;
    s->keep = hist_capacity / 2;
    s->n_stop = n_stop;
    const size_t r = (size_t)rows;
    bool ok = true;
    for (int i = 0; i < 2 && ok; i++) {
        ok = cudaMallocHost(&s->h_params[i], r * sizeof(MantleSampleParams)) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&s->params_free[i], cudaEventDisableTiming) == cudaSuccess;
        if (ok) memset(s->h_params[i], 0, r * sizeof(MantleSampleParams));
    }
    ok = ok && cudaMallocHost(&s->h_next, r * 4) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_ended, r * 4) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_status, 4) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->h_stage, ((size_t)hist_capacity + 4 + (size_t)(n_stop > 0 ? n_stop : 1)) * 4) == cudaSuccess;
    s->ended = new (std::nothrow) uint8_t[r];
    ok = ok && s->ended;
    ok = ok && cudaMalloc(&s->d_params, r * sizeof(MantleSampleParams)) == cudaSuccess;
    ok = ok && cudaMalloc(&s->d_history, r * (size_t)hist_capacity * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&s->d_hist_len, r * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&s->d_ended, r * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&s->d_next, r * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&s->d_status, 4) == cudaSuccess;
    ok = ok && cudaMalloc(&s->d_stop, (size_t)(n_stop > 0 ? n_stop : 1) * 4) == cudaSuccess;
    s->d_ws_bytes = workspace_bound(rows);
    ok = ok && cudaMalloc(&s->d_ws, s->d_ws_bytes) == cudaSuccess;
    if (ok) {
        // every row starts ended, with an empty history; the stop tokens go up once
        memset(s->ended, 1, r);
        for (size_t i = 0; i < r; i++) {
            s->h_ended[i] = 1;
            s->h_next[i] = -1;
        }
        *s->h_status = 0;
        int32_t* h_stop = s->h_stage + hist_capacity + 4;
        for (int i = 0; i < n_stop; i++) h_stop[i] = mantle_internal_narrow_id(stop[i]);
        ok = cudaMemcpy(s->d_ended, s->h_ended, r * 4, cudaMemcpyHostToDevice) == cudaSuccess;
        ok = ok && cudaMemcpy(s->d_next, s->h_next, r * 4, cudaMemcpyHostToDevice) == cudaSuccess;
        ok = ok && cudaMemset(s->d_hist_len, 0, r * 4) == cudaSuccess;
        ok = ok && cudaMemset(s->d_status, 0, 4) == cudaSuccess;
        if (n_stop > 0) ok = ok && cudaMemcpy(s->d_stop, h_stop, (size_t)n_stop * 4, cudaMemcpyHostToDevice) == cudaSuccess;
    }
    if (!ok) {
        (void)cudaGetLastError();
        mantleBatchSamplerFree(s);
        return nullptr;
    }
    return s;
}

extern "C" void mantleBatchSamplerFree(MantleBatchSampler* s) {
    if (!s) return;
    for (int i = 0; i < 2; i++) {
        if (s->h_params[i]) cudaFreeHost(s->h_params[i]);
        if (s->params_free[i]) cudaEventDestroy(s->params_free[i]);
    }
    if (s->h_next) cudaFreeHost(s->h_next);
    if (s->h_ended) cudaFreeHost(s->h_ended);
    if (s->h_status) cudaFreeHost(s->h_status);
    if (s->h_stage) cudaFreeHost(s->h_stage);
    delete[] s->ended;
    if (s->d_params) cudaFree(s->d_params);
    if (s->d_history) cudaFree(s->d_history);
    if (s->d_hist_len) cudaFree(s->d_hist_len);
    if (s->d_ended) cudaFree(s->d_ended);
    if (s->d_next) cudaFree(s->d_next);
    if (s->d_status) cudaFree(s->d_status);
    if (s->d_stop) cudaFree(s->d_stop);
    if (s->d_ws) cudaFree(s->d_ws);
    delete s;
}

extern "C" int mantleBatchSamplerSetRow(MantleBatchSampler* s, int row, const MantleSamplerConfig* cfg,
                                        const int64_t* context, int n_context, mantleCudaStream_t stream_) {
    if (!s || !cfg || row < 0 || row >= s->rows || n_context < 0 || (n_context > 0 && !context)) return kInvalid;
    MantleSampleParams p;
    mantle_internal_normalise(*cfg, &p);
    if (p.repeat_last_n > s->keep) {
        mantle_internal_set_last_error("repeat_last_n exceeds half the history capacity the batch sampler was made with");
        return kInvalid;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // toks := copy(ContextTokens) (engine.go:189): the most recent ids that fit
    const int n = n_context < s->cap ? n_context : s->cap;
    for (int i = 0; i < n; i++) s->h_stage[i] = mantle_internal_narrow_id(context[n_context - n + i]);
    int32_t* small = s->h_stage + s->cap;
    small[0] = n;  // hist_len
    small[1] = 0;  // ended
    small[2] = -1; // next
    cudaError_t e = cudaSuccess;
    if (n > 0)
        e = cudaMemcpyAsync(s->d_history + (size_t)row * (size_t)s->cap, s->h_stage, (size_t)n * 4, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s->d_hist_len + row, small + 0, 4, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s->d_ended + row, small + 1, 4, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s->d_next + row, small + 2, 4, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);  // the staging buffer is free again
    if (e != cudaSuccess) return (int)e;
    // an upload of either parameter buffer may be in flight: wait for it before rewriting the row
    for (int i = 0; i < 2; i++) {
        e = cudaEventSynchronize(s->params_free[i]);
        if (e != cudaSuccess) return (int)e;
        s->h_params[i][row] = p;
    }
    s->ended[row] = 0;
    s->h_ended[row] = 0;
    s->h_next[row] = -1;
    return 0;
}

extern "C" int mantleBatchSamplerEndRow(MantleBatchSampler* s, int row, mantleCudaStream_t stream_) {
    if (!s || row < 0 || row >= s->rows) return kInvalid;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int32_t* small = s->h_stage + s->cap;
    small[3] = 1;
    cudaError_t e = cudaMemcpyAsync(s->d_ended + row, small + 3, 4, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return (int)e;
    s->ended[row] = 1;
    s->h_ended[row] = 1;
    return 0;
}

extern "C" int mantleBatchSamplerNeedsUniform(const MantleBatchSampler* s, int row) {
    if (!s || row < 0 || row >= s->rows) return 0;
    return !s->ended[row] && !mantle_internal_argmax_shortcut(s->h_params[0][row]);
}

extern "C" int mantleBatchSamplerCanUseDeviceGreedy(const MantleBatchSampler* s, int row) {  // sampler.go:56-58
    if (!s || row < 0 || row >= s->rows) return 0;
    const MantleSampleParams& p = s->h_params[0][row];
    return p.greedy && p.repeat_penalty <= 1.0f;
}

extern "C" int mantleBatchSamplerStep(MantleBatchSampler* s, const void* dev_logits, int dtype, int64_t row_stride,
                                      const double* uniforms, float logit_scale, float logit_softcap,
                                      mantleCudaStream_t stream_) {
    if (!s || !dev_logits || !uniforms || row_stride < s->vocab) return kInvalid;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // this step's parameter records: the rows' configurations and their uniform draws
    const int t = s->turn;
    s->turn ^= 1;
    cudaError_t e = cudaEventSynchronize(s->params_free[t]);  // the upload of two steps ago; normally long done
    if (e != cudaSuccess) return (int)e;
    MantleSampleParams* hp = s->h_params[t];
    int max_k = 1;
    for (int r = 0; r < s->rows; r++) {
        hp[r].uniform = uniforms[r];
        if (!s->ended[r]) {
            const int k = hp[r].top_k < s->vocab ? hp[r].top_k : s->vocab;  // sampler.go:147
            if (!mantle_internal_argmax_shortcut(hp[r]) && k > max_k) max_k = k;
        }
    }
    e = cudaMemcpyAsync(s->d_params, hp, (size_t)s->rows * sizeof(MantleSampleParams), cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(s->params_free[t], stream);
    if (e != cudaSuccess) return (int)e;

    MantleSampleBatch b;
    memset(&b, 0, sizeof b);
    b.logits = dev_logits;
    b.dtype = dtype;
    b.rows = s->rows;
    b.vocab = s->vocab;
    b.max_top_k = max_k;
    b.row_stride = row_stride;
    b.history = s->d_history;
    b.hist_len = s->d_hist_len;
    b.hist_stride = s->cap;
    b.exclude = s->n_stop > 0 ? s->d_stop : nullptr;  // excludePenalty = StopTokens (engine.go:233)
    b.n_exclude = s->n_stop;
    b.params = s->d_params;
    b.next = s->d_next;
    b.status = s->d_status;
    b.skip = s->d_ended;
    b.logit_scale = logit_scale;
    b.logit_softcap = logit_softcap;
    size_t need = 0;
    int rc = mantleCudaSamplerWorkspaceBytes(&b, &need);
    if (rc) return rc;
    if (need > s->d_ws_bytes) return kInvalid;
    rc = mantleCudaSampleRows(&b, need ? s->d_ws : nullptr, need, stream_);
    if (rc) return rc;
    // toks = append(toks, next), or the end of the row on a stop token (engine.go:244-250)
    rc = mantleCudaHistoryAppendRows(s->d_history, s->d_hist_len, s->cap, s->rows, s->d_next, s->keep,
                                     s->n_stop > 0 ? s->d_stop : nullptr, s->n_stop, s->d_ended, stream_);
    if (rc) return rc;
    e = cudaMemcpyAsync(s->h_next, s->d_next, (size_t)s->rows * 4, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s->h_ended, s->d_ended, (size_t)s->rows * 4, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s->h_status, s->d_status, 4, cudaMemcpyDeviceToHost, stream);
    return (int)e;
}

extern "C" int mantleBatchSamplerResults(MantleBatchSampler* s, const int32_t** next, const int32_t** ended,
                                         int32_t* status, const int32_t** dev_next) {
    if (!s) return kInvalid;
    for (int r = 0; r < s->rows; r++) s->ended[r] = s->h_ended[r] != 0;
    if (next) *next = s->h_next;
    if (ended) *ended = s->h_ended;
    if (status) *status = *s->h_status;
    if (dev_next) *dev_next = s->d_next;
    return 0;
}
