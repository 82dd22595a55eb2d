// Per-row set-up shared by the kernels: a row's parameters, its k and its geometry, the penalty
// bitmap of the history window, and the small kernels beside the sampler (in-place penalty,
// history append, head post-processing).
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

__device__ __forceinline__ MantleSampleParams row_params(const KArgs& a, int row) {
    MantleSampleParams P;
    if (a.params) {
        P = a.params[row];
    } else {  // plain argmax of every row
        P.temperature = 1.0f; P.top_p = 1.0f; P.min_p = 0.0f; P.repeat_penalty = 1.0f;
        P.top_k = 1; P.repeat_last_n = 1; P.greedy = 1; P.reserved = 0; P.uniform = 0.0;
    }
    return P;
}

// The effective shortlist length of a row and whether it takes the argmax shortcut.
__device__ __forceinline__ int row_k(const KArgs& a, const MantleSampleParams& P, int kcap, bool* greedy, bool* bad) {
    // sampler.go:140: greedy, or the top-1 / top_p >= 1 / temperature == 1 shortcut
    *greedy = P.greedy != 0 || (P.top_k == 1 && P.top_p >= 1.0f && P.temperature == 1.0f);
    int k = *greedy ? 1 : min(P.top_k, a.vocab_total);  // sampler.go:147
    *bad = false;
    if (!*greedy && (k > a.max_top_k || k > kcap || k < 1)) {
        *bad = true;
        k = max(1, min(min(k, a.max_top_k), kcap));
    }
    return k;
}

// Which part of a row one work item (row, split) covers.
template <typename T, class S>
struct ItemGeom {
    const uint4* vbase;  // the row rounded down to 16 bytes
    const void* row;
    int mis;       // elements between vbase and the row pointer
    int a0, b0;    // complete vectors [a0, b0) of this item
    int elo, ehi;  // columns [elo, ehi) of this item
    int nchunks;   // regions of NT * U vectors
};

template <typename T, class S>
__device__ __forceinline__ ItemGeom<T, S> item_geom(const KArgs& a, int item) {
    constexpr int VEC = Elem<T>::VEC;
    constexpr int CV = S::NT * S::U;
    ItemGeom<T, S> g;
    const int row = item / a.splits;
    const int split = item - row * a.splits;
    g.row = reinterpret_cast<const T*>(a.logits) + (size_t)row * (size_t)a.row_stride;
    g.mis = (int)((reinterpret_cast<uintptr_t>(g.row) & 15u) / sizeof(T));
    g.vbase = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(g.row) - (size_t)g.mis * sizeof(T));
    const int nvec = (g.mis + a.vocab + VEC - 1) / VEC;
    const int per = (nvec + a.splits - 1) / a.splits;
    const int vlo = min(split * per, nvec);
    const int vhi = min(vlo + per, nvec);
    g.elo = max(vlo * VEC - g.mis, 0);
    g.ehi = min(vhi * VEC - g.mis, a.vocab);
    g.a0 = max(vlo, g.mis != 0 ? 1 : 0);
    g.b0 = min(vhi, (g.mis + a.vocab) / VEC);
    g.nchunks = g.b0 > g.a0 ? (g.b0 - g.a0 + CV - 1) / CV : 0;
    return g;
}

// ---------------------------------------------------------------------------------------
// The repeat penalty (sampler.go:99-138): the bitmap of the de-duplicated history window.

// The history window of one row.
struct WinPlan {
    bool active;  // the penalty runs on this row (sampler.go:99)
    int start;    // window = ids [start, hl) of the row's history (sampler.go:100-101)
};

__device__ __forceinline__ WinPlan win_plan(const MantleSampleParams& P, int hl) {
    WinPlan w;
    w.active = P.repeat_penalty > 1.0f && hl > 0;
    w.start = max(hl - P.repeat_last_n, 0);
    return w;
}

__device__ void build_penalty_bitmap(const KArgs& a, int row, const WinPlan& w, int hl, int V, int voff,
                                     uint32_t* bm, int tid, int nt) {
    const int nwords = (int)bitmap_words(V);
    for (int i = tid; i < nwords; i += nt) bm[i] = 0;
    __syncthreads();
    const int32_t* h = a.history + (size_t)row * (size_t)a.hist_stride;
    for (int j = w.start + tid; j < hl; j += nt) {
        int id = h[j];
        if (id >= 0 && id < a.vocab_total) {  // sampler.go:116
            id -= voff;
            if (id >= 0 && id < V) atomicOr(&bm[id >> 5], 1u << (id & 31));
        }
    }
    __syncthreads();
    for (int j = tid; j < a.n_exclude; j += nt) {  // sampler.go:122-126
        int id = a.exclude[j];
        if (id >= 0 && id < a.vocab_total) {
            id -= voff;
            if (id >= 0 && id < V) atomicAnd(&bm[id >> 5], ~(1u << (id & 31)));
        }
    }
    __syncthreads();
}

// The same bitmap for the streaming kernels, arranged for latency.  The most recent HIST_PRE * NT ids of
// the row's history are requested at the very start of the kernel (history_tail), before the row's
// parameters -- which say how long the window is -- have arrived, so that the two loads travel together
// instead of one behind the other (measured under load: several thousand cycles each); they also travel
// while the bitmap is zeroed (with 16-byte stores).  The barrier after the clears is the caller's.
constexpr int HIST_PRE = 4;
template <int NT>
__device__ __forceinline__ void history_tail(const KArgs& a, int row, int hl, int tid, int (&ids)[HIST_PRE]) {
    const int32_t* h = a.history + (size_t)row * (size_t)a.hist_stride;
#pragma unroll
    for (int u = 0; u < HIST_PRE; u++) {
        const int j = hl - 1 - (u * NT + tid);
        ids[u] = j >= 0 ? __ldg(h + j) : -1;
    }
}
template <int NT>
__device__ __forceinline__ void build_penalty_bitmap_early(const KArgs& a, int row, const WinPlan& w, int hl, int V,
                                                           int voff, uint32_t* bm, int tid, const int (&ids)[HIST_PRE]) {
    const int32_t* h = a.history + (size_t)row * (size_t)a.hist_stride;
    uint4* bm4 = reinterpret_cast<uint4*>(bm);
    const int nvec = (int)(bitmap_words(V) / 4);
    for (int i = tid; i < nvec; i += NT) bm4[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    auto mark = [&](int id) {
        if (id >= 0 && id < a.vocab_total) {  // sampler.go:116
            id -= voff;
            if (id >= 0 && id < V) atomicOr(&bm[id >> 5], 1u << (id & 31));
        }
    };
#pragma unroll
    for (int u = 0; u < HIST_PRE; u++)
        if (hl - 1 - (u * NT + tid) >= w.start) mark(ids[u]);  // inside the window (sampler.go:100-101)
    for (int j = w.start + tid; j < hl - HIST_PRE * NT; j += NT) mark(h[j]);  // what a longer window holds beyond
    if (a.n_exclude > 0) {  // sampler.go:122-126, after every set
        __syncthreads();
        for (int j = tid; j < a.n_exclude; j += NT) {
            int id = a.exclude[j];
            if (id >= 0 && id < a.vocab_total) {
                id -= voff;
                if (id >= 0 && id < V) atomicAnd(&bm[id >> 5], ~(1u << (id & 31)));
            }
        }
    }
}

__device__ __forceinline__ int history_len(const KArgs& a, int row) {
    if (!a.history || (a.flags & MANTLE_SAMPLE_PENALTY_PREAPPLIED)) return 0;
    int hl = a.hist_len ? a.hist_len[row] : a.hist_stride;
    return max(0, min(hl, a.hist_stride));
}

// The penalty alone, in place: one CTA per row rewrites each flagged logit once.
constexpr int PENALTY_NT = 512;

__global__ void __launch_bounds__(PENALTY_NT) penalty_rows_kernel(const KArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint32_t* bm = reinterpret_cast<uint32_t*>(smem_raw);
    const int tid = threadIdx.x;
    const int row = blockIdx.x;
    const MantleSampleParams P = row_params(a, row);
    const int hl = history_len(a, row);
    const WinPlan w = win_plan(P, hl);
    if (!w.active) return;
    build_penalty_bitmap(a, row, w, hl, a.vocab, a.vocab_offset, bm, tid, PENALTY_NT);
    float* wrow = const_cast<float*>(reinterpret_cast<const float*>(a.logits)) + (size_t)row * (size_t)a.row_stride;
    const int nwords = (int)bitmap_words(a.vocab);
    for (int i = tid; i < nwords; i += PENALTY_NT) {
        uint32_t bits = bm[i];
        while (bits) {
            int b = __ffs(bits) - 1;
            bits &= bits - 1;
            int e = i * 32 + b;
            wrow[e] = penalise(wrow[e], P.repeat_penalty);
        }
    }
}

// The decode loop's `toks = append(toks, next)` (inference/engine.go:244-250) for a batch whose
// histories live on the device: one warp per row.  A row whose token is a stop token (or
// negative: the sampler reported an error) is marked done and left alone, as the reference
// leaves the loop before it appends; rows already done stay untouched.  A full buffer first
// moves its `keep` most recent ids to the front (keep <= hist_stride / 2, so the two ranges
// never overlap): the penalty window, the last repeat_last_n ids, is unchanged while keep
// covers it.
__global__ void __launch_bounds__(256) history_append_rows_kernel(int32_t* history, int32_t* hist_len, int hist_stride,
                                                                  int rows, const int32_t* next, int keep,
                                                                  const int32_t* stop, int n_stop, int32_t* done) {
    const int row = (int)((blockIdx.x * (unsigned)blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    if (done && done[row] != 0) return;
    const int tok = next[row];
    bool is_stop = tok < 0;
    for (int j = lane; j < n_stop; j += 32) is_stop |= stop[j] == tok;
    is_stop = __any_sync(0xffffffffu, is_stop);
    if (is_stop) {
        if (done && lane == 0) done[row] = 1;
        return;
    }
    int32_t* h = history + (size_t)row * (size_t)hist_stride;
    int len = min(max(hist_len[row], 0), hist_stride);
    if (len == hist_stride) {
        for (int j = lane; j < keep; j += 32) h[j] = h[len - keep + j];
        len = keep;
        __syncwarp();
    }
    if (lane == 0) {
        h[len] = tok;
        hist_len[row] = len + 1;
    }
}

// The post-processing alone, in place: what the reference does to the whole logits vector before
// it samples (simd/runtime.go:258-272; device form native/softmax.cu:963-970).  For callers that
// want the rewritten logits; the sampler itself applies it on the fly and writes nothing.
__global__ void __launch_bounds__(256) postprocess_rows_kernel(float* logits, int rows, int vocab, int64_t row_stride,
                                                               Post post) {
    const int64_t n = (int64_t)rows * vocab;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vocab;
        float* p = logits + r * row_stride + (i - r * vocab);
        *p = post_logit(*p, post);
    }
}

}  // namespace
