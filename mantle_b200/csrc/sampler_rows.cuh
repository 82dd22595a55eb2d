// Per-row set-up shared by the kernels: the penalty bitmap of the history window, the
// in-place penalty, history append and head post-processing kernels, a row's geometry and its k.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// ---------------------------------------------------------------------------------------
// The repeat penalty (sampler.go:99-138): the bitmap of the de-duplicated history window.

// The history window of one row and how it reaches the CTA.
struct WinPlan {
    bool active;  // the penalty runs on this row (sampler.go:99)
    bool staged;  // the window is copied to shared memory ahead of time
    int start;    // window = ids [start, hl) of the row's history (sampler.go:100-101)
    int a4, n4;   // 16-byte aligned superset [a4, a4 + n4) that the copy moves
};

__device__ __forceinline__ WinPlan win_plan(const KArgs& a, const MantleSampleParams& P, int hl) {
    WinPlan w;
    w.active = P.repeat_penalty > 1.0f && hl > 0;
    w.start = max(hl - P.repeat_last_n, 0);
    w.a4 = w.start & ~3;
    w.n4 = min((hl + 3) & ~3, a.hist_stride) - w.a4;
    w.staged = w.active && a.hist_tma_ok && w.n4 > 0 && w.n4 <= HIST_CAP;
    return w;
}

__device__ void build_penalty_bitmap(const KArgs& a, int row, const WinPlan& w, int hl, const int32_t* win, int V,
                                     int voff, uint32_t* bm, int tid, int nt) {
    const int nwords = (int)bitmap_words(V);
    for (int i = tid; i < nwords; i += nt) bm[i] = 0;
    __syncthreads();
    const int32_t* h = w.staged ? win - w.a4 : a.history + (size_t)row * (size_t)a.hist_stride;
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

// The same bitmap for the plain-load kernel, arranged for latency: the window's ids are requested
// first and travel while the bitmap is zeroed (with 16-byte stores); the barrier after the clears
// is the caller's.  (Measured: the bitmap phase cost a tenth of the kernel's time before.)
template <int NT>
__device__ __forceinline__ void build_penalty_bitmap_early(const KArgs& a, int row, const WinPlan& w, int hl, int V,
                                                           int voff, uint32_t* bm, int tid) {
    constexpr int PRE = 4;  // ids per thread fetched ahead: windows of up to PRE * NT ids
    const int32_t* h = a.history + (size_t)row * (size_t)a.hist_stride;
    int ids[PRE];
#pragma unroll
    for (int u = 0; u < PRE; u++) {
        const int j = w.start + u * NT + tid;
        ids[u] = j < hl ? __ldg(h + j) : -1;
    }
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
    for (int u = 0; u < PRE; u++) mark(ids[u]);
    for (int j = w.start + PRE * NT + tid; j < hl; j += NT) mark(h[j]);
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
    WinPlan w = win_plan(a, P, hl);
    if (!w.active) return;
    w.staged = false;
    build_penalty_bitmap(a, row, w, hl, nullptr, a.vocab, a.vocab_offset, bm, tid, PENALTY_NT);
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

}  // namespace
