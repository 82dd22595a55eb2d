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

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/mantle_cuda_sampler.h"

namespace {

constexpr int KMAX = MANTLE_SAMPLE_MAX_TOP_K;
constexpr int SLOW_EPT = 4;   // columns per thread per step of the careful path
constexpr int RANK_MAX = 256; // largest buffer the counting select takes

// Launch shape of one kernel instantiation.
//   NT    threads per CTA            U     16-byte vectors per thread per region
//   CAP   candidate buffer entries   KCAP  largest top_k this shape serves
//   MINB  CTAs per SM the register budget is held to
template <int NT_, int U_, int CAP_, int KCAP_, int MINB_>
struct Shape {
    static constexpr int NT = NT_, U = U_, CAP = CAP_, KCAP = KCAP_, MINB = MINB_;
    static constexpr int NWARP = NT / 32;
    static constexpr int EPT = CAP / NT;  // candidate entries per thread during compaction
    static_assert(KCAP + NT * SLOW_EPT <= CAP, "careful path needs room for one full step");
    static_assert(KCAP * 24 <= CAP * 8, "ordered shortlist must fit behind the survivors");
    static_assert(RANK_MAX <= NT, "counting select: one entry per thread");
    // shared memory: [Cand buf[CAP]] [hist[256]] [Ctl] [bitmap words]
    static constexpr size_t SMEM_FIXED = 8 * (size_t)CAP + 4 * 256 + 512;
};
using ShapeSmallK = Shape<256, 4, 2048, 256, 4>;   // top_k <= 256: four CTAs per SM
using ShapeLargeK = Shape<512, 4, 4096, KMAX, 2>;  // top_k <= 1024: two CTAs per SM
constexpr int MAX_NWARP = 32;
constexpr int MERGE_CAP = ShapeLargeK::CAP;

constexpr int MODE_FUSED = 0;    // one CTA per row, tail in the same kernel
constexpr int MODE_PARTS = 1;    // several CTAs per row (or one vocabulary shard): write the local shortlist
constexpr int MODE_PENALTY = 2;  // repeat penalty only, in place

struct Cand {
    uint32_t key;  // order-preserving image of the scaled value
    uint32_t idx;  // token id (global)
};

// Per-CTA control block in shared memory.
struct Ctl {
    int cnt;            // live entries in the candidate buffer
    int sel_bin;        // radix select: chosen digit
    int sel_need;       //               entries still wanted inside the chosen digit
    int sel_cnt;        //               entries inside the chosen digit
    uint32_t kmin, kmax;
    int n_after;        // shortlist length after min-p
    int cut;
    int pos;
    int pad;
    double sum;
    double new_sum;
    float warpv[MAX_NWARP];
    uint32_t warpk_min[MAX_NWARP];
    uint32_t warpk_max[MAX_NWARP];
};
static_assert(sizeof(Ctl) <= 512, "control block outgrew its slot");

struct KArgs {
    const void* logits;
    int64_t row_stride;
    int rows;
    int vocab;         // columns held here
    int vocab_offset;  // global id of column 0
    int vocab_total;   // width of the whole row (for k = min(top_k, V))
    const int32_t* history;
    const int32_t* hist_len;
    int hist_stride;
    int n_exclude;
    const int32_t* exclude;
    const MantleSampleParams* params;  // NULL: every row is a plain argmax
    int splits;
    int max_top_k;
    uint32_t flags;
    int32_t* next;
    int32_t* cand_idx;
    double* cand_prob;
    int32_t* n_kept;
    int32_t* cut;
    int32_t* status;
    int cand_stride;
    // MODE_PARTS outputs / merge inputs: part p of row r at (p*rows + r)*part_cap
    float* part_val;
    int32_t* part_idx;
    int32_t* part_cnt;
    int part_cap;
    int parts;
};

// ---------------------------------------------------------------------------------------
// small helpers

__device__ __forceinline__ uint32_t f2key(float v) {
    v = __fadd_rn(v, 0.0f);  // -0.0 -> +0.0: the reference compares floats, for which they are equal
    uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float key2f(uint32_t k) {
    uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

// fastExp, sampler.go:10-31, operation for operation in float32.
__device__ __forceinline__ float fast_exp(float x) {
    if (x > 88.0f) return 3.4028235e38f;
    if (x < -88.0f) return 0.0f;
    const float ln2 = 0.693147180559945309417f;
    const float ln2inv = 1.44269504088896340736f;
    float t = __fmul_rn(x, ln2inv);
    int k = (x < 0.0f) ? __float2int_rz(__fsub_rn(t, 0.5f)) : __float2int_rz(__fadd_rn(t, 0.5f));
    float r = __fsub_rn(x, __fmul_rn((float)k, ln2));
    float r2 = __fmul_rn(r, r);
    float r3 = __fmul_rn(r2, r);
    float r4 = __fmul_rn(r2, r2);
    float poly = __fadd_rn(1.0f, r);
    poly = __fadd_rn(poly, __fmul_rn(r2, 0.5f));
    poly = __fadd_rn(poly, __fmul_rn(r3, 0.16666667f));
    poly = __fadd_rn(poly, __fmul_rn(r4, 0.041666667f));
    poly = __fadd_rn(poly, __fmul_rn(__fmul_rn(r4, r), 0.008333333f));
    float scale = __uint_as_float((uint32_t)(k + 127) << 23);
    return __fmul_rn(poly, scale);
}

// sampler.go:132-136
__device__ __forceinline__ float penalise(float l, float p) {
    return l > 0.0f ? __fdiv_rn(l, p) : __fmul_rn(l, p);
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
    static constexpr int VEC = 4;
    __device__ static __forceinline__ void widen(const uint4& r, float* o) {
        o[0] = __uint_as_float(r.x);
        o[1] = __uint_as_float(r.y);
        o[2] = __uint_as_float(r.z);
        o[3] = __uint_as_float(r.w);
    }
    __device__ static __forceinline__ float load1(const void* p, int64_t e) {
        return __ldcs(reinterpret_cast<const float*>(p) + e);
    }
};
struct bf16_t {
    uint16_t bits;
};
template <>
struct Elem<bf16_t> {
    static constexpr int VEC = 8;
    __device__ static __forceinline__ void widen(const uint4& r, float* o) {
        o[0] = __uint_as_float(r.x << 16);
        o[1] = __uint_as_float(r.x & 0xffff0000u);
        o[2] = __uint_as_float(r.y << 16);
        o[3] = __uint_as_float(r.y & 0xffff0000u);
        o[4] = __uint_as_float(r.z << 16);
        o[5] = __uint_as_float(r.z & 0xffff0000u);
        o[6] = __uint_as_float(r.w << 16);
        o[7] = __uint_as_float(r.w & 0xffff0000u);
    }
    __device__ static __forceinline__ float load1(const void* p, int64_t e) {
        uint16_t h = __ldcs(reinterpret_cast<const uint16_t*>(p) + e);
        return __uint_as_float((uint32_t)h << 16);
    }
};

// What a CTA knows about its row while it streams.
struct RowCtx {
    const void* row;      // row pointer
    int mis;              // elements between the 16-byte boundary below the row pointer and the pointer
    int V;                // columns
    int voff;             // global id of column 0
    float inv_temp;
    float pen;
    bool pen_bitmap;      // the penalty is applied from the bitmap (logits stay read-only)
    const uint32_t* bm;   // bitmap, bit e set: column e is penalised
};

__device__ __forceinline__ bool bm_test(const uint32_t* bm, int e) { return (bm[e >> 5] >> (e & 31)) & 1u; }

__device__ __forceinline__ int live_count(const Ctl* ctl) {
    return *reinterpret_cast<const volatile int*>(&ctl->cnt);
}

template <class S>
__device__ __forceinline__ void append(Cand* buf, Ctl* ctl, float v, int gidx) {
    int slot = atomicAdd(&ctl->cnt, 1);
    if (slot < S::CAP) {
        Cand e;
        e.key = f2key(v);
        e.idx = (uint32_t)gidx;
        buf[slot] = e;
    }
}

// One column whose scaled RAW value reached the filter.  The penalty only ever lowers a
// logit (l/p < l for l > 0, l*p < l for l < 0, p > 1), so filtering raw values first is
// conservative: only here, on the rare survivor, is the bitmap consulted, the penalty
// applied and the filter repeated on the true value.
template <class S, bool INCL>
__device__ __forceinline__ void consider(Cand* buf, Ctl* ctl, const RowCtx& c, float raw, float v, int e, float thr) {
    if (c.pen_bitmap && bm_test(c.bm, e)) {
        v = __fmul_rn(penalise(raw, c.pen), c.inv_temp);
        if (!(INCL ? v >= thr : v > thr)) return;
    }
    append<S>(buf, ctl, v, e + c.voff);
}

// The largest scaled value of one complete vector, with the penalty applied to the flagged
// columns: used for the first region only, whose thread-maxima seed the threshold.
template <typename T>
__device__ __forceinline__ float vec_max_penalised(const uint4& rawv, int vec, const RowCtx& c) {
    constexpr int VEC = Elem<T>::VEC;
    float raw[VEC];
    Elem<T>::widen(rawv, raw);
    const int e0 = vec * VEC - c.mis;
    float m = __uint_as_float(0xff800000u);
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        float l = raw[j];
        if (c.pen_bitmap && bm_test(c.bm, e0 + j)) l = penalise(l, c.pen);
        m = fmaxf(m, __fmul_rn(l, c.inv_temp));
    }
    return m;
}

// The hot loop body: one complete 16-byte vector.  Scale, take the maximum, and leave
// unless some column reaches the threshold (NaN never does; fmaxf ignores it).  The rare
// survivors are walked one at a time so that the slow code exists once per vector.
template <class S, typename T, bool INCL>
__device__ __forceinline__ void filter_vec(const uint4& rawv, int vec, const RowCtx& c, float thr, Cand* buf,
                                           Ctl* ctl) {
    constexpr int VEC = Elem<T>::VEC;
    float raw[VEC];
    Elem<T>::widen(rawv, raw);
    float m = __fmul_rn(raw[0], c.inv_temp);
#pragma unroll
    for (int j = 1; j < VEC; j++) m = fmaxf(m, __fmul_rn(raw[j], c.inv_temp));
    if (INCL ? m >= thr : m > thr) {
        uint32_t pass = 0;
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            float x = __fmul_rn(raw[j], c.inv_temp);
            pass |= (INCL ? x >= thr : x > thr) ? (1u << j) : 0u;
        }
        const int e0 = vec * VEC - c.mis;
        while (pass) {
            const int j = __ffs(pass) - 1;
            pass &= pass - 1;
            float r = raw[0];
#pragma unroll
            for (int q = 1; q < VEC; q++) r = (j == q) ? raw[q] : r;
            consider<S, INCL>(buf, ctl, c, r, __fmul_rn(r, c.inv_temp), e0 + j, thr);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Shared-memory radix select: cut the candidate buffer to its k best entries in the order
// (key descending, index ascending).  Called by every thread of the CTA with the buffer
// quiescent (a barrier after the last append).  Leaves min(k, n) entries, unordered, and
// returns the key of the k-th one when n > k (*have_kth set).
//
// Digits are taken from (key - smallest key), most significant first, so the first
// histogram already spreads the candidates over up to 256 bins however narrow their
// value range is.  Ties at the k-th key are resolved by a second select over the index.
template <class S>
__device__ __noinline__ uint32_t select_topk(Cand* buf, Ctl* ctl, uint32_t* hist, int k, int tid, bool* have_kth) {
    constexpr int NT = S::NT, NWARP = S::NWARP, EPT = S::EPT;
    const int lane = tid & 31, warp = tid >> 5;
    __syncthreads();
    const int n = min(live_count(ctl), S::CAP);
    __syncthreads();  // every thread has read the count before a caller may append again
    *have_kth = false;
    if (n <= k) return 0;

    // range of the keys
    uint32_t lo = 0xffffffffu, hi = 0;
    for (int i = tid; i < n; i += NT) {
        uint32_t key = buf[i].key;
        lo = min(lo, key);
        hi = max(hi, key);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane == 0) {
        ctl->warpk_min[warp] = lo;
        ctl->warpk_max[warp] = hi;
    }
    __syncthreads();
    lo = ctl->warpk_min[0];
    hi = ctl->warpk_max[0];
#pragma unroll
    for (int w = 1; w < NWARP; w++) {
        lo = min(lo, ctl->warpk_min[w]);
        hi = max(hi, ctl->warpk_max[w]);
    }
    const uint32_t range = hi - lo;
    int rem = range == 0 ? 0 : 32 - __clz(range);  // significant bits of (key - lo)

    int need = k;           // entries wanted among those matching the prefix
    int ties = n;           // entries matching the whole prefix so far
    uint32_t prefix = 0;    // chosen high bits of (key - lo)
    while (rem > 0) {
        const int d = rem < 8 ? rem : 8;
        const int shift = rem - d;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i = tid; i < n; i += NT) {
            uint32_t o = buf[i].key - lo;
            uint32_t hi_bits = rem >= 32 ? 0u : (o >> rem);  // a 32-bit shift by 32 must give 0
            if (hi_bits == prefix) atomicAdd(&hist[(o >> shift) & ((1u << d) - 1u)], 1u);
        }
        __syncthreads();
        if (warp == 0) {
            // lane L owns bins 8L..8L+7; find the bin where the count from the top reaches `need`
            uint32_t c[8];
            uint32_t tot = 0;
#pragma unroll
            for (int b = 0; b < 8; b++) {
                c[b] = hist[lane * 8 + b];
                tot += c[b];
            }
            uint32_t above = tot;  // inclusive suffix sum over lanes >= me
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t y = __shfl_down_sync(0xffffffffu, above, o);
                if (lane + o < 32) above += y;
            }
            above -= tot;  // exclusive: entries in bins owned by higher lanes
            if (above < (uint32_t)need && (uint32_t)need <= above + tot) {
                uint32_t run = above;
#pragma unroll
                for (int b = 7; b >= 0; b--) {
                    if (run < (uint32_t)need && (uint32_t)need <= run + c[b]) {
                        ctl->sel_bin = lane * 8 + b;
                        ctl->sel_need = need - (int)run;
                        ctl->sel_cnt = (int)c[b];
                    }
                    run += c[b];
                }
            }
        }
        __syncthreads();
        prefix = (prefix << d) | (uint32_t)ctl->sel_bin;
        need = ctl->sel_need;
        ties = ctl->sel_cnt;
        rem = shift;
    }
    const uint32_t kth = lo + prefix;

    // `ties` entries carry the k-th key and `need` of them are wanted: the lowest indices.
    uint32_t idx_max = 0xffffffffu;
    if (need < ties) {
        int irem = 32;
        uint32_t iprefix = 0;
        int ineed = need;
        while (irem > 0) {
            const int shift = irem - 8;
            if (tid < 256) hist[tid] = 0;
            __syncthreads();
            for (int i = tid; i < n; i += NT) {
                Cand e = buf[i];
                uint32_t hi_bits = irem >= 32 ? 0u : (e.idx >> irem);
                if (e.key == kth && hi_bits == iprefix) atomicAdd(&hist[(e.idx >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (warp == 0) {
                uint32_t c[8];
                uint32_t tot = 0;
#pragma unroll
                for (int b = 0; b < 8; b++) {
                    c[b] = hist[lane * 8 + b];
                    tot += c[b];
                }
                uint32_t below = tot;  // inclusive prefix sum over lanes <= me
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    uint32_t y = __shfl_up_sync(0xffffffffu, below, o);
                    if (lane >= o) below += y;
                }
                below -= tot;
                if (below < (uint32_t)ineed && (uint32_t)ineed <= below + tot) {
                    uint32_t run = below;
#pragma unroll
                    for (int b = 0; b < 8; b++) {
                        if (run < (uint32_t)ineed && (uint32_t)ineed <= run + c[b]) {
                            ctl->sel_bin = lane * 8 + b;
                            ctl->sel_need = ineed - (int)run;
                        }
                        run += c[b];
                    }
                }
            }
            __syncthreads();
            iprefix = (iprefix << 8) | (uint32_t)ctl->sel_bin;
            ineed = ctl->sel_need;
            irem = shift;
        }
        idx_max = iprefix;  // indices are unique: exactly `need` tied entries have idx <= idx_max
    }

    // compaction through registers (reads and writes overlap in the buffer)
    Cand mine[EPT];
    uint32_t keep = 0;
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        int i = tid + j * NT;
        if (i < n) {
            mine[j] = buf[i];
            if (mine[j].key > kth || (mine[j].key == kth && mine[j].idx <= idx_max)) keep |= 1u << j;
        }
    }
    __syncthreads();
    if (tid == 0) ctl->cnt = 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        if ((keep >> j) & 1u) {
            int slot = atomicAdd(&ctl->cnt, 1);
            buf[slot] = mine[j];
        }
    }
    __syncthreads();
    *have_kth = true;
    return kth;
}

// Exact cut for a small buffer (n <= RANK_MAX entries): every entry counts the entries that
// precede it in the order (key descending, index ascending) and moves to that position,
// which leaves the best min(k, n) entries in order.  Two barriers, no atomics.
__device__ __forceinline__ uint32_t rank_select(Cand* buf, Ctl* ctl, int n, int k, int tid, bool* have_kth) {
    Cand me;
    me.key = 0;
    me.idx = 0;
    int rank = 0x7fffffff;
    if (tid < n) {
        me = buf[tid];
        rank = 0;
        for (int j = 0; j < n; j++) {
            Cand o = buf[j];
            rank += (o.key > me.key || (o.key == me.key && o.idx < me.idx)) ? 1 : 0;
        }
    }
    __syncthreads();
    if (rank < k) buf[rank] = me;
    if (rank == k - 1) ctl->sel_bin = (int)me.key;
    if (tid == 0) ctl->cnt = min(n, k);
    __syncthreads();
    *have_kth = n >= k;
    return (uint32_t)ctl->sel_bin;
}

// Cut the buffer to its k best entries, by counting when it is small and by radix select
// otherwise.  Called by every thread with the buffer quiescent.
template <class S>
__device__ __forceinline__ uint32_t refresh_topk(Cand* buf, Ctl* ctl, uint32_t* hist, int k, int tid,
                                                 bool* have_kth) {
    __syncthreads();
    const int n = live_count(ctl);
    __syncthreads();
    if (n <= RANK_MAX) return rank_select(buf, ctl, n, k, tid, have_kth);
    return select_topk<S>(buf, ctl, hist, k, tid, have_kth);
}

// Orders the n <= KCAP entries of the buffer (key descending, index ascending) by
// counting, into sval/sidx.  Entries are distinct under that order, so ranks are a
// permutation.
template <class S>
__device__ void rank_sort(const Cand* buf, int n, float* sval, int32_t* sidx, int tid) {
    for (int i = tid; i < n; i += S::NT) {
        Cand me = buf[i];
        int rank = 0;
        for (int j = 0; j < n; j++) {
            Cand o = buf[j];
            rank += (o.key > me.key || (o.key == me.key && o.idx < me.idx)) ? 1 : 0;
        }
        sval[rank] = key2f(me.key);
        sidx[rank] = (int32_t)me.idx;
    }
}

// The tail of Sampler.Sample, sampler.go:154-233, on the ordered shortlist in shared
// memory.  Probabilities are doubles summed in shortlist order by one thread, which is
// what makes the result identical to the reference's; everything elementwise is spread
// over the CTA.
template <class S>
__device__ void sample_tail(const KArgs& a, int row, const MantleSampleParams& P, bool greedy, int n,
                            float* sval, int32_t* sidx, double* sprob, Ctl* ctl, int tid) {
    constexpr int NT = S::NT;
    if (n == 0) {  // only an all-NaN row ends here; the reference's behaviour there is undefined
        if (tid == 0) {
            a.next[row] = 0;
            if (a.n_kept) a.n_kept[row] = 0;
            if (a.cut) a.cut[row] = 0;
        }
        return;
    }
    if (greedy) {
        if (tid == 0) {
            a.next[row] = sidx[0];
            if (a.n_kept) a.n_kept[row] = 0;
            if (a.cut) a.cut[row] = 0;
        }
        return;
    }
    const float maxv = sval[0];
    for (int i = tid; i < n; i += NT) sprob[i] = (double)fast_exp(__fsub_rn(sval[i], maxv));
    __syncthreads();
    if (tid == 0) {
        double s = 0.0;
        for (int i = 0; i < n; i++) s = __dadd_rn(s, sprob[i]);
        ctl->sum = s;
    }
    __syncthreads();
    const double sum = ctl->sum;
    if (sum == 0.0) {  // sampler.go:170-172
        if (tid == 0) {
            a.next[row] = sidx[0];
            if (a.n_kept) a.n_kept[row] = n;
            if (a.cut) a.cut[row] = 0;
        }
        return;
    }
    const double inv = __ddiv_rn(1.0, sum);
    for (int i = tid; i < n; i += NT) sprob[i] = __dmul_rn(sprob[i], inv);
    __syncthreads();

    if (P.min_p > 0.0f) {  // sampler.go:180-210
        if (tid == 0) {
            const double thr = __dmul_rn(sprob[0], (double)P.min_p);
            int m = 0;
            double ns = 0.0;
            for (int i = 0; i < n; i++) {
                double p = sprob[i];
                if (p >= thr) {
                    sprob[m] = p;
                    sidx[m] = sidx[i];
                    ns = __dadd_rn(ns, p);
                    m++;
                }
            }
            ctl->n_after = m;
            ctl->new_sum = ns;
        }
        __syncthreads();
        const int m = ctl->n_after;
        if (m < n) {
            n = m;
            const double ns = ctl->new_sum;
            if (ns > 0.0) {
                const double sc = __ddiv_rn(1.0, ns);
                for (int i = tid; i < n; i += NT) sprob[i] = __dmul_rn(sprob[i], sc);
            }
            __syncthreads();
        }
    }

    if (tid == 0) {
        int token;
        int cut = n;
        if (n == 0) {  // min_p > 1 dropped everything: the reference indexes topIdx[-1] and panics
            token = -1;
            cut = 0;
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_EMPTY);
        } else {
            // sampler.go:212-233: the nucleus prefix and the inverse-CDF walk add the same
            // doubles in the same order, so one running sum serves both
            const bool nucleus = P.top_p < 1.0f;
            const double r = P.uniform;
            double c = 0.0;
            int pos = -1;
            for (int i = 0; i < n; i++) {
                c = __dadd_rn(c, sprob[i]);
                if (pos < 0 && r <= c) pos = i;
                if (nucleus && __double2float_rn(c) >= P.top_p) {
                    cut = i + 1;
                    break;
                }
                if (!nucleus && pos >= 0) break;
            }
            if (pos < 0) pos = cut - 1;
            token = sidx[pos];
        }
        a.next[row] = token;
        if (a.n_kept) a.n_kept[row] = n;
        if (a.cut) a.cut[row] = cut;
    }
    if (a.cand_idx || a.cand_prob) {
        const int m = min(n, a.cand_stride);
        for (int i = tid; i < m; i += NT) {
            if (a.cand_idx) a.cand_idx[(size_t)row * a.cand_stride + i] = sidx[i];
            if (a.cand_prob) a.cand_prob[(size_t)row * a.cand_stride + i] = sprob[i];
        }
    }
}

__host__ __device__ inline size_t bitmap_words(int vocab) { return (size_t)((vocab + 31) / 32 + 2); }

// After the select: order the survivors and either finish the row or publish the local
// shortlist.  The ordered arrays live in the part of the candidate buffer the survivors
// (at most KCAP entries) do not occupy.
template <class S, int MODE>
__device__ void finish_row(const KArgs& a, int row, int split, const MantleSampleParams& P, bool greedy,
                           Cand* buf, Ctl* ctl, int tid) {
    constexpr int KC = S::KCAP;
    const int n = min(ctl->cnt, KC);
    float* sval = reinterpret_cast<float*>(buf + KC);
    int32_t* sidx = reinterpret_cast<int32_t*>(sval + KC);
    double* sprob = reinterpret_cast<double*>(sidx + KC);
    rank_sort<S>(buf, n, sval, sidx, tid);
    __syncthreads();
    if (MODE == MODE_FUSED) {
        sample_tail<S>(a, row, P, greedy, n, sval, sidx, sprob, ctl, tid);
    } else {
        const size_t base = ((size_t)split * a.rows + row) * a.part_cap;
        const int m = min(n, a.part_cap);
        for (int i = tid; i < m; i += S::NT) {
            a.part_val[base + i] = sval[i];
            a.part_idx[base + i] = sidx[i];
        }
        if (tid == 0) a.part_cnt[(size_t)split * a.rows + row] = m;
    }
}

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

// ---------------------------------------------------------------------------------------
// The streaming kernel.

template <class S, typename T, int MODE>
__global__ void __launch_bounds__(S::NT, S::MINB) scan_rows_kernel(const KArgs a) {
    constexpr int VEC = Elem<T>::VEC;
    constexpr int NT = S::NT, NWARP = S::NWARP, U = S::U, CAP = S::CAP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(hist + 256);
    uint32_t* bm = reinterpret_cast<uint32_t*>(smem_raw + S::SMEM_FIXED);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x / a.splits;
    const int split = blockIdx.x - row * a.splits;

    // ---- the row's parameters --------------------------------------------------------
    const MantleSampleParams P = row_params(a, row);
    // sampler.go:140: greedy, or the top-1 / top_p >= 1 / temperature == 1 shortcut
    const bool greedy = P.greedy != 0 || (P.top_k == 1 && P.top_p >= 1.0f && P.temperature == 1.0f);
    int k = greedy ? 1 : min(P.top_k, a.vocab_total);  // sampler.go:147
    bool bad_k = false;
    if (!greedy && (k > a.max_top_k || k > S::KCAP || k < 1)) {
        bad_k = true;
        k = max(1, min(min(k, a.max_top_k), S::KCAP));
    }

    RowCtx c;
    c.row = reinterpret_cast<const T*>(a.logits) + (size_t)row * (size_t)a.row_stride;
    c.mis = (int)((reinterpret_cast<uintptr_t>(c.row) & 15u) / sizeof(T));
    c.V = a.vocab;
    c.voff = a.vocab_offset;
    c.inv_temp = greedy ? 1.0f : __fdiv_rn(1.0f, P.temperature);  // sampler.go:144-145
    c.pen = P.repeat_penalty;
    c.bm = bm;
    c.pen_bitmap = false;
    const uint4* vbase = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(c.row) -
                                                        (size_t)c.mis * sizeof(T));
    const int nvec = (c.mis + c.V + VEC - 1) / VEC;

    // This CTA's share of the row, in vectors and in columns.  Vectors [a0, b0) of the share
    // lie wholly inside the row and are streamed; the columns of the (at most two) partial
    // vectors at the row's ends are taken one by one afterwards.
    const int per = (nvec + a.splits - 1) / a.splits;
    const int vlo = min(split * per, nvec);
    const int vhi = min(vlo + per, nvec);
    const int elo = max(vlo * VEC - c.mis, 0);
    const int ehi = min(vhi * VEC - c.mis, c.V);
    constexpr int RV = NT * U;  // vectors per region
    const int a0 = max(vlo, c.mis != 0 ? 1 : 0);
    const int b0 = min(vhi, (c.mis + c.V) / VEC);
    const int nreg = b0 > a0 ? (b0 - a0 + RV - 1) / RV : 0;

    int hl = 0;
    if (a.history && !(a.flags & MANTLE_SAMPLE_PENALTY_PREAPPLIED)) {
        hl = a.hist_len ? a.hist_len[row] : a.hist_stride;
        hl = max(0, min(hl, a.hist_stride));
    }
    const bool pen_active = P.repeat_penalty > 1.0f && hl > 0;
    const bool in_place = MODE == MODE_PENALTY || (a.flags & MANTLE_SAMPLE_WRITE_BACK_PENALTY) != 0;
    bool careful = k > 32 * NWARP;

    // The first region's loads go out before anything else, so that they are in flight while
    // the bitmap is built -- unless the penalty is about to rewrite the row in place.
    uint4 ra[U], rb[U];
    const bool early = MODE != MODE_PENALTY && !careful && nreg > 0 && !(pen_active && in_place);
    if (early) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            int v = a0 + u * NT + tid;
            ra[u] = v < b0 ? __ldcs(vbase + v) : make_uint4(0, 0, 0, 0);
        }
    }
    if (tid == 0) ctl->cnt = 0;

    // ---- repeat penalty: bitmap of the de-duplicated window (sampler.go:99-138) --------
    if (pen_active) {
        const int nwords = (int)bitmap_words(c.V);
        for (int w = tid; w < nwords; w += NT) bm[w] = 0;
        __syncthreads();
        const int start = max(hl - P.repeat_last_n, 0);
        const int32_t* h = a.history + (size_t)row * (size_t)a.hist_stride;
        for (int j = start + tid; j < hl; j += NT) {
            int id = h[j];
            if (id >= 0 && id < a.vocab_total) {  // sampler.go:116
                id -= c.voff;
                if (id >= 0 && id < c.V) atomicOr(&bm[id >> 5], 1u << (id & 31));
            }
        }
        __syncthreads();
        for (int j = tid; j < a.n_exclude; j += NT) {  // sampler.go:122-126
            int id = a.exclude[j];
            if (id >= 0 && id < a.vocab_total) {
                id -= c.voff;
                if (id >= 0 && id < c.V) atomicAnd(&bm[id >> 5], ~(1u << (id & 31)));
            }
        }
        __syncthreads();
        if (in_place) {
            // the reference's in-place form: one read-modify-write per distinct id this CTA owns
            if (sizeof(T) == 4) {
                float* wrow = const_cast<float*>(reinterpret_cast<const float*>(c.row));
                for (int w = tid; w < nwords; w += NT) {
                    uint32_t bits = bm[w];
                    while (bits) {
                        int b = __ffs(bits) - 1;
                        bits &= bits - 1;
                        int e = w * 32 + b;
                        if (e >= elo && e < ehi) wrow[e] = penalise(wrow[e], c.pen);
                    }
                }
            }
        } else {
            c.pen_bitmap = true;
        }
    }
    if (MODE == MODE_PENALTY) return;
    __syncthreads();

    // ---- stream the row ------------------------------------------------------------------
    const int trig = min(k + max(k >> 1, 16), CAP / 2);  // refresh the threshold at this many entries
    float thr = __uint_as_float(0xff800000u);            // -inf

    if (!careful && nreg > 0) {
        if (!early) {
#pragma unroll
            for (int u = 0; u < U; u++) {
                int v = a0 + u * NT + tid;
                ra[u] = v < b0 ? __ldcs(vbase + v) : make_uint4(0, 0, 0, 0);
            }
        }
        // `load(dst, r)`: region r into dst (predicated: only the last region can be partial)
        auto load = [&](uint4(&dst)[U], int r) {
#pragma unroll
            for (int u = 0; u < U; u++) {
                int v = a0 + r * RV + u * NT + tid;
                dst[u] = v < b0 ? __ldcs(vbase + v) : make_uint4(0, 0, 0, 0);
            }
        };
        // `later(src, r)`: regions after the first.  The buffer already holds k entries >= thr
        // with lower indices, so an equal value can no longer enter (sampler.go:268-275).
        auto later = [&](const uint4(&src)[U], int r) {
            const int v0 = a0 + r * RV + tid;
            if (r + 1 < nreg) {
#pragma unroll
                for (int u = 0; u < U; u++) filter_vec<S, T, false>(src[u], v0 + u * NT, c, thr, buf, ctl);
            } else {
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (v0 + u * NT < b0) filter_vec<S, T, false>(src[u], v0 + u * NT, c, thr, buf, ctl);
            }
        };
        // One barrier per region.  The thread that made the last append of the region reads
        // the final count before it arrives, so the OR is the same for every thread.
        auto region_end = [&](int lim) {
            if (__syncthreads_or(live_count(ctl) >= lim)) {
                if (live_count(ctl) > CAP) {
                    careful = true;  // entries were dropped: start over on the careful path
                } else {
                    bool have;
                    uint32_t kth = refresh_topk<S>(buf, ctl, hist, k, tid, &have);
                    if (have) thr = key2f(kth);
                }
            }
        };

        // -- region 0 --
        if (nreg > 1) load(rb, 1);
        {
            // A threshold that at least k columns of this region reach: with
            // j = ceil(k / warps), every warp holds j thread-maxima >= its j-th largest one,
            // so the smallest of those per-warp values is reached by >= k columns.
            const int v0 = a0 + tid;
            float tmax = __uint_as_float(0xff800000u);
#pragma unroll
            for (int u = 0; u < U; u++)
                if (v0 + u * NT < b0) tmax = fmaxf(tmax, vec_max_penalised<T>(ra[u], v0 + u * NT, c));
            float x = tmax;  // bitonic sort across the warp, descending
#pragma unroll
            for (int k2 = 2; k2 <= 32; k2 <<= 1) {
#pragma unroll
                for (int j2 = k2 >> 1; j2 > 0; j2 >>= 1) {
                    float y = __shfl_xor_sync(0xffffffffu, x, j2);
                    bool desc = (lane & k2) == 0;
                    bool lower = (lane & j2) == 0;
                    x = (lower == desc) ? fmaxf(x, y) : fminf(x, y);
                }
            }
            const int j = (k + NWARP - 1) / NWARP;
            float wj = __shfl_sync(0xffffffffu, x, j - 1);
            if (lane == 0) ctl->warpv[warp] = wj;
            __syncthreads();
            float t0 = ctl->warpv[0];
#pragma unroll
            for (int w = 1; w < NWARP; w++) t0 = fminf(t0, ctl->warpv[w]);
            thr = t0;
#pragma unroll
            for (int u = 0; u < U; u++)
                if (v0 + u * NT < b0) filter_vec<S, T, true>(ra[u], v0 + u * NT, c, thr, buf, ctl);
        }
        region_end(k + 1);

        // -- regions 1.. : two register sets, each refilled while the other is filtered --
        int r = 1;
        while (r < nreg && !careful) {
            if (r + 1 < nreg) load(ra, r + 1);
            later(rb, r);
            region_end(trig);
            if (++r >= nreg || careful) break;
            if (r + 1 < nreg) load(rb, r + 1);
            later(ra, r);
            region_end(trig);
            ++r;
        }
    }

    if (!careful) {
        // the columns of the partial vectors at the ends of this CTA's share
        int r1_lo = elo, r1_hi = ehi, r2_lo = ehi, r2_hi = ehi;
        if (b0 > a0) {
            r1_hi = min(ehi, max(elo, a0 * VEC - c.mis));
            r2_lo = max(elo, b0 * VEC - c.mis);
        }
        const int n1 = r1_hi - r1_lo, n2 = r2_hi - r2_lo;
        if (tid < n1 + n2) {  // at most 4 * VEC columns
            int e = tid < n1 ? r1_lo + tid : r2_lo + (tid - n1);
            float raw = Elem<T>::load1(c.row, e);
            float v = __fmul_rn(raw, c.inv_temp);
            if (v >= thr) consider<S, true>(buf, ctl, c, raw, v, e, thr);
        }
        __syncthreads();
        if (live_count(ctl) > CAP) careful = true;
        __syncthreads();
    }

    if (careful) {
        // Careful path: any input, any order.  Steps of NT*SLOW_EPT columns with room for a
        // whole step guaranteed before it starts; the buffer is cut to k whenever it could
        // overflow.  Reached for k beyond 32 per warp, for rows whose first region ties
        // massively, and for adversarial orders (e.g. ascending logits).
        __syncthreads();
        if (tid == 0) ctl->cnt = 0;
        __syncthreads();
        thr = __uint_as_float(0xff800000u);
        bool strict = false;
        constexpr int STEP = NT * SLOW_EPT;
        for (int e0 = elo; e0 < ehi; e0 += STEP) {
            __syncthreads();
            if (ctl->cnt + STEP > CAP) {
                bool have;
                uint32_t kth = select_topk<S>(buf, ctl, hist, k, tid, &have);
                if (have) {
                    thr = key2f(kth);
                    strict = true;
                }
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < SLOW_EPT; j++) {
                int e = e0 + j * NT + tid;
                if (e < ehi) {
                    float l = Elem<T>::load1(c.row, e);
                    if (c.pen_bitmap && bm_test(bm, e)) l = penalise(l, c.pen);
                    float v = __fmul_rn(l, c.inv_temp);
                    if (strict ? (v > thr) : (v >= thr)) append<S>(buf, ctl, v, e + c.voff);
                }
            }
        }
        __syncthreads();
    }

    // ---- cut to k, order, finish ------------------------------------------------------------
    bool have;
    refresh_topk<S>(buf, ctl, hist, k, tid, &have);
    __syncthreads();
    if (bad_k) {
        if (tid == 0) {
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_TOPK_RANGE);
            if (MODE == MODE_FUSED) {
                a.next[row] = -1;
                if (a.n_kept) a.n_kept[row] = 0;
                if (a.cut) a.cut[row] = 0;
            } else {
                a.part_cnt[(size_t)split * a.rows + row] = 0;
            }
        }
        return;
    }
    finish_row<S, MODE>(a, row, split, P, greedy, buf, ctl, tid);
}

// Merge of `parts` local shortlists per row (several CTAs of one GPU, or one per
// vocabulary shard after an all-gather), then the tail.
__global__ void __launch_bounds__(ShapeLargeK::NT, ShapeLargeK::MINB) merge_parts_kernel(const KArgs a) {
    using S = ShapeLargeK;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + S::CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(hist + 256);
    const int tid = threadIdx.x;
    const int row = blockIdx.x;

    const MantleSampleParams P = row_params(a, row);
    const bool greedy = P.greedy != 0 || (P.top_k == 1 && P.top_p >= 1.0f && P.temperature == 1.0f);
    int k = greedy ? 1 : min(P.top_k, a.vocab_total);
    const bool bad_k = !greedy && (k > a.max_top_k || k > KMAX || k < 1);

    if (tid == 0) ctl->cnt = 0;
    __syncthreads();
    for (int p = 0; p < a.parts; p++) {
        const size_t slot = (size_t)p * a.rows + row;
        const int m = min(a.part_cnt[slot], a.part_cap);
        for (int i = tid; i < m; i += S::NT)
            append<S>(buf, ctl, a.part_val[slot * a.part_cap + i], a.part_idx[slot * a.part_cap + i]);
    }
    if (bad_k) {
        if (tid == 0) {
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_TOPK_RANGE);
            a.next[row] = -1;
            if (a.n_kept) a.n_kept[row] = 0;
            if (a.cut) a.cut[row] = 0;
        }
        return;
    }
    bool have;
    refresh_topk<S>(buf, ctl, hist, k, tid, &have);
    __syncthreads();
    finish_row<S, MODE_FUSED>(a, row, 0, P, greedy, buf, ctl, tid);
}

// ---------------------------------------------------------------------------------------
// host side

constexpr int kInvalid = (int)cudaErrorInvalidValue;

int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    return n;
}

bool batch_ok(const MantleSampleBatch* b, bool need_outputs) {
    if (!b || !b->logits || b->rows <= 0 || b->vocab <= 0) return false;
    if (b->vocab > MANTLE_SAMPLE_MAX_VOCAB) return false;
    if (b->dtype != MANTLE_DTYPE_F32 && b->dtype != MANTLE_DTYPE_BF16) return false;
    if (b->row_stride < b->vocab) return false;
    if (b->hist_stride < 0 || b->n_exclude < 0) return false;
    if (b->n_exclude > 0 && !b->exclude) return false;
    if (b->splits < 0 || b->reserved != 0) return false;
    if (b->flags & ~(MANTLE_SAMPLE_WRITE_BACK_PENALTY | MANTLE_SAMPLE_PENALTY_PREAPPLIED)) return false;
    if ((b->flags & MANTLE_SAMPLE_WRITE_BACK_PENALTY) && b->dtype != MANTLE_DTYPE_F32) return false;
    const size_t esz = b->dtype == MANTLE_DTYPE_F32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(b->logits) % esz) return false;
    if (need_outputs) {
        if (!b->params || !b->next) return false;
        if (b->max_top_k < 1 || b->max_top_k > KMAX) return false;
        if ((b->cand_idx || b->cand_prob) && b->cand_stride <= 0) return false;
    }
    return true;
}

// Shape selection.  MANTLE_SAMPLER_SHAPE=small|large overrides it (a tuning aid: `small`
// is refused, by falling back, for batches whose top_k it cannot serve).
bool use_small_shape(int max_top_k) {
    static const int forced = [] {
        const char* e = getenv("MANTLE_SAMPLER_SHAPE");
        if (!e) return 0;
        return strcmp(e, "small") == 0 ? 1 : (strcmp(e, "large") == 0 ? 2 : 0);
    }();
    if (max_top_k > ShapeSmallK::KCAP) return false;
    return forced != 2;
}

int choose_splits(const MantleSampleBatch* b) {
    const int vec = b->dtype == MANTLE_DTYPE_F32 ? 4 : 8;
    const int nvec = (b->vocab + vec - 1) / vec + 1;
    const bool small = use_small_shape(b->max_top_k);
    const int region = small ? ShapeSmallK::NT * ShapeSmallK::U : ShapeLargeK::NT * ShapeLargeK::U;
    const int per_sm = small ? ShapeSmallK::MINB : ShapeLargeK::MINB;
    const int max_by_k = MERGE_CAP / b->max_top_k;  // the merge holds splits * k candidates
    if (b->splits > 0) return max(1, min(min(b->splits, max_by_k), min(nvec, 64)));
    const int max_by_work = nvec / (2 * region);  // at least two regions per CTA
    const int cap = max(1, min(min(max_by_k, max_by_work), 64));
    const int target = per_sm * sm_count();  // one full wave
    if (b->rows >= target) return 1;
    return max(1, min(cap, (target + b->rows - 1) / b->rows));
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
    a.cand_stride = b->cand_stride;
    a.part_val = nullptr;
    a.part_idx = nullptr;
    a.part_cnt = nullptr;
    a.part_cap = 0;
    a.parts = 0;
}

template <typename K>
int launch(K kernel, const KArgs& a, int grid, int threads, size_t smem, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    kernel<<<grid, threads, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

template <class S, int MODE>
int launch_scan_shape(const KArgs& a, int dtype, cudaStream_t stream) {
    const size_t smem = S::SMEM_FIXED + bitmap_words(a.vocab) * sizeof(uint32_t);
    const long long grid = (long long)a.rows * a.splits;
    if (grid > 0x7fffffffLL) return kInvalid;
    if (dtype == MANTLE_DTYPE_F32)
        return launch(scan_rows_kernel<S, float, MODE>, a, (int)grid, S::NT, smem, stream);
    return launch(scan_rows_kernel<S, bf16_t, MODE>, a, (int)grid, S::NT, smem, stream);
}

template <int MODE>
int launch_scan(const KArgs& a, int dtype, cudaStream_t stream) {
    if (use_small_shape(a.max_top_k)) return launch_scan_shape<ShapeSmallK, MODE>(a, dtype, stream);
    return launch_scan_shape<ShapeLargeK, MODE>(a, dtype, stream);
}

int launch_merge(const KArgs& a, cudaStream_t stream) {
    return launch(merge_parts_kernel, a, a.rows, ShapeLargeK::NT, ShapeLargeK::SMEM_FIXED, stream);
}

size_t parts_bytes(int rows, int parts, int cap) {
    size_t n = (size_t)rows * parts;
    size_t bytes = n * cap * (sizeof(float) + sizeof(int32_t)) + n * sizeof(int32_t);
    return (bytes + 255) & ~(size_t)255;
}

}  // namespace

extern "C" int mantleCudaSamplerAbiVersion(void) { return 1; }

extern "C" int mantleCudaSamplerSplits(const MantleSampleBatch* batch, int* splits) {
    if (!splits || !batch_ok(batch, true)) return kInvalid;
    *splits = choose_splits(batch);
    return 0;
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
    int rc = launch_scan<MODE_PARTS>(a, batch->dtype, stream);
    if (rc) return rc;
    return launch_merge(a, stream);
}

extern "C" int mantleCudaRepeatPenaltyRowsF32(const MantleSampleBatch* batch, mantleCudaStream_t stream_) {
    if (!batch_ok(batch, false) || batch->dtype != MANTLE_DTYPE_F32 || !batch->params) return kInvalid;
    if (batch->flags & MANTLE_SAMPLE_PENALTY_PREAPPLIED) return kInvalid;
    KArgs a;
    fill_args(a, batch);
    a.max_top_k = 1;
    return launch_scan<MODE_PENALTY>(a, MANTLE_DTYPE_F32, static_cast<cudaStream_t>(stream_));
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
    return launch_scan<MODE_PARTS>(a, batch->dtype, static_cast<cudaStream_t>(stream_));
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
    size_t logits, history, hist_len, exclude, params, next, cand_idx, cand_prob, n_kept, cut, status, split, total;
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
    if (hb->flags & MANTLE_SAMPLE_WRITE_BACK_PENALTY)
        MANTLE_TRY(cudaMemcpyAsync(const_cast<void*>(hb->logits), ws + p.logits, p.logits_bytes, cudaMemcpyDeviceToHost, stream));
#undef MANTLE_TRY
    return 0;
}
