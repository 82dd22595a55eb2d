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
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>

#include "../../include/mantle_cuda_sampler.h"

// Development aid, compiled out of the shipped library: with -DMANTLE_DEBUG_SWITCHES the
// environment variable MANTLE_SAMPLER_DEBUG switches pieces of the kernel off to cost them.
#ifdef MANTLE_DEBUG_SWITCHES
#define DEBUG_OFF(a, bit) (((a).debug >> (bit)) & 1)
#else
#define DEBUG_OFF(a, bit) 0
#endif

namespace {

constexpr int KMAX = MANTLE_SAMPLE_MAX_TOP_K;
constexpr int RANK_MAX = 256;  // largest buffer the counting select takes
constexpr int HIST_CAP = 1024; // history-window ids staged in shared memory ahead of their row
constexpr int MAX_STAGES = 8;

// Launch shape of one kernel instantiation.
//   NT    threads per CTA            U     16-byte vectors per thread per chunk
//   CAP   candidate buffer entries   KCAP  largest top_k this shape serves
//   MINB  CTAs per SM the register budget is held to
template <int NT_, int U_, int CAP_, int KCAP_, int MINB_>
struct Shape {
    static constexpr int NT = NT_, U = U_, CAP = CAP_, KCAP = KCAP_, MINB = MINB_;
    static constexpr int NWARP = NT / 32;
    static constexpr int EPT = (CAP + NT - 1) / NT;  // candidate entries per thread during compaction
    // columns per thread per step of the careful path: a whole step always fits the buffer
    static constexpr int SLOW_EPT = (CAP - KCAP) / NT < 4 ? (CAP - KCAP) / NT : 4;
    static_assert(SLOW_EPT >= 1, "careful path needs room");
    static_assert(KCAP + NT * SLOW_EPT <= CAP, "careful path needs room for one full step");
    static_assert(KCAP * 24 <= CAP * 8, "ordered shortlist must fit behind the survivors");
    static_assert(RANK_MAX <= NT, "counting select: one entry per thread");
    // shared memory: [Cand buf[CAP]] [hist[256]] [Ctl] [Pre] [window ids[HIST_CAP]] [ring] [bitmap]
    static constexpr size_t SMEM_FIXED = 8 * (size_t)CAP + 4 * 256 + 512 + 256 + 4 * (size_t)HIST_CAP;
};
// Measured on B200 (a bare copy loop over 2.5 GB): the time one bulk copy takes to land hardly
// depends on its size (about 0.6 us for 8, 16 and 32 KB alike) and deeper rings do not raise a
// CTA's copy rate, so bandwidth comes from chunk size times CTAs per SM.  With the sampler's
// serial phases per row (bitmap, cuts, tail) three CTAs of 256 threads with 16 KB chunks
// overlap better than two with 32 KB chunks (71 % against 69 % of measured HBM bandwidth).
using ShapeSmallK = Shape<256, 4, 2048, 256, 3>;   // top_k <= 256: 16 KB candidate buffer
using ShapeLargeK = Shape<512, 4, 4096, KMAX, 1>;  // top_k <= 1024: 32 KB candidate buffer
#ifndef LDG_VOTE_EVERY
#define LDG_VOTE_EVERY 2
#endif
#ifndef LDG_PREFETCH
#define LDG_PREFETCH 1
#endif
#ifndef LDG_NT
#define LDG_NT 256
#define LDG_U 4
#define LDG_MINB 4
#endif
using ShapeLdg = Shape<LDG_NT, LDG_U, 2048, 256, LDG_MINB>;  // the plain-load kernel: four CTAs per SM
using ShapeLdgLargeK = Shape<512, 4, 4096, KMAX, 1>;         // the plain-load kernel for top_k <= 1024
using ShapeAlt = Shape<256, 8, 2048, 256, 2>;      // tuning: MANTLE_SAMPLER_SHAPE=alt (32 KB chunks)
constexpr int MAX_NWARP = 32;
constexpr int MERGE_CAP = ShapeLargeK::CAP;

constexpr int POST_SCALE = 1, POST_CAP = 2, POST_TANHF = 4;

constexpr int MODE_FUSED = 0;    // one CTA per row, tail in the same kernel
constexpr int MODE_PARTS = 1;    // several CTAs per row (or one vocabulary shard): write the local shortlist

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
    uint64_t full[MAX_STAGES];  // one mbarrier per ring stage: "the chunk has landed"
    int abort;                  // a wait on a copy ran out
};
static_assert(sizeof(Ctl) <= 512 && sizeof(Ctl) % 8 == 0, "control block outgrew its slot");

// What thread 0 fetches ahead for the item after the current one -- its parameters and history
// length (small asynchronous copies) and, tracked by `win_full`, its history window -- and the
// producer's own state, kept here rather than in registers that every thread would set aside.
struct Pre {
    MantleSampleParams p[2];
    int hl[2];
    int pad[2];
    uint64_t win_full;
    uint64_t pol;          // L2 eviction policy of the bulk copies
    const uint4* p_vbase;  // item being issued: its row rounded down to 16 bytes,
    int p_item, p_chunk, p_nchunks, p_a0, p_b0;  // its id, next chunk, chunk count, vector range
    uint32_t g_issued;     // chunks issued so far
    uint32_t w_issued;     // staged windows requested so far
};
static_assert(sizeof(Pre) <= 256, "prefetch block outgrew its slot");

// Post-processing of the model head's output, applied to every logit before the sampler sees
// it: POST_SCALE l *= scale; POST_CAP l = tanh(l / cap) * cap (POST_TANHF picks tanhf).
struct Post {
    int mode;
    float scale, cap;
};

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
    int hist_tma_ok;  // history base 16-byte aligned and hist_stride a multiple of 4
    Post post;  // read from the kernel's parameter space where it is used, never copied to registers
#ifdef MANTLE_DEBUG_SWITCHES
    int debug;
#endif
};

// ---------------------------------------------------------------------------------------
// small helpers

// Barrier among the N threads of a CTA launched with exactly N threads.
template <int N>
__device__ __forceinline__ void csync() {
    __syncthreads();
}

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

// fastTanh, simd/ops.go:165-175, operation for operation in float32.
__device__ __forceinline__ float fast_tanh(float x) {
    if (x > 10.0f) return 1.0f;
    if (x < -10.0f) return -1.0f;
    const float e2x = fast_exp(__fmul_rn(2.0f, x));
    return __fdiv_rn(__fsub_rn(e2x, 1.0f), __fadd_rn(e2x, 1.0f));
}

// What the model head does to a logit before the sampler sees it (simd/runtime.go:258-272):
// the multiplier first, then the soft cap, with the host path's fastTanh or, on request, with
// tanhf as the reference's device kernel has it (native/softmax.cu:963-970).
__device__ __forceinline__ float post_logit(float l, const Post& p) {
    if (p.mode & POST_SCALE) l = __fmul_rn(l, p.scale);
    if (p.mode & POST_CAP) {
        const float b = __fdiv_rn(l, p.cap);
        const float t = (p.mode & POST_TANHF) ? tanhf(b) : fast_tanh(b);
        l = __fmul_rn(t, p.cap);
    }
    return l;
}

// The streaming kernels never evaluate post_logit on a column that cannot matter.  The true map
// g(l) = inv_temp * cap * tanh(l * scale / cap) is increasing, and what the device computes
// differs from it by less than POST_EPS * cap * inv_temp (fastTanh: 1.7e-6 absolute, the
// worst over every float32 in [-10, 10]; tanhf: 3e-7; the roundings of the multiplies and
// divides: 3e-7 relative), so a threshold on the computed values turns into a threshold on the raw
// logits: every column whose computed value reaches `thr` has a raw logit of at least
// post_raw_bound(thr).  The margins are several times the error they cover; a wider margin only
// lets a few more columns through to the exact test.
constexpr float POST_EPS = 1e-5f;
__device__ __forceinline__ float post_raw_bound(float thr, float inv_temp, const Post& p) {
    const float ninf = __uint_as_float(0xff800000u);
    if (!(thr > ninf)) return ninf;
    float q = thr / inv_temp;
    if (!(fabsf(q) > 1e-30f) || !(fabsf(q) < 1e30f)) return ninf;  // at zero the roundings are not relative
    if (p.mode & POST_CAP) {
        float y = q / p.cap - 10.0f * POST_EPS;
        if (y <= -1.0f) return ninf;
        y = fminf(y, 1.0f - 1e-6f);
        q = 0.5f * logf((1.0f + y) / (1.0f - y)) * p.cap;  // atanh
        if (!(fabsf(q) > 1e-30f)) return ninf;
    }
    if (p.mode & POST_SCALE) q = q / p.scale;
    return q - fabsf(q) * 1e-4f;
}
// A post-processed logit that every column with a raw logit >= raw0 reaches (the seed of the threshold).
__device__ __forceinline__ float post_seed_logit(float raw0, const Post& p) {
    const float l0 = post_logit(raw0, p);
    if (!(fabsf(l0) < 3.0e38f)) return l0;  // an infinite value is its own bound
    const float slack = (p.mode & POST_CAP) ? 4.0f * POST_EPS * p.cap : 0.0f;
    return l0 - slack - fabsf(l0) * 1e-5f;
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
// A survivor that carries a penalty is rarer still (a column of the history window among the few
// that pass the filter); its divide lives out of line, once per kernel, so that the streaming
// loop stays small.  The candidate buffer and the control block sit at fixed offsets.
template <class S>
__device__ __noinline__ void penalised_survivor(float raw, int gidx, float thr, bool incl, float inv_temp, float pen) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + 8 * (size_t)S::CAP + 4 * 256);
    const float v = __fmul_rn(penalise(raw, pen), inv_temp);
    if (incl ? v >= thr : v > thr) append<S>(buf, ctl, v, gidx);
}
template <class S, bool INCL>
__device__ __forceinline__ void consider(Cand* buf, Ctl* ctl, const RowCtx& c, float raw, float v, int e, float thr) {
    if (c.pen_bitmap && bm_test(c.bm, e)) {
        penalised_survivor<S>(raw, e + c.voff, thr, INCL, c.inv_temp, c.pen);
        return;
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

// The largest scaled value of one complete vector (no penalty: raw values bound the true ones).
template <typename T>
__device__ __forceinline__ float vec_max_scaled(const uint4& rawv, float inv_temp) {
    constexpr int VEC = Elem<T>::VEC;
    float raw[VEC];
    Elem<T>::widen(rawv, raw);
    float m = __fmul_rn(raw[0], inv_temp);
#pragma unroll
    for (int j = 1; j < VEC; j++) m = fmaxf(m, __fmul_rn(raw[j], inv_temp));
    return m;
}

// One complete 16-byte vector that may hold a survivor.  Survivors are walked one at a time
// (NaN never passes a compare), so the slow code exists once per call site.
template <class S, typename T, bool INCL>
__device__ __forceinline__ void filter_vec(const uint4& rawv, int vec, const RowCtx& c, float thr, Cand* buf,
                                           Ctl* ctl) {
    constexpr int VEC = Elem<T>::VEC;
    float raw[VEC];
    Elem<T>::widen(rawv, raw);
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

// The same three steps for a batch with post-processing: the hot test runs on the raw logits
// against a raw bound (post_raw_bound), and only a column that passes it pays for the exact value.
// The exact value of a survivor is a few hundred instructions (two divides, fastExp or tanhf).
// Inlined at every place a survivor can turn up it made the streaming loop too large for the
// instruction cache (measured: as many stalls waiting for instructions as at barriers), so it
// exists once per kernel, out of line, with everything it needs passed by value; the candidate
// buffer and the control block sit at fixed offsets of the CTA's shared memory.
template <class S>
__device__ __noinline__ void post_survivor(float raw, int e, float thr, bool incl, float inv_temp, float pen,
                                           int voff, int mode, float scale, float cap) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + 8 * (size_t)S::CAP + 4 * 256);
    const Post post = {mode, scale, cap};
    float l = post_logit(raw, post);
    if (pen != 0.0f) l = penalise(l, pen);  // 0: this column carries no penalty
    const float v = __fmul_rn(l, inv_temp);
    if (incl ? v >= thr : v > thr) append<S>(buf, ctl, v, e + voff);
}
template <class S, bool INCL>
__device__ __forceinline__ void consider_post(Cand* buf, Ctl* ctl, const RowCtx& c, const Post& post, float raw,
                                              int e, float thr) {
    post_survivor<S>(raw, e, thr, INCL, c.inv_temp, (c.pen_bitmap && bm_test(c.bm, e)) ? c.pen : 0.0f, c.voff,
                     post.mode, post.scale, post.cap);
}

// The largest raw logit of one complete vector.
template <typename T>
__device__ __forceinline__ float vec_max_raw(const uint4& rawv) {
    constexpr int VEC = Elem<T>::VEC;
    float raw[VEC];
    Elem<T>::widen(rawv, raw);
    float m = raw[0];
#pragma unroll
    for (int j = 1; j < VEC; j++) m = fmaxf(m, raw[j]);
    return m;
}

template <class S, typename T, bool INCL>
__device__ __forceinline__ void filter_vec_post(const uint4& rawv, int vec, const RowCtx& c, const Post& post,
                                                float rthr, float thr, Cand* buf, Ctl* ctl) {
    constexpr int VEC = Elem<T>::VEC;
    float raw[VEC];
    Elem<T>::widen(rawv, raw);
    uint32_t pass = 0;
#pragma unroll
    for (int j = 0; j < VEC; j++) pass |= (raw[j] >= rthr) ? (1u << j) : 0u;
    const int e0 = vec * VEC - c.mis;
    while (pass) {
        const int j = __ffs(pass) - 1;
        pass &= pass - 1;
        float r = raw[0];
#pragma unroll
        for (int q = 1; q < VEC; q++) r = (j == q) ? raw[q] : r;
        consider_post<S, INCL>(buf, ctl, c, post, r, e0 + j, thr);
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
                                                 bool* have_kth, bool* ordered = nullptr) {
    __syncthreads();
    const int n = live_count(ctl);
    __syncthreads();
    if (ordered) *ordered = n <= RANK_MAX;  // the counting select leaves its survivors in order
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

// words of the penalty bitmap: V bits, padded to whole 16-byte vectors
__host__ __device__ inline size_t bitmap_words(int vocab) { return (size_t)(((vocab + 31) / 32 + 2 + 3) & ~3); }

// The same tail for shortlists of at most 64 entries, run by one warp with the shortlist in
// registers (lane L holds entries L and L+32): no CTA barrier, no shared-memory round trips.
// The sums that the reference accumulates in shortlist order are accumulated in that order
// here too -- every lane walks the same chain, fed by shuffles -- so the doubles are the
// same doubles.  `buf` holds the n ordered survivors; sidx/sprob are scratch for the min-p
// compaction.
__device__ void sample_tail_warp(const KArgs& a, int row, const MantleSampleParams& P, bool greedy, int n,
                                 const Cand* buf, int32_t* sidx, double* sprob, int lane) {
    const unsigned full = 0xffffffffu;
    int token, n_kept = 0, cut = 0;
    if (n == 0) {
        token = 0;
    } else if (greedy) {
        token = (int)buf[0].idx;
    } else {
        Cand c0, c1;
        c0.key = c0.idx = c1.key = c1.idx = 0;
        if (lane < n) c0 = buf[lane];
        if (lane + 32 < n) c1 = buf[lane + 32];
        int i0 = (int)c0.idx, i1 = (int)c1.idx;
        const float maxv = key2f(__shfl_sync(full, c0.key, 0));
        double p0 = lane < n ? (double)fast_exp(__fsub_rn(key2f(c0.key), maxv)) : 0.0;
        double p1 = lane + 32 < n ? (double)fast_exp(__fsub_rn(key2f(c1.key), maxv)) : 0.0;
        double sum = 0.0;
        for (int i = 0; i < n; i++) sum = __dadd_rn(sum, __shfl_sync(full, i < 32 ? p0 : p1, i & 31));
        if (sum == 0.0) {  // sampler.go:170-172
            token = __shfl_sync(full, i0, 0);
            n_kept = n;
        } else {
            const double inv = __ddiv_rn(1.0, sum);
            p0 = __dmul_rn(p0, inv);
            p1 = __dmul_rn(p1, inv);
            if (P.min_p > 0.0f) {  // sampler.go:180-210
                const double thr = __dmul_rn(__shfl_sync(full, p0, 0), (double)P.min_p);
                const bool k0 = lane < n && p0 >= thr, k1 = lane + 32 < n && p1 >= thr;
                const unsigned b0 = __ballot_sync(full, k0), b1 = __ballot_sync(full, k1);
                const int m = __popc(b0) + __popc(b1);
                double ns = 0.0;
                for (int i = 0; i < n; i++) {
                    const double pi = __shfl_sync(full, i < 32 ? p0 : p1, i & 31);
                    if (((i < 32 ? b0 : b1) >> (i & 31)) & 1u) ns = __dadd_rn(ns, pi);
                }
                if (m < n) {
                    const unsigned lt = (1u << lane) - 1u;
                    if (k0) {
                        const int q = __popc(b0 & lt);
                        sprob[q] = p0;
                        sidx[q] = i0;
                    }
                    if (k1) {
                        const int q = __popc(b0) + __popc(b1 & lt);
                        sprob[q] = p1;
                        sidx[q] = i1;
                    }
                    __syncwarp();
                    n = m;
                    p0 = lane < n ? sprob[lane] : 0.0;
                    i0 = lane < n ? sidx[lane] : 0;
                    p1 = lane + 32 < n ? sprob[lane + 32] : 0.0;
                    i1 = lane + 32 < n ? sidx[lane + 32] : 0;
                    __syncwarp();
                    if (ns > 0.0) {
                        const double sc = __ddiv_rn(1.0, ns);
                        p0 = __dmul_rn(p0, sc);
                        p1 = __dmul_rn(p1, sc);
                    }
                }
            }
            n_kept = n;
            if (n == 0) {  // min_p > 1 dropped everything: the reference indexes topIdx[-1] and panics
                token = -1;
                if (lane == 0 && a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_EMPTY);
            } else {
                // sampler.go:212-233: the nucleus prefix and the inverse-CDF walk add the same
                // doubles in the same order, so one running sum serves both
                double c = 0.0, c0v = 0.0, c1v = 0.0;
                for (int i = 0; i < n; i++) {
                    c = __dadd_rn(c, __shfl_sync(full, i < 32 ? p0 : p1, i & 31));
                    if (i == lane) c0v = c;
                    if (i == lane + 32) c1v = c;
                }
                const bool nucleus = P.top_p < 1.0f;
                const unsigned q0 = __ballot_sync(full, nucleus && lane < n && __double2float_rn(c0v) >= P.top_p);
                const unsigned q1 = __ballot_sync(full, nucleus && lane + 32 < n && __double2float_rn(c1v) >= P.top_p);
                const int first = q0 ? __ffs(q0) - 1 : (q1 ? 31 + __ffs(q1) : -1);
                cut = first < 0 ? n : first + 1;
                const double r = P.uniform;
                const unsigned r0 = __ballot_sync(full, lane < cut && r <= c0v);
                const unsigned r1 = __ballot_sync(full, lane + 32 < cut && r <= c1v);
                const int pos = r0 ? __ffs(r0) - 1 : (r1 ? 31 + __ffs(r1) : cut - 1);
                token = __shfl_sync(full, pos < 32 ? i0 : i1, pos & 31);
            }
            if (a.cand_idx || a.cand_prob) {
                const size_t base = (size_t)row * a.cand_stride;
                if (lane < n && lane < a.cand_stride) {
                    if (a.cand_idx) a.cand_idx[base + lane] = i0;
                    if (a.cand_prob) a.cand_prob[base + lane] = p0;
                }
                if (lane + 32 < n && lane + 32 < a.cand_stride) {
                    if (a.cand_idx) a.cand_idx[base + lane + 32] = i1;
                    if (a.cand_prob) a.cand_prob[base + lane + 32] = p1;
                }
            }
        }
    }
    if (lane == 0) {
        a.next[row] = token;
        if (a.n_kept) a.n_kept[row] = n_kept;
        if (a.cut) a.cut[row] = cut;
    }
}

// After the select: order the survivors and either finish the row or publish the local
// shortlist.  The ordered arrays live in the part of the candidate buffer the survivors
// (at most KCAP entries) do not occupy.  `ordered`: the select already left them in order.
template <class S, int MODE>
__device__ void finish_row(const KArgs& a, int row, int split, const MantleSampleParams& P, bool greedy,
                           bool ordered, Cand* buf, Ctl* ctl, int tid) {
    constexpr int KC = S::KCAP;
    const int n = min(ctl->cnt, KC);
    float* sval = reinterpret_cast<float*>(buf + KC);
    int32_t* sidx = reinterpret_cast<int32_t*>(sval + KC);
    double* sprob = reinterpret_cast<double*>(sidx + KC);
    if (MODE == MODE_FUSED && ordered && n <= 64) {
        if (tid < 32) sample_tail_warp(a, row, P, greedy, n, buf, sidx, sprob, tid);
        return;
    }
    if (ordered) {
        for (int i = tid; i < n; i += S::NT) {
            sval[i] = key2f(buf[i].key);
            sidx[i] = (int32_t)buf[i].idx;
        }
    } else {
        rank_sort<S>(buf, n, sval, sidx, tid);
    }
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
// Asynchronous bulk copies (TMA, untiled form) and the mbarriers that track them.
// Both addresses are 16-byte aligned and sizes are multiples of 16 bytes by construction:
// copies move whole 16-byte vectors from the row rounded down to a 16-byte boundary.

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

constexpr uint32_t WAIT_HINT_NS = 20000;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s

// One poll.  The suspend-time hint lets the hardware park the thread until the phase completes
// (or the hint, in nanoseconds, runs out) instead of spinning through issue slots that the
// other CTA on the SM could use.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(WAIT_HINT_NS)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Every wait on a copy is bounded by wall time: after WAIT_LIMIT_NS without the phase
// completing the caller gives up, raises MANTLE_SAMPLE_STATUS_TIMEOUT and leaves the kernel
// in an orderly way.  A copy normally lands within a microsecond or two.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > limit_ns) return false;
    }
}

// Self-test of the bounded wait: waits on an mbarrier that nothing ever completes.  The wait
// must give up after limit_ns, report it in the status word and leave the context usable.
__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, int32_t* status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool landed = mbar_wait(&bar, 0, limit_ns);
    if (!landed && threadIdx.x == 0) atomicOr(status, MANTLE_SAMPLE_STATUS_TIMEOUT);
}

__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}

// Small asynchronous copies (8 or 4 bytes) for the next item's parameters.
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

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

// ---------------------------------------------------------------------------------------
// The streaming kernel: persistent CTAs, rows fed through a ring of shared-memory stages
// by asynchronous bulk copies.
//
// A CTA owns work items (row, split) blockIdx.x, blockIdx.x + gridDim.x, ...  The complete
// 16-byte vectors of an item are cut into chunks of NT*U vectors; thread 0 keeps `stages`
// chunks in flight or landed at all times, in item order, running ahead across item
// boundaries -- so the copies of the next row proceed while the current row's shortlist
// is cut, ordered and sampled.  All threads consume a chunk from shared memory, meet at
// one barrier (which also carries the "buffer needs a cut" vote), and thread 0 refills
// the stage just freed.  Thread 0 also looks one item ahead: the next item's parameters,
// history length and history window are in shared memory before the item starts.

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

template <typename T, class S>
struct ItemGeom {
    const uint4* vbase;  // the row rounded down to 16 bytes
    const void* row;
    int mis;       // elements between vbase and the row pointer
    int a0, b0;    // complete vectors [a0, b0) of this item
    int elo, ehi;  // columns [elo, ehi) of this item
    int nchunks;
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

template <class S, typename T, int MODE>
__global__ void __launch_bounds__(S::NT, S::MINB) scan_rows_kernel(const KArgs a, const int stages) {
    constexpr int VEC = Elem<T>::VEC;
    constexpr int NT = S::NT, NWARP = S::NWARP, U = S::U, CAP = S::CAP;
    constexpr int CV = NT * U;                 // vectors per chunk
    constexpr uint32_t CHUNK_BYTES = CV * 16;  // bytes per stage
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(hist + 256);
    Pre* pre = reinterpret_cast<Pre*>(reinterpret_cast<unsigned char*>(ctl) + 512);
    int32_t* win = reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(pre) + 256);
    unsigned char* ring = smem_raw + S::SMEM_FIXED;
    uint32_t* bm = reinterpret_cast<uint32_t*>(ring + (size_t)stages * CHUNK_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nitems = a.rows * a.splits;

    if (tid == 0) {
        for (int s = 0; s < stages; s++) mbar_init(&ctl->full[s], 1);
        mbar_init(&pre->win_full, 1);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // ---- look-ahead (thread 0): the next item's parameters, history length and window -------
    const bool per_row_len = a.history != nullptr && a.hist_len != nullptr &&
                             !(a.flags & MANTLE_SAMPLE_PENALTY_PREAPPLIED);
    auto item_hl = [&](int slot) {  // history length of the item whose look-ahead sits in `slot`
        if (!a.history || (a.flags & MANTLE_SAMPLE_PENALTY_PREAPPLIED)) return 0;
        const int hl = a.hist_len ? pre->hl[slot] : a.hist_stride;
        return max(0, min(hl, a.hist_stride));
    };
    auto fetch_params = [&](int item, int slot) {  // asynchronous; completed by cp_async_wait_all
        const int r = item / a.splits;
        if (a.params) {
            const char* src = reinterpret_cast<const char*>(a.params + r);
            char* dst = reinterpret_cast<char*>(&pre->p[slot]);
#pragma unroll
            for (int q = 0; q < (int)sizeof(MantleSampleParams); q += 8) cp_async8(dst + q, src + q);
        }
        if (per_row_len) cp_async4(&pre->hl[slot], a.hist_len + r);
        cp_async_commit();
    };
    auto slot_params = [&](int slot) {
        if (a.params) return pre->p[slot];
        return row_params(a, 0);  // plain argmax rows
    };
    auto fetch_window = [&](int item, int slot) {  // needs the slot's parameters to have landed
        const MantleSampleParams Pn = slot_params(slot);
        const WinPlan w = win_plan(a, Pn, item_hl(slot));
        if (w.staged) {
            pre->w_issued++;
            const int32_t* src = a.history + (size_t)(item / a.splits) * (size_t)a.hist_stride + w.a4;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&pre->win_full, (uint32_t)w.n4 * 4u);
            bulk_load(win, src, (uint32_t)w.n4 * 4u, &pre->win_full, pre->pol);
        }
    };

    // ---- producer (thread 0; its state lives in `pre`) ---------------------------------------
    // items whose shortlist is too long for the seeded threshold stream nothing: they go
    // straight to the careful path
    auto fast_item = [&](int item) {
        if (a.max_top_k <= 32 * NWARP) return true;  // no row can exceed the bound: nothing to look up
        bool greedy, bad;
        const MantleSampleParams Pq = row_params(a, item / a.splits);
        return row_k(a, Pq, S::KCAP, &greedy, &bad) <= 32 * NWARP;
    };
    auto producer_open = [&]() {  // geometry of item pre->p_item
        pre->p_chunk = 0;
        pre->p_nchunks = 0;
        if (pre->p_item < nitems) {
            const ItemGeom<T, S> g = item_geom<T, S>(a, pre->p_item);
            pre->p_vbase = g.vbase;
            pre->p_a0 = g.a0;
            pre->p_b0 = g.b0;
            pre->p_nchunks = fast_item(pre->p_item) ? g.nchunks : 0;
        }
    };
    auto issue_next = [&]() {  // thread 0: the next chunk in item order, if any is left
        while (pre->p_item < nitems) {
            const int pc = pre->p_chunk;
            if (pc < pre->p_nchunks) {
                const int v = pre->p_a0 + pc * CV;
                const uint32_t bytes = (uint32_t)min(CV, pre->p_b0 - v) * 16u;
                const uint32_t s = pre->g_issued % (uint32_t)stages;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(&ctl->full[s], bytes);
                bulk_load(ring + (size_t)s * CHUNK_BYTES, pre->p_vbase + v, bytes, &ctl->full[s], pre->pol);
                pre->p_chunk = pc + 1;
                pre->g_issued++;
                return;
            }
            pre->p_item += gridDim.x;
            producer_open();
        }
    };
    if (tid == 0) {
        pre->pol = evict_first_policy();
        pre->p_item = blockIdx.x;
        pre->g_issued = 0;
        pre->w_issued = 0;
        producer_open();
        for (int s = 0; s < stages; s++) issue_next();
        if ((int)blockIdx.x < nitems) {
            fetch_params(blockIdx.x, 0);
            cp_async_wait_all();
            fetch_window(blockIdx.x, 0);
        }
    }

    uint32_t g_done = 0;  // chunks consumed so far (same in every thread)
    uint32_t w_done = 0;  // staged windows consumed so far (same in every thread)
    int it_index = 0;
    bool aborted = false;

    for (int item = blockIdx.x; item < nitems && !aborted; item += gridDim.x, it_index++) {
        const int row = item / a.splits;
        const int split = item - row * a.splits;
        const int slot = it_index & 1;
        const int next_item = item + gridDim.x;

        __syncthreads();  // the previous item is done with buffer and bitmap; the look-ahead is visible
        if (tid == 0) ctl->cnt = 0;
        const MantleSampleParams P = slot_params(slot);
        const int hl = item_hl(slot);
        bool greedy, bad_k;
        const int k = row_k(a, P, S::KCAP, &greedy, &bad_k);
        const ItemGeom<T, S> g = item_geom<T, S>(a, item);
        if (tid == 0 && next_item < nitems) fetch_params(next_item, slot ^ 1);
        bool looked_ahead = false;  // thread 0: the next item's window has been requested

        RowCtx c;
        c.row = g.row;
        c.mis = g.mis;
        c.V = a.vocab;
        c.voff = a.vocab_offset;
        c.inv_temp = greedy ? 1.0f : __fdiv_rn(1.0f, P.temperature);  // sampler.go:144-145
        c.pen = P.repeat_penalty;
        c.bm = bm;
        c.pen_bitmap = false;
        const int a0 = g.a0, b0 = g.b0, elo = g.elo, ehi = g.ehi;
        bool careful = k > 32 * NWARP;
        const int nchunks = careful ? 0 : g.nchunks;

        // ---- repeat penalty: bitmap of the de-duplicated window (sampler.go:99-138) --------
        const WinPlan wp = win_plan(a, P, hl);
        if (wp.staged) {
            if (!mbar_wait(&pre->win_full, w_done & 1u)) ctl->abort = 1;
            w_done++;
        }
        if (wp.active && !DEBUG_OFF(a, 0)) {
            build_penalty_bitmap(a, row, wp, hl, win, c.V, c.voff, bm, tid, NT);
            c.pen_bitmap = true;
        }
        __syncthreads();

        // ---- stream the item's chunks -------------------------------------------------------
#ifdef MANTLE_TRIG_EXTRA
        const int trig = min(k + MANTLE_TRIG_EXTRA, CAP / 2);
#else
        const int trig = min(k + max(k >> 1, 16), CAP / 2);  // cut the buffer at this many entries
#endif
        float thr = __uint_as_float(0xff800000u);            // -inf

        for (int cc = 0; cc < nchunks; cc++, g_done++) {
            const uint32_t s = g_done % (uint32_t)stages;
            const uint32_t parity = (g_done / (uint32_t)stages) & 1u;
            bool landed = mbar_wait(&ctl->full[s], parity);
            if (!landed) ctl->abort = 1;
            // the first chunk's filter meets at a barrier of its own: enter it all together or not at all
            if (cc == 0 && !careful) landed = __syncthreads_and(landed);
            const uint4* stage = reinterpret_cast<const uint4*>(ring + (size_t)s * CHUNK_BYTES);
            const int v0 = a0 + cc * CV + tid;  // this thread's first vector of the chunk
            if (landed && !careful) {
                if (cc == 0) {
                    // A threshold that at least k columns of this chunk reach: with
                    // j = ceil(k / warps), every warp holds j thread-maxima >= its j-th largest
                    // one, so the smallest of those per-warp values is reached by >= k columns.
                    // The maxima are taken over penalised values: the bound must hold for them.
                    float tmax = __uint_as_float(0xff800000u);
#pragma unroll
                    for (int u = 0; u < U; u++)
                        if (v0 + u * NT < b0)
                            tmax = fmaxf(tmax, vec_max_penalised<T>(stage[u * NT + tid], v0 + u * NT, c));
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
                        if (v0 + u * NT < b0)
                            filter_vec<S, T, true>(stage[u * NT + tid], v0 + u * NT, c, thr, buf, ctl);
                } else {
                    // Later columns: the buffer already holds k entries >= thr with lower
                    // indices, so an equal value can no longer enter (sampler.go:268-275).
                    // One test per thread and chunk in the common case: the largest of its
                    // U * VEC scaled values against the threshold.
                    const bool whole = cc + 1 < nchunks;  // only the last chunk can be partial
                    uint4 rv[U];
                    float mu[U];
                    float m = __uint_as_float(0xff800000u);
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        mu[u] = __uint_as_float(0xff800000u);
                        if (whole || v0 + u * NT < b0) {
                            rv[u] = stage[u * NT + tid];
                            mu[u] = vec_max_scaled<T>(rv[u], c.inv_temp);
                        }
                        m = fmaxf(m, mu[u]);
                    }
                    if (m > thr) {
#pragma unroll
                        for (int u = 0; u < U; u++)
                            if (mu[u] > thr) filter_vec<S, T, false>(rv[u], v0 + u * NT, c, thr, buf, ctl);
                    }
                }
            }
            // One barrier per chunk.  The thread that made the last append of the chunk reads
            // the final count before it arrives, so the OR is the same for every thread.
            int lim = cc == 0 ? k + 1 : trig;
            if (DEBUG_OFF(a, 3)) lim = CAP + 1;
            if (DEBUG_OFF(a, 2)) thr = __uint_as_float(0x7f800000u);
            const bool vote = __syncthreads_or(live_count(ctl) >= lim || !landed);
            if (tid == 0) {
                issue_next();  // the stage is free again
                if (!looked_ahead && next_item < nitems) {
                    // by now the next item's parameters have long landed, and this item is done
                    // with the window buffer: request the next window
                    cp_async_wait_all();
                    fetch_window(next_item, slot ^ 1);
                    looked_ahead = true;
                }
            }
            if (vote) {
                if (*reinterpret_cast<volatile int*>(&ctl->abort)) {
                    aborted = true;
                    g_done++;
                    break;
                }
                if (!careful) {
                    if (live_count(ctl) > CAP) {
                        careful = true;  // entries were dropped: redo the item on the careful path
                    } else {
                        bool have;
                        uint32_t kth = refresh_topk<S>(buf, ctl, hist, k, tid, &have);
                        if (have) thr = key2f(kth);
                    }
                }
            }
        }
        if (aborted) break;

        if (!careful) {
            // the columns of the partial vectors at the ends of this item
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
            // Careful path: any input, any order, plain loads.  Steps of NT*SLOW_EPT columns
            // with room for a whole step guaranteed before it starts; the buffer is cut to k
            // whenever it could overflow.  Reached for k beyond 32 per warp, for rows whose
            // first chunk ties massively, and for adversarial orders (e.g. ascending logits).
            __syncthreads();
            if (tid == 0) ctl->cnt = 0;
            __syncthreads();
            thr = __uint_as_float(0xff800000u);
            bool strict = false;
            constexpr int STEP = NT * S::SLOW_EPT;
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
                for (int j = 0; j < S::SLOW_EPT; j++) {
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

        // ---- cut to k, order, finish --------------------------------------------------------
        bool have, ordered;
        refresh_topk<S>(buf, ctl, hist, k, tid, &have, &ordered);
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
        } else if (!DEBUG_OFF(a, 1)) {
            finish_row<S, MODE>(a, row, split, P, greedy, ordered, buf, ctl, tid);
        }
        if (tid == 0 && !looked_ahead && next_item < nitems) {  // items that streamed no chunk
            cp_async_wait_all();
            fetch_window(next_item, slot ^ 1);
        }
    }

    if (aborted) {
        // A copy never landed.  Report it, give the copies still in flight a bounded time to
        // land (their destination is this CTA's shared memory), and leave.
        if (tid == 0) {
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_TIMEOUT);
            for (uint32_t q = g_done; q < pre->g_issued; q++)
                mbar_wait(&ctl->full[q % (uint32_t)stages], (q / (uint32_t)stages) & 1u);
            cp_async_wait_all();
            if (pre->w_issued > w_done) mbar_wait(&pre->win_full, w_done & 1u);
        }
        __syncthreads();
    } else if (tid == 0 && ctl->abort && a.status) {
        atomicOr(a.status, MANTLE_SAMPLE_STATUS_TIMEOUT);  // a history window never landed
    }
}

// ---------------------------------------------------------------------------------------
// The same streaming pass with plain 16-byte loads instead of the bulk-copy ring: one CTA per
// item (row, split), two register sets per thread, each refilled from global memory while the
// other is filtered, one barrier per region of NT*U vectors.  No shared-memory staging, so the
// CTA is small (candidate buffer + bitmap) and four of them share an SM; which of the two
// kernels is faster for a batch is a matter of measurement (see launch_scan).

template <class S>
struct LdgLayout {
    // shared memory: [Cand buf[CAP]] [hist[256]] [Ctl] [bitmap words]
    static constexpr size_t FIXED = 8 * (size_t)S::CAP + 4 * 256 + 512;
};

template <class S, typename T, int MODE, bool POST>
__global__ void __launch_bounds__(S::NT, S::MINB) scan_rows_ldg_kernel(const KArgs a) {
    constexpr int VEC = Elem<T>::VEC;
    constexpr int NT = S::NT, NWARP = S::NWARP, U = S::U, CAP = S::CAP;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(hist + 256);
    uint32_t* bm = reinterpret_cast<uint32_t*>(smem_raw + LdgLayout<S>::FIXED);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int item = blockIdx.x;
    const int row = item / a.splits;
    const int split = item - row * a.splits;

    const MantleSampleParams P = row_params(a, row);
    bool greedy, bad_k;
    const int k = row_k(a, P, S::KCAP, &greedy, &bad_k);
    const ItemGeom<T, S> g = item_geom<T, S>(a, item);

    RowCtx c;
    c.row = g.row;
    c.mis = g.mis;
    c.V = a.vocab;
    c.voff = a.vocab_offset;
    c.inv_temp = greedy ? 1.0f : __fdiv_rn(1.0f, P.temperature);  // sampler.go:144-145
    c.pen = P.repeat_penalty;
    c.bm = bm;
    c.pen_bitmap = false;
    const uint4* vbase = g.vbase;
    const int a0 = g.a0, b0 = g.b0, elo = g.elo, ehi = g.ehi;
    constexpr int RV = NT * U;  // vectors per region
    const int nreg = g.nchunks;
    bool careful = k > 32 * NWARP;

    // The first region's loads go out before anything else: they are in flight while the bitmap is built.
    uint4 ra[U], rb[U];
    auto load = [&](uint4(&dst)[U], int r) {  // region r (only the last region can be partial)
#pragma unroll
        for (int u = 0; u < U; u++) {
            int v = a0 + r * RV + u * NT + tid;
            // the zero fill is not read (the tests below mask what lies beyond the item), but a load
            // that kept the register's old value would have to wait for its last reader (measured: 1.6 % slower)
            dst[u] = v < b0 ? __ldcs(vbase + v) : make_uint4(0, 0, 0, 0);
        }
    };
    // `ahead(r)`: ask the L2 for region r (one request per 128-byte line), two regions before its
    // loads are issued, so that those loads find their lines on the way or already there
    auto ahead = [&](int r) {
#if LDG_PREFETCH
        // a warp's share of a region is U runs of 512 bytes: lane i asks for line i & 3 of run i >> 2
        if (r < nreg && lane < 4 * U) {
            const int v = a0 + r * RV + (lane >> 2) * NT + (tid & ~31) + (lane & 3) * 8;
            if (v < b0) asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(vbase + v));
        }
#endif
    };
    if (!careful && nreg > 0) {
        load(ra, 0);
        ahead(1);
        ahead(2);
    }
    if (tid == 0) ctl->cnt = 0;

    // ---- repeat penalty: bitmap of the de-duplicated window (sampler.go:99-138) --------
    const int hl = history_len(a, row);
    WinPlan wp = win_plan(a, P, hl);
    wp.staged = false;
    if (wp.active) {
        build_penalty_bitmap_early<NT>(a, row, wp, hl, c.V, c.voff, bm, tid);
        c.pen_bitmap = true;
    }
    __syncthreads();

    // ---- stream the item ------------------------------------------------------------------
    const int trig = min(k + max(k >> 1, 16), CAP / 2);  // cut the buffer at this many entries
    float thr = __uint_as_float(0xff800000u);            // -inf
    float rthr = thr;  // POST: the raw logit every column that can reach thr has at least
    const Post& POSTP = a.post;

    if (!careful && nreg > 0) {
        // later regions: the buffer already holds k entries >= thr with lower indices, so an equal
        // value can no longer enter (sampler.go:268-275); one test per thread and region
        auto later = [&](const uint4(&src)[U], int r) {
            const int v0 = a0 + r * RV + tid;
            const bool whole = r + 1 < nreg;
            float mu[U];
            float m = __uint_as_float(0xff800000u);
#pragma unroll
            for (int u = 0; u < U; u++) {
                mu[u] = __uint_as_float(0x7fc00000u);  // NaN: beyond the item, admitted by no compare
                if (whole || v0 + u * NT < b0)
                    mu[u] = POST ? vec_max_raw<T>(src[u]) : vec_max_scaled<T>(src[u], c.inv_temp);
                m = fmaxf(m, mu[u]);
            }
            if (POST) {
                if (m >= rthr) {
#pragma unroll
                    for (int u = 0; u < U; u++)
                        if (mu[u] >= rthr) filter_vec_post<S, T, false>(src[u], v0 + u * NT, c, POSTP, rthr, thr, buf, ctl);
                }
            } else if (m > thr) {
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (mu[u] > thr) filter_vec<S, T, false>(src[u], v0 + u * NT, c, thr, buf, ctl);
            }
        };
        // one barrier per region; the thread that made the region's last append reads the final
        // count before it arrives, so the OR is the same for every thread
        auto region_end = [&](int lim) {
            if (__syncthreads_or(live_count(ctl) >= lim)) {
                if (live_count(ctl) > CAP) {
                    careful = true;  // entries were dropped: redo the item on the careful path
                } else {
                    bool have;
                    uint32_t kth = refresh_topk<S>(buf, ctl, hist, k, tid, &have);
                    if (have) {
                        thr = key2f(kth);
                        if (POST) rthr = post_raw_bound(thr, c.inv_temp, POSTP);
                    }
                }
            }
        };

        // -- region 0 seeds the threshold (see scan_rows_kernel) --
        if (nreg > 1) load(rb, 1);
        {
            const int v0 = a0 + tid;
            // Thread maxima of the RAW logits: everything between a raw logit and its final value
            // (post-processing up to its slack, penalty, temperature) is non-decreasing, and a
            // column's value is at least what it would be with the penalty, so the image of a raw
            // logit that k columns reach is a value that k columns reach -- no bitmap lookups here.
            float tmax = __uint_as_float(0xff800000u);
#pragma unroll
            for (int u = 0; u < U; u++)
                if (v0 + u * NT < b0) tmax = fmaxf(tmax, vec_max_raw<T>(ra[u]));
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
            if (POST) t0 = post_seed_logit(t0, POSTP);
            if (c.pen_bitmap) t0 = penalise(t0, c.pen);
            t0 = __fmul_rn(t0, c.inv_temp);
            if (POST) {
                thr = t0;
                rthr = post_raw_bound(thr, c.inv_temp, POSTP);
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (v0 + u * NT < b0) filter_vec_post<S, T, true>(ra[u], v0 + u * NT, c, POSTP, rthr, thr, buf, ctl);
            } else {
                thr = t0;
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (v0 + u * NT < b0) filter_vec<S, T, true>(ra[u], v0 + u * NT, c, thr, buf, ctl);
            }
        }
        region_end(k + 1);

        // -- regions 1.. : two register sets, each refilled while the other is filtered --
        // The barrier carries only the vote (the register sets are private), so it need not follow
        // every region: the threshold is refreshed at most every LDG_VOTE_EVERY regions, at the
        // price of a few more survivors under a threshold that is that much staler.
        int r = 1;
        while (r < nreg && !careful) {
            if (r + 1 < nreg) load(ra, r + 1);
            ahead(r + 3);
            later(rb, r);
            if (r % LDG_VOTE_EVERY == 0 || r + 1 == nreg) region_end(trig);
            if (++r >= nreg || careful) break;
            if (r + 1 < nreg) load(rb, r + 1);
            ahead(r + 3);
            later(ra, r);
            if (r % LDG_VOTE_EVERY == 0 || r + 1 == nreg) region_end(trig);
            ++r;
        }
    }

    if (!careful) {
        // the columns of the partial vectors at the ends of this item
        int r1_lo = elo, r1_hi = ehi, r2_lo = ehi, r2_hi = ehi;
        if (b0 > a0) {
            r1_hi = min(ehi, max(elo, a0 * VEC - c.mis));
            r2_lo = max(elo, b0 * VEC - c.mis);
        }
        const int n1 = r1_hi - r1_lo, n2 = r2_hi - r2_lo;
        if (tid < n1 + n2) {  // at most 4 * VEC columns
            int e = tid < n1 ? r1_lo + tid : r2_lo + (tid - n1);
            float raw = Elem<T>::load1(c.row, e);
            if (POST) {
                if (raw >= rthr) consider_post<S, true>(buf, ctl, c, POSTP, raw, e, thr);
            } else {
                float v = __fmul_rn(raw, c.inv_temp);
                if (v >= thr) consider<S, true>(buf, ctl, c, raw, v, e, thr);
            }
        }
        __syncthreads();
        if (live_count(ctl) > CAP) careful = true;
        __syncthreads();
    }

    if (careful) {  // the careful path of scan_rows_kernel
        __syncthreads();
        if (tid == 0) ctl->cnt = 0;
        __syncthreads();
        thr = __uint_as_float(0xff800000u);
        bool strict = false;
        constexpr int STEP = NT * S::SLOW_EPT;
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
            for (int j = 0; j < S::SLOW_EPT; j++) {
                int e = e0 + j * NT + tid;
                if (e < ehi) {
                    float l = Elem<T>::load1(c.row, e);
                    if (POST) l = post_logit(l, POSTP);
                    if (c.pen_bitmap && bm_test(bm, e)) l = penalise(l, c.pen);
                    float v = __fmul_rn(l, c.inv_temp);
                    if (strict ? (v > thr) : (v >= thr)) append<S>(buf, ctl, v, e + c.voff);
                }
            }
        }
        __syncthreads();
    }

    bool have, ordered;
    refresh_topk<S>(buf, ctl, hist, k, tid, &have, &ordered);
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
    finish_row<S, MODE>(a, row, split, P, greedy, ordered, buf, ctl, tid);
}

// ---------------------------------------------------------------------------------------
// Long shortlists: top_k above MANTLE_SAMPLE_MAX_TOP_K, up to the whole vocabulary.
//
// The reference's Sample with a shortlist of tens of thousands of entries (TopK >= V is its
// only way to a whole-vocabulary nucleus, sampler.go:147) needs the shortlist in order only to
// walk its prefix sums.  This kernel never orders it.  One CTA per row answers three questions
// of the same form -- "at which position of the order (key descending, index ascending) does a
// monotone predicate on the running (mass, count) first hold?" -- by a radix search over the
// key: each pass streams the row, sums the mass and the count of the 16 sub-ranges of the
// current key range, and descends into the sub-range where the predicate turns true.  The
// search ends at one key; entries sharing a key share a probability, so the position inside
// the tie group follows by arithmetic and the index by one counting pass in index order.
//   KTH   count >= k                                   -> shortlist membership (top_k < V)
//   CUT   float32(prefix) >= top_p                     -> nucleus length   (sampler.go:212-222)
//   DRAW  r <= prefix, or CUT                          -> the token        (sampler.go:224-233)
// Sums are taken in double like the reference's but in tree order, not shortlist order: the
// prefix can differ from the reference's in the last bits (about 1e-16 relative), which moves a
// token only when r lies that close to a boundary -- far inside the contract's 1e-6.
// The row is read once per pass (11 to 30 passes; it stays in L2 after the first), so this
// path is compute-bound by design and meant for the rare request, not for throughput.

constexpr int WIDE_NT = 512;
constexpr int WIDE_FAN = 16;  // sub-ranges per pass (4 key bits)

struct WideCtl {
    double mass[WIDE_FAN];
    unsigned long long count[WIDE_FAN];
    double red_d[WIDE_NT / 32][WIDE_FAN];
    unsigned long long red_c[WIDE_NT / 32][WIDE_FAN];
    uint32_t red_min[WIDE_NT / 32], red_max[WIDE_NT / 32];
    double scalar_d;
    unsigned long long scalar_c;
    uint32_t kmin, kmax;
    int decided;     // radix search: chosen sub-range
    int found_flag;  //               the predicate turned true inside it
};

enum { WIDE_KTH = 0, WIDE_CUT = 1, WIDE_DRAW = 2 };

// Where a search ended: the key, the mass and count of everything before that key's tie
// group, the size of the group and the probability each member carries.
struct WideHit {
    uint32_t key;
    double mass_before;
    unsigned long long count_before;
    unsigned long long ties;
    double p_each;
    bool found;  // the predicate turned true somewhere (else: the search ended on the last entry)
};

template <typename T>
__global__ void __launch_bounds__(WIDE_NT, 1) wide_rows_kernel(const KArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    WideCtl* w = reinterpret_cast<WideCtl*>(smem_raw);
    uint32_t* bm = reinterpret_cast<uint32_t*>(smem_raw + ((sizeof(WideCtl) + 127) / 128) * 128);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x;
    const int V = a.vocab;

    const MantleSampleParams P = row_params(a, row);
    bool greedy, bad_k;
    const int k = row_k(a, P, 0x7fffffff, &greedy, &bad_k);  // no cap on this path
    if (bad_k) {
        if (tid == 0) {
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_TOPK_RANGE);
            a.next[row] = -1;
            if (a.n_kept) a.n_kept[row] = 0;
            if (a.cut) a.cut[row] = 0;
        }
        return;
    }
    const float inv_temp = greedy ? 1.0f : __fdiv_rn(1.0f, P.temperature);
    const void* rowp = reinterpret_cast<const T*>(a.logits) + (size_t)row * (size_t)a.row_stride;

    const int hl = history_len(a, row);
    WinPlan wp = win_plan(a, P, hl);
    wp.staged = false;
    const bool pen = wp.active;
    if (pen) build_penalty_bitmap(a, row, wp, hl, nullptr, V, a.vocab_offset, bm, tid, WIDE_NT);

    // scaled, penalised value of column e and its key
    const Post& post = a.post;
    auto value = [&](int e) {
        float l = Elem<T>::load1(rowp, e);
        if (post.mode) l = post_logit(l, post);
        if (pen && bm_test(bm, e)) l = penalise(l, P.repeat_penalty);
        return __fmul_rn(l, inv_temp);
    };

    // ---- block reductions ---------------------------------------------------------------------
    auto reduce_minmax = [&](uint32_t lo, uint32_t hi) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if (lane == 0) {
            w->red_min[warp] = lo;
            w->red_max[warp] = hi;
        }
        csync<WIDE_NT>();
        if (tid == 0) {
            for (int i = 1; i < WIDE_NT / 32; i++) {
                lo = min(lo, w->red_min[i]);
                hi = max(hi, w->red_max[i]);
            }
            w->kmin = lo;
            w->kmax = hi;
        }
        csync<WIDE_NT>();
    };
    auto reduce_sum = [&](double d, unsigned long long c) {  // -> w->scalar_d, w->scalar_c
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            d = __dadd_rn(d, __shfl_xor_sync(0xffffffffu, d, o));
            c += __shfl_xor_sync(0xffffffffu, c, o);
        }
        if (lane == 0) {
            w->red_d[warp][0] = d;
            w->red_c[warp][0] = c;
        }
        csync<WIDE_NT>();
        if (tid == 0) {
            for (int i = 1; i < WIDE_NT / 32; i++) {
                d = __dadd_rn(d, w->red_d[i][0]);
                c += w->red_c[i][0];
            }
            w->scalar_d = d;
            w->scalar_c = c;
        }
        csync<WIDE_NT>();
    };

    // ---- pass 1: the key range of the row ------------------------------------------------------
    {
        uint32_t lo = 0xffffffffu, hi = 0;
        for (int e = tid; e < V; e += WIDE_NT) {
            const float v = value(e);
            if (v == v) {  // NaN is outside the contract and takes no part
                const uint32_t key = f2key(v);
                lo = min(lo, key);
                hi = max(hi, key);
            }
        }
        reduce_minmax(lo, hi);
    }
    const uint32_t row_kmin = w->kmin, row_kmax = w->kmax;
    if (row_kmax < row_kmin || greedy) {  // an all-NaN row, or argmax rows routed here by a long-shortlist batch
        // argmax with the lowest index: the DRAW machinery is not needed
        unsigned long long best = 0xffffffffffffffffull;
        if (row_kmax >= row_kmin)
            for (int e = tid; e < V; e += WIDE_NT) {
                const float v = value(e);
                if (v == v && f2key(v) == row_kmax) best = min(best, (unsigned long long)e);
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (lane == 0) w->red_c[warp][0] = best;
        csync<WIDE_NT>();
        if (tid == 0) {
            for (int i = 1; i < WIDE_NT / 32; i++) best = min(best, w->red_c[i][0]);
            a.next[row] = best == 0xffffffffffffffffull ? 0 : (int)best + a.vocab_offset;
            if (a.n_kept) a.n_kept[row] = 0;
            if (a.cut) a.cut[row] = 0;
        }
        return;
    }
    const float maxv = key2f(row_kmax);  // the shortlist's maximum: its first entry (sampler.go:154-160)

    // Shortlist membership (set by the KTH search when k < V).
    uint32_t member_key = 0;        // keys above it are in
    int member_idx = 0x7fffffff;    // entries with that key are in up to this column
    // Probability stages (sampler.go:165-210): e -> e * inv_sum -> (min-p) -> * scale.
    double inv_sum = 1.0, minp_thr = -1.0, scale = 1.0;
    int stage = 0;  // 0: count only (KTH search); 1: e; 2: final probabilities
    auto member = [&](uint32_t key, int e) { return key > member_key || (key == member_key && e <= member_idx); };
    // mass an element contributes at the current stage; false: it is not part of the shortlist (any more)
    auto weigh = [&](float v, uint32_t key, int e, double* p) {
        if (!member(key, e)) return false;
        if (stage == 0) {
            *p = 0.0;
            return true;
        }
        const double ex = (double)fast_exp(__fsub_rn(v, maxv));
        if (stage == 1) {
            *p = ex;
            return true;
        }
        double q = __dmul_rn(ex, inv_sum);
        if (q < minp_thr) return false;  // sampler.go:188: kept iff prob >= threshold
        *p = __dmul_rn(q, scale);
        return true;
    };

    // ---- the radix search ----------------------------------------------------------------------
    auto search = [&](int mode, unsigned long long want_count, double r, float top_p, bool nucleus) {
        WideHit hit;
        hit.mass_before = 0.0;
        hit.count_before = 0;
        hit.found = false;
        uint32_t lo = row_kmin, hi = row_kmax;  // current key range, inclusive
        unsigned long long in_range = 0;
        double in_mass = 0.0;
        for (;;) {
            // sub-range j covers keys (hi - (j+1)*width, hi - j*width]; j = 0 holds the largest keys
            const uint32_t span = hi - lo;  // >= 0
            const uint32_t width = span / WIDE_FAN + 1;
            double m[WIDE_FAN];
            unsigned long long c[WIDE_FAN];
#pragma unroll
            for (int j = 0; j < WIDE_FAN; j++) {
                m[j] = 0.0;
                c[j] = 0;
            }
            for (int e = tid; e < V; e += WIDE_NT) {
                const float v = value(e);
                if (!(v == v)) continue;
                const uint32_t key = f2key(v);
                if (key < lo || key > hi) continue;
                double p;
                if (!weigh(v, key, e, &p)) continue;
                const int j = (int)((hi - key) / width);
#pragma unroll
                for (int q = 0; q < WIDE_FAN; q++)
                    if (q == j) {
                        m[q] = __dadd_rn(m[q], p);
                        c[q]++;
                    }
            }
#pragma unroll
            for (int j = 0; j < WIDE_FAN; j++) {
                double d = m[j];
                unsigned long long n = c[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    d = __dadd_rn(d, __shfl_xor_sync(0xffffffffu, d, o));
                    n += __shfl_xor_sync(0xffffffffu, n, o);
                }
                if (lane == 0) {
                    w->red_d[warp][j] = d;
                    w->red_c[warp][j] = n;
                }
            }
            csync<WIDE_NT>();
            if (tid < WIDE_FAN) {
                double d = 0.0;
                unsigned long long n = 0;
                for (int i = 0; i < WIDE_NT / 32; i++) {
                    d = __dadd_rn(d, w->red_d[i][tid]);
                    n += w->red_c[i][tid];
                }
                w->mass[tid] = d;
                w->count[tid] = n;
            }
            csync<WIDE_NT>();
            if (tid == 0) {
                // walk the sub-ranges from the largest keys down; stop where the predicate turns true
                double cum = hit.mass_before;
                unsigned long long cnt = hit.count_before;
                int chosen = -1, last_nonempty = -1;
                bool turned = false;
                for (int j = 0; j < WIDE_FAN; j++) {
                    if (w->count[j] == 0) continue;
                    last_nonempty = j;
                    const double cum_end = __dadd_rn(cum, w->mass[j]);
                    const unsigned long long cnt_end = cnt + w->count[j];
                    bool ok;
                    if (mode == WIDE_KTH) ok = cnt_end >= want_count;
                    else {
                        ok = nucleus && __double2float_rn(cum_end) >= top_p;
                        if (mode == WIDE_DRAW) ok = ok || r <= cum_end;
                    }
                    if (ok) {
                        chosen = j;
                        turned = true;
                        break;
                    }
                    cum = cum_end;
                    cnt = cnt_end;
                }
                if (chosen < 0) {  // never true: end on the last entry of the order
                    chosen = last_nonempty;
                    cum = hit.mass_before;
                    cnt = hit.count_before;
                    for (int j = 0; j < chosen; j++) {
                        cum = __dadd_rn(cum, w->mass[j]);
                        cnt += w->count[j];
                    }
                }
                w->decided = chosen;
                w->found_flag = turned ? 1 : 0;
                w->scalar_d = cum;
                w->scalar_c = cnt;
            }
            csync<WIDE_NT>();
            const int j = w->decided;
            hit.found = w->found_flag != 0;
            hit.mass_before = w->scalar_d;
            hit.count_before = w->scalar_c;
            in_range = w->count[j];
            in_mass = w->mass[j];
            csync<WIDE_NT>();
            const uint32_t new_hi = hi - (uint32_t)j * width;
            const uint32_t below = new_hi - lo;  // keys available under new_hi inside the range
            const uint32_t new_lo = below >= width - 1 ? new_hi - (width - 1) : lo;
            hi = new_hi;
            lo = new_lo;
            if (width == 1) break;  // the range is one key
        }
        hit.key = hi;
        hit.ties = in_range;
        hit.p_each = in_range ? in_mass / (double)in_range : 0.0;
        return hit;
    };

    // position (1-based) inside a tie group at which the predicate first holds; the group's
    // members carry equal probabilities, added one by one
    auto tie_position = [&](const WideHit& h, int mode, unsigned long long want_count, double r, float top_p,
                            bool nucleus) {
        if (mode == WIDE_KTH) return want_count - h.count_before;
        if (!h.found) return h.ties;
        // exact element probability: recomputed by whoever owns the key; here the mean of the group,
        // which is the same number because equal keys have equal values
        unsigned long long lo = 1, hi = h.ties;
        auto holds = [&](unsigned long long j) {
            const double c = __dadd_rn(h.mass_before, __dmul_rn((double)j, h.p_each));
            bool ok = nucleus && __double2float_rn(c) >= top_p;
            if (mode == WIDE_DRAW) ok = ok || r <= c;
            return ok;
        };
        if (!holds(hi)) return hi;
        while (lo < hi) {
            const unsigned long long mid = (lo + hi) / 2;
            if (holds(mid)) hi = mid;
            else lo = mid + 1;
        }
        return lo;
    };

    // column of the j-th (1-based) shortlist member with the given key, in index order
    auto nth_with_key = [&](uint32_t key, unsigned long long j) {
        const int per = (V + WIDE_NT - 1) / WIDE_NT;
        const int e0 = tid * per, e1 = min(V, e0 + per);
        unsigned long long mine = 0;
        for (int e = e0; e < e1; e++) {
            const float v = value(e);
            double p;
            if (v == v && f2key(v) == key && weigh(v, key, e, &p)) mine++;
        }
        // exclusive scan over threads (contiguous column ranges in thread order)
        unsigned long long incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            unsigned long long y = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += y;
        }
        if (lane == 31) w->red_c[warp][0] = incl;
        csync<WIDE_NT>();
        unsigned long long base = 0;
        for (int i = 0; i < warp; i++) base += w->red_c[i][0];
        const unsigned long long before = base + incl - mine;
        if (tid == 0) w->decided = -1;
        csync<WIDE_NT>();
        if (mine > 0 && before < j && j <= before + mine) {
            unsigned long long seen = before;
            for (int e = e0; e < e1; e++) {
                const float v = value(e);
                double p;
                if (v == v && f2key(v) == key && weigh(v, key, e, &p)) {
                    if (++seen == j) {
                        w->decided = e;
                        break;
                    }
                }
            }
        }
        csync<WIDE_NT>();
        const int e = w->decided;
        csync<WIDE_NT>();
        return e;
    };

    // ---- shortlist membership: the k best (sampler.go:255-296) ---------------------------------
    if (k < V) {
        stage = 0;
        const WideHit h = search(WIDE_KTH, (unsigned long long)k, 0.0, 1.0f, false);
        const unsigned long long j = tie_position(h, WIDE_KTH, (unsigned long long)k, 0.0, 1.0f, false);
        member_key = 0;  // the counting pass must see every entry with the key
        member_idx = 0x7fffffff;
        const int cut_col = j >= h.ties ? 0x7fffffff : nth_with_key(h.key, j);
        member_key = h.key;
        member_idx = cut_col;
    }

    // ---- softmax over the shortlist (sampler.go:154-177) ----------------------------------------
    stage = 1;
    {
        double s = 0.0;
        unsigned long long n = 0;
        for (int e = tid; e < V; e += WIDE_NT) {
            const float v = value(e);
            if (!(v == v)) continue;
            double p;
            if (weigh(v, f2key(v), e, &p)) {
                s = __dadd_rn(s, p);
                n++;
            }
        }
        reduce_sum(s, n);
    }
    const double sum = w->scalar_d;
    unsigned long long n_kept = w->scalar_c;
    csync<WIDE_NT>();
    if (sum == 0.0) {  // sampler.go:170-172: cannot happen (the maximum contributes fastExp(0) = 1), kept for form
        if (tid == 0) {
            a.next[row] = 0;
            if (a.n_kept) a.n_kept[row] = (int)n_kept;
            if (a.cut) a.cut[row] = 0;
        }
        return;
    }
    inv_sum = __ddiv_rn(1.0, sum);
    stage = 2;

    // ---- min-p (sampler.go:180-210) --------------------------------------------------------------
    if (P.min_p > 0.0f) {
        // prob[0] = fastExp(0) * inv_sum = inv_sum
        minp_thr = __dmul_rn(__dmul_rn((double)fast_exp(0.0f), inv_sum), (double)P.min_p);
        double s = 0.0;
        unsigned long long n = 0;
        for (int e = tid; e < V; e += WIDE_NT) {
            const float v = value(e);
            if (!(v == v)) continue;
            double p;
            if (weigh(v, f2key(v), e, &p)) {
                s = __dadd_rn(s, p);
                n++;
            }
        }
        reduce_sum(s, n);
        const double new_sum = w->scalar_d;
        const unsigned long long kept = w->scalar_c;
        csync<WIDE_NT>();
        if (kept < n_kept && new_sum > 0.0) scale = __ddiv_rn(1.0, new_sum);
        n_kept = kept;
        if (kept == 0) {  // min_p > 1 dropped everything: the reference indexes topIdx[-1] and panics
            if (tid == 0) {
                a.next[row] = -1;
                if (a.n_kept) a.n_kept[row] = 0;
                if (a.cut) a.cut[row] = 0;
                if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_EMPTY);
            }
            return;
        }
    }

    // ---- top-p cut and draw (sampler.go:212-233) ---------------------------------------------------
    const bool nucleus = P.top_p < 1.0f;
    int cut = (int)n_kept;
    if (a.cut && nucleus) {
        const WideHit h = search(WIDE_CUT, 0, 0.0, P.top_p, true);
        if (h.found) cut = (int)(h.count_before + tie_position(h, WIDE_CUT, 0, 0.0, P.top_p, true));
    }
    const WideHit h = search(WIDE_DRAW, 0, P.uniform, P.top_p, nucleus);
    const unsigned long long j = tie_position(h, WIDE_DRAW, 0, P.uniform, P.top_p, nucleus);
    const int col = nth_with_key(h.key, j);
    if (tid == 0) {
        a.next[row] = col < 0 ? -1 : col + a.vocab_offset;
        if (a.n_kept) a.n_kept[row] = (int)n_kept;
        if (a.cut) a.cut[row] = cut;
    }
}

// Merge of `parts` local shortlists per row (several CTAs of one GPU, or one per
// vocabulary shard after an all-gather), then the tail.
__global__ void __launch_bounds__(ShapeLargeK::NT, ShapeLargeK::MINB) merge_parts_kernel(const KArgs a) {
    using S = ShapeLargeK;
    extern __shared__ __align__(128) unsigned char smem_raw[];
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
    bool have, ordered;
    refresh_topk<S>(buf, ctl, hist, k, tid, &have, &ordered);
    __syncthreads();
    finish_row<S, MODE_FUSED>(a, row, 0, P, greedy, ordered, buf, ctl, tid);
}

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

// Shape selection.  MANTLE_SAMPLER_SHAPE=small|large overrides it (a tuning aid: `small`
// is refused, by falling back, for batches whose top_k it cannot serve).
int forced_shape() {
    static const int forced = [] {
        const char* e = getenv("MANTLE_SAMPLER_SHAPE");
        if (!e) return 0;
        return strcmp(e, "small") == 0 ? 1 : (strcmp(e, "large") == 0 ? 2 : (strcmp(e, "alt") == 0 ? 3 : 0));
    }();
    return forced;
}

// MANTLE_SAMPLER_KERNEL=ldg|tma picks the streaming kernel for shortlists of at most 256 entries.
int forced_kernel() {
    static const int forced = [] {
        const char* e = getenv("MANTLE_SAMPLER_KERNEL");
        if (!e) return 0;
        return strcmp(e, "ldg") == 0 ? 1 : (strcmp(e, "tma") == 0 ? 2 : 0);
    }();
    return forced;
}

bool use_small_shape(int max_top_k) {
    if (max_top_k > ShapeSmallK::KCAP) return false;
    return forced_shape() != 2;
}

// Which streaming kernel serves a batch: plain loads, unless MANTLE_SAMPLER_KERNEL=tma asks for
// the bulk-copy ring (which has no post-processing form).  Measured on 151 936-column float32
// rows, plain loads against the ring: 0.437 against 0.541 ms for 4096 rows at top_k 20;
// 0.93 against 1.06 ms (top_k 300), 1.22 against 1.46 ms (512), 3.70 against 3.86 ms (1024)
// for 2048 rows.
bool use_ldg(int max_top_k, bool post) {
    (void)max_top_k;
    return post || forced_kernel() != 2;
}

bool use_alt_shape(int max_top_k) { return forced_shape() == 3 && max_top_k <= ShapeAlt::KCAP; }

struct SmemBudget {
    int per_sm;     // shared memory of one SM
    int per_block;  // largest opt-in dynamic shared memory of one CTA
    int sms;
};

SmemBudget smem_budget() {
    SmemBudget b = {233472, 232448, 148};  // B200 figures, used when no device can be asked
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return b;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess && v > 0) b.per_sm = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess && v > 0) b.per_block = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) b.sms = v;
    return b;
}

// Ring depth and CTAs per SM for one shape and vocabulary: as many stages as fit beside the
// candidate buffer and the bitmap with MINB CTAs on an SM; one CTA per SM with a deeper ring
// when fewer than two stages would fit.
template <class S>
bool plan_ring(int vocab, const SmemBudget& bud, int* stages, int* ctas_per_sm, size_t* smem) {
    const size_t chunk = (size_t)S::NT * S::U * 16;
    const size_t fixed = S::SMEM_FIXED + bitmap_words(vocab) * sizeof(uint32_t);
    for (int ctas = S::MINB; ctas >= 1; ctas--) {
        const long long room = std::min<long long>(bud.per_sm / ctas - 1024, bud.per_block) - (long long)fixed;
        int st = room > 0 ? (int)(room / (long long)chunk) : 0;
        st = std::min(st, ctas == 1 ? 6 : 3);
        if (st >= 2) {
            *stages = st;
            *ctas_per_sm = ctas;
            *smem = fixed + (size_t)st * chunk;
            return true;
        }
    }
    return false;
}

int choose_splits(const MantleSampleBatch* b) {
    if (b->max_top_k > KMAX) return 1;  // long shortlists: one CTA per row, no merge
    const int vec = b->dtype == MANTLE_DTYPE_F32 ? 4 : 8;
    const int nvec = (b->vocab + vec - 1) / vec + 1;
    const bool ldg = use_ldg(b->max_top_k, post_mode_of(b->logit_scale, b->logit_softcap, b->flags) != 0);
    const bool small = ldg ? b->max_top_k <= ShapeLdg::KCAP : use_small_shape(b->max_top_k);
    const int chunk = ldg ? (small ? ShapeLdg::NT * ShapeLdg::U : ShapeLdgLargeK::NT * ShapeLdgLargeK::U)
                          : (small ? ShapeSmallK::NT * ShapeSmallK::U : ShapeLargeK::NT * ShapeLargeK::U);
    const int per_sm = ldg ? (small ? ShapeLdg::MINB : ShapeLdgLargeK::MINB)
                           : (small ? ShapeSmallK::MINB : ShapeLargeK::MINB);
    const int max_by_k = MERGE_CAP / b->max_top_k;  // the merge holds splits * k candidates
    if (b->splits > 0) return std::max(1, std::min(std::min(b->splits, max_by_k), std::min(nvec, 64)));
    const int max_by_work = nvec / (2 * chunk);  // at least two chunks per CTA
    const int cap = std::max(1, std::min(std::min(max_by_k, max_by_work), 64));
    const int target = per_sm * smem_budget().sms;  // one full wave
    if (b->rows >= target) return 1;
    return std::max(1, std::min(cap, (target + b->rows - 1) / b->rows));
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
    a.hist_tma_ok = a.history && reinterpret_cast<uintptr_t>(a.history) % 16 == 0 && a.hist_stride % 4 == 0;
    a.post.mode = post_mode_of(b->logit_scale, b->logit_softcap, b->flags);
    a.post.scale = b->logit_scale;
    a.post.cap = b->logit_softcap;
#ifdef MANTLE_DEBUG_SWITCHES
    const char* dbg = getenv("MANTLE_SAMPLER_DEBUG");
    a.debug = dbg ? atoi(dbg) : 0;
#endif
}

template <class S, int MODE>
int launch_scan_shape(const KArgs& a, int dtype, cudaStream_t stream) {
    const SmemBudget bud = smem_budget();
    int stages = 0, ctas = 0;
    size_t smem = 0;
    if (!plan_ring<S>(a.vocab, bud, &stages, &ctas, &smem)) return kInvalid;
    const long long items = (long long)a.rows * a.splits;
    if (items > 0x7fffffffLL) return kInvalid;
    const int grid = (int)std::min<long long>(items, (long long)ctas * bud.sms);
    cudaError_t e;
    if (dtype == MANTLE_DTYPE_F32) {
        auto kern = scan_rows_kernel<S, float, MODE>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, S::NT, smem, stream>>>(a, stages);
    } else {
        auto kern = scan_rows_kernel<S, bf16_t, MODE>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, S::NT, smem, stream>>>(a, stages);
    }
    return (int)cudaGetLastError();
}

template <class S, typename T, int MODE, bool POST>
int launch_scan_ldg_as(const KArgs& a, cudaStream_t stream) {
    const size_t smem = LdgLayout<S>::FIXED + bitmap_words(a.vocab) * sizeof(uint32_t);
    const long long items = (long long)a.rows * a.splits;
    if (items > 0x7fffffffLL) return kInvalid;
    auto kern = scan_rows_ldg_kernel<S, T, MODE, POST>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    kern<<<(int)items, S::NT, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

template <class S, int MODE>
int launch_scan_ldg(const KArgs& a, int dtype, cudaStream_t stream) {
    if (a.post.mode)
        return dtype == MANTLE_DTYPE_F32 ? launch_scan_ldg_as<S, float, MODE, true>(a, stream)
                                         : launch_scan_ldg_as<S, bf16_t, MODE, true>(a, stream);
    return dtype == MANTLE_DTYPE_F32 ? launch_scan_ldg_as<S, float, MODE, false>(a, stream)
                                     : launch_scan_ldg_as<S, bf16_t, MODE, false>(a, stream);
}

template <int MODE>
int launch_scan(const KArgs& a, int dtype, cudaStream_t stream) {
    if (use_ldg(a.max_top_k, a.post.mode != 0)) {
        if (a.max_top_k <= ShapeLdg::KCAP) return launch_scan_ldg<ShapeLdg, MODE>(a, dtype, stream);
        return launch_scan_ldg<ShapeLdgLargeK, MODE>(a, dtype, stream);
    }
    if (use_alt_shape(a.max_top_k)) return launch_scan_shape<ShapeAlt, MODE>(a, dtype, stream);
    if (use_small_shape(a.max_top_k)) return launch_scan_shape<ShapeSmallK, MODE>(a, dtype, stream);
    return launch_scan_shape<ShapeLargeK, MODE>(a, dtype, stream);
}

int launch_merge(const KArgs& a, cudaStream_t stream) {
    const size_t smem = ShapeLargeK::SMEM_FIXED;
    cudaError_t e = cudaFuncSetAttribute(merge_parts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    merge_parts_kernel<<<a.rows, ShapeLargeK::NT, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

int launch_wide(const KArgs& a, int dtype, cudaStream_t stream) {
    const size_t smem = ((sizeof(WideCtl) + 127) / 128) * 128 + bitmap_words(a.vocab) * sizeof(uint32_t);
    cudaError_t e;
    if (dtype == MANTLE_DTYPE_F32) {
        e = cudaFuncSetAttribute(wide_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        wide_rows_kernel<float><<<a.rows, WIDE_NT, smem, stream>>>(a);
    } else {
        e = cudaFuncSetAttribute(wide_rows_kernel<bf16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        wide_rows_kernel<bf16_t><<<a.rows, WIDE_NT, smem, stream>>>(a);
    }
    return (int)cudaGetLastError();
}

int launch_penalty(const KArgs& a, cudaStream_t stream) {
    const size_t smem = bitmap_words(a.vocab) * sizeof(uint32_t);
    cudaError_t e = cudaFuncSetAttribute(penalty_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
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

extern "C" int mantleCudaSamplerAbiVersion(void) { return 2; }

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
    return launch_merge(a, stream);
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
    const int grid = (int)std::min<long long>((n + 255) / 256, (long long)smem_budget().sms * 32);
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

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices];    // device address of g_split_scratch, per device ordinal
bool g_scratch_known[kMaxDevices];
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
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_known[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_split_scratch);
        if (e != cudaSuccess) {
            set_last_error("cudaGetSymbolAddress failed with cudaError %llu", (unsigned long long)e);
            return (int)e;
        }
        g_scratch_addr[dev] = p;
        g_scratch_known[dev] = true;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" const char* mantleCudaSamplerLastError(void) { return g_last_error; }

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
