// Shapes, shared-memory records, kernel arguments and the per-column helpers (keys, fastExp,
// penalty, head post-processing, the filter and the candidate buffer) every sampler kernel shares.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

constexpr int KMAX = MANTLE_SAMPLE_MAX_TOP_K;
constexpr int RANK_MAX = 256;  // largest buffer the counting select takes
constexpr int HBINS = 256;     // bins of the running histogram of the candidate buffer

// Launch shape of one kernel instantiation.
//   NT    threads per CTA            U     16-byte vectors per thread per region
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
    // shared memory: [Cand buf[CAP]] [hist[HBINS]] [Ctl] [staged survivors[NWARP][STG]] [their counts[NWARP]] [bitmap]
    // raw survivors a warp sets aside before it works them off together.  (Sixty-four in the smaller shape
    // were measured slower at every shortlist length, the other kernel included: four CTAs of 41 KB push the
    // SM's shared-memory carve-out from 164 to 196 KB and leave the L1 a third less.)
    static constexpr int STG = 32;
    static constexpr size_t CTL_OFF = 8 * (size_t)CAP + 4 * (size_t)HBINS;
    static constexpr size_t STG_OFF = CTL_OFF + 512;
    static constexpr size_t WCNT_OFF = STG_OFF + 8 * (size_t)(NWARP * STG);
    static constexpr size_t SMEM_FIXED = WCNT_OFF + ((4 * (size_t)NWARP + 15) & ~(size_t)15);
    // the streaming loop compacts the buffer at its next meeting once it holds this many entries
    // (the shape for shortlists of up to 224 entries sees at most that many arrive between two meetings)
    static constexpr int FORCE = KCAP > 256 ? CAP / 2 : CAP / 4 * 3;
};
// Four small CTAs per SM overlap the serial phases of a row (bitmap, cuts, tail) with the
// streaming of three other rows; measured against three CTAs fed by a ring of bulk copies
// (0.541 against 0.403 ms for 4096 rows of 151 936 float32 columns at top_k 20) and against
// larger CTAs at every shortlist length.
using ShapeK256 = Shape<256, 4, 2048, 256, 4>;    // top_k <= 256: 16 KB candidate buffer, four CTAs per SM
using ShapeK1024 = Shape<256, 4, 4096, KMAX, 4>;  // top_k <= 1024: 32 KB candidate buffer
using ShapeMerge = Shape<512, 4, 4096, KMAX, 1>;  // the merge kernel where the parts hold more than ShapeK256 takes
constexpr int MAX_NWARP = 32;
constexpr int MERGE_CAP = ShapeMerge::CAP;

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
    int k;              // shortlist length wanted (for the warp that refreshes the threshold)
    // running histogram of the buffer's values: bin = (v - hbase) * hscale, clamped to [0, HBINS)
    uint32_t thr_key;   // key of the admission threshold: at least k buffered entries reach it
    float thr;          // the same as a value, for the streaming loop (any value once valid stays valid)
    float hbase, hscale;  // read as one float2
    float htop;
    float hwidth;       // 1 / hscale
    int walked;         // entries in the buffer when the histogram was last walked
    // what the out-of-line survivor code needs to know about the row
    int pen_on;         // the penalty is applied from the bitmap
    float inv_temp, pen;
    int voff;           // global id of column 0
    int post_mode;
    float post_scale, post_cap;
    int pad;
    double sum;
    double new_sum;
    float warpv[MAX_NWARP];
    uint32_t warpk_min[MAX_NWARP];
    uint32_t warpk_max[MAX_NWARP];
};
static_assert(sizeof(Ctl) <= 512 && sizeof(Ctl) % 8 == 0, "control block outgrew its slot");

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
    double* token_prob;
    double* softmax_sum;
    const int32_t* skip;  // rows with a non-zero entry are not sampled
    int cand_stride;
    // MODE_PARTS outputs / merge inputs: part p of row r at (p*rows + r)*part_cap
    float* part_val;
    int32_t* part_idx;
    int32_t* part_cnt;
    int part_cap;
    long long part_stride;  // elements from one part's values (ids) to the next part's: rows * part_cap unless packed
    long long cnt_stride;   // the same for the counts: rows unless packed
    int parts;
    Post post;  // read from the kernel's parameter space where it is used, never copied to registers
#ifdef MANTLE_DEBUG_SWITCHES
    int debug;
#endif
};

// ---------------------------------------------------------------------------------------
// small helpers

// One row's results, written by one thread.  Rows that end in argmax, or in an error, report
// zero lengths and probabilities.
__device__ __forceinline__ void publish_row(const KArgs& a, int row, int token, int n_kept = 0, int cut = 0,
                                            double token_prob = 0.0, double sum = 0.0) {
    a.next[row] = token;
    if (a.n_kept) a.n_kept[row] = n_kept;
    if (a.cut) a.cut[row] = cut;
    if (a.token_prob) a.token_prob[row] = token_prob;
    if (a.softmax_sum) a.softmax_sum[row] = sum;
}

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

// ---------------------------------------------------------------------------------------
// The running histogram.  While a row streams, every entry that enters the candidate buffer is
// also counted in one of HBINS bins of its value.  The bin is a non-decreasing map of the value, so
// walking the counts from the top bin down to the bin b where they reach k gives a threshold --
// the lower edge of bin b -- that at least k buffered entries reach, without a barrier and without
// touching the buffer: one warp does it after every region while the others stream on.  A column
// below such a threshold is below k buffered entries and can be in no shortlist; a column AT it
// may be (the entries that reach the threshold can have higher indices), so admission is `>=`.
__device__ __forceinline__ int hist_bin(float v, float base, float scale) {
    const float d = __fmul_rn(__fsub_rn(v, base), scale);
    return d > 0.0f ? (d < (float)(HBINS - 1) ? (int)d : HBINS - 1) : 0;  // NaN (inf - inf, inf * 0): bin 0
}

// The buffer entry and its count.  A count seen by the warp that walks the histogram stands for
// an entry that is in the buffer by the next barrier, which is before anything reads the buffer.
template <class S>
__device__ __forceinline__ void append_binned(Cand* buf, Ctl* ctl, float v, int gidx) {
    int slot = atomicAdd(&ctl->cnt, 1);
    if (slot < S::CAP) {
        Cand e;
        e.key = f2key(v);
        e.idx = (uint32_t)gidx;
        buf[slot] = e;
        uint32_t* hist = reinterpret_cast<uint32_t*>(buf + S::CAP);
        const float2 bs = *reinterpret_cast<const float2*>(&ctl->hbase);  // base, scale
        atomicAdd(&hist[hist_bin(v, bs.x, bs.y)], 1u);
    }
}

// Called by one whole warp: the key of the smallest value of the highest bin at which the counts
// from the top reach `need`, or 0 when they never do or do so only in the lowest bin.  Every
// counted value whose bin is that one or higher has a key of at least the returned one.
template <class S>
__device__ __noinline__ uint32_t hist_threshold(int need_) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const volatile uint32_t* hist = reinterpret_cast<const volatile uint32_t*>(smem_raw + 8 * (size_t)S::CAP);
    const Ctl* ctl = reinterpret_cast<const Ctl*>(smem_raw + S::CTL_OFF);
    static_assert(HBINS == 256, "a lane owns eight bins");
    const int lane = threadIdx.x & 31;
    const uint32_t need = (uint32_t)need_;
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
    above -= tot;  // entries in bins owned by higher lanes
    uint32_t key = 0u;
    if (above < need && need <= above + tot) {
        int bin = 0;
        uint32_t run = above;
#pragma unroll
        for (int b = 7; b >= 0; b--) {
            if (run < need && need <= run + c[b]) bin = lane * 8 + b;
            run += c[b];
        }
        const float base = ctl->hbase, scale = ctl->hscale;
        if (bin > 0 && scale > 0.0f) {
            // A value half a bin below the edge, which the bin function puts into a lower bin (checked):
            // whatever is counted in `bin` or above is larger (the map is non-decreasing), so the next
            // key up is reached by all of it.
            const float t = __fadd_rn(base, __fmul_rn((float)bin - 0.5f, ctl->hwidth));
            if (hist_bin(t, base, scale) < bin) key = f2key(t) + 1u;
        }
    }
    const uint32_t who = __ballot_sync(0xffffffffu, key != 0u);
    return who ? __shfl_sync(0xffffffffu, key, __ffs(who) - 1) : 0u;
}

// One column whose RAW value reached the filter.  The penalty only ever lowers a logit
// (l/p < l for l > 0, l*p < l for l < 0, p > 1) and post-processing is filtered through a raw bound
// (post_raw_bound), so filtering raw values first is conservative: only here, on the rare
// survivor, are the exact value computed (a few hundred instructions with post-processing: two
// divides, fastExp or tanhf), the bitmap consulted, the penalty applied and the filter repeated
// -- against the threshold of this moment, which may have risen since the caller read its own.
// Out of line and once per kernel: inlined wherever a survivor can turn up, this code made the
// streaming loop outgrow the instruction cache (as many stalls waiting for instructions as at
// barriers).  What it needs of the row sits in the control block; the candidate buffer, the
// control block and the bitmap are at fixed offsets of the CTA's shared memory.
template <class S, bool POST>
__device__ __noinline__ void survivor(float raw, int e) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
    const uint32_t* bm = reinterpret_cast<const uint32_t*>(smem_raw + S::SMEM_FIXED);
    float l = raw;
    if (POST) {
        const Post post = {ctl->post_mode, ctl->post_scale, ctl->post_cap};
        l = post_logit(l, post);
    }
    if (ctl->pen_on && bm_test(bm, e)) l = penalise(l, ctl->pen);
    const float v = __fmul_rn(l, ctl->inv_temp);
    if (v >= *reinterpret_cast<const volatile float*>(&ctl->thr)) append_binned<S>(buf, ctl, v, e + ctl->voff);
}

// In the streaming loop a lane that finds a survivor only sets it aside -- raw value and column,
// two shared-memory operations -- in its warp's staging area; the warp works its staged survivors
// off together at the end of a region (flush_staged: one lane each, everything above in lock step,
// one reservation in the candidate buffer for all of them).  A lane that finds the area full takes
// the survivor through the code above at once.
template <class S, bool POST>
__device__ __forceinline__ void stage(float raw, int e) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    int* wcnt = reinterpret_cast<int*>(smem_raw + S::WCNT_OFF);
    const int warp = threadIdx.x >> 5;
    const int slot = atomicAdd(&wcnt[warp], 1);
    if (slot < S::STG)
        reinterpret_cast<uint2*>(smem_raw + S::STG_OFF)[warp * S::STG + slot] = make_uint2(__float_as_uint(raw), (uint32_t)e);
    else
        survivor<S, POST>(raw, e);
}

// Called by one whole warp between two regions.
template <class S, bool POST>
__device__ __noinline__ void flush_staged() {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + S::CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
    const uint32_t* bm = reinterpret_cast<const uint32_t*>(smem_raw + S::SMEM_FIXED);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int* wc = reinterpret_cast<int*>(smem_raw + S::WCNT_OFF) + warp;
    __syncwarp();
    const int n = min(*reinterpret_cast<volatile int*>(wc), S::STG);
    if (n == 0) return;
    for (int first = 0; first < n; first += 32) {  // 32 staged survivors at a time, one per lane
        bool pass = false;
        float v = 0.0f;
        int e = 0;
        if (first + lane < n) {
            const uint2 st = reinterpret_cast<const uint2*>(smem_raw + S::STG_OFF)[warp * S::STG + first + lane];
            e = (int)st.y;
            float l = __uint_as_float(st.x);
            if (POST) {
                const Post post = {ctl->post_mode, ctl->post_scale, ctl->post_cap};
                l = post_logit(l, post);
            }
            if (ctl->pen_on && bm_test(bm, e)) l = penalise(l, ctl->pen);
            v = __fmul_rn(l, ctl->inv_temp);
            pass = v >= *reinterpret_cast<const volatile float*>(&ctl->thr);
        }
        const uint32_t m = __ballot_sync(0xffffffffu, pass);
        if (m) {
            int base = 0;
            if (lane == 0) base = atomicAdd(&ctl->cnt, __popc(m));
            base = __shfl_sync(0xffffffffu, base, 0);
            const int slot = base + __popc(m & ((1u << lane) - 1u));
            if (pass && slot < S::CAP) {
                Cand c;
                c.key = f2key(v);
                c.idx = (uint32_t)(e + ctl->voff);
                buf[slot] = c;
                const float2 bs = *reinterpret_cast<const float2*>(&ctl->hbase);
                atomicAdd(&hist[hist_bin(v, bs.x, bs.y)], 1u);
            }
        }
    }
    __syncwarp();
    if (lane == 0) *wc = 0;
    __syncwarp();
}

// One complete 16-byte vector that may hold a survivor: the columns whose raw value reaches `rawthr`
// (for a batch without post-processing: whose scaled value reaches `thr`) are walked one at a time
// (NaN never passes a compare).
template <class S, typename T, bool POST>
__device__ __forceinline__ void filter_vec(const uint4& rawv, int vec, int mis, float inv_temp, float thr, float rawthr) {
    constexpr int VEC = Elem<T>::VEC;
    float raw[VEC];
    Elem<T>::widen(rawv, raw);
    uint32_t pass = 0;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        const bool in = POST ? raw[j] >= rawthr : __fmul_rn(raw[j], inv_temp) >= thr;
        pass |= in ? (1u << j) : 0u;
    }
    const int e0 = vec * VEC - mis;
    while (pass) {
        const int j = __ffs(pass) - 1;
        pass &= pass - 1;
        float r = raw[0];
#pragma unroll
        for (int q = 1; q < VEC; q++) r = (j == q) ? raw[q] : r;
        stage<S, POST>(r, e0 + j);
    }
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
// bfloat16: the eight values are compared as four packed pairs (three two-wide maxima) and only
// the winning pair is widened -- six instructions instead of fifteen.  Like fmaxf, the packed
// maximum returns the other operand when one is NaN, and -0.0 against +0.0 may return either,
// which no compare downstream can tell apart.
template <>
__device__ __forceinline__ float vec_max_raw<bf16_t>(const uint4& rawv) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&rawv.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&rawv.y);
    const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&rawv.z);
    const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(&rawv.w);
    const __nv_bfloat162 m2 = __hmax2(__hmax2(a, b), __hmax2(c, d));
    return fmaxf(__low2float(m2), __high2float(m2));
}

// The streaming loop's one test per thread and region is on the largest raw logit of the region's
// U vectors.  It is built from one partial maximum per vector, which the rarer path that follows a
// passed test finishes into that vector's own maximum (one more instruction) instead of starting over.
// float32: three-input maxima (sm_100) -- eight instructions for sixteen values; the partial is the
// maximum of the first three lanes of the vector.
__device__ __forceinline__ float max3f(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
template <typename T>
struct VecPart;
template <>
struct VecPart<float> {
    typedef float part_t;
    __device__ static __forceinline__ part_t part(const uint4& v) {
        return max3f(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z));
    }
    __device__ static __forceinline__ float finish(part_t p, const uint4& v) { return fmaxf(p, __uint_as_float(v.w)); }
    template <int U>
    __device__ static __forceinline__ float region(const part_t (&p)[U], const uint4 (&v)[U]) {
        float m = p[0];
#pragma unroll
        for (int u = 1; u < U; u++) m = max3f(m, __uint_as_float(v[u - 1].w), p[u]);
        return fmaxf(m, __uint_as_float(v[U - 1].w));
    }
};
// bfloat16: packed two-wide maxima; the partial is the vector's maximum still packed as a pair.
template <>
struct VecPart<bf16_t> {
    typedef __nv_bfloat162 part_t;
    __device__ static __forceinline__ part_t part(const uint4& v) {
        return __hmax2(__hmax2(*reinterpret_cast<const __nv_bfloat162*>(&v.x), *reinterpret_cast<const __nv_bfloat162*>(&v.y)),
                       __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&v.z), *reinterpret_cast<const __nv_bfloat162*>(&v.w)));
    }
    __device__ static __forceinline__ float finish(part_t p, const uint4&) { return fmaxf(__low2float(p), __high2float(p)); }
    template <int U>
    __device__ static __forceinline__ float region(const part_t (&p)[U], const uint4 (&)[U]) {
        part_t m = p[0];
#pragma unroll
        for (int u = 1; u < U; u++) m = __hmax2(m, p[u]);
        return fmaxf(__low2float(m), __high2float(m));
    }
};

}  // namespace
