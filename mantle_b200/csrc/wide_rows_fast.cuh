// wide_hist_kernel: shortlists longer than 1024 entries, up to the whole vocabulary, in three to
// five passes over the row.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// ---------------------------------------------------------------------------------------
// Long shortlists without ordering them.
//
// The reference's Sample with tens of thousands of shortlist entries (TopK >= V is its only way
// to a whole-vocabulary nucleus, sampler.go:147) needs the order only to walk prefix sums.  One
// CTA per row finds the few hundred entries around the place where the walk stops, orders only
// those, and walks only them:
//
//   pass 1   the row's largest and smallest scaled value (the softmax shifts by the largest,
//            sampler.go:154-160)
//   pass 2   a COUNT histogram of d = max - value over 8192 linear bins, and in the same pass
//            the softmax normaliser, sum of fastExp(value - max) (sampler.go:161-168)
//   locate   every entry of bin b has d inside the bin's edges, so fastExp(-d) lies between
//            exp of the edges (fastExp is within 4e-6 of exp: measured over 8e7 points); bin
//            counts times those bounds bracket every prefix of the order from both sides.
//            The walk (top-p cut, sampler.go:212-222; draw, :224-233) stops where a prefix first
//            reaches a target: all bins where that can happen, given the brackets, are the range.
//   pass 3   the exact mass and count of everything before the range (per-thread sums, one
//            block reduction) and the entries of the range into shared memory
//   finish   a bitonic sort of those entries by (value descending, index ascending), their
//            probabilities, and the reference's own sequential walk over them from the exact prefix
//
// A range too large for shared memory (a bracket that is wide in entries: the thin tail of the
// distribution, heavy ties) is histogrammed again on its own, with its exact prefix, until it
// fits.  top_k < V first finds the k-th entry the same way (counts are exact, so the range is
// one bin), min-p adds one pass for the renormaliser.  A row this cannot settle (ties by the
// thousand around the stopping place, k-th entry among values 96 or more below the maximum,
// an all-NaN row) is left marked for wide_rows_kernel, which is launched behind this kernel, takes
// only marked rows and handles everything.
//
// Sums are doubles like the reference's, the same addends in a different association (per-thread
// chains, then a tree), so a prefix can differ from the reference's in the last bits (about 1e-16
// relative): the token can differ only when the uniform lies that close to a boundary, far
// inside the 1e-6 the contract allows.  Counts are integers and exact.

constexpr int WF_NT = 512;
constexpr int WF_NWARP = WF_NT / 32;
constexpr int WF_BINS = 8192;
constexpr int WF_BPT = WF_BINS / WF_NT;  // bins per thread when the histogram is scanned
constexpr int WF_CAND = 2048;            // entries of a range held in shared memory
constexpr float WF_RCLAMP = 96.0f;       // entries this far below the maximum weigh exactly 0 (fastExp(x) = 0 for x < -87.7)
constexpr double WF_EXP_EPS = 1e-5;      // fastExp against exp, relative (measured 3.9e-6), with margin
constexpr double WF_EDGE_EPS = 4e-7;     // float roundings between an entry's d and its bin, relative
constexpr int WF_MAX_ZOOM = 4;
constexpr int WF_CTL_BYTES = 2048;

enum { WF_KTH = 0, WF_CUT = 1, WF_DRAW = 2 };

struct WFCtl {
    double red_d[2][WF_NWARP];
    unsigned long long red_c[2][WF_NWARP];
    float red_f[2][WF_NWARP];
    double scan_l[WF_NWARP], scan_h[WF_NWARP];
    unsigned long long scan_c[WF_NWARP];
    int b1, b2;
    int cand_cnt;
    int pos, flipped;
};

struct WFRow {
    const void* rowp;
    const uint4* vbase;
    int mis, a0, b0, V;
    float inv_temp, pen;
    bool has_pen;
    const uint32_t* bm;
};

// The head's post-processing is rare on this path and large: one copy per kernel.
__device__ __noinline__ float wf_post(float l, int mode, float scale, float cap) {
    const Post p = {mode, scale, cap};
    return post_logit(l, p);
}

// Every column of the row, as (raw logit, column): complete 16-byte vectors two at a time, the
// columns of the partial vectors at both ends one by one.
template <typename T, class F>
__device__ __forceinline__ void wf_for_each(const WFRow& g, int tid, F&& f) {
    constexpr int VEC = Elem<T>::VEC;
    auto vec = [&](const uint4& r, int v) {
        float x[VEC];
        Elem<T>::widen(r, x);
        const int e0 = v * VEC - g.mis;
#pragma unroll
        for (int j = 0; j < VEC; j++) f(x[j], e0 + j);
    };
    int v = g.a0 + tid;
    for (; v + WF_NT < g.b0; v += 2 * WF_NT) {
        const uint4 r0 = __ldg(g.vbase + v), r1 = __ldg(g.vbase + v + WF_NT);
        vec(r0, v);
        vec(r1, v + WF_NT);
    }
    if (v < g.b0) vec(__ldg(g.vbase + v), v);
    int head = g.V, tail0 = g.V;
    if (g.b0 > g.a0) {
        head = g.a0 * VEC - g.mis;
        tail0 = g.b0 * VEC - g.mis;
    }
    for (int t = tid; t < head + (g.V - tail0); t += WF_NT) {
        const int e = t < head ? t : tail0 + (t - head);
        f(Elem<T>::load1(g.rowp, e), e);
    }
}

// Block sums of two doubles and two counts; every thread returns with the totals.  The warps'
// partial sums are added in warp order, so the result does not depend on timing.
__device__ __forceinline__ void wf_reduce(WFCtl* w, int tid, double& d0, double& d1, unsigned long long& c0,
                                          unsigned long long& c1) {
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        d0 = __dadd_rn(d0, __shfl_xor_sync(0xffffffffu, d0, o));
        d1 = __dadd_rn(d1, __shfl_xor_sync(0xffffffffu, d1, o));
        c0 += __shfl_xor_sync(0xffffffffu, c0, o);
        c1 += __shfl_xor_sync(0xffffffffu, c1, o);
    }
    __syncthreads();  // the slots' previous readers are done
    if (lane == 0) {
        w->red_d[0][warp] = d0;
        w->red_d[1][warp] = d1;
        w->red_c[0][warp] = c0;
        w->red_c[1][warp] = c1;
    }
    __syncthreads();
    d0 = d1 = 0.0;
    c0 = c1 = 0;
#pragma unroll
    for (int i = 0; i < WF_NWARP; i++) {
        d0 = __dadd_rn(d0, w->red_d[0][i]);
        d1 = __dadd_rn(d1, w->red_d[1][i]);
        c0 += w->red_c[0][i];
        c1 += w->red_c[1][i];
    }
}

// One range of d = max - value and its histogram geometry: bin(d) = min(int((d - lo) * scale), BINS - 1)
// for lo <= d <= hi.
struct WFRange {
    float lo, hi, scale;
};

template <typename T>
__global__ void __launch_bounds__(WF_NT, 2) wide_hist_kernel(const KArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    WFCtl* w = reinterpret_cast<WFCtl*>(smem_raw);
    uint32_t* hist_top = reinterpret_cast<uint32_t*>(smem_raw + WF_CTL_BYTES);     // the whole row's histogram
    uint32_t* hist_zoom = hist_top + WF_BINS;                              // a range's own; later the range's probabilities
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(hist_zoom + WF_BINS);  // (key << 32 | ~column)
    uint32_t* bm = reinterpret_cast<uint32_t*>(cand + WF_CAND);
    static_assert(sizeof(WFCtl) <= WF_CTL_BYTES, "control block outgrew its slot");
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x;
    const int V = a.vocab;

    if (a.skip && a.skip[row] != 0) {
        if (tid == 0) publish_row(a, row, -1);
        return;
    }
    const MantleSampleParams P = row_params(a, row);
    bool greedy, bad_k;
    const int k = row_k(a, P, 0x7fffffff, &greedy, &bad_k);  // no cap on this path
    if (bad_k) {
        if (tid == 0) {
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_TOPK_RANGE);
            publish_row(a, row, -1);
        }
        return;
    }
    auto give_up = [&]() {  // leave the row to wide_rows_kernel
        if (tid == 0) a.next[row] = WIDE_UNRESOLVED;
    };

    WFRow g;
    g.rowp = reinterpret_cast<const T*>(a.logits) + (size_t)row * (size_t)a.row_stride;
    g.mis = (int)((reinterpret_cast<uintptr_t>(g.rowp) & 15u) / sizeof(T));
    g.vbase = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(g.rowp) - (size_t)g.mis * sizeof(T));
    g.a0 = g.mis != 0 ? 1 : 0;
    g.b0 = (g.mis + V) / Elem<T>::VEC;
    g.V = V;
    g.inv_temp = greedy ? 1.0f : __fdiv_rn(1.0f, P.temperature);
    g.pen = P.repeat_penalty;
    g.bm = bm;
    const int hl = history_len(a, row);
    const WinPlan wp = win_plan(P, hl);
    g.has_pen = wp.active;
    if (wp.active) build_penalty_bitmap(a, row, wp, hl, V, a.vocab_offset, bm, tid, WF_NT);
    const Post& post = a.post;
    // scaled, penalised value of a column (sampler.go:132-136, 267)
    auto value = [&](float raw, int e) {
        float l = raw;
        if (post.mode) l = wf_post(l, post.mode, post.scale, post.cap);
        if (g.has_pen && bm_test(bm, e)) l = penalise(l, g.pen);
        return __fmul_rn(l, g.inv_temp);
    };

    // ---- pass 1: the largest and smallest value ------------------------------------------------
    float vmax = __uint_as_float(0xff800000u), vmin = __uint_as_float(0x7f800000u);
    wf_for_each<T>(g, tid, [&](float raw, int e) {
        const float v = value(raw, e);
        vmax = fmaxf(vmax, v);  // fmaxf / fminf return the other operand on NaN: NaN takes no part
        vmin = fminf(vmin, v);
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
    }
    if (lane == 0) {
        w->red_f[0][warp] = vmax;
        w->red_f[1][warp] = vmin;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < WF_NWARP; i++) {
        vmax = fmaxf(vmax, w->red_f[0][i]);
        vmin = fminf(vmin, w->red_f[1][i]);
    }
    __syncthreads();
    if (!(vmax > __uint_as_float(0xff800000u)) || !(vmax < __uint_as_float(0x7f800000u))) {
        give_up();  // nothing but NaN, or an infinite maximum: not this kernel's business
        return;
    }
    const float maxv = __fadd_rn(vmax, 0.0f);  // -0.0 and +0.0 are one value (sampler.go compares floats)
    const uint32_t max_key = f2key(maxv);

    if (greedy) {  // argmax rows routed here by a long-shortlist batch: lowest column of the maximum
        unsigned long long best = 0xffffffffffffffffull;
        wf_for_each<T>(g, tid, [&](float raw, int e) {
            const float v = value(raw, e);
            if (v == v && f2key(v) == max_key) best = min(best, (unsigned long long)e);
        });
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (lane == 0) w->red_c[0][warp] = best;
        __syncthreads();
        if (tid == 0) {
            for (int i = 1; i < WF_NWARP; i++) best = min(best, w->red_c[0][i]);
            publish_row(a, row, (int)best + a.vocab_offset);
        }
        return;
    }

    // ---- the row's range of d and its bins -----------------------------------------------------
    WFRange top;
    top.lo = 0.0f;
    top.hi = fminf(__fsub_rn(maxv, vmin), WF_RCLAMP);  // entries further down weigh exactly 0: counted apart ("far")
    if (!(top.hi > 1e-30f)) top.hi = 1e-30f;
    top.scale = (float)WF_BINS / top.hi * (1.0f - 1e-6f);

    // Shortlist membership (the k best when k < V; set by the KTH resolve) and the probability stages
    // (sampler.go:165-210): e -> e * inv_sum -> (min-p) -> * rescale.
    uint32_t member_key = 0;
    int member_col = 0x7fffffff;
    bool all_members = true;
    double inv_sum = 1.0, minp_thr = -1.0, rescale = 1.0;
    bool rescaled = false;
    auto member = [&](uint32_t key, int e) {
        return all_members || key > member_key || (key == member_key && e <= member_col);
    };
    // final probability of an entry from its fastExp; false: min-p dropped it (sampler.go:188)
    auto final_prob = [&](float ex, double* p) {
        double q = __dmul_rn((double)ex, inv_sum);
        if (q < minp_thr) return false;
        if (rescaled) q = __dmul_rn(q, rescale);
        *p = q;
        return true;
    };
    auto zero_hist = [&](uint32_t* h) {
        uint4* h4 = reinterpret_cast<uint4*>(h);
        for (int i = tid; i < WF_BINS / 4; i += WF_NT) h4[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
    };
    auto bin_of = [&](const WFRange& r, float d) {
        return min(__float2int_rz(__fmul_rn(__fsub_rn(d, r.lo), r.scale)), WF_BINS - 1);
    };

    // ---- statistics pass: histogram of the members over the row's range, their mass and count --
    //   stage 0  counts only (before the k-th entry is known)
    //   stage 1  mass = sum of fastExp                       (sampler.go:161-168)
    //   stage 2  mass = sum of the probabilities min-p keeps (sampler.go:186-196); only they are counted
    unsigned long long near_cnt = 0, far_cnt = 0;
    auto stat_pass = [&](int stage) {
        zero_hist(hist_top);
        double mass = 0.0, unused = 0.0;
        unsigned long long nc = 0, fc = 0;
        wf_for_each<T>(g, tid, [&](float raw, int e) {
            const float v = value(raw, e);
            if (!(v == v)) return;
            if (!all_members && !member(f2key(v), e)) return;
            const float x = __fsub_rn(v, maxv);  // the reference's argument of fastExp (sampler.go:167)
            if (stage >= 1) {
                const float ex = fast_exp(x);
                if (stage == 1) {
                    mass = __dadd_rn(mass, (double)ex);
                } else {
                    const double q = __dmul_rn((double)ex, inv_sum);
                    if (q < minp_thr) return;
                    mass = __dadd_rn(mass, q);
                }
            }
            const float d = -x;
            if (d <= top.hi) {
                atomicAdd(&hist_top[bin_of(top, d)], 1u);
                nc++;
            } else {
                fc++;
            }
        });
        wf_reduce(w, tid, mass, unused, nc, fc);
        near_cnt = nc;
        far_cnt = fc;
        return mass;
    };

    // ---- resolve: where in the order does the walk stop? ---------------------------------------
    // KTH:  the entry at position `want` (1-based) of the order           -> *out_key, *out_col
    // CUT:  first position whose prefix, rounded to float, reaches top_p   -> *out_pos (1-based)
    // DRAW: first position with r <= prefix, or the CUT position           -> *out_col, *out_prob
    // Returns 1 settled, 0 the walk never stops inside the members (CUT / DRAW: it ends on the last
    // member), -1 cannot be settled here.
    const double r = P.uniform;
    const bool nucleus = P.top_p < 1.0f;
    auto stops = [&](int mode, double c) {
        bool ok = nucleus && __double2float_rn(c) >= P.top_p;
        if (mode == WF_DRAW) ok = ok || r <= c;
        return ok;
    };
    auto resolve = [&](int mode, unsigned long long want, uint32_t* out_key, int* out_col, double* out_prob,
                       unsigned long long* out_pos) -> int {
        // target of the walk in probability units, with the slack the float compare of top_p needs
        double target = 0.0;
        if (mode != WF_KTH) {
            const double tp = nucleus ? (double)P.top_p * (1.0 - 1e-7) : 1e300;
            target = mode == WF_CUT ? tp : fmin(tp, r);
        }
        const double gain = rescaled ? inv_sum * rescale : inv_sum;  // probability per unit of fastExp
        WFRange cur = top;
        const uint32_t* hist = hist_top;
        double p0 = 0.0;               // exact probability mass before the range
        unsigned long long c0 = 0;     // exact count before the range
        for (int zoom = 0;; zoom++) {
            // -- locate on `hist`: per-thread partial sums of its bins, block scan, crossings --
            // Bounds of one entry's fastExp in bin b: its d lies between the bin's edges, widened by the
            // float roundings between d and the bin index; the last bin reaches to the end of the range.
            const double width = 1.0 / (double)cur.scale;
            const int bfirst = tid * WF_BPT;
            const double step_hi = exp(-width * (1.0 - WF_EDGE_EPS)), step_lo = exp(-width * (1.0 + WF_EDGE_EPS));
            const double e_hi0 = exp(-((double)cur.lo + (double)bfirst * width * (1.0 - WF_EDGE_EPS)));
            const double d_end0 = (double)cur.lo + (double)(bfirst + 1) * width * (1.0 + WF_EDGE_EPS);
            const double e_lo0 = exp(-d_end0);
            const double e_lo_last = exp(-(double)cur.hi * (1.0 + WF_EDGE_EPS));
            auto bounds = [&](int j, double e_hi, double e_lo, double d_end, double* lo_b, double* hi_b) {
                const bool last = bfirst + j == WF_BINS - 1;
                const double dl = last ? (double)cur.hi * (1.0 + WF_EDGE_EPS) : d_end;
                *hi_b = e_hi * (1.0 + WF_EXP_EPS) * gain;
                *lo_b = dl > 87.0 ? 0.0 : (last ? e_lo_last : e_lo) * (1.0 - WF_EXP_EPS) * gain;  // fastExp is 0 from 87.7 on
                if (mode == WF_KTH) *hi_b = *lo_b = 0.0;
            };
            unsigned long long tc = 0;
            double tl = 0.0, th = 0.0;
            {
                double e_hi = e_hi0, e_lo = e_lo0, d_end = d_end0;
#pragma unroll 4
                for (int j = 0; j < WF_BPT; j++) {
                    double lo_b, hi_b;
                    bounds(j, e_hi, e_lo, d_end, &lo_b, &hi_b);
                    const double c = (double)hist[bfirst + j];
                    tc += hist[bfirst + j];
                    tl = __dadd_rn(tl, __dmul_rn(c, lo_b));
                    th = __dadd_rn(th, __dmul_rn(c, hi_b));
                    e_hi *= step_hi;
                    e_lo *= step_lo;
                    d_end += width * (1.0 + WF_EDGE_EPS);
                }
            }
            // exclusive scan over threads
            unsigned long long sc = tc;
            double sl = tl, sh = th;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long yc = __shfl_up_sync(0xffffffffu, sc, o);
                const double yl = __shfl_up_sync(0xffffffffu, sl, o), yh = __shfl_up_sync(0xffffffffu, sh, o);
                if (lane >= o) {
                    sc += yc;
                    sl = __dadd_rn(sl, yl);
                    sh = __dadd_rn(sh, yh);
                }
            }
            __syncthreads();
            if (lane == 31) {
                w->scan_c[warp] = sc;
                w->scan_l[warp] = sl;
                w->scan_h[warp] = sh;
            }
            if (tid == 0) {
                w->b1 = WF_BINS;
                w->b2 = WF_BINS;
            }
            __syncthreads();
            unsigned long long bc = 0;
            double bl = 0.0, bh = 0.0;
            for (int i = 0; i < warp; i++) {
                bc += w->scan_c[i];
                bl = __dadd_rn(bl, w->scan_l[i]);
                bh = __dadd_rn(bh, w->scan_h[i]);
            }
            // Running inclusive prefixes through my bins (the same arithmetic as above, so the same
            // numbers).  b1: the first non-empty bin the walk can stop in (upper bracket reaches the
            // target); b2: the first bin by whose end it has stopped (lower bracket reaches it).
            {
                unsigned long long pc = c0 + bc + sc - tc;
                double pl = p0 + bl + sl - tl, ph = p0 + bh + sh - th;
                const double t_lo = target * (1.0 - 1e-9) - 1e-300, t_hi = target * (1.0 + 1e-9) + 1e-300;
                int my_b1 = WF_BINS, my_b2 = WF_BINS;
                double e_hi = e_hi0, e_lo = e_lo0, d_end = d_end0;
#pragma unroll 4
                for (int j = 0; j < WF_BPT; j++) {
                    double lo_b, hi_b;
                    bounds(j, e_hi, e_lo, d_end, &lo_b, &hi_b);
                    const uint32_t cj = hist[bfirst + j];
                    const unsigned long long pc0 = pc;
                    pc += cj;
                    pl = __dadd_rn(pl, __dmul_rn((double)cj, lo_b));
                    ph = __dadd_rn(ph, __dmul_rn((double)cj, hi_b));
                    e_hi *= step_hi;
                    e_lo *= step_lo;
                    d_end += width * (1.0 + WF_EDGE_EPS);
                    if (cj == 0) continue;
                    bool in1, in2;
                    if (mode == WF_KTH) {
                        in1 = in2 = pc0 < want && want <= pc;
                    } else {
                        in1 = ph >= t_lo;
                        in2 = pl >= t_hi;
                    }
                    if (in1 && my_b1 == WF_BINS) my_b1 = bfirst + j;
                    if (in2 && my_b2 == WF_BINS) my_b2 = bfirst + j;
                }
                if (my_b1 < WF_BINS) atomicMin(&w->b1, my_b1);
                if (my_b2 < WF_BINS) atomicMin(&w->b2, my_b2);
            }
            __syncthreads();
            int b1 = w->b1, b2 = w->b2;
            const bool open_end = b2 >= WF_BINS;  // the walk may run off the end of this range
            if (b1 >= WF_BINS) {
                // even the upper bracket never reaches the target inside this range
                if (mode == WF_KTH || zoom > 0) return -1;  // (a zoomed range was chosen to contain the stop)
                return 0;                                    // the walk ends on the last member
            }
            if (open_end) b2 = WF_BINS - 1;
            if (b2 < b1) b2 = b1;
            // the new range: bins b1..b2 of the current one, a hair wider than their edges
            WFRange nr;
            {
                const double lo_d = (double)cur.lo + (double)b1 * width * (1.0 - WF_EDGE_EPS);
                const double hi_d = b2 == WF_BINS - 1 ? (double)cur.hi
                                                      : (double)cur.lo + (double)(b2 + 1) * width * (1.0 + WF_EDGE_EPS);
                nr.lo = b1 == 0 ? cur.lo : fmaxf(cur.lo, __double2float_rd(lo_d));
                nr.hi = fminf(cur.hi, __double2float_ru(hi_d));
                const float span = __fsub_rn(nr.hi, nr.lo);
                nr.scale = span > 0.0f ? (float)WF_BINS / span * (1.0f - 1e-6f) : 0.0f;
            }
            // how many entries the new range holds, from the counts (its neighbours' share of the
            // hair is at most their own counts)
            unsigned long long in_range = 0;
            for (int b = max(b1 - 1, 0) + tid; b <= min(b2 + 1, WF_BINS - 1); b += WF_NT) in_range += hist[b];
            {
                double z0 = 0.0, z1 = 0.0;
                unsigned long long z = 0;
                wf_reduce(w, tid, z0, z1, in_range, z);
            }
            const bool fits = in_range <= (unsigned long long)WF_CAND;
            if (!fits && (zoom >= WF_MAX_ZOOM || !(nr.scale > 0.0f) || !(nr.scale < 3e38f))) return -1;

            // -- one pass: the exact mass and count between the old and the new lower edge, and either
            //    the range's entries (it fits) or its own histogram (it does not) --
            if (!fits) zero_hist(hist_zoom);
            if (tid == 0) w->cand_cnt = 0;
            __syncthreads();
            double add_p = 0.0, unused = 0.0;
            unsigned long long add_c = 0, unused_c = 0;
            const float old_lo = cur.lo;
            const bool first_range = zoom == 0;
            wf_for_each<T>(g, tid, [&](float raw, int e) {
                const float v = value(raw, e);
                if (!(v == v)) return;
                const float x = __fsub_rn(v, maxv);
                const float d = -x;
                if (d > nr.hi || (!first_range && d < old_lo)) return;  // behind the range, or summed earlier
                const uint32_t key = f2key(v);
                if (!all_members && !member(key, e)) return;
                double p = 0.0;
                if (mode != WF_KTH && !final_prob(fast_exp(x), &p)) return;
                if (d < nr.lo) {
                    add_p = __dadd_rn(add_p, p);
                    add_c++;
                } else if (fits) {
                    const int slot = atomicAdd(&w->cand_cnt, 1);
                    if (slot < WF_CAND) cand[slot] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)e);
                } else {
                    atomicAdd(&hist_zoom[bin_of(nr, d)], 1u);
                }
            });
            wf_reduce(w, tid, add_p, unused, add_c, unused_c);
            p0 = __dadd_rn(p0, add_p);
            c0 += add_c;
            cur = nr;
            if (!fits) {
                hist = hist_zoom;
                continue;
            }

            // -- the range's entries are in shared memory: order them and walk --
            __syncthreads();
            const int n = w->cand_cnt;
            if (n > WF_CAND) return -1;  // more entries in the hair than counted: not settled here
            int n2 = 64;
            while (n2 < n) n2 <<= 1;
            for (int i = n + tid; i < n2; i += WF_NT) cand[i] = 0ull;  // below every real entry
            __syncthreads();
            // bitonic sort, descending: (key descending, column ascending)
            for (int kk = 2; kk <= n2; kk <<= 1) {
                for (int jj = kk >> 1; jj > 0; jj >>= 1) {
                    for (int i = tid; i < n2; i += WF_NT) {
                        const int ixj = i ^ jj;
                        if (ixj > i) {
                            const unsigned long long x0 = cand[i], x1 = cand[ixj];
                            const bool desc = (i & kk) == 0;
                            if (desc ? x0 < x1 : x0 > x1) {
                                cand[i] = x1;
                                cand[ixj] = x0;
                            }
                        }
                    }
                    __syncthreads();
                }
            }
            if (mode == WF_KTH) {
                if (want <= c0 || want - c0 > (unsigned long long)n) return -1;
                const unsigned long long hit = cand[want - c0 - 1];
                *out_key = (uint32_t)(hit >> 32);
                *out_col = (int)(~(uint32_t)hit);
                __syncthreads();
                return 1;
            }
            double* prob = reinterpret_cast<double*>(hist_zoom);  // WF_CAND doubles fit the unused histogram
            for (int i = tid; i < n; i += WF_NT) {
                double p = 0.0;
                final_prob(fast_exp(__fsub_rn(key2f((uint32_t)(cand[i] >> 32)), maxv)), &p);
                prob[i] = p;
            }
            __syncthreads();
            if (tid == 0) {
                // the reference's own walk (sampler.go:214-231), entered with the exact prefix
                int pos = -1;
                bool early = stops(mode, p0) && c0 > 0;  // the walk stopped before the range: the brackets failed
                double c = p0;
                if (!early)
                    for (int i = 0; i < n; i++) {
                        c = __dadd_rn(c, prob[i]);
                        if (stops(mode, c)) {
                            pos = i;
                            break;
                        }
                    }
                w->pos = pos;
                w->flipped = early ? -1 : (pos >= 0 ? 1 : 0);
            }
            __syncthreads();
            const int flipped = w->flipped, pos = w->pos;
            int rc;
            if (flipped < 0) {
                rc = -1;
            } else if (flipped == 0) {
                rc = open_end && cur.hi >= top.hi ? 0 : -1;  // ran off the end of the members, or of a bad bracket
            } else {
                if (out_col) *out_col = (int)(~(uint32_t)cand[pos]);
                if (out_prob) *out_prob = prob[pos];
                if (out_pos) *out_pos = c0 + (unsigned long long)pos + 1;
                rc = 1;
            }
            __syncthreads();
            return rc;
        }
    };

    // ---- the k best (sampler.go:255-296), when that is not everything ----------------------------
    if (k < V) {
        stat_pass(0);
        if ((unsigned long long)k < near_cnt + far_cnt) {
            if ((unsigned long long)k > near_cnt) {  // the k-th entry weighs 0: among the "far" ones
                give_up();
                return;
            }
            uint32_t kk = 0;
            int kc = 0;
            if (resolve(WF_KTH, (unsigned long long)k, &kk, &kc, nullptr, nullptr) != 1) {
                give_up();
                return;
            }
            member_key = kk;
            member_col = kc;
            all_members = false;
        }
    }

    // ---- softmax over the shortlist (sampler.go:154-177) -----------------------------------------
    const double sum = stat_pass(1);
    unsigned long long n_kept = near_cnt + far_cnt;
    if (sum == 0.0) {  // sampler.go:170-172: cannot happen (the maximum contributes fastExp(0) = 1); kept for form
        give_up();
        return;
    }
    inv_sum = __ddiv_rn(1.0, sum);

    // ---- min-p (sampler.go:180-210) ----------------------------------------------------------------
    if (P.min_p > 0.0f) {
        // prob[0] = fastExp(0) * inv_sum
        minp_thr = __dmul_rn(__dmul_rn((double)fast_exp(0.0f), inv_sum), (double)P.min_p);
        const double new_sum = stat_pass(2);
        const unsigned long long kept = near_cnt + far_cnt;
        if (kept < n_kept && new_sum > 0.0) {
            rescale = __ddiv_rn(1.0, new_sum);
            rescaled = true;
        }
        n_kept = kept;
        if (kept == 0) {  // min_p > 1 dropped everything: the reference indexes topIdx[-1] and panics
            if (tid == 0) {
                publish_row(a, row, -1);
                if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_EMPTY);
            }
            return;
        }
    }

    // The last member of the order (smallest value, largest column): where a walk that never stops ends.
    auto last_member = [&](int* col, double* prob) {
        unsigned long long best = 0xffffffffffffffffull;
        wf_for_each<T>(g, tid, [&](float raw, int e) {
            const float v = value(raw, e);
            if (!(v == v)) return;
            const uint32_t key = f2key(v);
            if (!all_members && !member(key, e)) return;
            double p;
            if (!final_prob(fast_exp(__fsub_rn(v, maxv)), &p)) return;
            best = min(best, ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)e));
        });
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
        __syncthreads();
        if (lane == 0) w->red_c[0][warp] = best;
        __syncthreads();
        for (int i = 0; i < WF_NWARP; i++) best = min(best, w->red_c[0][i]);
        __syncthreads();
        *col = (int)(~(uint32_t)best);
        double p = 0.0;
        final_prob(fast_exp(__fsub_rn(key2f((uint32_t)(best >> 32)), maxv)), &p);
        *prob = p;
    };

    // ---- the draw (sampler.go:224-233), which the top-p cut may end early (:212-222) ---------------
    int col = -1;
    double tprob = 0.0;
    int rc = resolve(WF_DRAW, 0, nullptr, &col, &tprob, nullptr);
    if (rc < 0) {
        give_up();
        return;
    }
    if (rc == 0) last_member(&col, &tprob);
    int cut = (int)n_kept;
    if (a.cut && nucleus) {
        unsigned long long pos = 0;
        const int rc2 = resolve(WF_CUT, 0, nullptr, nullptr, nullptr, &pos);
        if (rc2 < 0) {
            give_up();
            return;
        }
        if (rc2 == 1) cut = (int)pos;
    }
    if (tid == 0) publish_row(a, row, col + a.vocab_offset, (int)n_kept, cut, tprob, sum);
}

}  // namespace
