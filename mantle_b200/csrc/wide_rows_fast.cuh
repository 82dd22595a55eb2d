// wide_hist_kernel: shortlists longer than 1024 entries, up to the whole vocabulary, in three to
// six passes over the row.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// ---------------------------------------------------------------------------------------
// Long shortlists without ordering them.
//
// The reference's Sample with tens of thousands of shortlist entries (TopK >= V is its only way
// to a whole-vocabulary nucleus, sampler.go:147) needs the order only to walk prefix sums.  One
// CTA per row finds the bin of a histogram in which the walk stops, orders only that bin's
// entries, and walks only them:
//
//   pass 1   the row's largest and smallest scaled value (the softmax shifts by the largest,
//            sampler.go:154-160)
//   pass 2   a histogram of d = max - value over 2048 linear bins: per bin the number of entries
//            and the EXACT sum of their fastExp(value - max) (sampler.go:161-168).  All entries of
//            a bin weigh within a factor of two of each other, so scaled by a power of two that
//            depends on the bin alone they are integers below 2^25; integer sums are exact and
//            do not depend on the order of the atomic adds.  One 64-bit word per bin carries
//            both: count << 43 | sum.
//   locate   a scan over the bins gives the softmax normaliser and every prefix of the order at
//            bin granularity; the walk (top-p cut, sampler.go:212-222; draw, :224-233) stops
//            in the first bin whose inclusive prefix reaches the target.
//   pass 3   that bin's entries into shared memory
//   finish   a bitonic sort of those entries by (value descending, index ascending), their
//            probabilities, and the reference's own sequential walk over them from the prefix
//            before the bin
//
// A bin with more entries than shared memory holds is histogrammed once more on its own.
// top_k < V first finds the k-th entry the same way (by count) and repeats pass 2 for the
// members only; min-p repeats it for what it keeps.  A row this cannot settle (ties by the
// thousand where the walk stops, a k-th entry among values 96 or more below the maximum, an
// all-NaN row, an infinite maximum) is left marked for wide_rows_kernel, which is launched behind
// this kernel, takes only marked rows and handles everything.
//
// Sums are doubles like the reference's, over the same addends in a different association
// (exact per bin, bins added in order), and a prefix is a sum times 1/sum where the reference
// adds products: a prefix can differ from the reference's in the last bits (about 1e-16
// relative), so the token can differ only when the uniform lies that close to a boundary, far
// inside the 1e-6 the contract allows.  Counts are integers and exact.

constexpr int WF_NT = 512;
constexpr int WF_NWARP = WF_NT / 32;
constexpr int WF_BINS = 2048;
constexpr int WF_BPT = WF_BINS / WF_NT;  // bins per thread when a histogram is scanned
constexpr int WF_CAND = 2048;            // entries of a bin held in shared memory
constexpr float WF_RCLAMP = 96.0f;       // entries this far below the maximum weigh exactly 0 (fastExp(x) = 0 for x < -87.7)
constexpr double WF_EXP_EPS = 1e-5;      // fastExp against exp, relative (measured 3.9e-6 over 8e7 points), with margin
constexpr double WF_EDGE_EPS = 4e-7;     // float roundings between an entry's d and its bin, relative
constexpr int WF_CTL_BYTES = 1024;
constexpr int WF_COUNT_SHIFT = 43;       // histogram word: count << 43 | sum of scaled weights
constexpr unsigned long long WF_MASS_MASK = (1ull << WF_COUNT_SHIFT) - 1;

enum { WF_KTH = 0, WF_CUT = 1, WF_DRAW = 2 };

struct WFCtl {
    double scan_m[WF_NWARP];
    unsigned long long scan_c[WF_NWARP];
    unsigned long long red_c[WF_NWARP];
    float red_f[2][WF_NWARP];
    int b1, b2;
    int cand_cnt;
    int pos, flipped;
};
static_assert(sizeof(WFCtl) <= WF_CTL_BYTES, "control block outgrew its slot");

// One histogram: words[b] = count << 43 | sum over the bin's entries of fastExp * scl[b], scl[b] a
// power of two; its geometry: bin(d) = min(int((d - lo) * scale), BINS - 1) for lo <= d <= hi.
struct WFHist {
    unsigned long long* words;
    float* scl;
    float lo, hi, scale;
};

struct WFRow {
    const void* rowp;
    const uint4* vbase;
    int mis, nvec, a0, b0, V;
    float inv_temp, pen;
    bool has_pen;
    const uint32_t* bm;
};

// A bin's sum in units of fastExp: the integer sum times 2^-(24 - E), the inverse of the bin's scale.
__device__ __forceinline__ double wf_mass(unsigned long long word, float scl) {
    const int e = (int)(__float_as_uint(scl) >> 23) - 127;  // scl = 2^e
    return __dmul_rn((double)(word & WF_MASS_MASK), __longlong_as_double((long long)(1023 - e) << 52));
}

// The head's post-processing is rare on this path and large: one copy per kernel.
__device__ __noinline__ float wf_post(float l, int mode, float scale, float cap) {
    const Post p = {mode, scale, cap};
    return post_logit(l, p);
}

template <typename T>
__device__ __forceinline__ uint32_t wf_nan_bits();
template <>
__device__ __forceinline__ uint32_t wf_nan_bits<float>() { return 0x7fc00000u; }
template <>
__device__ __forceinline__ uint32_t wf_nan_bits<bf16_t>() { return 0x7fc07fc0u; }

// The 16-byte vector `v` of the row.  A complete vector is one load; the partial vectors at the
// two ends of a row that does not start or end on a 16-byte boundary are put together from
// single loads, with NaN (which every pass skips) in the places outside the row.
template <typename T>
__device__ __forceinline__ uint4 wf_load(const WFRow& g, int v) {
    if (v >= g.a0 && v < g.b0) return __ldg(g.vbase + v);
    constexpr int VEC = Elem<T>::VEC;
    uint32_t wds[4] = {wf_nan_bits<T>(), wf_nan_bits<T>(), wf_nan_bits<T>(), wf_nan_bits<T>()};
    const int e0 = v * VEC - g.mis;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        const int e = e0 + j;
        if (e < 0 || e >= g.V) continue;
        if (sizeof(T) == 4) {
            wds[j & 3] = __float_as_uint(Elem<T>::load1(g.rowp, e));
        } else {
            const uint32_t h = __float_as_uint(Elem<T>::load1(g.rowp, e)) >> 16;
            const int sh = (j & 1) * 16;
            wds[(j >> 1) & 3] = (wds[(j >> 1) & 3] & ~(0xffffu << sh)) | (h << sh);
        }
    }
    return make_uint4(wds[0], wds[1], wds[2], wds[3]);
}

// Every column of the row as f(raw logit, column), one copy of f's code per call: the next vector's
// load is in flight while the current one is worked on.  Places outside the row arrive as NaN with
// a column outside [0, V).
template <typename T, class F>
__device__ __forceinline__ void wf_for_each(const WFRow& g, int tid, F&& f) {
    constexpr int VEC = Elem<T>::VEC;
    int v = tid;
    uint4 cur = make_uint4(0, 0, 0, 0);
    if (v < g.nvec) cur = wf_load<T>(g, v);
#pragma unroll 1
    while (v < g.nvec) {
        const int vn = v + WF_NT;
        uint4 nxt = make_uint4(0, 0, 0, 0);
        if (vn < g.nvec) nxt = wf_load<T>(g, vn);
        float x[VEC];
        Elem<T>::widen(cur, x);
        const int e0 = v * VEC - g.mis;
#pragma unroll
        for (int j = 0; j < VEC; j++) f(x[j], e0 + j);
        cur = nxt;
        v = vn;
    }
}

template <typename T>
__global__ void __launch_bounds__(WF_NT, 2) wide_hist_kernel(const KArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    WFCtl* w = reinterpret_cast<WFCtl*>(smem_raw);
    // [ctl][row histogram words][bin histogram words][row scl][bin scl][counts of the histogram being built][entries][bitmap]
    unsigned long long* words0 = reinterpret_cast<unsigned long long*>(smem_raw + WF_CTL_BYTES);
    unsigned long long* words1 = words0 + WF_BINS;
    float* scl0 = reinterpret_cast<float*>(words1 + WF_BINS);
    float* scl1 = scl0 + WF_BINS;
    uint32_t* cnt32 = reinterpret_cast<uint32_t*>(scl1 + WF_BINS);
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(cnt32 + WF_BINS);  // (key << 32 | ~column)
    uint32_t* bm = reinterpret_cast<uint32_t*>(cand + WF_CAND);
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

    WFRow g;
    g.rowp = reinterpret_cast<const T*>(a.logits) + (size_t)row * (size_t)a.row_stride;
    g.mis = (int)((reinterpret_cast<uintptr_t>(g.rowp) & 15u) / sizeof(T));
    g.vbase = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(g.rowp) - (size_t)g.mis * sizeof(T));
    g.nvec = (g.mis + V + Elem<T>::VEC - 1) / Elem<T>::VEC;
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
    // scaled, penalised value of a column (sampler.go:132-136, 267); NaN stays NaN
    auto value = [&](float raw, int e) {
        float l = raw;
        if (post.mode) l = wf_post(l, post.mode, post.scale, post.cap);
        if (g.has_pen && (unsigned)e < (unsigned)V && bm_test(bm, e)) l = penalise(l, g.pen);
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
        if (tid == 0) a.next[row] = WIDE_UNRESOLVED;  // nothing but NaN, or an infinite maximum
        return;
    }
    const float maxv = __fadd_rn(vmax, 0.0f);  // -0.0 and +0.0 are one value (sampler.go compares floats)

    if (greedy) {  // argmax rows routed here by a long-shortlist batch: lowest column of the maximum
        const uint32_t max_key = f2key(maxv);
        unsigned long long best = 0xffffffffffffffffull;
        wf_for_each<T>(g, tid, [&](float raw, int e) {
            const float v = value(raw, e);
            if (v == v && f2key(v) == max_key) best = min(best, (unsigned long long)e);
        });
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (lane == 0) w->red_c[warp] = best;
        __syncthreads();
        if (tid == 0) {
            for (int i = 1; i < WF_NWARP; i++) best = min(best, w->red_c[i]);
            publish_row(a, row, (int)best + a.vocab_offset);
        }
        return;
    }

    // ---- histograms ----------------------------------------------------------------------------
    WFHist top;
    top.words = words0;
    top.scl = scl0;
    top.lo = 0.0f;
    top.hi = fminf(__fsub_rn(maxv, vmin), WF_RCLAMP);  // entries further down weigh exactly 0: counted apart ("far")
    if (!(top.hi > 1e-30f)) top.hi = 1e-30f;
    top.scale = (float)WF_BINS / top.hi * (1.0f - 1e-6f);
    WFHist sub;
    sub.words = words1;
    sub.scl = scl1;
    sub.lo = sub.hi = sub.scale = 0.0f;

    auto bin_of = [&](const WFHist& h, float d) {
        return min(max(__float2int_rz(__fmul_rn(__fsub_rn(d, h.lo), h.scale)), 0), WF_BINS - 1);
    };
    // Clears a histogram and sets its bins' scales: every entry of bin b has d between the bin's
    // edges (widened by the float roundings between d and the bin index), so its fastExp is at
    // most exp(-lower edge) * (1 + eps) < 2^(E+1); times 2^(24 - E) it is below 2^25, and an
    // integer as long as it is at least 2^(E-1), which holds within a bin narrower than ln 2.
    // (Far below 1e-30 the scale stops growing and such weights lose low bits: 1e-37 of the sum.)
    auto prepare = [&](const WFHist& h) {
        const double width = 1.0 / (double)h.scale;
        for (int b = tid; b < WF_BINS; b += WF_NT) {
            const double top_e = exp(-((double)h.lo + (double)b * width * (1.0 - WF_EDGE_EPS))) * (1.0 + WF_EXP_EPS);
            int E = 0;
            (void)frexp(top_e, &E);  // top_e = m * 2^E, m in [0.5, 1): top_e < 2^E
            E = max(E - 1, -100);
            h.scl[b] = __uint_as_float((uint32_t)(24 - E + 127) << 23);  // 2^(24 - E)
            h.words[b] = 0ull;
            cnt32[b] = 0u;
        }
        __syncthreads();
    };
    // While a histogram is built its word holds two 32-bit sums -- the low twelve bits of the scaled
    // weights and the rest -- and the counts sit apart: three 32-bit atomics per entry, which the
    // shared-memory unit serves several times faster than one 64-bit one.  `pack` (every thread, ends with
    // a barrier) then puts count << 43 | sum into the word.  A bin of more than 2^18 entries could
    // overflow a partial sum: its count is packed as 0, which the totals' check turns into "not settled".
    auto hist_add = [&](const WFHist& h, int b, float ex) {
        const uint32_t x = __float2uint_rz(__fmul_rn(ex, h.scl[b]));
        uint32_t* halves = reinterpret_cast<uint32_t*>(&h.words[b]);
        if (x) {  // a pass that only counts, or a weight of exactly 0
            atomicAdd(&halves[0], x & 0xfffu);
            atomicAdd(&halves[1], x >> 12);
        }
        atomicAdd(&cnt32[b], 1u);
    };
    auto pack = [&](const WFHist& h) {
        __syncthreads();
        for (int b = tid; b < WF_BINS; b += WF_NT) {
            const uint32_t* halves = reinterpret_cast<const uint32_t*>(&h.words[b]);
            const unsigned long long sum = ((unsigned long long)halves[1] << 12) + halves[0];
            const uint32_t c = cnt32[b] <= (1u << 18) ? cnt32[b] : 0u;
            h.words[b] = ((unsigned long long)c << WF_COUNT_SHIFT) | sum;
            cnt32[b] = 0u;
        }
        __syncthreads();
    };

    // Shortlist membership (the k best when k < V; set by the KTH query) and the probability stages
    // (sampler.go:165-210): e -> e * inv_sum -> (min-p) -> * rescale.
    uint32_t member_key = 0;
    int member_col = 0x7fffffff;
    bool all_members = true;
    double inv_sum = 1.0, minp_thr = -1.0, rescale = 1.0;
    bool rescaled = false;
    // final probability of an entry from its fastExp; false: min-p dropped it (sampler.go:188)
    auto final_prob = [&](float ex, double* p) {
        double q = __dmul_rn((double)ex, inv_sum);
        if (q < minp_thr) return false;
        if (rescaled) q = __dmul_rn(q, rescale);
        *p = q;
        return true;
    };

    // ---- the program of a row --------------------------------------------------------------------
    //   op 0  histogram of counts            (only when k < V)
    //   op 1  query KTH -> membership        (only when k < V)
    //   op 2  histogram of the members: counts and sums of fastExp -> the softmax normaliser
    //   op 3  histogram of what min-p keeps  (only with min-p)     -> the renormaliser
    //   op 4  query DRAW -> the token
    //   op 5  query CUT  -> the nucleus length (only when the caller asks for it)
    // One loop runs them, so that the code of a pass and of a query exists once.
    const double r = P.uniform;
    const bool nucleus = P.top_p < 1.0f;
    unsigned long long near_cnt = 0, far_cnt = 0;
    double sum = 0.0;
    unsigned long long n_kept = 0;
    int token_col = -1, cut = 0;
    double token_prob = 0.0;
    bool unresolved = false, done = false;

#pragma unroll 1
    for (int op = 0; op < 6 && !unresolved && !done; op++) {
        if ((op == 0 || op == 1) && !(k < V)) continue;
        if (op == 3 && !(P.min_p > 0.0f)) continue;
        if (op == 5 && !(a.cut && nucleus)) continue;

        if (op == 0 || op == 2 || op == 3) {
            // -- a histogram pass over the whole row --
            const int stage = op == 0 ? 0 : (op == 2 ? 1 : 2);
            prepare(top);
            uint32_t nc = 0, fc = 0;
            wf_for_each<T>(g, tid, [&](float raw, int e) {
                const float v = value(raw, e);
                const float x = __fsub_rn(v, maxv);  // the reference's argument of fastExp (sampler.go:167)
                const float d = -x;
                if (!(d >= 0.0f)) return;  // NaN
                if (!all_members) {
                    const uint32_t key = f2key(v);
                    if (!(key > member_key || (key == member_key && e <= member_col))) return;
                }
                float ex = 0.0f;
                if (stage >= 1) {
                    ex = fast_exp(x);
                    if (stage == 2 && __dmul_rn((double)ex, inv_sum) < minp_thr) return;
                }
                if (d <= top.hi) {
                    const int b = bin_of(top, d);
                    hist_add(top, b, ex);
                    nc++;
                } else {
                    fc++;
                }
            });
            pack(top);
            // totals: counts over threads (the check on the packed words), sums over the bins
            unsigned long long tc = nc, tf = fc;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                tc += __shfl_xor_sync(0xffffffffu, tc, o);
                tf += __shfl_xor_sync(0xffffffffu, tf, o);
            }
            __syncthreads();
            if (lane == 0) {
                w->scan_c[warp] = tc;
                w->red_c[warp] = tf;
            }
            __syncthreads();
            tc = tf = 0;
            for (int i = 0; i < WF_NWARP; i++) {
                tc += w->scan_c[i];
                tf += w->red_c[i];
            }
            near_cnt = tc;
            far_cnt = tf;
            // sum of the bins, in bin order within a thread, threads in a fixed tree
            double m = 0.0;
            unsigned long long hc = 0;
            for (int j = 0; j < WF_BPT; j++) {
                const int b = tid * WF_BPT + j;
                const unsigned long long wd = top.words[b];
                hc += wd >> WF_COUNT_SHIFT;
                m = __dadd_rn(m, wf_mass(wd, top.scl[b]));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                m = __dadd_rn(m, __shfl_xor_sync(0xffffffffu, m, o));
                hc += __shfl_xor_sync(0xffffffffu, hc, o);
            }
            __syncthreads();
            if (lane == 0) {
                w->scan_m[warp] = m;
                w->scan_c[warp] = hc;
            }
            __syncthreads();
            m = 0.0;
            hc = 0;
            for (int i = 0; i < WF_NWARP; i++) {
                m = __dadd_rn(m, w->scan_m[i]);
                hc += w->scan_c[i];
            }
            __syncthreads();
            if (hc != near_cnt) {  // a bin's sum ran into its count: more than 2^18 entries in one bin
                unresolved = true;
                continue;
            }
            if (op == 0) {
                if ((unsigned long long)k >= near_cnt + far_cnt) {
                    op = 1;  // every entry is a member: no k-th entry to look for
                } else if ((unsigned long long)k > near_cnt) {
                    unresolved = true;  // the k-th entry weighs 0: among the "far" ones
                }
            } else if (op == 2) {
                sum = m;  // sampler.go:165-168
                n_kept = near_cnt + far_cnt;
                if (sum == 0.0) {  // sampler.go:170-172: cannot happen (the maximum contributes fastExp(0) = 1)
                    unresolved = true;
                    continue;
                }
                inv_sum = __ddiv_rn(1.0, sum);
                if (P.min_p > 0.0f)  // prob[0] = fastExp(0) * inv_sum (sampler.go:181)
                    minp_thr = __dmul_rn(__dmul_rn((double)fast_exp(0.0f), inv_sum), (double)P.min_p);
            } else {
                // m is the sum of the kept fastExp; the reference sums the kept probabilities
                const double new_sum = __dmul_rn(m, inv_sum);
                const unsigned long long kept = near_cnt + far_cnt;
                if (kept < n_kept && new_sum > 0.0) {  // sampler.go:199-207
                    rescale = __ddiv_rn(1.0, new_sum);
                    rescaled = true;
                }
                n_kept = kept;
                if (kept == 0) {  // min_p > 1 dropped everything: the reference indexes topIdx[-1] and panics
                    if (tid == 0) {
                        publish_row(a, row, -1);
                        if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_EMPTY);
                    }
                    done = true;
                }
            }
            continue;
        }

        // -- a query: where in the order does the walk stop? --
        //   KTH   the entry at position k (1-based)                               -> membership
        //   CUT   first position whose prefix, rounded to float, reaches top_p    -> cut
        //   DRAW  first position with r <= prefix, or the CUT position            -> the token
        const int mode = op == 1 ? WF_KTH : (op == 4 ? WF_DRAW : WF_CUT);
        const unsigned long long want = (unsigned long long)k;
        auto stops = [&](double c) {
            bool ok = nucleus && __double2float_rn(c) >= P.top_p;
            if (mode == WF_DRAW) ok = ok || r <= c;
            return ok;
        };
        // target of the walk in probability units, with the slack the float compare of top_p needs
        double target = 0.0;
        if (mode != WF_KTH) {
            const double tp = nucleus ? (double)P.top_p * (1.0 - 1e-7) : 1e300;
            target = mode == WF_CUT ? tp : fmin(tp, r);
        }
        const double gain = rescaled ? __dmul_rn(inv_sum, rescale) : inv_sum;  // probability per unit of fastExp
        double p0 = 0.0;            // probability mass before the current histogram's range
        unsigned long long c0 = 0;  // entries before it
        int lvl_b1 = 0, lvl_b2 = WF_BINS - 1;  // the row histogram's bins the bin histogram covers
        unsigned long long expect_c = 0;  // entries the bins' own histogram must hold
        int result = 2;             // 1 settled, 0 the walk never stops among the members, -1 not settled here
#pragma unroll 1
        for (int level = 0; level < 2 && result == 2; level++) {
            const WFHist& h = level == 0 ? top : sub;
            // -- locate: per-thread sums of its bins, block scan, the bins where the walk can stop --
            unsigned long long tc = 0;
            double tm = 0.0;
            for (int j = 0; j < WF_BPT; j++) {
                const int b = tid * WF_BPT + j;
                const unsigned long long wd = h.words[b];
                tc += wd >> WF_COUNT_SHIFT;
                tm = __dadd_rn(tm, wf_mass(wd, h.scl[b]));
            }
            unsigned long long sc = tc;
            double sm = tm;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long yc = __shfl_up_sync(0xffffffffu, sc, o);
                const double ym = __shfl_up_sync(0xffffffffu, sm, o);
                if (lane >= o) {
                    sc += yc;
                    sm = __dadd_rn(sm, ym);
                }
            }
            __syncthreads();
            if (lane == 31) {
                w->scan_c[warp] = sc;
                w->scan_m[warp] = sm;
            }
            if (tid == 0) {
                w->b1 = WF_BINS;
                w->b2 = WF_BINS;
            }
            __syncthreads();
            unsigned long long bc = 0, all_c = 0;
            double bmass = 0.0;
            for (int i = 0; i < WF_NWARP; i++) {
                if (i < warp) {
                    bc += w->scan_c[i];
                    bmass = __dadd_rn(bmass, w->scan_m[i]);
                }
                all_c += w->scan_c[i];
            }
            if (level == 1 && all_c != expect_c) {  // a sum ran into its count in the bins' own histogram
                result = -1;
                break;
            }
            // inclusive prefixes through my bins: entries, and fastExp mass since the range's start
            unsigned long long pc = c0 + bc + sc - tc;
            double pm = bmass + sm - tm;
            // b1: the first bin the walk can stop in; b2: the first bin by whose end it has stopped
            // (the two differ only when the target sits on a bin's edge to within rounding)
            const double t_lo = target * (1.0 - 1e-12) - 1e-300, t_hi = target * (1.0 + 1e-12) + 1e-300;
            int my_b1 = WF_BINS, my_b2 = WF_BINS;
            for (int j = 0; j < WF_BPT; j++) {
                const int b = tid * WF_BPT + j;
                const unsigned long long wd = h.words[b];
                const unsigned long long cj = wd >> WF_COUNT_SHIFT;
                const unsigned long long pc0 = pc;
                pc += cj;
                pm = __dadd_rn(pm, wf_mass(wd, h.scl[b]));
                if (cj == 0) continue;
                bool in1, in2;
                if (mode == WF_KTH) {
                    in1 = in2 = pc0 < want && want <= pc;
                } else {
                    const double c = __dadd_rn(p0, __dmul_rn(pm, gain));
                    in1 = c * (1.0 + 1e-12) >= t_lo;
                    in2 = c * (1.0 - 1e-12) >= t_hi;
                }
                if (in1 && my_b1 == WF_BINS) my_b1 = b;
                if (in2 && my_b2 == WF_BINS) my_b2 = b;
            }
            if (my_b1 < WF_BINS) atomicMin(&w->b1, my_b1);
            if (my_b2 < WF_BINS) atomicMin(&w->b2, my_b2);
            __syncthreads();
            const int b1 = w->b1;
            int b2 = w->b2;
            const bool open_end = b2 >= WF_BINS;  // the walk may run off the end of the members
            if (b1 >= WF_BINS) {
                // no prefix reaches the target: the walk ends on the last member (DRAW / CUT at the
                // row's histogram); anything else contradicts the level above
                result = (mode != WF_KTH && level == 0) ? 0 : -1;
                break;
            }
            if (open_end) b2 = WF_BINS - 1;
            if (b2 < b1) b2 = b1;
            // what lies before bin b1 and how many entries bins b1..b2 hold: their owners say
            __syncthreads();
            if (b1 / WF_BPT == tid || b2 / WF_BPT == tid) {
                unsigned long long c = bc + sc - tc;
                double m2 = bmass + sm - tm;
                for (int j = 0; j < WF_BPT; j++) {
                    const int b = tid * WF_BPT + j;
                    const unsigned long long wd = h.words[b];
                    if (b == b1) {
                        w->red_c[0] = c;
                        w->scan_m[0] = m2;
                    }
                    c += wd >> WF_COUNT_SHIFT;
                    m2 = __dadd_rn(m2, wf_mass(wd, h.scl[b]));
                    if (b == b2) w->red_c[1] = c;
                }
            }
            __syncthreads();
            const unsigned long long before_c = w->red_c[0];
            const double before_m = w->scan_m[0];
            const unsigned long long in_range = w->red_c[1] - before_c;
            __syncthreads();
            p0 = __dadd_rn(p0, __dmul_rn(before_m, gain));
            c0 += before_c;
            const bool fits = in_range <= (unsigned long long)WF_CAND;
            if (!fits && level == 1) {
                result = -1;  // ties by the thousand: not settled here
                break;
            }
            if (level == 0) {
                lvl_b1 = b1;
                lvl_b2 = b2;
                expect_c = in_range;
            }
            if (!fits) {
                // the bins' own histogram: their range of d, a hair wider than their edges
                const double width = 1.0 / (double)top.scale;
                const double lo_d = (double)top.lo + (double)b1 * width * (1.0 - WF_EDGE_EPS);
                const double hi_d = b2 == WF_BINS - 1 ? (double)top.hi
                                                      : (double)top.lo + (double)(b2 + 1) * width * (1.0 + WF_EDGE_EPS);
                sub.lo = b1 == 0 ? top.lo : fmaxf(top.lo, __double2float_rd(lo_d));
                sub.hi = fminf(top.hi, __double2float_ru(hi_d));
                const float span = __fsub_rn(sub.hi, sub.lo);
                sub.scale = span > 0.0f ? (float)WF_BINS / span * (1.0f - 1e-6f) : 0.0f;
                if (!(sub.scale > 0.0f) || !(sub.scale < 3e38f)) {
                    result = -1;  // the bins hold one value: ties
                    break;
                }
                prepare(sub);
            }
            const int sb1 = level == 1 ? b1 : 0, sb2 = level == 1 ? b2 : WF_BINS - 1;
            if (tid == 0) w->cand_cnt = 0;
            __syncthreads();
            // -- one pass: the entries of the chosen bins into shared memory (they fit), or into
            //    their own histogram (they do not) --
            const bool collect = fits;
            const int at_level = level;
            wf_for_each<T>(g, tid, [&](float raw, int e) {
                const float v = value(raw, e);
                const float x = __fsub_rn(v, maxv);
                const float d = -x;
                if (!(d >= 0.0f) || d > top.hi) return;  // NaN, or far
                const int b0 = bin_of(top, d);
                if (b0 < lvl_b1 || b0 > lvl_b2) return;
                const uint32_t key = f2key(v);
                if (!all_members && !(key > member_key || (key == member_key && e <= member_col))) return;
                float ex = 0.0f;
                if (mode != WF_KTH) {
                    ex = fast_exp(x);
                    if (__dmul_rn((double)ex, inv_sum) < minp_thr) return;
                }
                if (!collect) {
                    const int b = bin_of(sub, d);
                    hist_add(sub, b, ex);
                    return;
                }
                if (at_level == 1) {
                    const int b = bin_of(sub, d);
                    if (b < sb1 || b > sb2) return;
                }
                const int slot = atomicAdd(&w->cand_cnt, 1);
                if (slot < WF_CAND) cand[slot] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)e);
            });
            __syncthreads();
            if (!collect) {
                pack(sub);
                continue;  // locate again, on the bins' own histogram
            }

            // -- the entries are in shared memory: order them and walk --
            const int n = w->cand_cnt;
            if (n != (int)in_range) {  // cannot happen: the histogram counted these very entries
                result = -1;
                break;
            }
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
                if (want <= c0 || want - c0 > (unsigned long long)n) {
                    result = -1;
                    break;
                }
                const unsigned long long hit = cand[want - c0 - 1];
                member_key = (uint32_t)(hit >> 32);
                member_col = (int)(~(uint32_t)hit);
                all_members = false;
                __syncthreads();
                result = 1;
                break;
            }
            double* prob = reinterpret_cast<double*>(sub.words);  // WF_CAND doubles fit the histogram not in use any more
            for (int i = tid; i < n; i += WF_NT) {
                double p = 0.0;
                final_prob(fast_exp(__fsub_rn(key2f((uint32_t)(cand[i] >> 32)), maxv)), &p);
                prob[i] = p;
            }
            __syncthreads();
            if (tid == 0) {
                // the reference's own walk (sampler.go:214-231), entered with the prefix before the bins
                int pos = -1;
                const bool early = c0 > 0 && stops(p0);  // the walk stopped before the bins: a wrong bracket
                double c = p0;
                if (!early)
                    for (int i = 0; i < n; i++) {
                        c = __dadd_rn(c, prob[i]);
                        if (stops(c)) {
                            pos = i;
                            break;
                        }
                    }
                w->pos = pos;
                w->flipped = early ? -1 : (pos >= 0 ? 1 : 0);
            }
            __syncthreads();
            const int flipped = w->flipped, pos = w->pos;
            if (flipped < 0) {
                result = -1;
            } else if (flipped == 0) {
                result = open_end ? 0 : -1;  // ran off the end of the members, or of a wrong bracket
            } else {
                if (mode == WF_DRAW) {
                    token_col = (int)(~(uint32_t)cand[pos]);
                    token_prob = prob[pos];
                } else {
                    cut = (int)(c0 + (unsigned long long)pos + 1);
                }
                result = 1;
            }
            __syncthreads();
        }
        if (result == 2 || result < 0) {
            unresolved = true;
            continue;
        }
        if (op == 4) cut = (int)n_kept;  // unless the CUT query says otherwise
        if (result == 0) {
            // The walk never stops: it ends on the last member of the order (smallest value, largest
            // column), which may be one of the "far" entries; the nucleus is everything.
            unsigned long long best = 0xffffffffffffffffull;
            wf_for_each<T>(g, tid, [&](float raw, int e) {
                const float v = value(raw, e);
                if (!(v == v) || (unsigned)e >= (unsigned)V) return;
                const uint32_t key = f2key(v);
                if (!all_members && !(key > member_key || (key == member_key && e <= member_col))) return;
                double p;
                if (!final_prob(fast_exp(__fsub_rn(v, maxv)), &p)) return;
                best = min(best, ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)e));
            });
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
            __syncthreads();
            if (lane == 0) w->red_c[warp] = best;
            __syncthreads();
            for (int i = 0; i < WF_NWARP; i++) best = min(best, w->red_c[i]);
            __syncthreads();
            if (mode == WF_DRAW) {
                token_col = (int)(~(uint32_t)best);
                double p = 0.0;
                final_prob(fast_exp(__fsub_rn(key2f((uint32_t)(best >> 32)), maxv)), &p);
                token_prob = p;
            } else {
                cut = (int)n_kept;
            }
        }
    }
    if (done) return;
    if (tid == 0) {
        if (unresolved) a.next[row] = WIDE_UNRESOLVED;  // wide_rows_kernel, launched behind this one, takes the row
        else publish_row(a, row, token_col + a.vocab_offset, (int)n_kept, cut, token_prob, sum);
    }
}

}  // namespace
