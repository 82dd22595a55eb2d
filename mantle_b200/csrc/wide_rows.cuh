// wide_rows_kernel: shortlists longer than 1024 entries, up to the whole vocabulary -- the
// thorough kernel behind wide_hist_kernel, for the rows that one leaves unsettled.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

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
// kernel is compute-bound by design.  It is launched behind wide_hist_kernel (three to five
// passes) and takes only the rows that kernel marked as unsettled: ties by the thousand around
// the place where the walk stops, rows with an infinite maximum, rows of nothing but NaN.

constexpr int WIDE_NT = 512;
constexpr int WIDE_UNRESOLVED = (int)0x80000000;  // next[row] of a row wide_hist_kernel left to this kernel
constexpr int WIDE_MINB = 2;  // two CTAs per SM at 64 registers: 3 to 15 % faster than one at 128, spills included
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
    // Every thread's partial sums of a pass, one column per thread: a read-add-write of shared
    // memory per element instead of sixteen predicated adds on registers (and 48 registers less).
    // A thread sees at most MAX_VOCAB / WIDE_NT = 2048 elements per pass, so 16 bits count them.
    double col_mass[WIDE_FAN][WIDE_NT];
    uint16_t col_count[WIDE_FAN][WIDE_NT];
};
static_assert(MANTLE_SAMPLE_MAX_VOCAB / WIDE_NT < 65536, "per-thread counts are 16 bits wide");

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
__global__ void __launch_bounds__(WIDE_NT, WIDE_MINB) wide_rows_kernel(const KArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    WideCtl* w = reinterpret_cast<WideCtl*>(smem_raw);
    uint32_t* bm = reinterpret_cast<uint32_t*>(smem_raw + ((sizeof(WideCtl) + 127) / 128) * 128);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x;
    const int V = a.vocab;

    if (a.next[row] != WIDE_UNRESOLVED) return;  // settled by wide_hist_kernel (skipped rows included)
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
    const float inv_temp = greedy ? 1.0f : __fdiv_rn(1.0f, P.temperature);
    const void* rowp = reinterpret_cast<const T*>(a.logits) + (size_t)row * (size_t)a.row_stride;

    const int hl = history_len(a, row);
    const WinPlan wp = win_plan(P, hl);
    const bool pen = wp.active;
    if (pen) build_penalty_bitmap(a, row, wp, hl, V, a.vocab_offset, bm, tid, WIDE_NT);

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
            publish_row(a, row, best == 0xffffffffffffffffull ? 0 : (int)best + a.vocab_offset);
            if (best == 0xffffffffffffffffull && a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_NAN);
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
            // a power of two just above span / WIDE_FAN: the sub-range of a key is a shift, not a divide
            const int wshift = 32 - __clz((int)(span / WIDE_FAN));
            const uint32_t width = 1u << wshift;
#pragma unroll
            for (int j = 0; j < WIDE_FAN; j++) {
                w->col_mass[j][tid] = 0.0;
                w->col_count[j][tid] = 0;
            }
            for (int e = tid; e < V; e += WIDE_NT) {
                const float v = value(e);
                if (!(v == v)) continue;
                const uint32_t key = f2key(v);
                if (key < lo || key > hi) continue;
                double p;
                if (!weigh(v, key, e, &p)) continue;
                const int j = (int)((hi - key) >> wshift);
                w->col_mass[j][tid] = __dadd_rn(w->col_mass[j][tid], p);
                w->col_count[j][tid]++;
            }
#pragma unroll
            for (int j = 0; j < WIDE_FAN; j++) {
                double d = w->col_mass[j][tid];
                unsigned long long n = w->col_count[j][tid];
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
        if (tid == 0) publish_row(a, row, 0, (int)n_kept, 0);
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
                publish_row(a, row, -1);
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
    if (tid == 0) publish_row(a, row, col < 0 ? -1 : col + a.vocab_offset, (int)n_kept, cut, h.p_each, sum);
}

}  // namespace
