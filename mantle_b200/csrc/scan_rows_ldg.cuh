// scan_rows_ldg_kernel: the streaming pass for short shortlists (top_k up to CUT_KMAX), with plain
// 16-byte loads and an exact cut of the candidate buffer whenever it fills.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// Up to this shortlist length the buffer is cut exactly, by counting, every time it holds half as
// many entries again: the cuts rank a few dozen entries and give the exact k-th value as the next
// threshold.  Longer shortlists go to scan_rows_hist_kernel, whose threshold comes from a running
// histogram and which never ranks more than the final shortlist (measured on 4096 rows of 151 936
// float32 columns: 0.405 against 0.420 ms at top_k 20, 0.428 against 0.430 ms at 28, 0.439 against
// 0.435 ms at 32, 0.470 against 0.446 ms at 40, 0.721 against 0.522 ms at 100).
constexpr int CUT_KMAX = 28;
constexpr int VOTE_EVERY = 2;  // regions between two "does the buffer need a cut" votes

namespace cut {

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
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
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
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
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


}  // namespace cut


// ---------------------------------------------------------------------------------------
// The streaming pass: one CTA per item (row, split), plain 16-byte loads, two register sets per
// thread, each refilled from global memory while the other is filtered, a barrier every second
// region of NT*U vectors.  No shared-memory staging, so the CTA is small (candidate buffer +
// bitmap) and four of them share an SM.

template <class S, typename T, int MODE, bool POST>
__global__ void __launch_bounds__(S::NT, S::MINB) scan_rows_ldg_kernel(const KArgs a) {
    constexpr int VEC = Elem<T>::VEC;
    constexpr int NT = S::NT, NWARP = S::NWARP, U = S::U, CAP = S::CAP;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
    uint32_t* bm = reinterpret_cast<uint32_t*>(smem_raw + S::SMEM_FIXED);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int item = blockIdx.x;
    const int row = item / a.splits;
    const int split = item - row * a.splits;

    // Split rows: the merge kernel queued behind this one may start as CTAs here retire (it waits
    // for this grid's writes before it reads a part); a no-op for any other successor.
    if (MODE == MODE_PARTS) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (a.skip && a.skip[row] != 0) {  // a request that has ended: nothing is read, nothing is drawn
        if (tid == 0) {
            if (MODE == MODE_FUSED) publish_row(a, row, -1);
            else a.part_cnt[(size_t)split * a.rows + row] = 0;
        }
        return;
    }
    // the history's most recent ids are asked for before anything else is
    const int hl = history_len(a, row);
    int recent[HIST_PRE];
    if (hl > 0) history_tail<NT>(a, row, hl, tid, recent);
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
    // (a shape whose longest shortlist the thread maxima can seed never starts on the careful path: its first
    // loads then do not wait for the row's parameters)
    bool careful = S::KCAP > 32 * NWARP && k > 32 * NWARP;

    // The first region's loads go out before anything else: they are in flight while the bitmap is built.
    uint4 ra[U], rb[U];
    // Only an item's last region can be partial.  Measured alternatives, each with fewer instructions
    // and each slower: loads that leave a register beyond the item as it is (they wait for its last
    // reader, 1.6 %), loads without bounds tests for whole regions (2 %), a -inf fill that spares the
    // masks below (1 %).
    auto load = [&](uint4(&dst)[U], int r) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            int v = a0 + r * RV + u * NT + tid;
            dst[u] = v < b0 ? __ldcs(vbase + v) : make_uint4(0, 0, 0, 0);
        }
    };
    // `ahead(r)`: ask the L2 for region r (one request per 128-byte line), two regions before its
    // loads are issued, so that those loads find their lines on the way or already there
    auto ahead = [&](int r) {
        // a warp's share of a region is U runs of 512 bytes: lane i asks for line i & 3 of run i >> 2
        if (r < nreg && lane < 4 * U) {
            const int v = a0 + r * RV + (lane >> 2) * NT + (tid & ~31) + (lane & 3) * 8;
            if (v < b0) asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(vbase + v));
        }
    };
    if (!careful && nreg > 0) {
        load(ra, 0);
        ahead(1);
        ahead(2);
    }
    if (tid == 0) ctl->cnt = 0;

    // ---- repeat penalty: bitmap of the de-duplicated window (sampler.go:99-138) --------
    const WinPlan wp = win_plan(P, hl);
    if (wp.active) {
        build_penalty_bitmap_early<NT>(a, row, wp, hl, c.V, c.voff, bm, tid, recent);
        c.pen_bitmap = true;
    }
    __syncthreads();

    // ---- stream the item ------------------------------------------------------------------
    // cut the buffer at this many entries (measured: k + k/4, k + k, k + 16 and k + 32 are all within
    // 2 % of this up to top_k 100 and worse beyond; votes every third region gain 2 % from top_k 64 on)
    const int trig = min(k + max(k >> 1, 16), CAP / 2);
    float thr = __uint_as_float(0xff800000u);            // -inf
    float rthr = thr;  // POST: the raw logit every column that can reach thr has at least
    const Post& POSTP = a.post;

    if (!careful && nreg > 0) {
        // later regions: the buffer already holds k entries >= thr with lower indices, so an equal
        // value can no longer enter (sampler.go:268-275); one test per thread and region
        auto later = [&](const uint4(&src)[U], int r) {
            const int v0 = a0 + r * RV + tid;
            float mu[U];
            float m = __uint_as_float(0xff800000u);
            const bool whole = r + 1 < nreg;
#pragma unroll
            for (int u = 0; u < U; u++) {
                mu[u] = __uint_as_float(0x7fc00000u);  // NaN: beyond the item, admitted by no compare
                if (whole || v0 + u * NT < b0) mu[u] = vec_max_raw<T>(src[u]);
                m = fmaxf(m, mu[u]);
            }
            if (POST) {
                if (m >= rthr) {
#pragma unroll
                    for (int u = 0; u < U; u++)
                        if (mu[u] >= rthr) cut::filter_vec_post<S, T, false>(src[u], v0 + u * NT, c, POSTP, rthr, thr, buf, ctl);
                }
            } else if (__fmul_rn(m, c.inv_temp) > thr) {
                // A rounded multiply by a positive factor is non-decreasing, so the largest scaled value
                // is the scaled largest raw value, exactly: one multiply per thread and region here,
                // one per vector below, and the sixteen only where a vector holds a survivor.
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (__fmul_rn(mu[u], c.inv_temp) > thr) cut::filter_vec<S, T, false>(src[u], v0 + u * NT, c, thr, buf, ctl);
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

        // -- region 0 seeds the threshold --
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
                    if (v0 + u * NT < b0) cut::filter_vec_post<S, T, true>(ra[u], v0 + u * NT, c, POSTP, rthr, thr, buf, ctl);
            } else {
                thr = t0;
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (v0 + u * NT < b0) cut::filter_vec<S, T, true>(ra[u], v0 + u * NT, c, thr, buf, ctl);
            }
        }
        region_end(k + 1);

        // -- regions 1.. : two register sets, each refilled while the other is filtered --
        // The barrier carries only the vote (the register sets are private), so it need not follow
        // every region: the threshold is refreshed at most every VOTE_EVERY regions, at the price of
        // a few more survivors under a threshold that is that much staler.
        // (Measured and not kept: no periodic barrier at all -- a warp that finds the buffer at `trig`
        // entries goes to the barrier and the others follow when they find the same, warps of one CTA
        // drifting apart in between.  2 to 5 % faster at top_k 40 to 64, 1 to 2.5 % slower at 20 and
        // 100, slower on the split-row batches.  Such a scheme must take the decision with a warp-wide
        // vote: lanes of one warp that read the count at different moments reached different barrier
        // instructions, which hung the kernel until the process was killed.)
        int r = 1;
        while (r < nreg && !careful) {
            if (r + 1 < nreg) load(ra, r + 1);
            ahead(r + 3);
            later(rb, r);
            if (r % VOTE_EVERY == 0 || r + 1 == nreg) region_end(trig);
            if (++r >= nreg || careful) break;
            if (r + 1 < nreg) load(rb, r + 1);
            ahead(r + 3);
            later(ra, r);
            if (r % VOTE_EVERY == 0 || r + 1 == nreg) region_end(trig);
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
                if (raw >= rthr) cut::consider_post<S, true>(buf, ctl, c, POSTP, raw, e, thr);
            } else {
                float v = __fmul_rn(raw, c.inv_temp);
                if (v >= thr) cut::consider<S, true>(buf, ctl, c, raw, v, e, thr);
            }
        }
        __syncthreads();
        if (live_count(ctl) > CAP) careful = true;
        __syncthreads();
    }

    if (careful) {  // the careful path: steps that always fit the buffer
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
                uint32_t kth = select_topk<S>(buf, ctl, hist, k, tid, &have);  // leaves no order
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
                publish_row(a, row, -1);
            } else {
                a.part_cnt[(size_t)split * a.rows + row] = 0;
            }
        }
        return;
    }
    finish_row<S, MODE>(a, row, split, P, greedy, ordered, buf, ctl, tid);
}

}  // namespace
