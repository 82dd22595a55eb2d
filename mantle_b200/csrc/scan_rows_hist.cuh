// scan_rows_hist_kernel: the streaming pass for shortlists of 29 to 1024 entries, with plain 16-byte
// loads and a threshold that comes from a running histogram of the candidate buffer.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// ---------------------------------------------------------------------------------------
// One CTA per item (row, split), plain 16-byte loads, two register sets per thread, each refilled
// from global memory while the other is filtered.  No shared-memory staging of the row, so the
// CTA is small (candidate buffer, histogram, staged survivors, bitmap) and four of them share an SM.
//
// Where scan_rows_ldg_kernel cuts its buffer exactly whenever it fills -- which ranks n entries
// against each other, n growing with the shortlist -- this kernel never ranks anything while the
// row streams.  Every entry that enters the buffer is counted in a histogram of its value; one
// warp per region walks the counts from the top to the bin at which they reach k and raises the
// threshold to that bin's edge (sampler_common.cuh: hist_bin, hist_threshold); the buffer keeps
// every entry ever admitted and is compacted by the last threshold once, before the one exact
// select at the end of the row.  A lane that finds a survivor only sets it aside; its warp works
// the staged survivors off together between two regions (stage, flush_staged).  The CTA meets at
// a barrier only after regions 1, 2, 4, 8, ... (sampler_select.cuh: forced_cut).

template <class S, typename T, int MODE, bool POST>
__global__ void __launch_bounds__(S::NT, S::MINB) scan_rows_hist_kernel(const KArgs a) {
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
    // shortlists longer than the thread maxima can seed take their seed from a histogram of region 0
    constexpr bool SEED_HIST = S::KCAP > 32 * NWARP;
    bool careful = false;

    // The first region's loads go out before anything else: they are in flight while the bitmap is built.
    uint4 ra[U], rb[U];
    // A region that may reach beyond the item (its last one): every vector tested against the end.
    auto load_checked = [&](uint4(&dst)[U], int r) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            int v = a0 + r * RV + u * NT + tid;
            dst[u] = v < b0 ? __ldcs(vbase + v) : make_uint4(0, 0, 0, 0);
        }
    };
    // A region that lies inside the item: U loads at fixed offsets from a pointer that walks the row.
    const int nwhole = (b0 - a0) / RV;  // regions [0, nwhole) are complete
    const uint4* q = vbase + a0 + tid + RV;  // this thread's first vector of region 1
    auto load_whole = [&](uint4(&dst)[U]) {
#pragma unroll
        for (int u = 0; u < U; u++) dst[u] = __ldcs(q + u * NT);
        q += RV;
    };
    // The L2 is asked for a region (one request per 128-byte line: a warp's share of a region is U
    // runs of 512 bytes, lane i asks for line i & 3 of run i >> 2) two regions before its loads are
    // issued, so that those loads find their lines on the way or already there.
    const uint4* pf = vbase + a0 + (lane >> 2) * NT + (tid & ~31) + (lane & 3) * 8;  // region 0's line of this lane
    const bool pf_lane = lane < 4 * U;
    auto ahead = [&](int r) {  // any region: the line tested against the end
        if (r < nreg && pf_lane) {
            const uint4* l = pf + (size_t)r * RV;
            if (l < vbase + b0) asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(l));
        }
    };
    if (nreg > 0) {
        load_checked(ra, 0);
        ahead(1);
        ahead(2);
        ahead(3);
    }
    if (tid == 0) {
        ctl->cnt = 0;
        ctl->k = k;
        ctl->thr_key = 0u;
        ctl->thr = __uint_as_float(0xff800000u);
        ctl->walked = 0;
        ctl->hbase = ctl->hscale = ctl->htop = ctl->hwidth = 0.0f;  // one bin until region 0 has laid them out
    }
    for (int i = tid; i < HBINS; i += NT) hist[i] = 0u;
    volatile int* wcnt = reinterpret_cast<volatile int*>(smem_raw + S::WCNT_OFF);
    if (tid < NWARP) wcnt[tid] = 0;

    // ---- repeat penalty: bitmap of the de-duplicated window (sampler.go:99-138) --------
    const WinPlan wp = win_plan(P, hl);
    if (wp.active) {
        build_penalty_bitmap_early<NT>(a, row, wp, hl, c.V, c.voff, bm, tid, recent);
        c.pen_bitmap = true;
    }
    if (tid == 0) {  // what the out-of-line survivor code reads
        ctl->pen_on = wp.active ? 1 : 0;
        ctl->inv_temp = c.inv_temp;
        ctl->pen = c.pen;
        ctl->voff = c.voff;
        ctl->post_mode = a.post.mode;
        ctl->post_scale = a.post.scale;
        ctl->post_cap = a.post.cap;
    }
    __syncthreads();

    // ---- stream the item ------------------------------------------------------------------
    float thr = __uint_as_float(0xff800000u);            // -inf
    float rthr = thr;  // POST: the raw logit every column that can reach thr has at least
    const Post& POSTP = a.post;

    if (nreg > 0) {
        // The threshold the running histogram has reached (sampler_common.cuh).
        auto fresh = [&]() {
            const float t = *reinterpret_cast<const volatile float*>(&ctl->thr);
            if (POST) {
                if (t != thr) rthr = post_raw_bound(t, c.inv_temp, POSTP);
            }
            thr = t;
        };
        typedef VecPart<T> VP;
        // One vector of a region in which this thread holds a column that reaches its threshold:
        // one test on the vector's maximum, the compares only where it holds a survivor.
        auto one_vector = [&](const uint4& v, float mu, int vec) {
            if (POST ? (mu >= rthr) : (__fmul_rn(mu, c.inv_temp) >= thr))
                filter_vec<S, T, POST>(v, vec, c.mis, c.inv_temp, thr, rthr);
        };
        // A complete region: one test per thread.  A rounded multiply by a positive factor is
        // non-decreasing, so the largest scaled value is the scaled largest raw value, exactly.
        auto whole_region = [&](const uint4(&src)[U], int r) {
            if constexpr (SEED_HIST) {
                // The larger shape's shortlists are long enough that nearly every warp holds a survivor in
                // nearly every vector: the tests in front of the compares only cost there.
                const int v0 = a0 + r * RV + tid;
#pragma unroll
                for (int u = 0; u < U; u++) filter_vec<S, T, POST>(src[u], v0 + u * NT, c.mis, c.inv_temp, thr, rthr);
                return;
            }
            typename VP::part_t part[U];
#pragma unroll
            for (int u = 0; u < U; u++) part[u] = VP::part(src[u]);
            const float m = VP::template region<U>(part, src);
            if (POST ? (m >= rthr) : (__fmul_rn(m, c.inv_temp) >= thr)) {
                const int v0 = a0 + r * RV + tid;
#pragma unroll
                for (int u = 0; u < U; u++) one_vector(src[u], VP::finish(part[u], src[u]), v0 + u * NT);
            }
        };
        // The item's last region: vectors beyond the end are skipped.
        auto last_region = [&](const uint4(&src)[U], int r) {
            const int v0 = a0 + r * RV + tid;
#pragma unroll
            for (int u = 0; u < U; u++)
                if (v0 + u * NT < b0) one_vector(src[u], vec_max_raw<T>(src[u]), v0 + u * NT);
        };
        // After region r one warp (they take turns) walks the histogram, if enough entries have come
        // since the last walk, and raises the threshold; nobody waits for it.  The CTA meets only after
        // regions 1, 2, 4, 8, ...: between two such meetings about k entries arrive however long the
        // row is, and a meeting that finds more than FORCE entries in the buffer compacts it.
        auto region_end = [&](int r) {
            // staged survivors are worked off once the area is three quarters full, and before the CTA meets
            // (the count is taken by one lane after the warp has come together again: lanes that read it
            // while others were still setting survivors aside would disagree on the call below, and a
            // warp split over two of its own meeting points does not return)
            __syncwarp();
            const int staged = __shfl_sync(0xffffffffu, wcnt[warp], 0);
            if (staged >= S::STG * 3 / 4 || (r & (r - 1)) == 0) flush_staged<S, POST>();
            if ((r & (NWARP - 1)) == warp) {
                const int n = live_count(ctl);
                const int fresh_entries = __shfl_sync(0xffffffffu, n - ctl->walked, 0);
                const int kk = ctl->k;
                if (fresh_entries >= (kk >> 2) + 8) {
                    const uint32_t key = hist_threshold<S>(kk);
                    if (lane == 0) {
                        ctl->walked = n;
                        if (key > ctl->thr_key) {
                            atomicMax(&ctl->thr_key, key);
                            ctl->thr = key2f(key);
                        }
                    }
                }
            }
            if ((r & (r - 1)) == 0) {
                if (__syncthreads_or(live_count(ctl) > S::FORCE)) careful = forced_cut<S>(tid);
            }
            fresh();
        };

        // -- region 0 seeds the threshold --
        if (nreg > 1) load_checked(rb, 1);
        if (nreg > 1 && nwhole > 1) q += RV;
        {
            const int v0 = a0 + tid;
            // The seed comes from RAW logits: everything between a raw logit and its final value
            // (post-processing up to its slack, penalty, temperature) is non-decreasing, and a
            // column's value is at least what it would be with the penalty, so the image of a raw
            // logit that k columns reach is a value that k columns reach -- no bitmap lookups here.
            float t0, h0;  // raw: what k columns of the region reach, and what about half as many reach
            if constexpr (!SEED_HIST) {
                // Up to 32 * NWARP entries: from a sort of each warp's thread maxima.  NWARP * j >= k
                // columns reach the smallest of the warps' j-th largest; the largest of their
                // (j / 2)-th largest spans the bins, so that a few outliers do not stretch them.
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
                const float wj = __shfl_sync(0xffffffffu, x, j - 1);
                const float wh = __shfl_sync(0xffffffffu, x, (j - 1) >> 1);
                if (lane == 0) {
                    ctl->warpv[warp] = wj;
                    ctl->warpk_min[warp] = __float_as_uint(wh);
                }
                __syncthreads();
                t0 = ctl->warpv[0];
                h0 = __uint_as_float(ctl->warpk_min[0]);
#pragma unroll
                for (int w = 1; w < NWARP; w++) {
                    t0 = fminf(t0, ctl->warpv[w]);
                    h0 = fmaxf(h0, __uint_as_float(ctl->warpk_min[w]));
                }
            } else {
                // Longer shortlists: every raw value of region 0 is counted in the histogram, laid
                // over the region's own range, and every warp walks it for itself.
                float lo = __uint_as_float(0x7f800000u), top = __uint_as_float(0xff800000u);
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (v0 + u * NT < b0) {
                        float raw[VEC];
                        Elem<T>::widen(ra[u], raw);
#pragma unroll
                        for (int i = 0; i < VEC; i++) {
                            if (raw[i] > -3.0e38f) lo = fminf(lo, raw[i]);
                            top = fmaxf(top, raw[i]);
                        }
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
                }
                if (lane == 0) {
                    ctl->warpv[warp] = top;
                    ctl->warpk_min[warp] = __float_as_uint(lo);
                }
                __syncthreads();
                lo = __uint_as_float(ctl->warpk_min[0]);
                top = ctl->warpv[0];
#pragma unroll
                for (int w = 1; w < NWARP; w++) {
                    lo = fminf(lo, __uint_as_float(ctl->warpk_min[w]));
                    top = fmaxf(top, ctl->warpv[w]);
                }
                const float sc = (top > lo && top - lo < 3.0e38f) ? (float)HBINS / (top - lo) : 0.0f;
                if (tid == 0) {
                    ctl->hbase = lo;
                    ctl->hscale = sc;
                    ctl->hwidth = sc > 0.0f ? (top - lo) / (float)HBINS : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (v0 + u * NT < b0) {
                        float raw[VEC];
                        Elem<T>::widen(ra[u], raw);
#pragma unroll
                        for (int i = 0; i < VEC; i++)
                            if (raw[i] >= lo) atomicAdd(&hist[hist_bin(raw[i], lo, sc)], 1u);
                    }
                }
                __syncthreads();
                const uint32_t kk = hist_threshold<S>(k);
                const uint32_t kh = hist_threshold<S>((k + 1) >> 1);
                // (with fewer than k columns in the region there is no seed)
                t0 = kk ? key2f(kk) : __uint_as_float(0xff800000u);
                h0 = kh ? key2f(kh) : top;
                __syncthreads();
                for (int i = tid; i < HBINS; i += NT) hist[i] = 0u;
            }
            if (POST) {
                t0 = post_seed_logit(t0, POSTP);
                h0 = post_seed_logit(h0, POSTP);
            }
            if (c.pen_bitmap) t0 = penalise(t0, c.pen);
            t0 = __fmul_rn(t0, c.inv_temp);
            h0 = __fmul_rn(h0, c.inv_temp);
            if (tid == 0) {
                // The bins of the running histogram start at the seed and span twelve times the
                // distance to the value half as many columns reach: the k-th value of the whole row
                // lies a few such distances up, and whatever lies beyond the span shares the top bin.
                const float span = __fmul_rn(SEED_HIST ? 12.0f : 8.0f, __fsub_rn(h0, t0));
                const bool ok = span > 0.0f && span < 3.0e38f;
                ctl->thr_key = f2key(t0);
                ctl->thr = t0;
                ctl->hbase = t0;
                ctl->htop = __fadd_rn(t0, span);
                ctl->hscale = ok ? __fdiv_rn((float)HBINS, span) : 0.0f;
                ctl->hwidth = ok ? __fdiv_rn(span, (float)HBINS) : 0.0f;
            }
            __syncthreads();
            thr = t0;
            if (POST) rthr = post_raw_bound(thr, c.inv_temp, POSTP);
            // (the seed admits a few entries more than k: for long shortlists, more than the staging area
            // holds, so it is emptied after every vector)
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (v0 + u * NT < b0) filter_vec<S, T, POST>(ra[u], v0 + u * NT, c.mis, c.inv_temp, thr, rthr);
                if (k >= 128 || u == U - 1) flush_staged<S, POST>();
            }
        }
        // the first meeting: every append of region 0 is counted before the threshold is read; every
        // warp walks the histogram for itself
        __syncthreads();
        if (live_count(ctl) > CAP) {
            careful = true;
        } else {
            const uint32_t key = hist_threshold<S>(k);
            if (key > f2key(thr)) thr = key2f(key);
            if (POST) rthr = post_raw_bound(thr, c.inv_temp, POSTP);
            if (tid == 0) {
                ctl->walked = live_count(ctl);
                ctl->thr_key = f2key(thr);
                ctl->thr = thr;
            }
        }

        // -- regions 1.. : two register sets, each refilled while the other is filtered --
        int r = 1;  // rb holds region r
        while (r + 2 < nwhole && !careful) {  // regions r + 1 and r + 2 are complete
            load_whole(ra);
            if (pf_lane && r + 3 < nwhole) asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(pf + (size_t)(r + 3) * RV));
            whole_region(rb, r);
            region_end(r);
            ++r;
            if (careful) break;
            load_whole(rb);
            if (pf_lane && r + 3 < nwhole) asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(pf + (size_t)(r + 3) * RV));
            whole_region(ra, r);
            region_end(r);
            ++r;
        }
        // the last regions (at most three), the item's end among them
        while (r < nreg && !careful) {
            if (r + 1 < nreg) load_checked(ra, r + 1);
            ahead(r + 3);
            if (r < nwhole) whole_region(rb, r);
            else last_region(rb, r);
            region_end(r);
            ++r;
#pragma unroll
            for (int u = 0; u < U; u++) rb[u] = ra[u];
        }
    }

    if (!careful) {
        flush_staged<S, POST>();
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
            if (POST ? (raw >= rthr) : (__fmul_rn(raw, c.inv_temp) >= thr)) survivor<S, POST>(raw, e);
        }
        __syncthreads();
        // what the histogram's threshold leaves is a few entries more than k: the exact cut's work
        if (live_count(ctl) > k + 32) careful = hist_compact<S>(buf, ctl, hist, tid, false);
        else __syncthreads();
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

    bool have, ordered = false;
    {
        // what is too long for a cheap counting select (from 129 entries on; the larger shape: 257) is
        // ordered by buckets of its value
        __syncthreads();
        if (!careful && live_count(ctl) > (SEED_HIST ? RANK_MAX : RANK_MAX / 2)) ordered = bucket_order<S>(k, tid);
    }
    if (!ordered) refresh_topk<S, true>(buf, ctl, hist, k, tid, &have, &ordered);
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
