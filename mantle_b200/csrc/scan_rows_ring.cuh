// scan_rows_kernel: the streaming pass fed by a ring of bulk copies (persistent CTAs).
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

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

}  // namespace
