// Cutting the candidate buffer to its k best entries: the shared-memory radix select, the
// counting select for small buffers, and the ordering of the survivors.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// a precedes b in the shortlist order (key descending, index ascending).  By value and without
// short-circuits: an entry read through a reference to shared memory became two dependent loads
// and a branch per compare, which cost the split-row batches a seventh of their time.
__device__ __forceinline__ bool cand_before(const Cand a, const Cand b) {
    return (a.key > b.key) | ((a.key == b.key) & (a.idx < b.idx));
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

// The counting select for NT < n <= 2 * NT: two entries per thread, one read of the buffer for both.
template <class S>
__device__ __forceinline__ uint32_t rank_select2(Cand* buf, Ctl* ctl, int n, int k, int tid, bool* have_kth) {
    static_assert(S::NT == RANK_MAX, "every thread holds a first entry");
    const Cand me0 = buf[tid];
    Cand me1;
    me1.key = 0;
    me1.idx = 0xffffffffu;
    const bool two = tid + S::NT < n;
    if (two) me1 = buf[tid + S::NT];
    int r0 = 0, r1 = 0;
    for (int j = 0; j < n; j++) {
        const Cand o = buf[j];
        r0 += ((o.key > me0.key) | ((o.key == me0.key) & (o.idx < me0.idx))) ? 1 : 0;
        r1 += ((o.key > me1.key) | ((o.key == me1.key) & (o.idx < me1.idx))) ? 1 : 0;
    }
    if (!two) r1 = 0x7fffffff;
    __syncthreads();
    if (r0 < k) buf[r0] = me0;
    if (r1 < k) buf[r1] = me1;
    if (r0 == k - 1) ctl->sel_bin = (int)me0.key;
    if (r1 == k - 1) ctl->sel_bin = (int)me1.key;
    if (tid == 0) ctl->cnt = min(n, k);
    __syncthreads();
    *have_kth = n >= k;
    return (uint32_t)ctl->sel_bin;
}

// Cut the buffer to its k best entries, by counting when it is small and by radix select
// otherwise.  Called by every thread with the buffer quiescent.
// RANK2: buffers of up to twice as many entries are still ranked by counting, two entries per thread.
template <class S, bool RANK2 = false>
__device__ __forceinline__ uint32_t refresh_topk(Cand* buf, Ctl* ctl, uint32_t* hist, int k, int tid,
                                                 bool* have_kth, bool* ordered = nullptr) {
    __syncthreads();
    const int n = live_count(ctl);
    __syncthreads();
    constexpr int RANKED = (RANK2 && S::NT == RANK_MAX) ? 2 * RANK_MAX : RANK_MAX;
    if (ordered) *ordered = n <= RANKED;  // the counting select leaves its survivors in order
    if (n <= RANK_MAX) return rank_select(buf, ctl, n, k, tid, have_kth);
    if constexpr (RANKED > RANK_MAX) {
        if (n <= RANKED) return rank_select2<S>(buf, ctl, n, k, tid, have_kth);
    }
    return select_topk<S>(buf, ctl, hist, k, tid, have_kth);
}

// ---------------------------------------------------------------------------------------
// The running histogram's side of the buffer (hist_bin, append_binned, hist_threshold).

// Zeroes the histogram and counts the first n entries of the buffer again.  Every thread; the
// buffer quiescent; ends with a barrier.
template <class S>
__device__ __forceinline__ void hist_rebuild(const Cand* buf, const Ctl* ctl, uint32_t* hist, int n, int tid) {
    for (int i = tid; i < HBINS; i += S::NT) hist[i] = 0u;
    __syncthreads();
    const float base = ctl->hbase, scale = ctl->hscale;
    for (int i = tid; i < n; i += S::NT) atomicAdd(&hist[hist_bin(key2f(buf[i].key), base, scale)], 1u);
    __syncthreads();
}

// Drops the entries below the histogram's threshold.  Called by every thread behind a barrier
// that follows the last append; returns true if the buffer has overflowed (the row is redone on
// the careful path).  With `rebuild` the histogram is counted again from what is left, so that
// it never counts an entry the buffer no longer holds.
template <class S>
__device__ __forceinline__ bool hist_compact(Cand* buf, Ctl* ctl, uint32_t* hist, int tid, bool rebuild) {
    constexpr int NT = S::NT, EPT = S::EPT;
    const int n = live_count(ctl);
    if (n > S::CAP) return true;
    if (tid < 32) {
        const uint32_t key = hist_threshold<S>(ctl->k);
        if (tid == 0 && key > ctl->thr_key) {
            ctl->thr_key = key;
            ctl->thr = key2f(key);
        }
    }
    __syncthreads();
    const uint32_t tk = ctl->thr_key;
    Cand mine[EPT];
    uint32_t keep = 0;
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        const int i = tid + j * NT;
        if (i < n) {
            mine[j] = buf[i];
            if (mine[j].key >= tk) keep |= 1u << j;
        }
    }
    __syncthreads();
    if (tid == 0) ctl->cnt = 0;
    __syncthreads();
    if constexpr (S::KCAP > RANK_MAX) {
        // long shortlists keep a thousand entries: one reservation per warp and round instead of one per entry
        const int lane = tid & 31;
#pragma unroll
        for (int j = 0; j < EPT; j++) {
            const bool kj = (keep >> j) & 1u;
            const uint32_t b = __ballot_sync(0xffffffffu, kj);
            if (b) {
                int base = 0;
                if (lane == 0) base = atomicAdd(&ctl->cnt, __popc(b));
                base = __shfl_sync(0xffffffffu, base, 0);
                if (kj) buf[base + __popc(b & ((1u << lane) - 1u))] = mine[j];
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < EPT; j++) {
            if ((keep >> j) & 1u) {
                const int slot = atomicAdd(&ctl->cnt, 1);
                buf[slot] = mine[j];
            }
        }
    }
    __syncthreads();
    if (tid == 0) ctl->walked = live_count(ctl);
    if (rebuild) hist_rebuild<S>(buf, ctl, hist, live_count(ctl), tid);
    return false;
}

// Orders the n entries of the buffer (key descending, index ascending) and keeps the best k, for a
// buffer too long for the counting select: the entries are dealt into HBINS buckets of their value
// (laid over the buffer's own range), bucket by bucket into the upper half of the buffer, and every
// entry then counts the entries of its own bucket that precede it -- the counting select, bucket by
// bucket.  n * (a bucket's length) compares in all, four barriers; the radix select followed by the
// bitonic sort it replaces has sixty.  Returns false, with
// the buffer as it was, when that does not work out (more than half the buffer in use, a bucket of
// more than BUCKET_MAX entries: ties, or one value far from the rest); the caller then takes the
// other way.  Every thread; the buffer quiescent.
constexpr int BUCKET_MAX = 256;
template <class S>
__device__ __noinline__ bool bucket_order(int k, int tid) {
    static_assert(S::NT == HBINS, "one bucket per thread");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* cnt = reinterpret_cast<uint32_t*>(buf + S::CAP);                 // the histogram's words
    uint32_t* off = reinterpret_cast<uint32_t*>(smem_raw + S::STG_OFF);      // the staging area: free by now
    static_assert(8 * S::NWARP * S::STG >= 4 * HBINS, "the offsets fit the staging area");
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
    Cand* dst = buf + S::CAP / 2;
    constexpr int NT = S::NT, EPT = (S::CAP / 2 + NT - 1) / NT;
    const int lane = tid & 31, warp = tid >> 5;
    const int n = live_count(ctl);
    if (n > S::CAP / 2) return false;

    // the range of the keys
    uint32_t lo = 0xffffffffu, hi = 0u;
    for (int i = tid; i < n; i += NT) {
        const uint32_t key = buf[i].key;
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
    cnt[tid] = 0u;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < S::NWARP; w++) {
        lo = min(lo, ctl->warpk_min[w]);
        hi = max(hi, ctl->warpk_max[w]);
    }
    const float flo = key2f(lo), fhi = key2f(hi);
    const float span = __fsub_rn(fhi, flo);
    const float sc = (span > 0.0f && span < 3.0e38f) ? __fmul_rn(__fdiv_rn((float)HBINS, span), 1.0f - 1e-6f) : 0.0f;

    // every entry takes a place in its bucket
    uint32_t place[EPT];  // bucket << 16 | place in it
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        const int i = tid + j * NT;
        if (i < n) {
            const int b = hist_bin(key2f(buf[i].key), flo, sc);
            place[j] = ((uint32_t)b << 16) | atomicAdd(&cnt[b], 1u);
        }
    }
    __syncthreads();
    // where a bucket starts: behind all higher ones
    if (warp == 0) {
        uint32_t c[8], tot = 0, most = 0;
#pragma unroll
        for (int b = 0; b < 8; b++) {
            c[b] = cnt[lane * 8 + b];
            tot += c[b];
            most = max(most, c[b]);
        }
        uint32_t above = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_down_sync(0xffffffffu, above, o);
            if (lane + o < 32) above += y;
            most = max(most, __shfl_xor_sync(0xffffffffu, most, o));
        }
        uint32_t run = above - tot;
#pragma unroll
        for (int b = 7; b >= 0; b--) {
            off[lane * 8 + b] = run;
            run += c[b];
        }
        if (lane == 0) ctl->sel_cnt = (int)most;
    }
    __syncthreads();
    if (ctl->sel_cnt > BUCKET_MAX) return false;
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        const int i = tid + j * NT;
        if (i < n) dst[off[place[j] >> 16] + (place[j] & 0xffffu)] = buf[i];
    }
    __syncthreads();
    // every entry counts the entries of its own bucket that precede it and goes to its place in the order;
    // only the best k places exist
    const int m = min(n, k);
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        const int i = tid + j * NT;
        if (i < n) {
            const uint32_t b = place[j] >> 16;
            const int first = (int)off[b], len = (int)cnt[b];
            const Cand me = dst[first + (int)(place[j] & 0xffffu)];
            int rank = 0;
            for (int t = 0; t < len; t++) rank += cand_before(dst[first + t], me) ? 1 : 0;
            if (first + rank < m) buf[first + rank] = me;
        }
    }
    if (tid == 0) ctl->cnt = m;
    __syncthreads();
    return true;
}

// A meeting of the streaming loop at which the buffer holds more than FORCE entries: compact it by
// the histogram's threshold and, if that does not free it (values tied in their thousands, bins
// too coarse for this row), cut it exactly and lay the bins over what is left.  Every warp is
// between two regions here, so every buffered entry has a lower index than every column still to
// come, and a column that only EQUALS the k-th key of an exact cut can no longer enter: the
// threshold becomes the next key above it.  Returns true if the buffer has overflowed.
template <class S>
__device__ __noinline__ bool forced_cut(int tid) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + S::CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
    if (hist_compact<S>(buf, ctl, hist, tid, true)) return true;
    if (live_count(ctl) <= S::FORCE) return false;
    bool have;
    if (tid == 0) ctl->kmax = 0u;
    const uint32_t kth = refresh_topk<S, true>(buf, ctl, hist, ctl->k, tid, &have);
    const int left = live_count(ctl);
    uint32_t top_key = 0u;
    for (int i = tid; i < left; i += S::NT) top_key = max(top_key, buf[i].key);
    atomicMax(&ctl->kmax, top_key);
    __syncthreads();
    if (tid == 0 && have) {
        // the bins now span what the cut left: its k-th value to its largest
        // thr_key is also what a later compaction keeps entries by: it stays at the k-th key, which
        // the cut's own ties carry; only the admission threshold moves past it
        const uint32_t keep = max(ctl->thr_key, kth);
        ctl->thr_key = keep;
        ctl->thr = key2f(max(keep, kth + 1u));
        const float base = key2f(kth), top = key2f(ctl->kmax);
        const bool ok = top > base && top - base < 3.0e38f;
        ctl->hbase = base;
        ctl->htop = top;
        ctl->hscale = ok ? (float)HBINS / (top - base) : 0.0f;
        ctl->hwidth = ok ? (top - base) / (float)HBINS : 0.0f;
    }
    __syncthreads();
    hist_rebuild<S>(buf, ctl, hist, live_count(ctl), tid);
    return false;
}

// Bitonic sort of the first n entries of the buffer into the shortlist order, in place; the
// buffer has room for the next power of two (n <= CAP / 2).
template <class S>
__device__ void sort_buf(Cand* buf, int n, int tid) {
    int n2 = 32;
    while (n2 < n) n2 <<= 1;
    Cand last;  // behind every real entry
    last.key = 0u;
    last.idx = 0xffffffffu;
    for (int i = n + tid; i < n2; i += S::NT) buf[i] = last;
    __syncthreads();
    for (int kk = 2; kk <= n2; kk <<= 1) {
        for (int jj = kk >> 1; jj > 0; jj >>= 1) {
            for (int i = tid; i < n2; i += S::NT) {
                const int ixj = i ^ jj;
                if (ixj > i) {
                    const Cand x0 = buf[i], x1 = buf[ixj];
                    const bool up = (i & kk) == 0;  // this pair is put into shortlist order
                    if (up ? cand_before(x1, x0) : cand_before(x0, x1)) {
                        buf[i] = x1;
                        buf[ixj] = x0;
                    }
                }
            }
            __syncthreads();
        }
    }
}

// Orders the n entries of the buffer (key descending, index ascending) by counting, into
// sval/sidx.  Entries are distinct under that order, so ranks are a permutation.  One independent
// read per entry and thread: n * n / NT steps, the shorter chain up to a few hundred entries.
template <class S>
__device__ void rank_sort(const Cand* buf, int n, float* sval, int32_t* sidx, int tid) {
    for (int i = tid; i < n; i += S::NT) {
        Cand me = buf[i];
        int rank = 0;
        for (int j = 0; j < n; j++) {
            const Cand o = buf[j];
            rank += cand_before(o, me) ? 1 : 0;
        }
        sval[rank] = key2f(me.key);
        sidx[rank] = (int32_t)me.idx;
    }
}

// (Measured and not kept for the cuts of the streaming loop: ranking only the newcomers of a cut
// against the ordered prefix the previous cut left -- by binary search, or with a histogram of
// their positions -- takes a third of the counting select's instructions and was 10 to 25 %
// slower at every shortlist length: a CTA streams nothing while it cuts, so what counts is the
// cut's longest dependent chain, and the counting select's is one independent read per entry.)

}  // namespace
