// Everything after the shortlist (sampler.go:154-233): softmax with fastExp, min-p, top-p and
// the draw, CTA-wide and as a single warp; publishing a row or its local shortlist.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

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
            publish_row(a, row, 0);
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_NAN);
        }
        return;
    }
    if (greedy) {
        if (tid == 0) publish_row(a, row, sidx[0]);
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
        if (tid == 0) publish_row(a, row, sidx[0], n, 0);
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
        double tprob = 0.0;
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
            tprob = sprob[pos];
        }
        publish_row(a, row, token, n, cut, tprob, sum);
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
    double tprob = 0.0, sum_out = 0.0;
    if (n == 0) {
        token = 0;
        if (lane == 0 && a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_NAN);
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
        sum_out = sum;
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
                tprob = __shfl_sync(full, pos < 32 ? p0 : p1, pos & 31);
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
    if (lane == 0) publish_row(a, row, token, n_kept, cut, tprob, sum_out);
}

// After the final cut: order the survivors where the cut did not (`ordered`: it did) and either
// finish the row or publish the local shortlist.  The value / id / probability arrays live in the
// part of the candidate buffer the shortlist (at most KCAP entries) does not occupy.
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
    if (!ordered && n > 512) {  // counting would take n * n / NT steps: sort in place instead
        sort_buf<S>(buf, n, tid);
        ordered = true;
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

}  // namespace
