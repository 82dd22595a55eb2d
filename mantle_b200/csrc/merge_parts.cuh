// merge_parts_kernel: merges the local shortlists of a split row or of vocabulary shards.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// Merge of `parts` local shortlists per row (several CTAs of one GPU, or one per
// vocabulary shard after an all-gather), then the tail.  In the small shape (256 threads, four
// CTAs per SM) when parts * top_k fits its buffer, else in the large one.
// Launched behind the kernel that writes the parts, where possible as a programmatic dependent
// launch: everything above griddepcontrol.wait (parameters, the control block) runs while that
// kernel drains, and the wait returns once its writes are visible.  Without the launch attribute
// the wait is a no-op.
template <class S>
__global__ void __launch_bounds__(S::NT, S::MINB) merge_parts_kernel(const KArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Cand* buf = reinterpret_cast<Cand*>(smem_raw);
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + S::CAP);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + S::CTL_OFF);
    const int tid = threadIdx.x;
    const int row = blockIdx.x;

    if (a.skip && a.skip[row] != 0) {
        if (tid == 0) publish_row(a, row, -1);
        return;
    }
    const MantleSampleParams P = row_params(a, row);
    const bool greedy = P.greedy != 0 || (P.top_k == 1 && P.top_p >= 1.0f && P.temperature == 1.0f);
    int k = greedy ? 1 : min(P.top_k, a.vocab_total);
    const bool bad_k = !greedy && (k > a.max_top_k || k > KMAX || k < 1);

    if (tid == 0) ctl->cnt = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Every part is in order, so its j-th value is reached by j of its entries: with
    // j = ceil(k / parts) the smallest of the parts' j-th values is reached by at least k entries
    // overall and bounds the k-th largest from below.  Only entries that reach it are gathered --
    // about k of them instead of parts * k, which usually lets the cheap counting cut finish the job.
    float floor_v = __uint_as_float(0xff800000u);
    if (a.parts <= 128 && !bad_k) {
        // the parts' lengths and j-th values are fetched side by side, then every (part, entry) pair
        // is one independent load: a loop over the parts would pay one trip to memory per part
        float* part_floor = reinterpret_cast<float*>(hist);
        int* part_len = reinterpret_cast<int*>(hist + 128);
        const int j = (k + a.parts - 1) / a.parts;
        if (tid < a.parts) {
            const int m = min(a.part_cnt[(size_t)tid * (size_t)a.cnt_stride + row], a.part_cap);
            const size_t at = (size_t)tid * (size_t)a.part_stride + (size_t)row * a.part_cap;
            part_len[tid] = m;
            part_floor[tid] = m >= j ? a.part_val[at + j - 1] : __uint_as_float(0xff800000u);  // a short part: no bound
        }
        __syncthreads();
        floor_v = part_floor[0];
        for (int p = 1; p < a.parts; p++) floor_v = fminf(floor_v, part_floor[p]);
        if (!(floor_v == floor_v)) floor_v = __uint_as_float(0xff800000u);
        const int total = a.parts * a.part_cap;
        for (int t = tid; t < total; t += S::NT) {
            const int p = t / a.part_cap, e = t - p * a.part_cap;
            if (e < part_len[p]) {
                const size_t at = (size_t)p * (size_t)a.part_stride + (size_t)row * a.part_cap + e;
                const float v = a.part_val[at];
                if (v >= floor_v) append<S>(buf, ctl, v, a.part_idx[at]);
            }
        }
    } else {
        __syncthreads();
        for (int p = 0; p < a.parts; p++) {
            const size_t at = (size_t)p * (size_t)a.part_stride + (size_t)row * a.part_cap;
            const int m = min(a.part_cnt[(size_t)p * (size_t)a.cnt_stride + row], a.part_cap);
            for (int e = tid; e < m; e += S::NT) append<S>(buf, ctl, a.part_val[at + e], a.part_idx[at + e]);
        }
    }
    if (bad_k) {
        if (tid == 0) {
            if (a.status) atomicOr(a.status, MANTLE_SAMPLE_STATUS_TOPK_RANGE);
            publish_row(a, row, -1);
        }
        return;
    }
    bool have, ordered;
    refresh_topk<S>(buf, ctl, hist, k, tid, &have, &ordered);
    __syncthreads();
    finish_row<S, MODE_FUSED>(a, row, 0, P, greedy, ordered, buf, ctl, tid);
}

}  // namespace
