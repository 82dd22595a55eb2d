/*
 * CPU oracle for the logits sampling path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference sampler, internal/logits/sampler.go, written
 * to be the checker the CUDA path is compared with.  Only the test-suite, the smoke
 * check and the benchmark's CPU-baseline legs load it; nothing in the shipped library
 * calls it or falls back to it.
 *
 * Arithmetic contract (must hold for bit-exact token ids):
 *   - fast_exp is evaluated in float32, left to right, every multiply and add rounded
 *     separately; build with -ffp-contract=off so the compiler fuses nothing
 *     (sampler.go:10-31; the reference's Go build for amd64 does not fuse either).
 *   - probabilities, their sums and the running CDF are IEEE doubles accumulated in
 *     shortlist order (sampler.go:165-177, 214-231).
 *   - the nucleus test is made on the double prefix rounded to float32 (sampler.go:217).
 *
 * Pinning: checked against every expected value the reference's own tests hold
 * (internal/logits/sampler_test.go:20-58: greedy -> 3, temperature 0 -> 3, top-p on
 * {10,0,0,0,0} -> 0 for every draw; the determinism test pins no value).  The mapping
 * seed -> uniform draw belongs to Go's math/rand, which is not part of the reference
 * tree and is pinned by none of its tests; here the uniform is an input.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <stdatomic.h>
#include <unistd.h>

#include "../include/mantle_sample_params.h"

/* sampler.go:10-31 */
float mantle_oracle_fast_exp(float x) {
    if (x > 88.0f) return 3.4028235e38f;
    if (x < -88.0f) return 0.0f;
    const float ln2 = 0.693147180559945309417f;
    const float ln2inv = 1.44269504088896340736f;
    int32_t k = (int32_t)(x * ln2inv + 0.5f);
    if (x < 0) k = (int32_t)(x * ln2inv - 0.5f);
    float r = x - (float)k * ln2;
    float r2 = r * r;
    float r3 = r2 * r;
    float r4 = r2 * r2;
    float poly = 1.0f + r + r2 * 0.5f + r3 * 0.16666667f + r4 * 0.041666667f + (r4 * r) * 0.008333333f;
    uint32_t bits = (uint32_t)(k + 127) << 23;
    float scale;
    memcpy(&scale, &bits, sizeof scale);
    return poly * scale;
}

/* internal/backend/simd/ops.go:165-175 -- fastTanh, built on the same fastExp
 * (simd/ops.go:111-150 is a copy of sampler.go:10-31). */
float mantle_oracle_fast_tanh(float x) {
    if (x > 10.0f) return 1.0f;
    if (x < -10.0f) return -1.0f;
    float e2x = mantle_oracle_fast_exp(2.0f * x);
    return (e2x - 1.0f) / (e2x + 1.0f);
}

/* internal/backend/simd/runtime.go:258-272 -- what the model head does to the logits before
 * they reach the sampler, in place: the LMHeadMultiplier loop (when the multiplier is
 * neither 0 nor 1), then the FinalLogitSoftcap loop of the host path (when the cap is
 * positive).  Pinned only loosely by the reference's tests: the cap is the identity when it
 * is not positive and damps large logits (internal/backend/cuda/graph_test.go:255-263). */
void mantle_oracle_postprocess(float *logits, int64_t n, float scale, float softcap) {
    if (scale != 0.0f && scale != 1.0f)
        for (int64_t i = 0; i < n; i++) logits[i] *= scale;
    if (softcap > 0.0f)
        for (int64_t i = 0; i < n; i++) logits[i] = mantle_oracle_fast_tanh(logits[i] / softcap) * softcap;
}

/* sampler.go:61-83 -- NewSampler's normalisation; the seed stays with the host RNG. */
void mantle_oracle_normalize_config(const MantleSamplerConfig *cfg, MantleSampleParams *out) {
    memset(out, 0, sizeof *out);
    out->greedy = cfg->temperature <= 0 ? 1 : 0;
    out->temperature = cfg->temperature <= 0 ? 1.0f : cfg->temperature;
    out->top_k = cfg->top_k <= 0 ? 40 : cfg->top_k;
    out->top_p = (cfg->top_p <= 0 || cfg->top_p > 1) ? 1.0f : cfg->top_p;
    out->min_p = cfg->min_p;
    out->repeat_penalty = cfg->repeat_penalty <= 0 ? 1.0f : cfg->repeat_penalty;
    out->repeat_last_n = cfg->repeat_last_n <= 0 ? 64 : cfg->repeat_last_n;
}

/* sampler.go:56-58 */
int mantle_oracle_can_use_device_greedy(const MantleSampleParams *p) {
    return p->greedy && p->repeat_penalty <= 1.0f;
}

/* sampler.go:99-138.  `mark` is a caller-owned scratch of V bytes, all zero on entry
 * and on return (the reference's epoch-stamped seenMark, restated with explicit clears). */
void mantle_oracle_apply_penalty(float *logits, int V, const int32_t *recent, int n_recent,
                                 const int32_t *exclude, int n_exclude, float penalty,
                                 int repeat_last_n, uint8_t *mark) {
    if (!(penalty > 1.0f) || n_recent <= 0) return;
    int start = n_recent - repeat_last_n;
    if (start < 0) start = 0;
    int n = n_recent - start;
    const int32_t *window = recent + start;
    int32_t *seen = (int32_t *)malloc(sizeof(int32_t) * (size_t)(n > 0 ? n : 1));
    int n_seen = 0;
    for (int i = 0; i < n; i++) {
        int32_t id = window[i];
        if (id >= 0 && id < V && !mark[id]) {
            mark[id] = 1;
            seen[n_seen++] = id;
        }
    }
    for (int i = 0; i < n_exclude; i++) {
        int32_t id = exclude[i];
        if (id >= 0 && id < V) mark[id] = 0;
    }
    for (int i = 0; i < n_seen; i++) {
        int32_t id = seen[i];
        if (!mark[id]) continue;
        if (logits[id] > 0)
            logits[id] /= penalty;
        else
            logits[id] *= penalty;
        mark[id] = 0;
    }
    free(seen);
}

/* sampler.go:237-250 */
int mantle_oracle_argmax(const float *x, int n) {
    int best_i = 0;
    float best_v = x[0];
    for (int i = 1; i < n; i++) {
        if (x[i] > best_v) {
            best_v = x[i];
            best_i = i;
        }
    }
    return best_i;
}

/* sampler.go:255-296 -- the insertion shortlist, O(V*k).  Returns the shortlist length. */
int mantle_oracle_topk_insertion(const float *logits, int V, int k, float inv_temp,
                                 int32_t *top_idx, float *top_val) {
    if (k <= 0) return 0;
    int len = 0;
    for (int i = 0; i < V; i++) {
        float v = logits[i] * inv_temp;
        int pos = len;
        while (pos > 0 && top_val[pos - 1] < v) pos--;
        if (pos >= k) continue;
        int newlen = len < k ? len + 1 : k;
        /* shift [pos, newlen-1) one place right; the element at k falls off */
        for (int j = newlen - 1; j > pos; j--) {
            top_idx[j] = top_idx[j - 1];
            top_val[j] = top_val[j - 1];
        }
        top_idx[pos] = i;
        top_val[pos] = v;
        len = newlen;
    }
    if (len == 0) { /* sampler.go:290-292: empty input */
        top_idx[0] = 0;
        top_val[0] = 0;
        return 1;
    }
    return len;
}

typedef struct {
    float v;
    int32_t i;
} oracle_pair;

static int pair_cmp(const void *pa, const void *pb) {
    const oracle_pair *a = (const oracle_pair *)pa, *b = (const oracle_pair *)pb;
    if (a->v > b->v) return -1;
    if (a->v < b->v) return 1;
    return a->i < b->i ? -1 : (a->i > b->i ? 1 : 0);
}

/* The same shortlist as the insertion loop, obtained by a full ordering: value
 * descending, ties by ascending index (an equal value never displaces an earlier one,
 * sampler.go:268-275).  Used where k is so large that O(V*k) is impractical; the tests
 * prove it equal to the insertion loop on small inputs.  Inputs hold no NaN. */
int mantle_oracle_topk_sorted(const float *logits, int V, int k, float inv_temp,
                              int32_t *top_idx, float *top_val) {
    if (k <= 0) return 0;
    if (V == 0) {
        top_idx[0] = 0;
        top_val[0] = 0;
        return 1;
    }
    oracle_pair *p = (oracle_pair *)malloc(sizeof(oracle_pair) * (size_t)V);
    for (int i = 0; i < V; i++) {
        p[i].v = logits[i] * inv_temp;
        p[i].i = i;
    }
    qsort(p, (size_t)V, sizeof(oracle_pair), pair_cmp);
    int len = k < V ? k : V;
    for (int i = 0; i < len; i++) {
        top_idx[i] = p[i].i;
        top_val[i] = p[i].v;
    }
    free(p);
    return len;
}

#define ORACLE_SORT_THRESHOLD 2048

/* Everything after the shortlist: sampler.go:154-233.  top_idx/top_val hold `len`
 * entries; prob has room for `len` doubles.  Writes the post-min-p shortlist length to
 * *n_kept, the nucleus length to *cut, the softmax normaliser (`sum`, sampler.go:165-168) to
 * *sum_out and the probability the returned token carries in prob[] to *token_prob (any of
 * them may be NULL). */
int mantle_oracle_tail(int32_t *top_idx, const float *top_val, int len, double *prob,
                       float top_p, float min_p, double r, int *n_kept, int *cut_out,
                       double *sum_out, double *token_prob) {
    float maxv = top_val[0];
    for (int i = 1; i < len; i++)
        if (top_val[i] > maxv) maxv = top_val[i];
    double sum = 0;
    for (int i = 0; i < len; i++) {
        double e = (double)mantle_oracle_fast_exp(top_val[i] - maxv);
        prob[i] = e;
        sum += e;
    }
    if (sum_out) *sum_out = sum;
    if (token_prob) *token_prob = 0;
    if (sum == 0) {
        if (n_kept) *n_kept = len;
        if (cut_out) *cut_out = 0;
        return top_idx[0];
    }
    double inv_sum = 1.0 / sum;
    for (int i = 0; i < len; i++) prob[i] *= inv_sum;

    int n = len;
    if (min_p > 0) {
        double threshold = prob[0] * (double)min_p;
        int new_len = 0;
        double new_sum = 0;
        for (int i = 0; i < n; i++) {
            if (prob[i] >= threshold) {
                prob[new_len] = prob[i];
                top_idx[new_len] = top_idx[i];
                new_sum += prob[i];
                new_len++;
            }
        }
        if (new_len < n) {
            n = new_len;
            if (new_sum > 0) {
                double scale = 1.0 / new_sum;
                for (int i = 0; i < n; i++) prob[i] *= scale;
            }
        }
    }
    int cut = n;
    if (top_p < 1) {
        double c = 0;
        for (int i = 0; i < n; i++) {
            c += prob[i];
            if ((float)c >= top_p) {
                cut = i + 1;
                break;
            }
        }
    }
    if (n_kept) *n_kept = n;
    if (cut_out) *cut_out = cut;
    double c = 0;
    for (int i = 0; i < cut; i++) {
        c += prob[i];
        if (r <= c) {
            if (token_prob) *token_prob = prob[i];
            return top_idx[i];
        }
    }
    if (token_prob) *token_prob = prob[cut - 1];
    return top_idx[cut - 1];
}

/*
 * One call of Sampler.Sample (sampler.go:98-234) on one row.
 *   logits       V floats, patched in place by the penalty exactly as the reference does
 *   recent       the token history (the reference's `recent`), n_recent ids
 *   exclude      the reference's `excludePenalty` (stop tokens)
 *   cand_idx / cand_prob   optional, cand_cap entries each: the shortlist after min-p,
 *                in order, with its (renormalised) probabilities
 *   n_kept / cut optional: shortlist length after min-p; nucleus length after top-p
 *   use_sort     0: the reference's insertion loop; 1: the equivalent full ordering;
 *                -1: insertion for k <= ORACLE_SORT_THRESHOLD, the ordering above it
 *   softmax_sum / token_prob   optional: the softmax normaliser and the probability of the
 *                returned token (after the min-p renormalisation)
 * Greedy rows write n_kept = cut = 0 and softmax_sum = token_prob = 0.  V must be > 0.
 */
int mantle_oracle_sample_row(float *logits, int V, const int32_t *recent, int n_recent,
                             const int32_t *exclude, int n_exclude, const MantleSampleParams *p,
                             int32_t *cand_idx, double *cand_prob, int cand_cap, int *n_kept,
                             int *cut, int use_sort, double *softmax_sum, double *token_prob) {
    if (p->repeat_penalty > 1.0f && n_recent > 0) {
        uint8_t *mark = (uint8_t *)calloc((size_t)V, 1);
        mantle_oracle_apply_penalty(logits, V, recent, n_recent, exclude, n_exclude,
                                    p->repeat_penalty, p->repeat_last_n, mark);
        free(mark);
    }
    if (n_kept) *n_kept = 0;
    if (cut) *cut = 0;
    if (softmax_sum) *softmax_sum = 0;
    if (token_prob) *token_prob = 0;
    if (p->greedy || (p->top_k == 1 && p->top_p >= 1 && p->temperature == 1))
        return mantle_oracle_argmax(logits, V);

    float inv_temp = 1.0f / p->temperature;
    int k = p->top_k < V ? p->top_k : V;
    int32_t *top_idx = (int32_t *)malloc(sizeof(int32_t) * (size_t)(k + 1));
    float *top_val = (float *)malloc(sizeof(float) * (size_t)(k + 1));
    double *prob = (double *)malloc(sizeof(double) * (size_t)(k + 1));
    int sorted = use_sort < 0 ? (k > ORACLE_SORT_THRESHOLD) : use_sort;
    int len = sorted ? mantle_oracle_topk_sorted(logits, V, k, inv_temp, top_idx, top_val)
                     : mantle_oracle_topk_insertion(logits, V, k, inv_temp, top_idx, top_val);
    int token;
    if (len == 0) {
        token = 0;
    } else {
        int nk = 0, ct = 0;
        token = mantle_oracle_tail(top_idx, top_val, len, prob, p->top_p, p->min_p, p->uniform, &nk, &ct,
                                   softmax_sum, token_prob);
        if (n_kept) *n_kept = nk;
        if (cut) *cut = ct;
        int m = nk < cand_cap ? nk : cand_cap;
        if (cand_idx) memcpy(cand_idx, top_idx, sizeof(int32_t) * (size_t)m);
        if (cand_prob) memcpy(cand_prob, prob, sizeof(double) * (size_t)m);
    }
    free(top_idx);
    free(top_val);
    free(prob);
    return token;
}

static float bf16_to_f32(uint16_t h) {
    uint32_t b = (uint32_t)h << 16;
    float f;
    memcpy(&f, &b, sizeof f);
    return f;
}

typedef struct {
    void *logits;
    int dtype, rows, V;
    int64_t row_stride;
    const int32_t *history;
    int hist_stride;
    const int32_t *hist_len, *exclude;
    int n_exclude;
    const MantleSampleParams *params;
    int32_t *next, *cand_idx;
    double *cand_prob;
    int cand_stride;
    int32_t *n_kept, *cut;
    int use_sort;
    double *softmax_sum, *token_prob;
    atomic_int next_row;
} oracle_job;

static void oracle_one_row(oracle_job *j, int r) {
    float *row;
    float *tmp = NULL;
    if (j->dtype == 0) {
        row = (float *)j->logits + (size_t)r * (size_t)j->row_stride;
    } else {
        const uint16_t *src = (const uint16_t *)j->logits + (size_t)r * (size_t)j->row_stride;
        tmp = (float *)malloc(sizeof(float) * (size_t)j->V);
        for (int i = 0; i < j->V; i++) tmp[i] = bf16_to_f32(src[i]);
        row = tmp;
    }
    int hl = j->hist_len ? j->hist_len[r] : j->hist_stride;
    const int32_t *h = j->history ? j->history + (size_t)r * (size_t)j->hist_stride : NULL;
    if (!h) hl = 0;
    int nk = 0, ct = 0;
    j->next[r] = mantle_oracle_sample_row(
        row, j->V, h, hl, j->exclude, j->n_exclude, &j->params[r],
        j->cand_idx ? j->cand_idx + (size_t)r * (size_t)j->cand_stride : NULL,
        j->cand_prob ? j->cand_prob + (size_t)r * (size_t)j->cand_stride : NULL, j->cand_stride,
        &nk, &ct, j->use_sort, j->softmax_sum ? j->softmax_sum + r : NULL,
        j->token_prob ? j->token_prob + r : NULL);
    if (j->n_kept) j->n_kept[r] = nk;
    if (j->cut) j->cut[r] = ct;
    free(tmp);
}

static void *oracle_worker(void *arg) {
    oracle_job *j = (oracle_job *)arg;
    for (;;) {
        int r = atomic_fetch_add(&j->next_row, 1);
        if (r >= j->rows) break;
        oracle_one_row(j, r);
    }
    return NULL;
}

int mantle_oracle_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/*
 * Batch driver: rows are independent, one sampler state per row, handed out one at a
 * time to `threads` POSIX threads (<= 0: one per online core).  Layout matches the CUDA
 * C-ABI: logits[row * row_stride + i]; history[row * hist_stride + j] with
 * hist_len[row] valid ids (NULL: hist_stride); one exclude list for the batch.
 * dtype 0: float32 logits, patched in place; dtype 1: bfloat16 logits, widened exactly
 * to float32 in a private copy (the input is left untouched).
 * softmax_sum / token_prob: optional [rows] doubles, see mantle_oracle_sample_row.
 * Returns the number of threads used.
 */
int mantle_oracle_sample_rows(void *logits, int dtype, int rows, int V, int64_t row_stride,
                              const int32_t *history, int hist_stride, const int32_t *hist_len,
                              const int32_t *exclude, int n_exclude,
                              const MantleSampleParams *params, int32_t *next,
                              int32_t *cand_idx, double *cand_prob, int cand_stride,
                              int32_t *n_kept, int32_t *cut, int use_sort, int threads,
                              double *softmax_sum, double *token_prob) {
    oracle_job j = {logits, dtype, rows, V, row_stride, history, hist_stride, hist_len, exclude,
                    n_exclude, params, next, cand_idx, cand_prob, cand_stride, n_kept, cut,
                    use_sort, softmax_sum, token_prob, 0};
    if (threads <= 0) threads = mantle_oracle_max_threads();
    if (threads > rows) threads = rows > 0 ? rows : 1;
    if (threads <= 1) {
        oracle_worker(&j);
        return 1;
    }
    pthread_t *t = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    int started = 0;
    for (int i = 0; i < threads; i++)
        if (pthread_create(&t[started], NULL, oracle_worker, &j) == 0) started++;
    if (started == 0) oracle_worker(&j);
    for (int i = 0; i < started; i++) pthread_join(t[i], NULL);
    free(t);
    return started > 0 ? started : 1;
}
