/*
 * C-ABI of the device-side logits sampler (sm_100a).
 *
 * These are the symbols a cgo file under internal/backend/cuda/native binds, next to
 * the reference's own wrappers.  They follow that package's conventions
 * (internal/backend/cuda/native/softmax.h:1-115, softmax.cu:972-988, 1151-1160):
 * `extern "C" int mantleCudaXxx(..., cudaStream_t stream)` returning a cudaError_t as
 * int, 0 on success, cudaErrorInvalidValue (1) for bad arguments; work is queued on
 * `stream` and the call returns without synchronising.  Unlike the reference's
 * ArgMaxF32 (native/argmax.go:32-53) nothing here allocates, frees or copies to the
 * host behind the caller's back: every buffer, the workspace included, is the caller's.
 * The current device must be the one that owns the buffers.
 *
 * What the kernels compute is Sampler.Sample of internal/logits/sampler.go:98-234 for
 * every row of a batch: repeat penalty over the de-duplicated history window, the
 * greedy test and lowest-index argmax, temperature scaling, the top-k shortlist
 * (value descending, ties by ascending index), fastExp softmax over the shortlist in
 * float32 with double sums, min-p, the top-p cut and the inverse-CDF draw from a
 * host-supplied uniform.
 *
 * What "equal to the reference" means.  For batches whose max_top_k is at most
 * MANTLE_SAMPLE_MAX_TOP_K every double is the reference's double (same operations, same
 * order): token ids, shortlists, lengths and probabilities are bit-equal.  Batches with a
 * larger max_top_k (up to the whole vocabulary) never materialise the shortlist; their sums
 * are taken in a different association than the reference's shortlist order, so a prefix
 * sum can differ from the reference's in its last bits (about 1e-16 relative).  There the
 * token, n_kept and cut can differ from the reference's only when the uniform or top_p lies
 * that close to a boundary of the cumulative distribution -- far inside the 1e-6 the
 * sampling contract allows -- token_prob and softmax_sum hold to 1e-5 relative (in practice
 * 1e-15), and cand_idx / cand_prob are not available.
 *
 * NaN logits are outside the contract (the reference's own result depends on where in the row
 * they sit).  Here a NaN is never admitted to a shortlist; a row with no other value returns
 * token 0 and raises MANTLE_SAMPLE_STATUS_NAN.  So is a row whose shortlist holds nothing but
 * -inf (a fully masked row) or whose largest value is +inf: the reference's softmax shifts by the
 * maximum, inf - inf is NaN, and every probability with it.  Such a row returns one of its shortlist's
 * ids, or -1 with MANTLE_SAMPLE_STATUS_EMPTY when min_p is set (no probability reaches a NaN threshold).
 *
 * The library keeps a little per-device state (device attributes, kernel attributes, the
 * address of the static scratch): it must not be used across a cudaDeviceReset.
 */
#ifndef MANTLE_CUDA_SAMPLER_H
#define MANTLE_CUDA_SAMPLER_H

#include <stddef.h>
#include <stdint.h>

#include "mantle_sample_params.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef MANTLE_CUDA_STREAM_T
#define MANTLE_CUDA_STREAM_T
typedef void* mantleCudaStream_t; /* a cudaStream_t, as in native/softmax.h:11 */
#endif

#define MANTLE_DTYPE_F32 0
#define MANTLE_DTYPE_BF16 1

/* Largest top_k the streaming shortlist kernels take.  The reference's shortlist loop is
 * O(V*k) and meant for small k (sampler.go:252-254); its default is 40.  Batches with a
 * larger max_top_k (up to the vocabulary: the reference's whole-vocabulary nucleus,
 * TopK >= V) run on a slower kernel that never materialises the shortlist. */
#define MANTLE_SAMPLE_MAX_TOP_K 1024
/* Largest vocabulary (per GPU) the kernels take: the penalty bitmap of V bits lives
 * in shared memory beside the candidate buffer. */
#define MANTLE_SAMPLE_MAX_VOCAB 1048576

/* flags */
/* Store the penalised logits back, as the reference does to the caller's slice
 * (sampler.go:132-136).  Without it the logits are read-only and the penalty is
 * applied on the fly while the row streams past.  float32 logits only. */
#define MANTLE_SAMPLE_WRITE_BACK_PENALTY 1u
/* The history is ignored: mantleCudaRepeatPenaltyRowsF32 already ran on these logits. */
#define MANTLE_SAMPLE_PENALTY_PREAPPLIED 2u

/* The soft cap uses tanhf, as the reference's device kernel does (native/softmax.cu:963-970),
 * instead of the host path's fastTanh (simd/ops.go:165-175), which is the default because a
 * CPU can reproduce it bit for bit. */
#define MANTLE_SAMPLE_SOFTCAP_TANHF 4u

/* bits of the optional device status word (OR-ed in by the kernels; never cleared) */
#define MANTLE_SAMPLE_STATUS_TOPK_RANGE 1  /* a row's top_k exceeded max_top_k          */
#define MANTLE_SAMPLE_STATUS_EMPTY 2       /* a row ended with an empty shortlist (the  */
                                           /* reference panics there); its token is -1  */
#define MANTLE_SAMPLE_STATUS_TIMEOUT 4     /* a bounded wait ran out (only the self-test  */
                                           /* raises it: no sampling kernel waits)        */
#define MANTLE_SAMPLE_STATUS_NAN 8         /* a row held nothing but NaN; its token is 0  */

/*
 * One batch of rows.  All pointers are device pointers on the current device.
 *
 *   logits      [rows][row_stride] elements of `dtype`; row r starts at r*row_stride;
 *               only the first `vocab` elements of a row are read
 *   history     [rows][hist_stride] int32 token ids, oldest first (the reference's
 *               `recent`); may be NULL (no penalty).  hist_len[r] <= hist_stride ids are
 *               valid; NULL means hist_stride for every row.  The window is the last
 *               params[r].repeat_last_n of them (sampler.go:100-101)
 *   exclude     n_exclude ids never penalised (the reference's excludePenalty: the stop
 *               tokens, engine.go:233); one list for the batch; may be NULL
 *   params      [rows] normalised per-row parameters
 *   next        [rows] out: the sampled token id of each row
 *   cand_idx, cand_prob  optional out, [rows][cand_stride]: the shortlist after min-p,
 *               in order, and its probabilities (double, as the reference holds them);
 *               at most cand_stride entries per row are written
 *   n_kept, cut optional out, [rows]: shortlist length after min-p and nucleus length
 *               after top-p; both 0 on greedy rows
 *   token_prob, softmax_sum  optional out, [rows] doubles: the probability the sampled token
 *               carries in the reference's prob[] (after the min-p renormalisation, before any
 *               top-p cut: sampler.go:176, 205) and the softmax normaliser `sum`
 *               (sampler.go:165-168); both 0 on greedy rows
 *   skip        optional, [rows] int32: a row whose entry is not 0 is not sampled (a request of
 *               a batched decode loop that has already ended); its token is -1, its other
 *               outputs 0, and nothing of its logits or history is read
 *   status      optional out: one int32 the kernels OR status bits into
 *   max_top_k   an upper bound of min(params[r].top_k, vocab) over the batch; sizes the
 *               workspace.  Above MANTLE_SAMPLE_MAX_TOP_K the whole batch takes the
 *               long-shortlist kernel: cand_idx/cand_prob must then be NULL
 *   splits      CTAs per row: 0 lets the library choose (1 for batches that fill the
 *               GPU, more for small batches); > 1 needs the workspace
 *   logit_scale, logit_softcap   the model head's post-processing, applied on the fly to every
 *               logit before the sampler sees it and gated as the reference gates it
 *               (simd/runtime.go:258-272): l *= logit_scale when it is neither 0 nor 1
 *               (LMHeadMultiplier), then l = tanh(l / logit_softcap) * logit_softcap when
 *               logit_softcap > 0 (FinalLogitSoftcap).  The logits themselves stay as they
 *               are, so neither penalty flag may be set with it.  A negative multiplier is
 *               refused.  Zero in both fields: no post-processing
 */
typedef struct MantleSampleBatch {
    const void* logits;
    int32_t dtype;
    int32_t rows;
    int32_t vocab;
    int32_t max_top_k;
    int64_t row_stride;
    const int32_t* history;
    const int32_t* hist_len;
    int32_t hist_stride;
    int32_t n_exclude;
    const int32_t* exclude;
    const MantleSampleParams* params;
    int32_t* next;
    int32_t* cand_idx;
    double* cand_prob;
    int32_t* n_kept;
    int32_t* cut;
    int32_t* status;
    int32_t cand_stride;
    int32_t splits;
    uint32_t flags;
    uint32_t reserved;
    float logit_scale;
    float logit_softcap;
    double* token_prob;
    double* softmax_sum;
    const int32_t* skip;
} MantleSampleBatch;

/*
 * Sampler.Sample for every row (replaces internal/logits/sampler.go:98-234, called from
 * internal/inference/engine.go:233,279,296).  `workspace` may be NULL when the batch
 * runs with one CTA per row; mantleCudaSamplerWorkspaceBytes says how much a batch needs.
 */
int mantleCudaSampleRows(const MantleSampleBatch* batch, void* workspace, size_t workspace_bytes,
                         mantleCudaStream_t stream);

/* Bytes of workspace mantleCudaSampleRows needs for this batch (0 when none). */
int mantleCudaSamplerWorkspaceBytes(const MantleSampleBatch* batch, size_t* bytes);

/* The number of CTAs per row mantleCudaSampleRows will use for this batch. */
int mantleCudaSamplerSplits(const MantleSampleBatch* batch, int* splits);

/* Name of the kernel that reads this batch's logits (for profiles and benchmark records; ""
 * for a descriptor mantleCudaSampleRows would refuse).  No counterpart in the reference. */
const char* mantleCudaSamplerKernelName(const MantleSampleBatch* batch);

/*
 * The repeat penalty alone, in place, one scatter over the de-duplicated history
 * window of each row (sampler.go:99-138).  Takes the same descriptor; reads logits
 * (float32), history, hist_len, exclude and params and writes only logits.
 */
int mantleCudaRepeatPenaltyRowsF32(const MantleSampleBatch* batch, mantleCudaStream_t stream);

/*
 * The model head's post-processing alone, in place over [rows][row_stride] float32 logits:
 * the multiplier loop and the soft cap of simd/runtime.go:258-272.  Replaces
 * mantleCudaLogitSoftcapF32 (native/softmax.cu:963-970, native/softmax.go:62-77), which
 * covers the cap only; `flags` takes MANTLE_SAMPLE_SOFTCAP_TANHF for that kernel's tanhf.
 * For callers that want the rewritten logits: mantleCudaSampleRows applies the same
 * arithmetic on the fly from the descriptor's logit_scale / logit_softcap and writes nothing.
 */
int mantleCudaLogitPostprocessRowsF32(float* logits, int rows, int vocab, int64_t row_stride,
                                      float logit_scale, float logit_softcap, uint32_t flags,
                                      mantleCudaStream_t stream);

/*
 * The decode loop's `toks = append(toks, next)` (internal/inference/engine.go:244-250) for a
 * batch whose histories stay on the device between steps, so that a step uploads no history:
 * history[r][hist_len[r]++] = next[r] for every row.  A row whose token is one of the `stop`
 * ids (the reference leaves its loop before appending a stop token) or negative is not
 * appended; it is marked in done[r] when `done` is given, and rows already marked are left
 * alone.  When a row's buffer is full its `keep` most recent ids move to the front first;
 * keep <= hist_stride / 2, and the penalty window stays exact while keep is at least the
 * largest repeat_last_n in use.  Queue it behind mantleCudaSampleRows on the same stream.
 */
int mantleCudaHistoryAppendRows(int32_t* history, int32_t* hist_len, int hist_stride, int rows,
                                const int32_t* next, int keep, const int32_t* stop, int n_stop,
                                int32_t* done, mantleCudaStream_t stream);

/*
 * Index of the maximum of each row, the lowest index on ties (argmax,
 * sampler.go:237-250).  Batched replacement for mantleCudaArgMaxF32
 * (native/softmax.cu:663-704,1151-1160), whose tie-break follows thread order.
 */
int mantleCudaArgMaxRowsF32(const float* x, int rows, int n, int64_t row_stride, int* out_idx,
                            mantleCudaStream_t stream);

/*
 * Vocabulary-sharded sampling, step 1: this GPU holds columns
 * [vocab_offset, vocab_offset + batch->vocab) of a vocab_total-wide row.  Applies the
 * penalty to the ids it owns, scales, and writes its local shortlist: for row r,
 * part_cnt[r] <= part_cap entries at part_val/part_idx[r*part_cap ...], value descending,
 * part_idx holding GLOBAL token ids.  history/exclude hold global ids.
 */
int mantleCudaSampleLocalTopK(const MantleSampleBatch* batch, int vocab_offset, int vocab_total,
                              float* part_val, int32_t* part_idx, int32_t* part_cnt, int part_cap,
                              mantleCudaStream_t stream);

/*
 * Vocabulary-sharded sampling, step 2 (after the caller's all-gather): merges `parts`
 * shortlists per row -- part p of row r at [(p*rows + r)*part_cap ...], its length at
 * part_cnt[p*rows + r] -- into the global shortlist and finishes the row (softmax,
 * min-p, top-p, draw).  Uses params, next and the optional outputs of `batch`;
 * parts * max_top_k must not exceed 4096.
 */
int mantleCudaSampleMergeParts(const MantleSampleBatch* batch, int parts, const float* part_val,
                               const int32_t* part_idx, const int32_t* part_cnt, int part_cap,
                               mantleCudaStream_t stream);

/*
 * The same merge for shortlists that travel as one block per rank, so that one all-gather
 * carries a step: a block is [rows * part_cap float values][rows * part_cap int32 ids]
 * [rows int32 counts], mantleCudaSamplePackedPartBytes() bytes long (padded to 256); `packed`
 * holds `parts` blocks in rank order.  A rank fills its block with
 * mantleCudaSampleLocalTopK(..., block, block + rows * part_cap, block + 2 * rows * part_cap, ...)
 * (pointers in 4-byte elements).
 */
int mantleCudaSamplePackedPartBytes(int rows, int part_cap, size_t* bytes);
int mantleCudaSampleMergePacked(const MantleSampleBatch* batch, int parts, const void* packed, int part_cap,
                                mantleCudaStream_t stream);

/*
 * Sampler.Sample for a batch that lives in HOST memory: the form of the reference's
 * call site, where the logits arrive as a host slice (internal/inference/engine.go:233,
 * 279, 296 pass `logitsVec []float32`).  Every pointer of `host_batch` (logits, history,
 * hist_len, exclude, params and all outputs) is a host pointer, pinned for the copies to
 * be asynchronous.  The call queues, on `stream`: the host-to-device copies of the inputs
 * into `device_workspace`, the same kernels as mantleCudaSampleRows, and the
 * device-to-host copies of next and of every optional output that is set.  With
 * MANTLE_SAMPLE_WRITE_BACK_PENALTY the penalised logits are copied back over the host
 * rows too, which is the reference's in-place side effect (sampler.go:132-136).
 * The caller synchronises `stream` before reading the outputs.
 */
int mantleCudaSampleRowsHost(const MantleSampleBatch* host_batch, void* device_workspace,
                             size_t workspace_bytes, mantleCudaStream_t stream);

/* Bytes of device workspace mantleCudaSampleRowsHost needs for this batch. */
int mantleCudaSamplerHostWorkspaceBytes(const MantleSampleBatch* host_batch, size_t* bytes);

/*
 * mantleCudaSampleRows for callers that cannot supply a workspace.  It has no counterpart in
 * the reference; it exists for hosts that must not allocate device memory where they sample
 * -- a runtime whose device-memory plan is frozen before the decode loop starts, an embedding
 * that keeps the allocator out of that loop -- and therefore have nowhere to take the split-row
 * scratch from.  The scratch is a fixed array of mantleCudaSamplerStaticScratchBytes() bytes
 * (4 MiB) inside the library image; every GPU that loads the library holds it until the
 * process exits.  Batches that need more (rows * splits * max_top_k * 8 bytes, plus counts) are
 * refused with cudaErrorInvalidValue and a message from mantleCudaSamplerLastError(); batches
 * that run one CTA per row need no scratch and always fit.  The call itself allocates and
 * frees nothing.  Its first call on a device looks the array's device address up
 * (cudaGetSymbolAddress, with that device current) and should therefore come before any
 * stream capture on that device.  All calls on a device share the one array, which keeps
 * whatever the last call left in it (each call overwrites every slot it reads): calls that
 * overlap on the GPU -- two streams, two host threads -- race on it and must be serialised
 * by the caller.
 */
int mantleCudaSampleRowsNoAlloc(const MantleSampleBatch* batch, mantleCudaStream_t stream);

/* Size of the static scratch behind mantleCudaSampleRowsNoAlloc. */
size_t mantleCudaSamplerStaticScratchBytes(void);

/* Text of the last refusal of mantleCudaSampleRowsNoAlloc on the calling thread ("" if none). */
const char* mantleCudaSamplerLastError(void);

/*
 * Failure-path self-test (no counterpart in the reference): launches a kernel that waits, with
 * the same bounded wait the bulk-copy ring uses, on a barrier nothing completes.  After
 * limit_ns (at most one second) the kernel sets MANTLE_SAMPLE_STATUS_TIMEOUT in *status_dev and
 * returns; the context stays usable.  Nothing faults, traps or spins without bound.
 */
int mantleCudaSamplerSelfTestBoundedWait(unsigned long long limit_ns, int32_t* status_dev,
                                         mantleCudaStream_t stream);

/* Library version, for the loader's sanity check. */
int mantleCudaSamplerAbiVersion(void);

#ifdef __cplusplus
}
#endif

#endif /* MANTLE_CUDA_SAMPLER_H */
