/*
 * The decode loop's sampling state for a whole batch of requests, on the device.
 *
 * The reference runs one request at a time (internal/api/engine_provider.go:56-71 holds one
 * engine behind a mutex) and its loop, Generator.RunWithContext
 * (internal/inference/engine.go:189, 233-300), is
 *
 *     toks := copy(ContextTokens)
 *     next := Sample(logits, toks, StopTokens)
 *     for {
 *         if next is a stop token { break }          // before the append
 *         toks = append(toks, next)
 *         logits = ForwardToken(next)
 *         next = Sample(logits, toks, StopTokens)
 *     }
 *
 * with a Sampler -- and its random generator -- made per request (engine_impl.go:133-158).
 * MantleBatchSampler is that loop's state for `rows` requests side by side: each row has its own
 * normalised configuration (NewSampler, sampler.go:61-83), its own token history on the device
 * and its own "has ended" flag.  One Step samples every live row from a [rows][row_stride]
 * matrix of device logits and appends each token to its row's history, all on the caller's
 * stream; per step the host sends one parameter record per row (which carries that row's
 * uniform draw) and reads back one token and one flag per row.
 *
 * The random generators stay with the caller, one per row as in the reference: a row consumes
 * exactly one uniform per step while it is live and does not end in argmax
 * (sampler.go:140-142, 224); mantleBatchSamplerNeedsUniform says which rows do.
 */
#ifndef MANTLE_BATCH_SAMPLER_H
#define MANTLE_BATCH_SAMPLER_H

#include <stdint.h>

#include "mantle_cuda_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MantleBatchSampler MantleBatchSampler;

/*
 * rows requests, logits rows of `vocab` columns, hist_capacity ids of history kept per row on
 * the device (at least twice the largest repeat_last_n that will be used: the penalty window
 * must survive the buffer wrapping), and the stop tokens shared by the batch (the reference's
 * StopTokens: never penalised, engine.go:233, and ending a row when sampled, engine.go:244).
 * Allocates all device and pinned memory here, on the current device.  NULL on failure.
 * Every row starts ended; mantleBatchSamplerSetRow starts one.
 */
MantleBatchSampler* mantleBatchSamplerNew(int rows, int vocab, int hist_capacity, const int64_t* stop, int n_stop);
void mantleBatchSamplerFree(MantleBatchSampler* s);

/*
 * Starts (or restarts) request `row`: NewSampler's normalisation of cfg and
 * toks := copy(ContextTokens) (the last hist_capacity ids are kept; ids are Go ints).
 * Synchronises `stream` before it returns (a request starts once; steps never synchronise).
 * cudaErrorInvalidValue when the normalised repeat_last_n exceeds hist_capacity / 2.
 */
int mantleBatchSamplerSetRow(MantleBatchSampler* s, int row, const MantleSamplerConfig* cfg, const int64_t* context,
                             int n_context, mantleCudaStream_t stream);

/* Ends request `row` without sampling a stop token (a length limit, a cancelled request). */
int mantleBatchSamplerEndRow(MantleBatchSampler* s, int row, mantleCudaStream_t stream);

/* 1 when the next Step consumes uniforms[row]: the row is live (as of the last results read)
 * and will not end in argmax.  The caller draws from that row's generator exactly then. */
int mantleBatchSamplerNeedsUniform(const MantleBatchSampler* s, int row);

/* Sampler.CanUseDeviceGreedy of one row (sampler.go:56-58). */
int mantleBatchSamplerCanUseDeviceGreedy(const MantleBatchSampler* s, int row);

/*
 * One step of the loop for every live row.  dev_logits: [rows][row_stride] elements of `dtype`
 * on the current device (the LM head's output, left untouched); uniforms: `rows` doubles on the
 * host, read before the call returns, entries of rows that need none ignored; logit_scale /
 * logit_softcap as in MantleSampleBatch.  Queues on `stream`: the parameter upload, the sampling
 * kernels, the append of every sampled token to its row's history (rows that drew a stop token
 * end instead), and the download of tokens and flags.  Returns without synchronising.
 */
int mantleBatchSamplerStep(MantleBatchSampler* s, const void* dev_logits, int dtype, int64_t row_stride,
                           const double* uniforms, float logit_scale, float logit_softcap, mantleCudaStream_t stream);

/*
 * The last step's results, valid once `stream` has been synchronised and until the next Step:
 * next[r] is the token row r sampled (-1 for a row that had already ended), ended[r] is 1 once
 * the row has sampled a stop token or was ended; status is the OR of the kernels' status bits
 * since the sampler was made.  The pointers are pinned host memory owned by the sampler.
 * dev_next is the same token array on the device, for a model that feeds from it directly.
 */
int mantleBatchSamplerResults(MantleBatchSampler* s, const int32_t** next, const int32_t** ended, int32_t* status,
                              const int32_t** dev_next);

#ifdef __cplusplus
}
#endif

#endif /* MANTLE_BATCH_SAMPLER_H */
