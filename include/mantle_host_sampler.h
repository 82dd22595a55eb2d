/*
 * Host-side sampler object: the C++ mirror of logits.Sampler (internal/logits/sampler.go:44-98)
 * on top of the CUDA C-ABI, written in C++ because no Go toolchain is at hand; the Go shim a
 * maintainer adds is a thin cgo wrapper over these calls.
 *
 *   mantleSamplerNew                = logits.NewSampler          (sampler.go:61-83)
 *   mantleSamplerCanUseDeviceGreedy = Sampler.CanUseDeviceGreedy (sampler.go:56-58)
 *   mantleSamplerSample             = Sampler.Sample             (sampler.go:98-234), host slice in
 *   mantleSamplerSampleDevice       = the same on logits that already live on the GPU, the
 *                                     hand-off the reference's device-greedy path uses
 *                                     (internal/backend/cuda/ops.go:1289-1346)
 *
 * The random generator stays with the caller: the reference draws rng.Float64() exactly once
 * per non-greedy Sample (sampler.go:224) and Go's math/rand is not part of the reference tree.
 * mantleSamplerNeedsUniform says whether the next call will consume a draw, so that the caller
 * draws under the same condition and its stream of draws stays aligned with the reference's.
 */
#ifndef MANTLE_HOST_SAMPLER_H
#define MANTLE_HOST_SAMPLER_H

#include <stdint.h>

#include "mantle_cuda_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MantleHostSampler MantleHostSampler;

/* NewSampler.  max_vocab bounds the logits length of later calls; the sampler allocates its
 * device workspace and pinned staging once, here.  Returns NULL on failure. */
MantleHostSampler* mantleSamplerNew(const MantleSamplerConfig* cfg, int max_vocab);
void mantleSamplerFree(MantleHostSampler* s);

/* The configuration after the constructor's normalisation (uniform left at 0). */
int mantleSamplerParams(const MantleHostSampler* s, MantleSampleParams* out);

int mantleSamplerCanUseDeviceGreedy(const MantleHostSampler* s);

/* 1 when Sample will take the stochastic path and consume `uniform`, 0 when it returns the argmax. */
int mantleSamplerNeedsUniform(const MantleHostSampler* s);

/*
 * Sampler.Sample(logits, recent, excludePenalty).  `logits` is a host slice of n floats and is
 * patched in place by the repeat penalty exactly as the reference patches it.  recent/exclude
 * are Go ints (64-bit).  Synchronous: returns a cudaError_t as int and the token in *token.
 * n == 0 returns cudaErrorInvalidValue (the reference panics on an empty slice, sampler.go:239).
 */
int mantleSamplerSample(MantleHostSampler* s, float* logits, int n, const int64_t* recent, int n_recent,
                        const int64_t* exclude, int n_exclude, double uniform, int* token);

/* The same for device-resident float32 logits (left untouched); queued on the sampler's stream
 * after `wait_stream`'s current work, then synchronised. */
int mantleSamplerSampleDevice(MantleHostSampler* s, const float* dev_logits, int n, const int64_t* recent,
                              int n_recent, const int64_t* exclude, int n_exclude, double uniform,
                              mantleCudaStream_t wait_stream, int* token);

#ifdef __cplusplus
}
#endif

#endif /* MANTLE_HOST_SAMPLER_H */
