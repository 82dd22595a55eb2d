/*
 * Per-row sampling parameters shared by the CUDA C-ABI and the CPU oracle.
 *
 * One record describes one row of a batch.  It carries the values the reference
 * sampler holds AFTER its constructor has normalised them
 * (internal/logits/sampler.go:61-83): temperature > 0, top_k >= 1, top_p in (0,1],
 * repeat_penalty > 0, repeat_last_n >= 1, and `greedy` set when the configured
 * temperature was <= 0.  The uniform draw `uniform` in [0,1) is supplied by the host,
 * which keeps the reference's random generator (sampler.go:224); it is read only on
 * the non-greedy path.
 */
#ifndef MANTLE_SAMPLE_PARAMS_H
#define MANTLE_SAMPLE_PARAMS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MantleSampleParams {
    float temperature;     /* SamplerConfig.Temperature after normalisation (> 0)          */
    float top_p;           /* SamplerConfig.TopP after normalisation, (0, 1]                */
    float min_p;           /* SamplerConfig.MinP; the filter runs iff > 0                   */
    float repeat_penalty;  /* SamplerConfig.RepeatPenalty; the penalty runs iff > 1.0       */
    int32_t top_k;         /* SamplerConfig.TopK after normalisation (>= 1); clamped to V   */
    int32_t repeat_last_n; /* SamplerConfig.RepeatLastN after normalisation (>= 1)          */
    int32_t greedy;        /* 1 when the configured temperature was <= 0                    */
    int32_t reserved;      /* must be 0                                                     */
    double uniform;        /* r in [0,1): the value rng.Float64() would have returned       */
} MantleSampleParams;      /* 40 bytes, 8-byte aligned */

/* Raw, un-normalised configuration: field for field logits.SamplerConfig
 * (internal/logits/sampler.go:34-42). */
typedef struct MantleSamplerConfig {
    int64_t seed;
    float temperature;
    int32_t top_k;
    float top_p;
    float min_p;
    float repeat_penalty;
    int32_t repeat_last_n;
} MantleSamplerConfig;

#ifdef __cplusplus
}
#endif

#endif /* MANTLE_SAMPLE_PARAMS_H */
