// Shared between the library's translation units; not part of the C-ABI.
#pragma once

#include <string.h>

#include "../../include/mantle_sample_params.h"

// Sets the text mantleCudaSamplerLastError() returns on the calling thread.
__attribute__((visibility("hidden"))) void mantle_internal_set_last_error(const char* msg);

// NewSampler's normalisation, internal/logits/sampler.go:61-83.
static inline void mantle_internal_normalise(const MantleSamplerConfig& cfg, MantleSampleParams* p) {
    memset(p, 0, sizeof *p);
    p->greedy = cfg.temperature <= 0 ? 1 : 0;
    p->temperature = cfg.temperature <= 0 ? 1.0f : cfg.temperature;
    p->top_k = cfg.top_k <= 0 ? 40 : cfg.top_k;
    p->top_p = (cfg.top_p <= 0 || cfg.top_p > 1) ? 1.0f : cfg.top_p;
    p->min_p = cfg.min_p;
    p->repeat_penalty = cfg.repeat_penalty <= 0 ? 1.0f : cfg.repeat_penalty;
    p->repeat_last_n = cfg.repeat_last_n <= 0 ? 64 : cfg.repeat_last_n;
}

// The test at sampler.go:140: such a row returns the argmax and consumes no uniform draw.
static inline bool mantle_internal_argmax_shortcut(const MantleSampleParams& p) {
    return p.greedy || (p.top_k == 1 && p.top_p >= 1.0f && p.temperature == 1.0f);
}

// Go ints to the device's int32 ids; an id that does not fit is out of every vocabulary and is
// ignored by the kernels like any other out-of-range id (sampler.go:116).
static inline int32_t mantle_internal_narrow_id(int64_t id) {
    return (id < 0 || id > 0x7fffffffLL) ? -1 : (int32_t)id;
}
