package simd

// ForwardTokenSample: one autoregressive step that ends in Sampler.Sample on the device, the
// sampling twin of ForwardTokenGreedy (runtime_greedy.go:13-73).  The layers run as there, the
// output head's result stays on the device (DeviceMatVecNoCopy) and is sampled in place
// (DeviceSampleLastResult); when the device path is not available the step falls back to the
// reference's own: logits to the host, then the caller's Sampler.  Not compiled here (no Go
// toolchain).

import (
	"fmt"

	instance "github.com/samcharles93/mantle/internal/backend/core"
	"github.com/samcharles93/mantle/internal/backend/cuda/native"
	"github.com/samcharles93/mantle/internal/logits"
)

// ErrNoDeviceSampler tells the decode loop to take its host path for this step (ForwardToken, then
// Sampler.Sample with the SAME uniform draw, which p carries: the sampler's generator has already
// been advanced by NextDeviceParams).
var ErrNoDeviceSampler = fmt.Errorf("device sampler not available")

func (m *Instance) ForwardTokenSample(tok int, p logits.DeviceParams, recent []int, exclude []int) (int, error) {
	rt, cleanup, err := prepareTokenRuntimeState(m, tok)
	if err != nil {
		return 0, err
	}
	defer cleanup()

	x := rt.x
	ops := rt.ops
	ds := rt.ds

	if err := runDecoderLayers(m, rt); err != nil {
		return 0, err
	}

	type sampleHeadOps interface {
		DeviceMatVecNoCopy(w *instance.Mat, x []float32) bool
		DeviceSampleLastResult(p logits.DeviceParams, recent, exclude []int, post native.HeadPost) (next int, ok bool)
	}

	// the head's multiplier and soft cap (runtime.go:258-272) ride along as two numbers: the device
	// sampler applies them on the fly, with the host path's fastTanh, and rewrites nothing
	post := native.HeadPost{
		Scale:   float32(m.Config.Config.LMHeadMultiplier),
		Softcap: float32(m.Config.Config.FinalLogitSoftcap),
	}
	if ds != nil && ds.DeviceRMSNorm(m.Scratch.Tmp, x, m.OutputNorm, m.RMSEpsilon) {
		if sh, ok := ops.(sampleHeadOps); ok && sh.DeviceMatVecNoCopy(m.Output, m.Scratch.Tmp) {
			if next, ok := sh.DeviceSampleLastResult(p, recent, exclude, post); ok {
				m.Pos++
				if skipper, ok := ds.(interface{ SetGreedyEndTokenSkipD2H() }); ok {
					skipper.SetGreedyEndTokenSkipD2H()
				}
				return next, nil
			}
		}
	}
	if err := consumeFastPathError(ops); err != nil {
		return 0, fmt.Errorf("output head fast path failed: %w", err)
	}
	// nothing was advanced that the host path cannot redo: the caller runs ForwardToken for this
	// token instead (the state prepared above is released by cleanup)
	return 0, ErrNoDeviceSampler
}
