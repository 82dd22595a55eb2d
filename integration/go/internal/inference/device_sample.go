//go:build cuda

package inference

// The decode loop's device-sampling hook, modelled on the greedyStepper idiom of
// Generator.RunWithContext (engine.go:190-194, 284-289).  Not compiled here (no Go toolchain).
//
// In RunWithContext, beside
//
//	gs, canDeviceGreedy := g.Model.(greedyStepper)
//
// add
//
//	ds, canDeviceSample := g.Model.(deviceSampler)
//
// and in the loop, before the host path (engine.go:291-300):
//
//	} else if canDeviceSample {
//		next, err = safeForwardTokenSample(ds, next, g.Sampler.NextDeviceParams(), toks, g.StopTokens)
//
// The model's ForwardTokenSample runs the layers as ForwardTokenGreedy does
// (simd/runtime_greedy.go:13-44), leaves the LM-head output on the device
// (Ops.DeviceMatVecNoCopy, cuda/ops.go:1289-1330) and calls Ops.DeviceSampleLastResult, which
// hands greedyResultDev to native.SampleRowsF32 the way DeviceArgMaxLastResult hands it to
// native.ArgMaxF32 (cuda/ops.go:1332-1346).  Errors are parked with recordFastPathErrorLocked
// like every other fast path.

import (
	"fmt"

	"github.com/samcharles93/mantle/internal/logits"
)

type deviceSampler interface {
	ForwardTokenSample(id int, p logits.DeviceParams, recent []int, exclude []int) (next int, err error)
}

func safeForwardTokenSample(m deviceSampler, id int, p logits.DeviceParams, recent, exclude []int) (next int, err error) {
	defer func() {
		if rec := recover(); rec != nil {
			err = fmt.Errorf("panic in ForwardTokenSample: %v", rec)
		}
	}()
	return m.ForwardTokenSample(id, p, recent, exclude)
}
