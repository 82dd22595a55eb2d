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
// and in the loop, between the device-greedy branch (engine.go:284-289) and the host path
// (engine.go:291-300):
//
//	} else if canDeviceSample {
//		next, err = g.stepDeviceSample(ds, next, toks)
//
// The model's ForwardTokenSample (cuda.go -> simd/runtime_sample.go) runs the layers as
// ForwardTokenGreedy does, leaves the LM-head output on the device (Ops.DeviceMatVecNoCopy,
// cuda/ops.go:1289-1330) and calls Ops.DeviceSampleLastResult, which hands greedyResultDev to
// native.SampleRows the way DeviceArgMaxLastResult hands it to native.ArgMaxF32
// (cuda/ops.go:1332-1346).  Errors are parked with recordFastPathErrorLocked like every other
// fast path.

import (
	"errors"
	"fmt"

	"github.com/samcharles93/mantle/internal/backend/simd"
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

// stepDeviceSample is one iteration of the loop with the sample taken on the device: the
// sampler's generator is advanced once (NextDeviceParams), and when the device path is not
// available for this step the host path runs with that same draw.
func (g *Generator) stepDeviceSample(ds deviceSampler, tok int, toks []int) (int, error) {
	p := g.Sampler.NextDeviceParams()
	next, err := safeForwardTokenSample(ds, tok, p, toks, g.StopTokens)
	if err == nil || !errors.Is(err, simd.ErrNoDeviceSampler) {
		return next, err
	}
	logitsVec, err := g.Model.ForwardToken(tok) // the reference's own step (engine.go:291-295)
	if err != nil {
		return 0, err
	}
	return safeSampleWith(g.Sampler, logitsVec, toks, g.StopTokens, p)
}

// safeSampleWith is safeSample (engine.go:339-346) around SampleWithParams.
func safeSampleWith(s *logits.Sampler, logitsVec []float32, recent, exclude []int, p logits.DeviceParams) (next int, err error) {
	defer func() {
		if rec := recover(); rec != nil {
			err = fmt.Errorf("panic in Sample: %v", rec)
		}
	}()
	return s.SampleWithParams(logitsVec, recent, exclude, p), nil
}
