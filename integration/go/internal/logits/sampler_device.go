//go:build cuda

package logits

// Additive to sampler.go: what the inference loop needs to run Sample on the device.
// Not compiled here (no Go toolchain).
//
// One change to sampler.go itself goes with it: the field `rng *rand.Rand` (sampler.go:47) becomes
// `rng interface{ Float64() float64 }`, which *rand.Rand satisfies, so that SampleWithParams below
// can replay a draw that NextDeviceParams already took.

// DeviceParams are the values NewSampler left in the Sampler, for one step.
type DeviceParams struct {
	Temperature, TopP, MinP, RepeatPenalty float32
	TopK, RepeatLastN                      int
	Greedy                                 bool
	Uniform                                float64
}

// usesArgmax mirrors the test at the top of Sample's second half (sampler.go:140).
func (s *Sampler) usesArgmax() bool {
	return s.greedy || (s.cfg.TopK == 1 && s.cfg.TopP >= 1 && s.cfg.Temperature == 1)
}

// NextDeviceParams returns the parameters of the next step.  It draws from the sampler's own
// generator exactly when Sample would (once per call that does not end in argmax,
// sampler.go:224), so a device-sampled stream consumes the same draws as a host-sampled one.
func (s *Sampler) NextDeviceParams() DeviceParams {
	p := DeviceParams{
		Temperature: s.cfg.Temperature, TopP: s.cfg.TopP, MinP: s.cfg.MinP, RepeatPenalty: s.cfg.RepeatPenalty,
		TopK: s.cfg.TopK, RepeatLastN: s.cfg.RepeatLastN, Greedy: s.greedy,
	}
	if !s.usesArgmax() {
		p.Uniform = s.rng.Float64()
	}
	return p
}

// constDraw replays one uniform.
type constDraw float64

func (c constDraw) Float64() float64 { return float64(c) }

// SampleWithParams is Sample for a step whose parameters were already taken with NextDeviceParams
// but whose device path turned out to be unavailable: the same computation as Sample on the host
// logits, with the uniform p carries instead of a fresh draw, so that the generator advances
// exactly once per step either way.
func (s *Sampler) SampleWithParams(logits []float32, recent []int, excludePenalty []int, p DeviceParams) int {
	saved := s.rng
	s.rng = constDraw(p.Uniform)
	defer func() { s.rng = saved }()
	return s.Sample(logits, recent, excludePenalty)
}
