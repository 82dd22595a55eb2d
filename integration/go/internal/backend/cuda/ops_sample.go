//go:build cuda

package cuda

// Device sampling on the LM head's output, added next to DeviceArgMaxLastResult
// (ops.go:1332-1346): the logits DeviceMatVecNoCopy left in o.yDev (ops.go:1289-1330,
// greedyResultDev / greedyResultLen) are sampled where they are, so that a non-greedy decode step
// downloads one token instead of V floats (today's path: flushLastResult, ops.go:360-377, then
// Sampler.Sample on the host).  Not compiled here (no Go toolchain).

import (
	"unsafe"

	"github.com/samcharles93/mantle/internal/backend/cuda/native"
	"github.com/samcharles93/mantle/internal/logits"
)

// deviceSampleState is what Ops keeps for the device sampler; a field `sample deviceSampleState`
// joins the greedyResult* fields of Ops (ops.go:93-99).  Everything is allocated on first use and
// freed in Ops.Close with the other device buffers.
type deviceSampleState struct {
	params    native.DeviceBuffer // one native.SampleParams
	history   native.DeviceBuffer // the penalty window, int32
	histCap   int
	exclude   native.DeviceBuffer // stop tokens, int32
	exclCap   int
	next      native.DeviceBuffer // one int32
	status    native.DeviceBuffer // one int32
	workspace native.DeviceBuffer // split-row scratch
	hostIDs   []int32             // staging for history + exclude
}

func (st *deviceSampleState) ensure(window, nExclude int, need int64) error {
	var err error
	alloc := func(buf *native.DeviceBuffer, bytes int64) {
		if err == nil && buf.Nbytes() < bytes {
			if buf.Ptr() != nil {
				_ = buf.Free()
			}
			*buf, err = native.AllocDevice(bytes)
		}
	}
	alloc(&st.params, int64(unsafe.Sizeof(native.SampleParams{})))
	alloc(&st.next, 4)
	alloc(&st.status, 4)
	alloc(&st.history, int64(max(window, 64))*4)
	alloc(&st.exclude, int64(max(nExclude, 16))*4)
	alloc(&st.workspace, need)
	return err
}

// DeviceSampleLastResult implements the sampling counterpart of DeviceArgMaxLastResult: Sample
// (logits/sampler.go:98-234) on the device-resident result of the last DeviceMatVecNoCopy.
// p carries the sampler's normalised configuration and this step's uniform draw; recent and
// exclude are the reference's `recent` and `excludePenalty`.  post is the model head's multiplier
// and soft cap, which the device path applies on the fly (the greedy device path skips them,
// simd/runtime_greedy.go:32-44, which is harmless for argmax but not for sampling).
func (o *Ops) DeviceSampleLastResult(p logits.DeviceParams, recent, exclude []int, post native.HeadPost) (next int, ok bool) {
	o.mu.Lock()
	defer o.mu.Unlock()

	if !o.greedyResultValid {
		return 0, false
	}
	vocab := o.greedyResultLen
	window := min(len(recent), p.RepeatLastN) // sampler.go:100-101
	recent = recent[len(recent)-window:]

	st := &o.sample
	b := native.SampleBatch{
		Logits: o.greedyResultDev, Rows: 1, Vocab: vocab, RowStride: int64(vocab),
		MaxTopK: min(p.TopK, vocab), HistStride: window, NExclude: len(exclude), Post: post,
	}
	// sizes first (the workspace depends on the shortlist length), then the buffers
	if err := st.ensure(window, len(exclude), 0); err != nil {
		o.recordFastPathErrorLocked(err)
		return 0, false
	}
	b.Params, b.Next, b.Status = st.params, st.next, st.status
	if window > 0 {
		b.History = st.history
	}
	if len(exclude) > 0 {
		b.Exclude = st.exclude
	}
	need, err := native.SamplerWorkspaceBytes(&b)
	if err == nil {
		err = st.ensure(window, len(exclude), need)
	}
	if err != nil {
		o.recordFastPathErrorLocked(err)
		return 0, false
	}

	// small inputs up: parameters, window, stop tokens (Go ints narrowed to the device's int32 ids;
	// an id that does not fit is out of every vocabulary and ignored like any other, sampler.go:116)
	hp := native.SampleParams{
		Temperature: p.Temperature, TopP: p.TopP, MinP: p.MinP, RepeatPenalty: p.RepeatPenalty,
		TopK: int32(p.TopK), RepeatLastN: int32(p.RepeatLastN), Uniform: p.Uniform,
	}
	if p.Greedy {
		hp.Greedy = 1
	}
	st.hostIDs = st.hostIDs[:0]
	for _, id := range recent {
		st.hostIDs = append(st.hostIDs, narrowID(id))
	}
	for _, id := range exclude {
		st.hostIDs = append(st.hostIDs, narrowID(id))
	}
	var zero int32
	steps := []func() error{
		func() error {
			return native.MemcpyH2DAsync(st.params, unsafe.Pointer(&hp), int64(unsafe.Sizeof(hp)), o.stream)
		},
		func() error { return native.MemcpyH2DAsync(st.status, unsafe.Pointer(&zero), 4, o.stream) },
		func() error {
			if window == 0 {
				return nil
			}
			return native.MemcpyH2DAsync(st.history, unsafe.Pointer(&st.hostIDs[0]), int64(window)*4, o.stream)
		},
		func() error {
			if len(exclude) == 0 {
				return nil
			}
			return native.MemcpyH2DAsync(st.exclude, unsafe.Pointer(&st.hostIDs[window]), int64(len(exclude))*4, o.stream)
		},
		func() error { return native.SampleRows(&b, st.workspace, o.stream) },
	}
	for _, step := range steps {
		if err := step(); err != nil {
			o.recordFastPathErrorLocked(err)
			return 0, false
		}
	}
	var out [2]int32 // token, status
	if err := native.MemcpyD2HAsync(unsafe.Pointer(&out[0]), st.next, 4, o.stream); err == nil {
		err = native.MemcpyD2HAsync(unsafe.Pointer(&out[1]), st.status, 4, o.stream)
	}
	if err == nil {
		err = o.stream.Synchronize()
	}
	if err != nil {
		o.recordFastPathErrorLocked(err)
		return 0, false
	}
	if out[1] != 0 {
		// min-p above 1 empties the shortlist: the reference panics in Sample there and the
		// engine reports "panic in Sample" (engine.go:339-346); here it is a fast-path error
		o.recordFastPathErrorLocked(sampleStatusError(out[1]))
		return 0, false
	}
	return int(out[0]), true
}

func narrowID(id int) int32 {
	if id < 0 || id > 0x7fffffff {
		return -1
	}
	return int32(id)
}

type sampleStatusError int32

func (e sampleStatusError) Error() string {
	switch {
	case int32(e)&native.SampleStatusEmpty != 0:
		return "device sampler: the shortlist was empty after min-p"
	case int32(e)&native.SampleStatusTopKRange != 0:
		return "device sampler: top_k exceeded the bound the launch was sized for"
	case int32(e)&native.SampleStatusNaN != 0:
		return "device sampler: the logits held nothing but NaN"
	}
	return "device sampler: unknown status"
}
