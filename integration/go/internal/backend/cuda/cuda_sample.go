//go:build cuda

package cuda

// ForwardTokenSample on the CUDA runtime, added next to ForwardTokenGreedy (cuda.go:174-199) and
// shaped like it: forward to the wrapped simd instance, turn panics into errors, count the token.
// Not compiled here (no Go toolchain).

import (
	"fmt"
	"os"

	"github.com/samcharles93/mantle/internal/backend/cuda/native"
	"github.com/samcharles93/mantle/internal/logits"
)

func (r *cudaRuntime) ForwardTokenSample(id int, p logits.DeviceParams, recent []int, exclude []int) (next int, err error) {
	if r.model == nil {
		return 0, fmt.Errorf("cuda runtime is closed")
	}
	s, ok := r.model.(interface {
		ForwardTokenSample(id int, p logits.DeviceParams, recent []int, exclude []int) (next int, err error)
	})
	if !ok {
		return 0, fmt.Errorf("runtime does not support device sampling")
	}
	defer func() {
		if rec := recover(); rec != nil {
			err = cudaExecutionError(rec)
		}
	}()
	next, err = s.ForwardTokenSample(id, p, recent, exclude)
	if err != nil {
		return 0, err
	}
	if !r.managedFallbackLog && native.ManagedFallbackUsed() {
		fmt.Fprintln(os.Stderr, "CUDA Unified Memory fallback active (device memory pressure detected)")
		r.managedFallbackLog = true
	}
	r.tokenCount.Add(1)
	return next, nil
}
