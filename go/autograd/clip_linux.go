//go:build linux && amd64

// ClipGradNorm on the device through liboptengine.so: replaces clipGPU and getClipPlan,
// autograd/cuda_clip.go:66-134, and the readback of GradientNormToHost, autograd/nn.go:17-27.
// Never compiled (no Go toolchain where it was written); reviewed against those lines.
package autograd

import (
	"github.com/yh2237/gograd/cuda"
)

// clipEngineState belongs, like clipState, to one (OS thread, device) pair (cuda_clip.go:25-53):
// independent training runs neither invalidate each other's plan nor read each other's norm.
type clipEngineState struct {
	plan *cuda.Plan
}

var clipEngineStates = map[clipStateKey]*clipEngineState{}

func clipEngineForThread() *clipEngineState {
	id := currentClipKey()
	clipMu.Lock()
	defer clipMu.Unlock()
	state := clipEngineStates[id]
	if state == nil {
		state = &clipEngineState{}
		clipEngineStates[id] = state
	}
	return state
}

// clipEngine is the body of clipGPU. Clipping observes gradients and must not create them, so a
// parameter without a gradient gets Grad = 0 and stays out of the device table (the rule at
// cuda_clip.go:71-77). The norm is the float64 sum the host code computes (nn.go:319-324), not
// the float32 atomics of global_norm_parts; maxNorm <= 0 computes the norm only (cuda_clip.go:130).
func clipEngine(params []Parameter, maxNorm float32) {
	state := clipEngineForThread()
	descs := make([]cuda.TensorDesc, 0, len(params))
	for _, p := range params {
		if p.Value == nil {
			continue
		}
		descs = append(descs, cuda.TensorDesc{Param: uint64(ptr(p.Value.buf)), Grad: uint64(ptr(p.Value.gradBuf)),
			Numel: uint64(p.Value.Numel())})
	}
	device, err := cuda.CurrentDevice()
	if err != nil {
		panic(err)
	}
	if state.plan == nil {
		if state.plan, err = cuda.NewPlan(device, descs); err != nil {
			panic(err)
		}
	} else if err = state.plan.Update(descs, cuda.CurrentStreamHandle()); err != nil {
		panic(err)
	}
	// the CUDA kernels' rule fminf(1, max/(norm+1e-6)) (cuda_kernels.go:676); drop the flag for
	// the host rule "scale only if norm > maxNorm" (nn.go:327)
	if err = state.plan.ClipGradNorm(maxNorm, cuda.ClipDevForm, cuda.CurrentStreamHandle()); err != nil {
		panic(err)
	}
}

// deferClip is the fused alternative for the usual Backward -> ClipGradNorm -> Step loop
// (cmd/transformer-bench/main.go:94,143), when nothing reads the gradients in between: the norm is
// computed on the optimizer's own plan now, and the next Step multiplies by the coefficient in
// registers instead of rewriting every gradient (8 bytes per parameter less). Parameters end
// bit-identical to clipEngine followed by Step; the stored gradients stay unscaled.
func deferClip(optimizer any, descs []cuda.TensorDesc, maxNorm float32) {
	state := engineStateFor(optimizer)
	plan := state.ensurePlan(descs)
	if err := plan.GradNorm(0, cuda.CurrentStreamHandle()); err != nil {
		panic(err)
	}
	state.pendingMaxNorm, state.pendingNorm = maxNorm, true
}

// gradientNormEngine is GradientNormToHost's readback: the last norm of this thread's clip plan.
func gradientNormEngine() float32 {
	id := currentClipKey()
	clipMu.Lock()
	state := clipEngineStates[id]
	clipMu.Unlock()
	if state == nil || state.plan == nil {
		return 0
	}
	norm, _, err := state.plan.ReadNorm(cuda.CurrentStreamHandle())
	if err != nil {
		panic(err)
	}
	return norm
}

// releaseClipEngine frees this thread's clip plan (the counterpart of ReleaseClipState).
func releaseClipEngine() {
	id := currentClipKey()
	clipMu.Lock()
	state := clipEngineStates[id]
	delete(clipEngineStates, id)
	clipMu.Unlock()
	if state != nil && state.plan != nil {
		if err := state.plan.Close(); err != nil {
			panic(err)
		}
	}
}
