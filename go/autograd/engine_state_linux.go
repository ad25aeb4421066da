//go:build linux && amd64

// Shared state of the optengine route through gograd's optimizers on Linux.
//
// Written against gograd's sources (autograd/nn.go, sgd.go, cuda_sgd.go, cuda_clip.go,
// cuda_autocast.go) and include/optengine.h; no Go toolchain was available, so this file has
// never been compiled. The optimizer structs are declared in files this change does not touch,
// so what the engine needs per optimizer lives in side tables keyed by the optimizer's address
// and is released from AdamW.Close / SGD.Close (autograd/optimizer_state.go:262-274,
// autograd/sgd.go:247-257).
//
// cuda.CurrentDevice and cuda.CurrentStreamHandle are the per-thread device state of the cuda
// package (cuda/cuda_windows.go:258, cuda_stub.go:34,74): on Linux they have to come from the
// device binding that takes cuda_stub.go's place (go/cuda/optengine_linux.go supplies the memory and
// copy calls such a binding wraps); with the stub still in place useEngine reports false and the
// optimizers keep their CPU branches.
package autograd

import (
	"sync"

	"github.com/yh2237/gograd/cuda"
)

// engineState is what one optimizer keeps for the engine: its plan, the descriptors the plan
// was last given, the shadow buffers the step writes, and a clip limit that ClipGradNorm left
// for the next Step to fold into the update.
type engineState struct {
	plan           *cuda.Plan
	descs          []cuda.TensorDesc
	shadows        []*cuda.Buffer
	pendingMaxNorm float32
	pendingNorm    bool
}

var (
	engineMu     sync.Mutex
	engineStates = map[any]*engineState{}
)

func engineStateFor(owner any) *engineState {
	engineMu.Lock()
	defer engineMu.Unlock()
	s := engineStates[owner]
	if s == nil {
		s = &engineState{}
		engineStates[owner] = s
	}
	return s
}

// releaseEngineState is called from the optimizers' Close: the plan's tables go back to the
// driver; parameters, gradients and optimizer state stay the caller's, as before.
func releaseEngineState(owner any) {
	engineMu.Lock()
	s := engineStates[owner]
	delete(engineStates, owner)
	engineMu.Unlock()
	if s != nil && s.plan != nil {
		if err := s.plan.Close(); err != nil {
			panic(err)
		}
	}
}

// ensurePlan creates the optimizer's plan on first use and afterwards hands it the current
// descriptors; the library uploads its tables only when an address, a size or a group value
// changed since the last call (the comparison getClipPlan makes, autograd/cuda_clip.go:80-93).
func (s *engineState) ensurePlan(descs []cuda.TensorDesc) *cuda.Plan {
	device, err := cuda.CurrentDevice()
	if err != nil {
		panic(err)
	}
	if s.plan == nil {
		if s.plan, err = cuda.NewPlan(device, descs); err != nil {
			panic(err)
		}
	} else if err = s.plan.Update(descs, cuda.CurrentStreamHandle()); err != nil {
		panic(err)
	}
	s.descs = descs
	return s.plan
}

// useEngine reports whether the parameters live on a CUDA device the engine serves.
func useEngine() bool {
	device, err := cuda.CurrentDevice()
	return err == nil && cuda.OptEngineAvailable(device)
}
