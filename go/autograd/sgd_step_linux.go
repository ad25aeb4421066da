//go:build linux && amd64

// SGD.stepGPU through liboptengine.so: replaces autograd/cuda_sgd.go:66-98 (sgd_step,
// sgd_update and sgd_mark launches per tensor) with one launch. Never compiled (no Go toolchain
// where it was written); reviewed against those lines. The body of stepGPU becomes
// `o.stepEngine(captured)`.
package autograd

import (
	"github.com/yh2237/gograd/cuda"
)

func (o *SGD) stepEngine(captured bool) {
	state := engineStateFor(o)
	writeShadow := BF16Autocast && !captured
	if writeShadow && len(state.shadows) != len(o.Params) {
		state.shadows = make([]*cuda.Buffer, len(o.Params))
	}
	descs := make([]cuda.TensorDesc, len(o.Params))
	for i, p := range o.Params {
		v := p.Value
		group := o.groups[o.groupOf[i]]
		// SGD.groupScale (sgd.go:127-130): the rate is LR*LRScale, the decay is the group's own
		// value, not multiplied by the rate; the device applies them in that order.
		d := cuda.TensorDesc{Param: uint64(ptr(v.buf)), Grad: uint64(ptr(v.gradBuf)), Numel: uint64(v.Numel()),
			LRScale: group.LRScale, WeightDecay: group.WeightDecay}
		if o.options.Momentum > 0 {
			// the momentum buffer and the per-tensor device float "buffer initialised" the
			// reference already keeps (cuda_sgd.go:39-65); the launch's last block sets the flag
			// of every tensor that took part, which sgd_mark did per tensor.
			d.State1, d.State2 = uint64(ptr(o.bufferGPU[i])), uint64(ptr(o.initializedGPU[i]))
		}
		if writeShadow && v.gradBuf != nil {
			state.shadows[i] = v.shadowForWriting()
			d.Shadow = uint64(ptr(state.shadows[i]))
		}
		descs[i] = d
	}
	plan := state.ensurePlan(descs)
	hp := cuda.SGDHParams{LR: o.LR, Momentum: o.options.Momentum, Dampening: o.options.Dampening}
	if o.options.Nesterov {
		hp.Flags |= cuda.Nesterov
	}
	if o.options.Maximize {
		hp.Flags |= cuda.Maximize
	}
	if writeShadow {
		hp.Flags |= cuda.WriteShadow
	}
	if captured {
		hp.StepDev = uint64(ptr(o.graphStep)) // the launch advances the counter (sgd_step, cuda_sgd.go:18)
	}
	if state.pendingNorm {
		hp.MaxNorm = state.pendingMaxNorm
		state.pendingNorm = false
	}
	if err := plan.SGDStep(&hp, cuda.CurrentStreamHandle()); err != nil {
		panic(err)
	}
	if captured {
		return
	}
	for i, p := range o.Params {
		if p.Value.gradBuf == nil {
			continue // skipped and left uninitialised, as the loop at cuda_sgd.go:73-75 does
		}
		if writeShadow {
			p.Value.installBF16(state.shadows[i])
		} else {
			p.Value.invalidateBF16()
		}
	}
}

// In SGD.Close (sgd.go:247-257) add: releaseEngineState(o).
