//go:build linux && amd64

// AdamW.Step through liboptengine.so: replaces the CUDA branches of AdamW.Step,
// autograd/nn.go:470-486 (captured) and autograd/nn.go:495-512 (eager).
//
// Never compiled (no Go toolchain where it was written); reviewed against those lines. The
// call sites in nn.go become:
//
//	if cuda.InCapture() { ...graphStep check...; o.stepEngine(0, 0, true); return }
//	...
//	if len(o.Params) > 0 && o.Params[0].Value.Device == tensor.CUDA { o.stepEngine(bc1, bc2, false); ...PrepareGraph as today...; return }
package autograd

import (
	"github.com/yh2237/gograd/cuda"
)

// descs builds one descriptor per parameter: Tensor.buf, Tensor.gradBuf (0 when the parameter
// has no gradient: the engine then skips it, as the loop at nn.go:496-498 does), mGPU, vGPU, the
// shadow buffer this step may write (0 without autocast) and the parameter's group values in
// float32 exactly as groupScale reads them (nn.go:461-465; the multiplication by LR happens on
// the device in the same order).
func (o *AdamW) descs(state *engineState, writeShadow bool) []cuda.TensorDesc {
	out := make([]cuda.TensorDesc, len(o.Params))
	if writeShadow && len(state.shadows) != len(o.Params) {
		state.shadows = make([]*cuda.Buffer, len(o.Params))
	}
	for i, p := range o.Params {
		group := o.groups[o.groupOf[i]]
		d := cuda.TensorDesc{
			Param: uint64(ptr(p.Value.buf)), Grad: uint64(ptr(p.Value.gradBuf)),
			State1: uint64(ptr(o.mGPU[i])), State2: uint64(ptr(o.vGPU[i])),
			Numel: uint64(p.Value.Numel()), LRScale: group.LRScale, WeightDecay: group.WeightDecay,
		}
		if writeShadow && p.Value.gradBuf != nil {
			state.shadows[i] = p.Value.shadowForWriting()
			d.Shadow = uint64(ptr(state.shadows[i]))
		}
		out[i] = d
	}
	return out
}

// stepEngine is one launch for the whole parameter list. bc1, bc2 are the host-computed bias
// corrections of nn.go:493-494; in a captured step they are ignored and the kernel derives them
// from the device step counter, which it also advances (graph_adam_inc + graph_adamw,
// autograd/cuda_kernels.go:595-597).
func (o *AdamW) stepEngine(bc1, bc2 float32, captured bool) {
	state := engineStateFor(o)
	writeShadow := BF16Autocast && !captured // a captured forward re-casts its leaf weights itself (cuda_autocast.go:82-88)
	plan := state.ensurePlan(o.descs(state, writeShadow))
	hp := cuda.AdamWHParams{LR: o.LR, Beta1: o.Beta1, Beta2: o.Beta2, Eps: o.Eps, BC1: bc1, BC2: bc2}
	if writeShadow {
		hp.Flags |= cuda.WriteShadow
	}
	if captured {
		hp.StepDev = uint64(ptr(o.graphStep))
	}
	// A ClipGradNorm that deferred its scaling (clip_linux.go) left the limit here: the update
	// multiplies each gradient element by the coefficient in registers, which rounds exactly
	// like the in-place scale followed by a reload.
	if state.pendingNorm {
		hp.MaxNorm = state.pendingMaxNorm
		state.pendingNorm = false
	}
	if err := plan.AdamWStep(&hp, cuda.CurrentStreamHandle()); err != nil {
		panic(err) // the optimizer level panics on a launch error, as nn.go:501-503 does
	}
	if captured {
		return // a captured Step does not invalidate shadows (nn.go:476-485)
	}
	for i, p := range o.Params {
		if p.Value.gradBuf == nil {
			continue
		}
		if writeShadow {
			p.Value.installBF16(state.shadows[i])
		} else {
			p.Value.invalidateBF16()
		}
	}
}

// In AdamW.Close (optimizer_state.go:262-274) add: releaseEngineState(o).
