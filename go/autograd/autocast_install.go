//go:build linux && amd64

// The bf16 shadow seam, autograd/cuda_autocast.go:30-60: an optimizer step that has already
// written the shadow installs it instead of invalidating it. Never compiled (no Go toolchain
// where it was written); reviewed against those lines and against the lease rule of
// ensureBF16Lease (cuda_autocast.go:77-94).
package autograd

import (
	"github.com/yh2237/gograd/cuda"
)

// shadowForWriting returns a bf16 buffer of this tensor's size that the coming optimizer step
// may overwrite. The tensor's cached shadow is reused when nobody else holds it: a graph node
// that leased it for its backward (savedLeases, cuda_blas.go:197-203) still reads the old
// values, so a shadow with more than one reference is left to its readers and a fresh buffer is
// allocated instead. After a non-retaining Backward the leases are gone (storage.go:115-118), so
// in the usual Backward -> Clip -> Step order no allocation happens here.
func (t *Tensor) shadowForWriting() *cuda.Buffer {
	if t.bf16Storage != nil && t.bf16Storage.references.Load() == 1 && t.bf16Storage.buffer != nil &&
		t.bf16Storage.buffer.Size() == t.Numel()*2 {
		return t.bf16Storage.buffer
	}
	return allocBF16(t.Numel())
}

// installBF16 is what Step calls instead of invalidateBF16 (nn.go:504, cuda_sgd.go:95) for a
// tensor whose shadow the update kernel just wrote into buffer: the master changed, so the
// version advances exactly as invalidateBF16 advances it, and the shadow is stamped with the new
// version, which keeps currentBF16 valid (cuda_autocast.go:43-51). Views share the parent's
// shadow through shareBF16 as before (views.go:181); a view created earlier holds the old
// storage with the old version and drops it on its next currentBF16, as it does today after any
// mutation through an alias.
func (t *Tensor) installBF16(buffer *cuda.Buffer) {
	t.storage.version.Add(1)
	if buffer == nil {
		t.dropBF16()
		return
	}
	if t.bf16Storage != nil && t.bf16Storage.buffer == buffer {
		// written in place: same storage, new version
		t.bf16Version = t.storage.version.Load()
		t.bf16CaptureID = cuda.CaptureID()
		return
	}
	t.setBF16(buffer) // drops the old lease of this tensor, keeps the readers' leases alive
}

// The profile counter "f32_to_bf16" keeps counting the casts castBF16 launches for activations
// (cuda_autocast_test.go:53); weight casts no longer happen, so tests that count weight casts
// per step expect zero on this route. castBF16 itself maps onto cuda.CastBF16:
//
//	func castBF16(src uintptr, count int) *cuda.Buffer {
//		b := allocBF16(count)
//		device, _ := cuda.CurrentDevice()
//		if err := cuda.CastBF16(device, src, ptr(b), count, cuda.CurrentStreamHandle()); err != nil { panic(err) }
//		return b
//	}
