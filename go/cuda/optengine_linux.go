//go:build linux && amd64

// Binding of liboptengine.so for gograd's cuda package on Linux.
//
// This file was written against gograd's sources and the C header include/optengine.h; no Go
// toolchain was available where it was written, so it has never been compiled. It adds names
// only (nothing in cuda_stub.go is redefined) and follows the loader the repository already
// uses on Linux for Vulkan: purego.Dlopen / Dlsym / SyscallN with integer and pointer
// arguments only, floats inside pointed-to structs (vulkan/loader_linux.go:16-47). It replaces,
// for the optimizer path, the Windows-only NVRTC route cuda.Compile -> Kernel.Launch
// (cuda/kernel_windows.go:131-310).
package cuda

import (
	"fmt"
	"runtime"
	"sync"
	"unsafe"

	"github.com/ebitengine/purego"
)

// TensorDesc mirrors oe_tensor_desc (56 bytes, no padding).
type TensorDesc struct {
	Param, Grad, State1, State2, Shadow, Numel uint64
	LRScale, WeightDecay                       float32
}

// AdamWHParams mirrors oe_adamw_hparams (48 bytes).
type AdamWHParams struct {
	LR, Beta1, Beta2, Eps, BC1, BC2, MaxNorm float32
	Flags                                    uint32
	StepDev, LRDev                           uint64
}

// SGDHParams mirrors oe_sgd_hparams (40 bytes).
type SGDHParams struct {
	LR, Momentum, Dampening, MaxNorm float32
	Flags, Reserved                  uint32
	StepDev, LRDev                   uint64
}

// Zero1Desc mirrors oe_zero1_desc (320 bytes): the ranks of a sharded step as seen from one GPU.
type Zero1Desc struct {
	Rank, World                  uint32
	FirstElem, Numel             uint64
	GradBases                    [8]uint64
	ShadowDeltas                 [8]int64
	ShadowMCDelta                int64
	SyncBlocks                   [8]uint64
	TimeoutMS, Flags             uint32
	Staging, StagingBytes        uint64 // caller-owned scratch for the copy-engine-assisted reduction, or 0
	CEPullSources, CEPushTargets uint32 // 0 = the library's choice, 0xffffffff = none
	StagingBases                 [8]uint64 // rank k's staging as mapped on this GPU, or all 0
}

// Flag bits of AdamWHParams.Flags / SGDHParams.Flags / GradNorm.
const (
	ClipDevForm uint32 = 0x1  // OE_CLIP_DEVFORM
	WriteShadow uint32 = 0x2  // OE_WRITE_SHADOW
	ZeroGrad    uint32 = 0x4  // OE_ZERO_GRAD
	Nesterov    uint32 = 0x8  // OE_NESTEROV
	Maximize    uint32 = 0x10 // OE_MAXIMIZE
	PartialOnly uint32 = 0x20 // OE_PARTIAL_ONLY
)

// Zero1SyncBytes is the size of the exchange area every rank of a sharded step provides.
const Zero1SyncBytes = 512

type optEngine struct {
	handle uintptr
	fn     map[string]uintptr
}

var (
	oeOnce sync.Once
	oeLib  *optEngine
	oeErr  error
)

var oeSymbols = []string{
	"oe_abi_version", "oe_last_error", "oe_init", "oe_plan_create", "oe_plan_update", "oe_plan_destroy",
	"oe_plan_norm_address", "oe_plan_set_grad_scale", "oe_grad_norm", "oe_norm_finalize", "oe_clip_grad_norm",
	"oe_read_norm", "oe_adamw_step", "oe_sgd_step", "oe_zero_grads", "oe_cast_bf16",
	"oe_peer_reduce_grads", "oe_adamw_step_peers", "oe_sgd_step_peers",
	"oe_zero1_create", "oe_zero1_destroy", "oe_zero1_adamw_step", "oe_zero1_sgd_step", "oe_zero1_status", "oe_zero1_info",
	"oe_ipc_export", "oe_ipc_import", "oe_ipc_close",
	"oe_mem_alloc", "oe_mem_free", "oe_memcpy_h2d", "oe_memcpy_d2h", "oe_memset_u32", "oe_stream_sync",
	"oe_launch_count",
}

// LoadOptEngine binds liboptengine.so once per process. It uses the dynamic linker's normal
// search (no path guessing), like openLinuxLibrary does for libvulkan.so.1.
func LoadOptEngine() error {
	oeOnce.Do(func() {
		handle, err := purego.Dlopen("liboptengine.so", purego.RTLD_NOW|purego.RTLD_LOCAL)
		if err != nil {
			oeErr = fmt.Errorf("%w: dlopen(liboptengine.so): %v", ErrUnavailable, err)
			return
		}
		lib := &optEngine{handle: handle, fn: make(map[string]uintptr, len(oeSymbols))}
		for _, name := range oeSymbols {
			address, err := purego.Dlsym(handle, name)
			if err != nil {
				oeErr = fmt.Errorf("%w: liboptengine.so lacks %s: %v", ErrUnavailable, name, err)
				return
			}
			lib.fn[name] = address
		}
		if version := oeCallRaw(lib.fn["oe_abi_version"]); int32(version) != 1 {
			oeErr = fmt.Errorf("%w: liboptengine.so has ABI version %d, this binding needs 1", ErrUnavailable, int32(version))
			return
		}
		oeLib = lib
	})
	return oeErr
}

// OptEngineAvailable reports whether the library is bound and device `device` is a B200 it accepts.
func OptEngineAvailable(device int) bool {
	if LoadOptEngine() != nil {
		return false
	}
	return oeCall("oe_init", uintptr(device)) == nil
}

// oeCallRaw enters the library. uintptrescapes keeps Go memory whose address was converted to
// uintptr alive and unmoved for the duration of the call.
//
//go:uintptrescapes
func oeCallRaw(fn uintptr, args ...uintptr) uintptr {
	r, _, _ := purego.SyscallN(fn, args...)
	return r
}

// goString copies a NUL-terminated C string owned by the library.
func goString(p uintptr) string {
	if p == 0 {
		return ""
	}
	n := 0
	for *(*byte)(unsafe.Add(unsafe.Pointer(p), n)) != 0 { //nolint:govet // address comes from C
		n++
	}
	return string(unsafe.Slice((*byte)(unsafe.Pointer(p)), n)) //nolint:govet
}

// oeCall turns a non-zero return code into the *Error the package already uses (Op, Code,
// Message): 0 is success, a positive value a CUresult, a negative value an OE_ERR_* code; the text
// comes from oe_last_error(), which is per OS thread — callers are pinned with
// runtime.LockOSThread as everywhere else in the CUDA path (autograd/cuda_context.go:29-54).
//
//go:uintptrescapes
func oeCall(name string, args ...uintptr) error {
	if err := LoadOptEngine(); err != nil {
		return err
	}
	rc := int32(oeCallRaw(oeLib.fn[name], args...))
	if rc == 0 {
		return nil
	}
	return &Error{Op: name, Code: int(rc), Message: goString(oeCallRaw(oeLib.fn["oe_last_error"]))}
}

// Plan is an oe_plan: the device-side tensor table and work-unit table of one parameter list. It
// takes the place of one Kernel.Launch per tensor and of the clip pointer table that
// getClipPlan builds with one write_clip_entry launch per tensor (autograd/cuda_clip.go:66-113).
type Plan struct {
	handle uintptr
	device int
}

func descPointer(tensors []TensorDesc) uintptr {
	if len(tensors) == 0 {
		return 0
	}
	return uintptr(unsafe.Pointer(&tensors[0]))
}

// NewPlan validates every descriptor, then builds and uploads the tables.
func NewPlan(device int, tensors []TensorDesc) (*Plan, error) {
	if err := oeCall("oe_init", uintptr(device)); err != nil {
		return nil, err
	}
	p := &Plan{device: device}
	err := oeCall("oe_plan_create", uintptr(device), descPointer(tensors), uintptr(len(tensors)), 0,
		uintptr(unsafe.Pointer(&p.handle)))
	runtime.KeepAlive(tensors) // descPointer handed out a bare address: the slice must outlive the call
	if err != nil {
		return nil, err
	}
	return p, nil
}

// Update hands the plan the current descriptors. Like getClipPlan's cache check it compares
// addresses and sizes (the pool may return a freed block to a parameter of another size,
// autograd/cuda_clip.go:80-93) and uploads, on stream, only when something changed.
func (p *Plan) Update(tensors []TensorDesc, stream uintptr) error {
	err := oeCall("oe_plan_update", p.handle, descPointer(tensors), uintptr(len(tensors)), stream)
	runtime.KeepAlive(tensors)
	return err
}

// SetGradScale makes norm and update read every gradient element as float32(g*scale).
func (p *Plan) SetGradScale(scale float32) error {
	return oeCall("oe_plan_set_grad_scale", p.handle, uintptr(unsafe.Pointer(&scale)))
}

// NormAddress is the device address of the float32 norm (the record's bytes 8..11).
func (p *Plan) NormAddress() uintptr {
	return oeCallRaw(oeLib.fn["oe_plan_norm_address"], p.handle) + 8
}

func (p *Plan) GradNorm(flags uint32, stream uintptr) error {
	return oeCall("oe_grad_norm", p.handle, uintptr(flags), stream)
}

func (p *Plan) NormFinalize(stream uintptr) error { return oeCall("oe_norm_finalize", p.handle, stream) }

func (p *Plan) ClipGradNorm(maxNorm float32, flags uint32, stream uintptr) error {
	return oeCall("oe_clip_grad_norm", p.handle, uintptr(unsafe.Pointer(&maxNorm)), uintptr(flags), stream)
}

// ReadNorm waits for stream and returns the last norm and its float64 sum of squares.
func (p *Plan) ReadNorm(stream uintptr) (norm float32, sumsq float64, err error) {
	err = oeCall("oe_read_norm", p.handle, uintptr(unsafe.Pointer(&norm)), uintptr(unsafe.Pointer(&sumsq)), stream)
	return norm, sumsq, err
}

func (p *Plan) AdamWStep(hp *AdamWHParams, stream uintptr) error {
	return oeCall("oe_adamw_step", p.handle, uintptr(unsafe.Pointer(hp)), stream)
}

func (p *Plan) SGDStep(hp *SGDHParams, stream uintptr) error {
	return oeCall("oe_sgd_step", p.handle, uintptr(unsafe.Pointer(hp)), stream)
}

func (p *Plan) ZeroGrads(stream uintptr) error { return oeCall("oe_zero_grads", p.handle, stream) }

// Close destroys the plan's tables; the tensors stay the caller's. Safe to call twice.
func (p *Plan) Close() error {
	if p == nil || p.handle == 0 {
		return nil
	}
	err := oeCall("oe_plan_destroy", p.handle)
	p.handle = 0
	return err
}

// CastBF16 is the stand-alone f32_to_bf16 pass (autograd/cuda_kernels.go:86) for every caller that
// is not a weight written by an optimizer step.
func CastBF16(device int, src, dst uintptr, count int, stream uintptr) error {
	return oeCall("oe_cast_bf16", uintptr(device), src, dst, uintptr(count), stream)
}

// Zero1 is an oe_zero1: a sharded step whose exchanges between the ranks are kernels of the
// library, for a host that has no collective library (gograd has none). With Staging set in the
// descriptor the step lets whole-shard copies carry part of the traffic from four ranks on; a host
// that keeps all ranks in one process then calls each rank's step from that rank's pinned OS
// thread on a stream created for it (autograd/cuda_context.go:29-54 pins the thread already).
type Zero1 struct{ handle uintptr }

func NewZero1(plan *Plan, desc *Zero1Desc) (*Zero1, error) {
	z := &Zero1{}
	if err := oeCall("oe_zero1_create", plan.handle, uintptr(unsafe.Pointer(desc)), uintptr(unsafe.Pointer(&z.handle))); err != nil {
		return nil, err
	}
	return z, nil
}

func (z *Zero1) AdamWStep(hp *AdamWHParams, stream uintptr) error {
	return oeCall("oe_zero1_adamw_step", z.handle, uintptr(unsafe.Pointer(hp)), stream)
}

func (z *Zero1) SGDStep(hp *SGDHParams, stream uintptr) error {
	return oeCall("oe_zero1_sgd_step", z.handle, uintptr(unsafe.Pointer(hp)), stream)
}

// CopyPlan reports how many peers' gradient ranges copies stage before the pull kernel and how
// many ranks receive their shadow values from a copy, as the library resolved them.
func (z *Zero1) CopyPlan() (stagedSources, shadowCopies int) {
	lib := oeLib
	return int(int64(oeCallRaw(lib.fn["oe_zero1_info"], z.handle, 0))), int(int64(oeCallRaw(lib.fn["oe_zero1_info"], z.handle, 1)))
}

// Status waits for stream; a rank that missed an exchange is reported as an *Error whose message
// names it.
func (z *Zero1) Status(stream uintptr) (uint32, error) {
	var word uint32
	err := oeCall("oe_zero1_status", z.handle, uintptr(unsafe.Pointer(&word)), stream)
	return word, err
}

func (z *Zero1) Close() error {
	if z == nil || z.handle == 0 {
		return nil
	}
	err := oeCall("oe_zero1_destroy", z.handle)
	z.handle = 0
	return err
}

// IPCExport returns the 64-byte handle of the allocation that contains address, and the
// address's offset inside it; IPCImport maps a peer's allocation on this device.
func IPCExport(device int, address uintptr) (handle [64]byte, offset uint64, err error) {
	err = oeCall("oe_ipc_export", uintptr(device), address, uintptr(unsafe.Pointer(&handle[0])), uintptr(unsafe.Pointer(&offset)))
	return handle, offset, err
}

func IPCImport(device int, handle [64]byte) (base uint64, err error) {
	err = oeCall("oe_ipc_import", uintptr(device), uintptr(unsafe.Pointer(&handle[0])), uintptr(unsafe.Pointer(&base)))
	return base, err
}

func IPCClose(device int, base uint64) error { return oeCall("oe_ipc_close", uintptr(device), uintptr(base)) }

// The few device-management calls the optimizer path needs on Linux, where cuda_stub.go has
// none (cuda.Alloc / Buffer.Free / CopyFromHost / CopyToHost / Memset, cuda/cuda_windows.go:324-700).
// A Linux Buffer type would wrap these one to one.
func EngineAlloc(device int, bytes int) (uintptr, error) {
	var address uint64
	err := oeCall("oe_mem_alloc", uintptr(device), uintptr(bytes), uintptr(unsafe.Pointer(&address)))
	return uintptr(address), err
}

func EngineFree(device int, address uintptr) error { return oeCall("oe_mem_free", uintptr(device), address) }

func EngineCopyFromHost(device int, dst uintptr, src []byte, stream uintptr) error {
	if len(src) == 0 {
		return nil
	}
	return oeCall("oe_memcpy_h2d", uintptr(device), dst, uintptr(unsafe.Pointer(&src[0])), uintptr(len(src)), stream)
}

func EngineCopyToHost(device int, dst []byte, src uintptr, stream uintptr) error {
	if len(dst) == 0 {
		return nil
	}
	if err := oeCall("oe_memcpy_d2h", uintptr(device), uintptr(unsafe.Pointer(&dst[0])), src, uintptr(len(dst)), stream); err != nil {
		return err
	}
	return oeCall("oe_stream_sync", uintptr(device), stream)
}

func EngineMemset32(device int, dst uintptr, value uint32, count int, stream uintptr) error {
	return oeCall("oe_memset_u32", uintptr(device), dst, uintptr(value), uintptr(count), stream)
}

// EngineLaunchCount is what the tests' "kernel X ran" assertions read instead of the profile
// counts of autograd/cuda_kernels.go:11-82 (sgd_test.go:119-121).
func EngineLaunchCount(kernel string) int64 {
	name := append([]byte(kernel), 0)
	return int64(oeCallRaw(oeLib.fn["oe_launch_count"], uintptr(unsafe.Pointer(&name[0]))))
}
