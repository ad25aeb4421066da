// Host-side mirror of gograd's optimizer surface for CUDA tensors, written over the
// C ABI of liboptengine (include/optengine.h). It shows — and lets the tests exercise —
// exactly what gograd's Go code does around the device work: parameter validation,
// parameter groups, the shared step counter and host-computed bias corrections, gradient
// presence, momentum initialisation flags, state snapshots, and the safetensors
// checkpoint layout. Names and behaviour follow the reference:
//
//   Parameter, ClipGradNorm, GradientNormToHost     autograd/nn.go:17-27,296-334
//   AdamW, NewAdamW, NewAdamWGroups, Step, ...       autograd/nn.go:336-537
//   SGD, SGDOptions, NewSGD, NewSGDGroups, ...       autograd/sgd.go:16-257, autograd/cuda_sgd.go
//   ParameterGroupSpec, resolveParameterGroups, ...  autograd/param_groups.go:21-251
//   OptimizerState, SGDState, snapshots, entries     autograd/optimizer.go, optimizer_state.go, sgd_state.go
//   OneCycle, Save/LoadTrainingCheckpoint            autograd/nn.go:539-571, autograd/training_checkpoint.go
//
// Where Go returns an error these functions return a message ("" = success); where Go
// panics they throw std::runtime_error. There is no host (CPU tensor) branch here: the
// reference keeps its own, and this library has no CPU fallback.
#ifndef GG_AUTOGRAD_HPP
#define GG_AUTOGRAD_HPP

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/optengine.h"
#include "safetensors.hpp"

namespace autograd {

// A contiguous float32 leaf tensor on one CUDA device (the part of autograd.Tensor the
// optimizer path touches: autograd/tensor.go:19-52): value buffer, optional gradient
// buffer, optional bf16 shadow with its version stamp (autograd/cuda_autocast.go:30-60).
class Tensor {
   public:
    std::vector<int> Shape;
    int Device = 0;
    bool RequiresGrad = true;
    uint64_t buf = 0, gradBuf = 0, bf16Buf = 0;
    uint64_t version = 0, bf16Version = 0;
    // True while the gradient buffer is known to hold zeros: freshly created, zeroed, or zeroed by an
    // optimizer step that was asked to do so. Anything that writes a gradient clears it (SetGrad here;
    // a backward pass that is handed the raw address must call MarkGradWritten).
    bool gradKnownZero = false;
    void MarkGradWritten() { gradKnownZero = false; }

    static std::string New(const std::vector<float>& values, const std::vector<int>& shape, int device,
                           bool requiresGrad, std::shared_ptr<Tensor>* out);
    ~Tensor();
    int Numel() const;
    std::string ToHost(std::vector<float>* out) const;
    std::string GradToHost(std::vector<float>* out) const;  // error when the gradient is absent
    std::string CopyFromHost(const std::vector<float>& values);
    std::string SetGrad(const std::vector<float>& values);  // creates the buffer when absent
    std::string EnsureGrad();                                // ensureGradGPU: present, zero-filled
    void FreeGrad();                                         // gradient becomes absent (nil gradBuf)
    std::string ZeroGrad();                                  // Tensor.ZeroGrad: memset when present
    std::string EnsureShadow();                              // allocates the bf16 buffer (not the cast)
    std::string ShadowToHost(std::vector<uint16_t>* out) const;
    bool ShadowCurrent() const { return bf16Buf != 0 && bf16Version == version; }
    // Leases (autograd/cuda_autocast.go:77-94): a graph node that keeps a raw pointer to the shadow
    // for its backward pass takes a lease; while leases are out, an optimizer step must not
    // overwrite that buffer — it gets a fresh one to write into, and the leased buffer lives until
    // its last lease is returned. AcquireShadowLease returns the leased address (0 without a shadow).
    uint64_t AcquireShadowLease();
    void ReleaseShadowLease(uint64_t address);
    std::string ShadowForWriting();  // EnsureShadow, or a fresh buffer when the current one is leased
    int LeasedShadowBuffers() const { return (int)retired_.size() + (leases_ > 0 ? 1 : 0); }
    void Close();

   private:
    bool closed_ = false;
    int leases_ = 0;                                  // leases on the current bf16Buf
    std::vector<std::pair<uint64_t, int>> retired_;   // replaced buffers that still have leases
};

struct Parameter {
    std::string Name;
    std::shared_ptr<Tensor> Value;
};

constexpr const char* DefaultParameterGroupName = "default";

struct ParameterGroupSpec {
    std::string Name;
    std::vector<Parameter> Params;
    float LRScale = 0;
    float WeightDecay = 0;
};

struct ParameterGroup {
    std::string Name;
    std::vector<int> Indexes;
    float LRScale = 1;
    float WeightDecay = 0;
};

struct OptimizerGroupState {
    std::string Name;
    std::vector<std::string> Names;
    float LRScale = 1;
    float WeightDecay = 0;
};

std::string normalizeLRScale(float scale, float* out);
std::string validateGroupDecay(float decay);
std::string validateLearningRate(float lr);
std::string resolveParameterGroups(const std::vector<Parameter>& params, const std::vector<ParameterGroupSpec>& specs,
                                   std::vector<ParameterGroup>* groups, std::vector<int>* owner);
std::string PartitionParameters(const std::vector<Parameter>& params, const std::vector<std::string>& labels,
                                std::vector<ParameterGroupSpec>* specs);
std::vector<OptimizerGroupState> groupStates(const std::vector<ParameterGroup>& groups, const std::vector<std::string>& names);
std::string validateGroupStates(const std::vector<ParameterGroup>& live, const std::vector<std::string>& names,
                                const std::vector<OptimizerGroupState>& states, float baseDecay,
                                std::vector<ParameterGroup>* resolved);

struct AdamWState {
    std::vector<float> M, V;
};

struct OptimizerState {
    int StepCount = 0;
    std::vector<AdamWState> Moments;
    std::vector<std::string> Names;
    std::vector<std::vector<int>> Shapes;
    float LR = 0, WeightDecay = 0, Beta1 = 0, Beta2 = 0, Eps = 0;
    std::vector<OptimizerGroupState> Groups;
};

struct SGDOptions {
    float LR = 0, Momentum = 0, Dampening = 0, WeightDecay = 0;
    bool Nesterov = false, Maximize = false;
    std::string validate() const;
};

struct SGDState {
    int StepCount = 0;
    std::vector<std::string> Names;
    std::vector<std::vector<int>> Shapes;
    SGDOptions Options;
    std::vector<bool> Initialized;
    std::vector<std::vector<float>> Buffers;
    std::vector<OptimizerGroupState> Groups;
};

struct OptimizerSnapshot {
    int Version = 0;
    std::string Kind;
    std::shared_ptr<OptimizerState> AdamW;
    std::shared_ptr<SGDState> SGD;
};

// The common eager training surface (autograd/optimizer.go:11-26).
class CheckpointOptimizer {
   public:
    virtual ~CheckpointOptimizer() = default;
    virtual void Step() = 0;
    virtual void ZeroGrad() = 0;
    virtual float LearningRate() const = 0;
    virtual void SetLearningRate(float lr) = 0;
    virtual void Close() = 0;
    virtual std::string Snapshot(OptimizerSnapshot* out) = 0;
    virtual std::string ValidateSnapshot(const OptimizerSnapshot& s) = 0;
    virtual std::string LoadSnapshot(const OptimizerSnapshot& s) = 0;
};

// Engine options that have no field in the reference's structs: whether Step also writes
// the bf16 shadows, and whether a preceding norm is folded into Step as a clip.
struct EngineOptions {
    bool WriteShadow = false;
    bool ClipDevForm = false;  // the CUDA kernels' fminf(1, .) rule instead of the host rule
    uint64_t Stream = 0;
    // Step stores zeros over every gradient it has read (the next group's ZeroGrad then finds nothing to do:
    // one pass and one launch less per update, autograd/training_loop.go:125-133). AdamW only: SGD's eager
    // ZeroGrad releases its gradients (autograd/sgd.go:231-246), and a zeroed buffer is not an absent one.
    bool ZeroGradInStep = false;
    // Step and StepClipped read every gradient element as (float)(g * GradScale): the 1/groups
    // factor of gradient accumulation, applied in the pass that reads the gradients anyway
    // instead of through the seed of every backward.
    float GradScale = 1.0f;
};

class AdamW : public CheckpointOptimizer {
   public:
    std::vector<Parameter> Params;
    float LR = 0, WeightDecay = 0, Beta1 = 0.9f, Beta2 = 0.999f, Eps = 1e-8f;
    int StepCount = 0;
    EngineOptions Engine;

    static std::string New(const std::vector<Parameter>& params, float lr, float decay, std::unique_ptr<AdamW>* out);
    static std::string NewGroups(const std::vector<Parameter>& params, float lr,
                                 const std::vector<ParameterGroupSpec>& specs, std::unique_ptr<AdamW>* out);
    ~AdamW() override;
    void Step() override;
    // Norm + update in two launches with the clip coefficient folded in; the gradients
    // are left unscaled. Same parameters as ClipGradNorm(params, maxNorm) then Step().
    void StepClipped(float maxNorm);
    float LastGradNorm();  // blocking read of the norm of the last StepClipped
    void ZeroGrad() override;
    float LearningRate() const override { return LR; }
    void SetLearningRate(float lr) override;
    void Close() override;
    std::string PrepareGraph();
    std::string GraphStepCount(int* out);
    std::string SyncGraphStepCount();
    void StepCaptured();  // the capture branch of Step: device step counter, no host state change
    std::string State(OptimizerState* out);
    std::string LoadState(const OptimizerState& state);
    std::string validateState(const OptimizerState& state);
    std::string SaveSafeTensors(const std::string& path);
    std::string LoadSafeTensors(const std::string& path);
    std::string Snapshot(OptimizerSnapshot* out) override;
    std::string ValidateSnapshot(const OptimizerSnapshot& s) override;
    std::string LoadSnapshot(const OptimizerSnapshot& s) override;
    const std::vector<ParameterGroup>& Groups() const { return groups_; }
    void groupScale(int n, float* stepSize, float* decay) const;

   private:
    std::vector<uint64_t> mGPU_, vGPU_;
    uint64_t graphStep_ = 0;
    std::vector<ParameterGroup> groups_;
    std::vector<int> groupOf_;
    oe_plan* plan_ = nullptr;
    int device_ = 0;
    bool closed_ = false;
    std::string refreshPlan();
    void run(float maxNorm, bool captured);
};

class SGD : public CheckpointOptimizer {
   public:
    std::vector<Parameter> Params;
    float LR = 0;
    int StepCount = 0;
    EngineOptions Engine;

    static std::string New(const std::vector<Parameter>& params, const SGDOptions& options, std::unique_ptr<SGD>* out);
    static std::string NewGroups(const std::vector<Parameter>& params, const SGDOptions& options,
                                 const std::vector<ParameterGroupSpec>& specs, std::unique_ptr<SGD>* out);
    ~SGD() override;
    void Step() override;
    void StepClipped(float maxNorm);
    // Eager: gradients become absent (set-to-none). Once prepared for graphs the buffers are kept
    // and zeroed, since a replay needs stable addresses (autograd/sgd.go:228-246).
    void ZeroGrad() override;
    float LearningRate() const override { return LR; }
    void SetLearningRate(float lr) override;
    void Close() override;
    std::string PrepareGraph();       // autograd/cuda_sgd.go:99-115
    std::string GraphStepCount(int* out);
    std::string SyncGraphStepCount();
    void StepCaptured();              // the capture branch of Step (autograd/sgd.go:167-172)
    SGDOptions config() const;
    std::string State(SGDState* out);
    std::string LoadState(const SGDState& state);
    std::string validateState(const SGDState& state);
    std::string SaveSafeTensors(const std::string& path);
    std::string LoadSafeTensors(const std::string& path);
    std::string Snapshot(OptimizerSnapshot* out) override;
    std::string ValidateSnapshot(const OptimizerSnapshot& s) override;
    std::string LoadSnapshot(const OptimizerSnapshot& s) override;
    void groupScale(int index, float* stepSize, float* decay) const;

   private:
    SGDOptions options_;
    std::vector<uint64_t> bufferGPU_, initializedGPU_;
    uint64_t graphStep_ = 0;
    std::vector<ParameterGroup> groups_;
    std::vector<int> groupOf_;
    oe_plan* plan_ = nullptr;
    int device_ = 0;
    bool closed_ = false;
    std::string validateOpen() const;
    std::string deviceStorage(std::vector<uint64_t>* buffers, std::vector<uint64_t>* flags);
    void freeStorage(std::vector<uint64_t>& buffers, std::vector<uint64_t>& flags);
    std::string refreshPlan();
    void run(float maxNorm, bool captured = false);
};

// ClipGradNorm for CUDA parameters (autograd/nn.go:310-317 + autograd/cuda_clip.go:114-134): the
// norm stays on the device, gradients are scaled in place when maxNorm > 0; returns NaN
// like the reference to avoid a host synchronisation. State is kept per (thread, device).
float ClipGradNorm(const std::vector<Parameter>& params, float maxNorm);
float GradientNormToHost();  // last norm of the calling thread on its device (autograd/nn.go:17-27)
void ReleaseClipState();     // frees the calling thread's clip plans

// GradAccumulator's bookkeeping (autograd/accumulate.go:15-71). Backward itself belongs to the
// autograd graph; MicroBatch() is what Backward does around it: it hands out the seed 1/groups,
// counts the micro-batch and reports whether the group is complete. A caller that accumulates
// unseeded gradients passes SeedScale() to EngineOptions::GradScale instead.
struct GradAccumulator {
    int groups = 0, pending = 0;
    static std::string New(int groups, GradAccumulator* out);
    std::string MicroBatch(float* seed, bool* complete);
    float SeedScale() const { return 1.0f / (float)groups; }
    int Pending() const { return pending; }
    int Groups() const { return groups; }
    void Reset() { pending = 0; }
};

// OneCycle schedule (autograd/nn.go:539-571).
struct OneCycle {
    double MaxLR = 0, PctStart = 0, DivFactor = 25, FinalDivFactor = 1e4;
    int Total = 0, StepCount = 0;
    static OneCycle New(double maxLR, int total, double pctStart);  // throws on an invalid configuration
    double LR() const;
    void Step(CheckpointOptimizer& o);
};
std::string validateOneCycle(const OneCycle& c);

// TrainingLoop (autograd/training_loop.go:53-214): the caller of ZeroGrad / Step / Schedule.Step.
// Reader, sampler, step, report and save are the caller's; they arrive as functions. A reader or a
// step reports how it ended with a status, the way the Go code tells io.EOF and context
// cancellation apart from other errors.
struct TrainingLoop {
    enum Status { Batch = 0, EndOfEpoch = 1, Cancelled = 2, Failed = 3 };
    std::function<int(std::string* err)> Next;                               // Reader.Next: a Status
    std::function<std::string()> NextEpoch;                                  // Reader.NextEpoch
    std::function<std::string(std::string* payload)> Position;               // Sampler.MarshalBinary; empty = no sampler
    std::function<int(float seed, double* loss, std::string* err)> Step;     // one micro-batch, backward seeded with seed: 0, Cancelled or Failed
    std::function<void(int update, double loss)> Report;                     // optional
    std::function<std::string(const std::string* savepoint)> Save;           // optional; savepoint may be null
    CheckpointOptimizer* Optimizer = nullptr;
    OneCycle* Schedule = nullptr;
    int Updates = 0, Applied = 0, Accumulate = 0, LogEvery = 0;
    // "" when the planned updates were applied (and saved); otherwise what stopped the run, with
    // *cancelled telling a cancellation (after which Save has run) from a failure.
    std::string Run(bool* cancelled);
};

// Entries / metadata of the checkpoint layout (autograd/optimizer_state.go:142-160,
// autograd/sgd_state.go:150-194, autograd/optimizer.go:85-120).
std::string optimizerEntries(OptimizerState state, EntryMap* entries, Metadata* metadata);
void optimizerMetadata(const OptimizerState& state, Metadata* metadata);
std::string optimizerStateFromEntries(const EntryMap& entries, const Metadata& metadata, int count, OptimizerState* out);
void sgdMetadata(const SGDState& state, Metadata* metadata);
std::string sgdEntries(SGDState state, EntryMap* entries, Metadata* metadata);
std::string sgdStateFromEntries(const EntryMap& entries, const Metadata& metadata, SGDState* out);
std::string snapshotEntries(const OptimizerSnapshot& s, EntryMap* entries, Metadata* metadata);
std::string snapshotFromEntries(const EntryMap& entries, Metadata metadata, OptimizerSnapshot* out);

// Training checkpoint "gograd-training-1" (autograd/training_checkpoint.go:13-132). The
// model is the list of named tensors a Module would report (parameters and buffers).
std::string SaveTrainingCheckpoint(const std::string& path, const std::vector<Parameter>& model,
                                   CheckpointOptimizer* optimizer, const OneCycle* scheduler,
                                   const std::map<std::string, std::string>& user);
std::string LoadTrainingCheckpoint(const std::string& path, const std::vector<Parameter>& model,
                                   CheckpointOptimizer* optimizer, OneCycle* scheduler,
                                   std::map<std::string, std::string>* user);
std::string TrainingCheckpointMetadata(const std::string& path, std::map<std::string, std::string>* user);

}  // namespace autograd
#endif
