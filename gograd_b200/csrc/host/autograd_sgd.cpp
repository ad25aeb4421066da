// SGD of the host mirror (PyTorch semantics as in autograd/sgd.go): validation before any
// mutation, lazily initialised momentum tracked by a per-parameter device flag, eager
// ZeroGrad that makes gradients absent, and two engine launches per step.
#include <climits>
#include <cmath>
#include <cstring>
#include <set>

#include "autograd.hpp"

namespace autograd {

namespace {
std::string engine_error(const char* op, int rc) {
    return std::string("cuda: ") + op + " failed (" + std::to_string(rc) + "): " + oe_last_error();
}

// validateSGDParameters (autograd/sgd.go:47-74): distinct named, non-empty float32 leaves with
// distinct storage on one device.
std::string validateSGDParameters(const std::vector<Parameter>& params) {
    std::set<std::string> names;
    std::set<const Tensor*> storage;
    int device = 0;
    for (size_t i = 0; i < params.size(); i++) {
        const Parameter& p = params[i];
        if (p.Name.empty() || names.count(p.Name) || !p.Value) return "autograd: SGD needs distinct named parameters";
        const Tensor& v = *p.Value;
        if (v.Numel() < 1 || storage.count(&v) || v.buf == 0) return "autograd: SGD requires distinct contiguous float32 leaves";
        if (i == 0) device = v.Device;
        if (v.Device != device) return "autograd: SGD parameters must use one device";
        names.insert(p.Name);
        storage.insert(&v);
    }
    return "";
}
}  // namespace

std::string SGDOptions::validate() const {
    for (float v : {LR, Momentum, Dampening, WeightDecay})
        if (v < 0 || std::isnan(v) || std::isinf(v)) return "autograd: invalid SGD configuration";
    if (Nesterov && (Momentum <= 0 || Dampening != 0)) return "autograd: Nesterov needs positive momentum and zero dampening";
    return "";
}

std::string SGD::New(const std::vector<Parameter>& params, const SGDOptions& options, std::unique_ptr<SGD>* out) {
    return NewGroups(params, options, {}, out);
}

std::string SGD::NewGroups(const std::vector<Parameter>& params, const SGDOptions& options_in,
                           const std::vector<ParameterGroupSpec>& specs, std::unique_ptr<SGD>* out) {
    // NewSGD passes no specs; NewSGDGroups requires some and refuses a decay in the options
    // (autograd/sgd.go:76-96). The caller distinguishes the two by passing specs or not.
    SGDOptions options = options_in;
    if (!specs.empty() && options.WeightDecay != 0) return "autograd: set weight decay on the parameter groups, not SGDOptions";
    std::string e = options.validate();
    if (!e.empty()) return e;
    if (!(e = validateSGDParameters(params)).empty()) return e;
    std::unique_ptr<SGD> o(new SGD());
    if (!(e = resolveParameterGroups(params, specs, &o->groups_, &o->groupOf_)).empty()) return e;
    if (specs.empty())
        o->groups_[0].WeightDecay = options.WeightDecay;
    else
        options.WeightDecay = o->groups_[0].WeightDecay;
    o->Params = params;
    o->LR = options.LR;
    o->options_ = options;
    o->device_ = params.empty() ? 0 : params[0].Value->Device;
    int rc = oe_init(o->device_);
    if (rc != 0) return engine_error("oe_init", rc);
    if (!params.empty() && options.Momentum > 0) {
        if (!(e = o->deviceStorage(&o->bufferGPU_, &o->initializedGPU_)).empty()) return e;
    }
    *out = std::move(o);
    return "";
}

// sgdDeviceStorage (autograd/cuda_sgd.go:39-65): a zeroed buffer and a zeroed one-float flag per parameter.
std::string SGD::deviceStorage(std::vector<uint64_t>* buffers, std::vector<uint64_t>* flags) {
    buffers->clear();
    flags->clear();
    for (const Parameter& p : Params) {
        uint64_t b = 0, f = 0, n = (uint64_t)p.Value->Numel();
        int rc;
        if ((rc = oe_mem_alloc(device_, n * 4, &b)) != 0 || (rc = oe_memset_u32(device_, b, 0, n, 0)) != 0 ||
            (rc = oe_mem_alloc(device_, 4, &f)) != 0 || (rc = oe_memset_u32(device_, f, 0, 1, 0)) != 0) {
            oe_mem_free(device_, b);
            oe_mem_free(device_, f);
            freeStorage(*buffers, *flags);
            return engine_error("SGD momentum storage", rc);
        }
        buffers->push_back(b);
        flags->push_back(f);
    }
    return "";
}

void SGD::freeStorage(std::vector<uint64_t>& buffers, std::vector<uint64_t>& flags) {
    for (uint64_t b : buffers) oe_mem_free(device_, b);
    for (uint64_t f : flags) oe_mem_free(device_, f);
    buffers.clear();
    flags.clear();
}

SGD::~SGD() { Close(); }

void SGD::Close() {
    if (closed_) return;
    oe_plan_destroy(plan_);
    plan_ = nullptr;
    freeStorage(bufferGPU_, initializedGPU_);
    if (graphStep_ != 0) oe_mem_free(device_, graphStep_);
    graphStep_ = 0;
    closed_ = true;
}

void SGD::groupScale(int index, float* stepSize, float* decay) const {
    const ParameterGroup& g = groups_[groupOf_[index]];
    *stepSize = LR * g.LRScale;  // autograd/sgd.go:127-130: the decay is not scaled by the rate
    *decay = g.WeightDecay;
}

void SGD::SetLearningRate(float lr) {
    std::string e = validateLearningRate(lr);
    if (!e.empty()) throw std::runtime_error(e);
    LR = lr;
}

SGDOptions SGD::config() const {
    SGDOptions c = options_;
    c.LR = LR;
    return c;
}

std::string SGD::validateOpen() const {
    if (closed_) return "autograd: SGD is closed";
    std::string e = config().validate();
    if (!e.empty()) return e;
    if (groups_.empty() || groupOf_.size() != Params.size()) return "autograd: SGD parameter group configuration is incomplete";
    if (!Params.empty() && options_.Momentum > 0 &&
        (bufferGPU_.size() != Params.size() || initializedGPU_.size() != Params.size()))
        return "autograd: incomplete SGD device storage";
    return validateSGDParameters(Params);
}

std::string SGD::refreshPlan() {
    std::vector<oe_tensor_desc> descs;
    for (size_t i = 0; i < Params.size(); i++) {
        Tensor& t = *Params[i].Value;
        if (Engine.WriteShadow && t.gradBuf != 0) {
            std::string e = t.ShadowForWriting();  // never the buffer a graph node still leases
            if (!e.empty()) return e;
        }
        const ParameterGroup& g = groups_[groupOf_[i]];
        oe_tensor_desc d;
        memset(&d, 0, sizeof d);
        d.param = t.buf;
        d.grad = t.gradBuf;
        if (options_.Momentum > 0) {
            d.state1 = bufferGPU_[i];
            d.state2 = initializedGPU_[i];
        }
        d.shadow = Engine.WriteShadow ? t.bf16Buf : 0;
        d.numel = (uint64_t)t.Numel();
        d.lr_scale = g.LRScale;
        d.weight_decay = g.WeightDecay;
        descs.push_back(d);
    }
    int rc = plan_ == nullptr ? oe_plan_create(device_, descs.data(), (uint32_t)descs.size(), 0, &plan_)
                              : oe_plan_update(plan_, descs.data(), (uint32_t)descs.size(), Engine.Stream);
    return rc == 0 ? "" : engine_error("optimizer plan", rc);
}

void SGD::run(float maxNorm, bool captured) {
    std::string e = validateOpen();
    if (!e.empty()) throw std::runtime_error(e);
    if (captured && graphStep_ == 0) throw std::runtime_error("autograd: call SGD.PrepareGraph before capture");
    if (!std::isfinite(Engine.GradScale) || !(Engine.GradScale > 0)) throw std::runtime_error("autograd: invalid gradient scale");
    // Zeroing inside Step equals ZeroGrad only where ZeroGrad zeroes: once prepared for graphs. Eager
    // ZeroGrad makes gradients absent, and a zeroed buffer is not an absent one.
    if (Engine.ZeroGradInStep && graphStep_ == 0)
        throw std::runtime_error("autograd: SGD.ZeroGrad releases its gradients; zeroing them inside Step would update parameters that are skipped today");
    if (!captured) {
        if (graphStep_ != 0 && !(e = SyncGraphStepCount()).empty()) throw std::runtime_error(e);
        if (StepCount >= INT32_MAX) throw std::runtime_error("autograd: SGD step count overflow");
        StepCount++;
    }
    if (!(e = refreshPlan()).empty()) throw std::runtime_error(e);
    int rc = oe_plan_set_grad_scale(plan_, &Engine.GradScale);
    if (rc != 0) throw std::runtime_error(engine_error("oe_plan_set_grad_scale", rc));
    oe_sgd_hparams hp;
    memset(&hp, 0, sizeof hp);
    hp.lr = LR;
    hp.momentum = options_.Momentum;
    hp.dampening = options_.Dampening;
    hp.max_norm = maxNorm;
    hp.flags = (options_.Nesterov ? OE_NESTEROV : 0u) | (options_.Maximize ? OE_MAXIMIZE : 0u) |
               (Engine.WriteShadow ? OE_WRITE_SHADOW : 0u) | (Engine.ClipDevForm ? OE_CLIP_DEVFORM : 0u) |
               (Engine.ZeroGradInStep ? OE_ZERO_GRAD : 0u);
    if (captured) hp.step_dev = graphStep_;  // the launch advances the device counter (sgd_step, autograd/cuda_sgd.go:67-70)
    if (maxNorm > 0 && (rc = oe_grad_norm(plan_, 0, Engine.Stream)) != 0) throw std::runtime_error(engine_error("oe_grad_norm", rc));
    if ((rc = oe_sgd_step(plan_, &hp, Engine.Stream)) != 0) throw std::runtime_error(engine_error("oe_sgd_step", rc));
    if (captured) return;  // a captured step changes no host state (autograd/cuda_sgd.go:94-96)
    for (Parameter& p : Params) {
        Tensor& t = *p.Value;
        if (t.gradBuf == 0) continue;
        t.version++;  // autograd/cuda_sgd.go:94-96 invalidates here; the engine rewrote the shadow instead
        if (Engine.WriteShadow && t.bf16Buf != 0) t.bf16Version = t.version;
        if (Engine.ZeroGradInStep) t.gradKnownZero = true;
    }
    if (graphStep_ != 0 && !(e = PrepareGraph()).empty()) throw std::runtime_error(e);
}

void SGD::Step() { run(0.0f); }
void SGD::StepClipped(float maxNorm) { run(maxNorm); }
void SGD::StepCaptured() { run(0.0f, true); }

void SGD::ZeroGrad() {
    std::string e = validateOpen();
    if (!e.empty()) throw std::runtime_error(e);
    if (graphStep_ != 0) {  // prepared for graphs: keep the buffers, zero them (autograd/sgd.go:236-239)
        for (Parameter& p : Params) {
            if (p.Value->gradBuf == 0 || p.Value->gradKnownZero) continue;
            if (!(e = p.Value->ZeroGrad()).empty()) throw std::runtime_error(e);
        }
        return;
    }
    for (Parameter& p : Params) p.Value->FreeGrad();  // set-to-none (autograd/sgd.go:240-245)
}

std::string SGD::PrepareGraph() {
    std::string e = validateOpen();
    if (!e.empty()) return e;
    if (Params.empty()) return "cuda: unavailable";
    int rc;
    if (graphStep_ == 0 && (rc = oe_mem_alloc(device_, 4, &graphStep_)) != 0) return engine_error("oe_mem_alloc", rc);
    int32_t step = (int32_t)StepCount;
    if ((rc = oe_memcpy_h2d(device_, graphStep_, &step, 4, Engine.Stream)) != 0) return engine_error("oe_memcpy_h2d", rc);
    if ((rc = oe_stream_sync(device_, Engine.Stream)) != 0) return engine_error("oe_stream_sync", rc);
    return "";
}

std::string SGD::GraphStepCount(int* out) {
    if (closed_ || graphStep_ == 0) return "cuda: unavailable";
    int32_t step = 0;
    int rc;
    if ((rc = oe_memcpy_d2h(device_, &step, graphStep_, 4, Engine.Stream)) != 0) return engine_error("oe_memcpy_d2h", rc);
    if ((rc = oe_stream_sync(device_, Engine.Stream)) != 0) return engine_error("oe_stream_sync", rc);
    *out = step;
    return "";
}

std::string SGD::SyncGraphStepCount() {
    int step = 0;
    std::string e = GraphStepCount(&step);
    if (e.empty()) StepCount = step;
    return e;
}

// ---- state (autograd/sgd_state.go) ------------------------------------------------------
std::string SGD::State(SGDState* out) {
    std::string e = validateOpen();
    if (!e.empty()) return e;
    SGDState s;
    s.StepCount = StepCount;
    if (graphStep_ != 0 && !(e = GraphStepCount(&s.StepCount)).empty()) return e;  // autograd/sgd_state.go:31-37
    s.Options = config();
    s.Initialized.assign(Params.size(), false);
    s.Buffers.resize(Params.size());
    for (size_t i = 0; i < Params.size(); i++) {
        s.Names.push_back(Params[i].Name);
        s.Shapes.push_back(Params[i].Value->Shape);
        if (initializedGPU_.empty()) continue;
        float flag = 0;
        int rc;
        if ((rc = oe_memcpy_d2h(device_, &flag, initializedGPU_[i], 4, Engine.Stream)) != 0 ||
            (rc = oe_stream_sync(device_, Engine.Stream)) != 0)
            return engine_error("oe_memcpy_d2h", rc);
        if (flag != 0 && flag != 1) return "autograd: invalid SGD initialization flag";
        s.Initialized[i] = flag == 1;
        if (s.Initialized[i]) {
            s.Buffers[i].assign((size_t)Params[i].Value->Numel(), 0.f);
            if ((rc = oe_memcpy_d2h(device_, s.Buffers[i].data(), bufferGPU_[i], s.Buffers[i].size() * 4, Engine.Stream)) != 0 ||
                (rc = oe_stream_sync(device_, Engine.Stream)) != 0)
                return engine_error("oe_memcpy_d2h", rc);
        }
    }
    s.Groups = groupStates(groups_, s.Names);
    *out = std::move(s);
    return "";
}

std::string SGD::validateState(const SGDState& s) {
    std::string e = validateOpen();
    if (!e.empty()) return e;
    if (!(e = s.Options.validate()).empty()) return e;
    size_t n = Params.size();
    if (s.StepCount < 0 || s.Names.size() != n || s.Shapes.size() != n || s.Buffers.size() != n || s.Initialized.size() != n)
        return "autograd: invalid SGD state count";
    for (size_t i = 0; i < n; i++) {
        if (s.Names[i] != Params[i].Name || s.Shapes[i] != Params[i].Value->Shape)
            return "autograd: SGD parameter " + std::to_string(i) + " name/shape mismatch";
        if (s.Initialized[i]) {
            if (s.Options.Momentum <= 0 || s.StepCount == 0 || (int)s.Buffers[i].size() != Params[i].Value->Numel())
                return "autograd: invalid SGD momentum buffer " + std::to_string(i);
        } else if (!s.Buffers[i].empty()) {
            return "autograd: uninitialized SGD buffer has values";
        }
        for (float v : s.Buffers[i])
            if (std::isnan(v) || std::isinf(v)) return "autograd: non-finite SGD momentum";
    }
    std::vector<ParameterGroup> resolved;
    return validateGroupStates(groups_, s.Names, s.Groups, s.Options.WeightDecay, &resolved);
}

std::string SGD::LoadState(const SGDState& s) {
    std::string e = validateState(s);
    if (!e.empty()) return e;
    // Fresh device storage is filled first and swapped in only when every copy succeeded.
    std::vector<uint64_t> buffers, flags;
    if (!Params.empty() && s.Options.Momentum > 0) {
        if (!(e = deviceStorage(&buffers, &flags)).empty()) return e;
        const float one = 1.0f;
        for (size_t i = 0; i < s.Initialized.size(); i++) {
            if (!s.Initialized[i]) continue;
            int rc;
            if ((rc = oe_memcpy_h2d(device_, buffers[i], s.Buffers[i].data(), s.Buffers[i].size() * 4, Engine.Stream)) != 0 ||
                (rc = oe_memcpy_h2d(device_, flags[i], &one, 4, Engine.Stream)) != 0 ||
                (rc = oe_stream_sync(device_, Engine.Stream)) != 0) {
                freeStorage(buffers, flags);
                return engine_error("oe_memcpy_h2d", rc);
            }
        }
    }
    freeStorage(bufferGPU_, initializedGPU_);
    bufferGPU_ = buffers;
    initializedGPU_ = flags;
    options_ = s.Options;
    LR = s.Options.LR;
    std::vector<ParameterGroup> groups;
    if (!(e = validateGroupStates(groups_, s.Names, s.Groups, s.Options.WeightDecay, &groups)).empty()) return e;
    groups_ = groups;
    groupOf_.assign(Params.size(), 0);
    for (size_t g = 0; g < groups_.size(); g++)
        for (int index : groups_[g].Indexes) groupOf_[index] = (int)g;
    options_.WeightDecay = groups_[0].WeightDecay;
    StepCount = s.StepCount;
    if (graphStep_ != 0) return PrepareGraph();  // autograd/sgd_state.go:145-147
    return "";
}

std::string SGD::SaveSafeTensors(const std::string& path) {
    SGDState s;
    std::string e = State(&s);
    if (!e.empty()) return e;
    if (!(e = validateState(s)).empty()) return e;
    EntryMap entries;
    Metadata metadata;
    if (!(e = sgdEntries(std::move(s), &entries, &metadata)).empty()) return e;
    return write_safetensors(path, entries, &metadata);
}

std::string SGD::LoadSafeTensors(const std::string& path) {
    EntryMap entries;
    Metadata metadata;
    std::string e = read_safetensors(path, &entries, &metadata);
    if (!e.empty()) return e;
    SGDState s;
    if (!(e = sgdStateFromEntries(entries, metadata, &s)).empty()) return e;
    return LoadState(s);
}

std::string SGD::Snapshot(OptimizerSnapshot* out) {
    auto s = std::make_shared<SGDState>();
    std::string e = State(s.get());
    if (!e.empty()) return e;
    out->Version = 1;
    out->Kind = "sgd";
    out->SGD = s;
    out->AdamW.reset();
    return "";
}

std::string SGD::ValidateSnapshot(const OptimizerSnapshot& s) {
    if (s.Version != 1 || s.Kind != "sgd" || !s.SGD || s.AdamW) return "autograd: incompatible SGD snapshot";
    return validateState(*s.SGD);
}

std::string SGD::LoadSnapshot(const OptimizerSnapshot& s) {
    std::string e = ValidateSnapshot(s);
    if (!e.empty()) return e;
    return LoadState(*s.SGD);
}

}  // namespace autograd
