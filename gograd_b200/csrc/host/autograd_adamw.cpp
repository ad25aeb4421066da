// AdamW of the host mirror: the reference's constructor checks, group scaling, shared step
// counter and host-side bias corrections around ONE engine launch per step.
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
}  // namespace

std::string AdamW::New(const std::vector<Parameter>& params, float lr, float decay, std::unique_ptr<AdamW>* out) {
    // NewAdamW (autograd/nn.go:385-395): one implicit group named "default" with the given decay.
    ParameterGroupSpec spec;
    spec.Name = DefaultParameterGroupName;
    spec.Params = params;
    spec.WeightDecay = decay;
    return NewGroups(params, lr, {spec}, out);
}

std::string AdamW::NewGroups(const std::vector<Parameter>& params, float lr,
                             const std::vector<ParameterGroupSpec>& specs, std::unique_ptr<AdamW>* out) {
    if (specs.empty()) return "autograd: NewAdamWGroups needs at least one parameter group";
    std::string e = validateLearningRate(lr);
    if (!e.empty()) return e;
    // newAdamW (autograd/nn.go:407-458): values present, distinct non-empty names, one device.
    std::set<std::string> seen;
    int device = 0;
    for (size_t i = 0; i < params.size(); i++) {
        const Parameter& p = params[i];
        if (!p.Value) return "autograd: AdamW needs parameter values";
        if (p.Name.empty() || seen.count(p.Name)) return "autograd: AdamW needs distinct named parameters";
        seen.insert(p.Name);
        if (i == 0) device = p.Value->Device;
        if (p.Value->Device != device) return "autograd: AdamW parameters must use one device";
    }
    std::unique_ptr<AdamW> o(new AdamW());
    if (!(e = resolveParameterGroups(params, specs, &o->groups_, &o->groupOf_)).empty()) return e;
    o->Params = params;
    o->LR = lr;
    o->WeightDecay = o->groups_[0].WeightDecay;
    o->device_ = device;
    int rc = oe_init(device);
    if (rc != 0) return engine_error("oe_init", rc);
    for (const Parameter& p : params) {
        uint64_t m = 0, v = 0;
        uint64_t n = (uint64_t)p.Value->Numel();
        if (n > 0) {
            if ((rc = oe_mem_alloc(device, n * 4, &m)) != 0 || (rc = oe_mem_alloc(device, n * 4, &v)) != 0 ||
                (rc = oe_memset_u32(device, m, 0, n, 0)) != 0 || (rc = oe_memset_u32(device, v, 0, n, 0)) != 0) {
                oe_mem_free(device, m);
                oe_mem_free(device, v);
                return engine_error("AdamW state allocation", rc);
            }
        }
        o->mGPU_.push_back(m);
        o->vGPU_.push_back(v);
    }
    *out = std::move(o);
    return "";
}

AdamW::~AdamW() { Close(); }

void AdamW::Close() {
    if (closed_) return;
    closed_ = true;
    oe_plan_destroy(plan_);
    plan_ = nullptr;
    for (uint64_t b : mGPU_) oe_mem_free(device_, b);
    for (uint64_t b : vGPU_) oe_mem_free(device_, b);
    oe_mem_free(device_, graphStep_);
    mGPU_.clear();
    vGPU_.clear();
    graphStep_ = 0;
}

void AdamW::groupScale(int n, float* stepSize, float* decay) const {
    // autograd/nn.go:461-465, in float32
    const ParameterGroup& g = groups_[groupOf_[n]];
    *stepSize = LR * g.LRScale;
    *decay = *stepSize * g.WeightDecay;
}

void AdamW::SetLearningRate(float lr) {
    std::string e = validateLearningRate(lr);
    if (!e.empty()) throw std::runtime_error(e);
    LR = lr;
}

// One descriptor per parameter; a parameter without a gradient keeps grad = 0 and is
// skipped by the engine exactly like a nil gradBuf (autograd/nn.go:497-499).
std::string AdamW::refreshPlan() {
    std::vector<oe_tensor_desc> descs;
    for (size_t i = 0; i < Params.size(); i++) {
        Tensor& t = *Params[i].Value;
        if (t.Numel() == 0) continue;
        if (Engine.WriteShadow && t.gradBuf != 0) {
            std::string e = t.ShadowForWriting();  // never the buffer a graph node still leases
            if (!e.empty()) return e;
        }
        const ParameterGroup& g = groups_[groupOf_[i]];
        oe_tensor_desc d;
        memset(&d, 0, sizeof d);
        d.param = t.buf;
        d.grad = t.gradBuf;
        d.state1 = mGPU_[i];
        d.state2 = vGPU_[i];
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

void AdamW::run(float maxNorm, bool captured) {
    if (closed_) throw std::runtime_error("autograd: AdamW is closed");
    if (captured && graphStep_ == 0) throw std::runtime_error("autograd: call AdamW.PrepareGraph before capture");
    if (!std::isfinite(Engine.GradScale) || !(Engine.GradScale > 0)) throw std::runtime_error("autograd: invalid gradient scale");
    if (!captured) {
        if (graphStep_ != 0) {
            std::string e = SyncGraphStepCount();
            if (!e.empty()) throw std::runtime_error(e);
        }
        StepCount++;  // one shared counter, even for parameters without gradients (autograd/nn.go:492)
    }
    std::string e = refreshPlan();
    if (!e.empty()) throw std::runtime_error(e);
    int rc = oe_plan_set_grad_scale(plan_, &Engine.GradScale);
    if (rc != 0) throw std::runtime_error(engine_error("oe_plan_set_grad_scale", rc));
    oe_adamw_hparams hp;
    memset(&hp, 0, sizeof hp);
    hp.lr = LR;
    hp.beta1 = Beta1;
    hp.beta2 = Beta2;
    hp.eps = Eps;
    if (captured) {
        hp.step_dev = graphStep_;
    } else {
        hp.bc1 = (float)(1.0 - std::pow((double)Beta1, (double)StepCount));  // autograd/nn.go:493-494
        hp.bc2 = (float)(1.0 - std::pow((double)Beta2, (double)StepCount));
    }
    hp.max_norm = maxNorm;
    hp.flags = (Engine.WriteShadow ? OE_WRITE_SHADOW : 0u) | (Engine.ClipDevForm ? OE_CLIP_DEVFORM : 0u) |
               (Engine.ZeroGradInStep ? OE_ZERO_GRAD : 0u);
    if (maxNorm > 0 && (rc = oe_grad_norm(plan_, 0, Engine.Stream)) != 0) throw std::runtime_error(engine_error("oe_grad_norm", rc));
    if ((rc = oe_adamw_step(plan_, &hp, Engine.Stream)) != 0) throw std::runtime_error(engine_error("oe_adamw_step", rc));
    if (!captured) {
        for (Parameter& p : Params) {
            Tensor& t = *p.Value;
            if (t.gradBuf == 0) continue;
            // Where the reference invalidates the shadow (autograd/nn.go:504), the engine has just
            // rewritten it: bump the version and stamp the shadow as current.
            t.version++;
            if (Engine.WriteShadow && t.bf16Buf != 0) t.bf16Version = t.version;
            if (Engine.ZeroGradInStep) t.gradKnownZero = true;  // the update stored zeros over what it read
        }
        if (graphStep_ != 0) {
            std::string e2 = PrepareGraph();
            if (!e2.empty()) throw std::runtime_error(e2);
        }
    }
}

void AdamW::Step() { run(0.0f, false); }
void AdamW::StepClipped(float maxNorm) { run(maxNorm, false); }
void AdamW::StepCaptured() { run(0.0f, true); }

float AdamW::LastGradNorm() {
    if (plan_ == nullptr) return 0.0f;
    float norm = 0;
    int rc = oe_read_norm(plan_, &norm, nullptr, Engine.Stream);
    if (rc != 0) throw std::runtime_error(engine_error("oe_read_norm", rc));
    return norm;
}

void AdamW::ZeroGrad() {
    // AdamW.ZeroGrad keeps the buffers and zeroes them (autograd/nn.go:533-537); one launch
    // when the plan already describes the current gradients, else per tensor; nothing at all when
    // every present gradient is known to hold zeros already (the last Step zeroed them).
    bool dirty = false;
    for (const Parameter& p : Params) dirty = dirty || (p.Value->gradBuf != 0 && !p.Value->gradKnownZero);
    if (!dirty) return;
    if (plan_ != nullptr && refreshPlan().empty()) {
        int rc = oe_zero_grads(plan_, Engine.Stream);
        if (rc != 0) throw std::runtime_error(engine_error("oe_zero_grads", rc));
        for (Parameter& p : Params)
            if (p.Value->gradBuf != 0) p.Value->gradKnownZero = true;
        return;
    }
    for (Parameter& p : Params) {
        std::string e = p.Value->ZeroGrad();
        if (!e.empty()) throw std::runtime_error(e);
    }
}

std::string AdamW::PrepareGraph() {
    if (Params.empty()) return "cuda: unavailable";
    int rc;
    if (graphStep_ == 0 && (rc = oe_mem_alloc(device_, 4, &graphStep_)) != 0) return engine_error("oe_mem_alloc", rc);
    int32_t step = (int32_t)StepCount;
    if ((rc = oe_memcpy_h2d(device_, graphStep_, &step, 4, Engine.Stream)) != 0) return engine_error("oe_memcpy_h2d", rc);
    if ((rc = oe_stream_sync(device_, Engine.Stream)) != 0) return engine_error("oe_stream_sync", rc);
    return "";
}

std::string AdamW::GraphStepCount(int* out) {
    if (graphStep_ == 0) return "cuda: unavailable";
    int32_t step = 0;
    int rc;
    if ((rc = oe_memcpy_d2h(device_, &step, graphStep_, 4, Engine.Stream)) != 0) return engine_error("oe_memcpy_d2h", rc);
    if ((rc = oe_stream_sync(device_, Engine.Stream)) != 0) return engine_error("oe_stream_sync", rc);
    *out = step;
    return "";
}

std::string AdamW::SyncGraphStepCount() {
    int step = 0;
    std::string e = GraphStepCount(&step);
    if (e.empty()) StepCount = step;
    return e;
}

// ---- state (autograd/optimizer_state.go) ---------------------------------------------
std::string AdamW::State(OptimizerState* out) {
    if (closed_ || mGPU_.size() != Params.size() || vGPU_.size() != Params.size())
        return "autograd: incomplete CUDA optimizer storage";
    OptimizerState s;
    s.StepCount = StepCount;
    if (graphStep_ != 0) {
        std::string e = GraphStepCount(&s.StepCount);
        if (!e.empty()) return e;
    }
    s.LR = LR;
    s.WeightDecay = WeightDecay;
    s.Beta1 = Beta1;
    s.Beta2 = Beta2;
    s.Eps = Eps;
    s.Moments.resize(Params.size());
    for (size_t i = 0; i < Params.size(); i++) {
        s.Names.push_back(Params[i].Name);
        s.Shapes.push_back(Params[i].Value->Shape);
        size_t n = (size_t)Params[i].Value->Numel();
        s.Moments[i].M.assign(n, 0.f);
        s.Moments[i].V.assign(n, 0.f);
        if (n > 0) {
            int rc;
            if ((rc = oe_memcpy_d2h(device_, s.Moments[i].M.data(), mGPU_[i], n * 4, Engine.Stream)) != 0 ||
                (rc = oe_memcpy_d2h(device_, s.Moments[i].V.data(), vGPU_[i], n * 4, Engine.Stream)) != 0)
                return engine_error("oe_memcpy_d2h", rc);
        }
    }
    int rc = oe_stream_sync(device_, Engine.Stream);
    if (rc != 0) return engine_error("oe_stream_sync", rc);
    s.Groups = groupStates(groups_, s.Names);
    *out = std::move(s);
    return "";
}

std::string AdamW::validateState(const OptimizerState& state) {
    // autograd/optimizer_state.go:228-259; nothing is mutated here.
    if (closed_ || mGPU_.size() != Params.size()) return "autograd: incomplete CUDA optimizer storage";
    size_t n = Params.size();
    if (state.StepCount < 0 || state.Moments.size() != n ||  // an int cannot exceed MaxInt32
       
        state.Names.size() != n || state.Shapes.size() != n)
        return "autograd: invalid optimizer step or parameter count";
    for (float v : {state.LR, state.WeightDecay, state.Beta1, state.Beta2, state.Eps})
        if (std::isnan(v) || std::isinf(v)) return "autograd: non-finite optimizer configuration";
    if (state.LR < 0 || state.WeightDecay < 0 || state.Beta1 < 0 || state.Beta1 >= 1 || state.Beta2 < 0 ||
        state.Beta2 >= 1 || state.Eps <= 0)
        return "autograd: invalid optimizer configuration";
    std::vector<std::string> names;
    for (const Parameter& p : Params) names.push_back(p.Name);
    std::vector<ParameterGroup> resolved;
    std::string e = validateGroupStates(groups_, names, state.Groups, state.WeightDecay, &resolved);
    if (!e.empty()) return e;
    for (size_t i = 0; i < n; i++) {
        size_t count = (size_t)Params[i].Value->Numel();
        if (state.Names[i] != Params[i].Name || state.Shapes[i] != Params[i].Value->Shape ||
            state.Moments[i].M.size() != count || state.Moments[i].V.size() != count)
            return "autograd: optimizer parameter " + std::to_string(i) + " name or shape mismatch";
        for (size_t j = 0; j < count; j++) {
            float m = state.Moments[i].M[j], v = state.Moments[i].V[j];
            if (std::isnan(m) || std::isinf(m) || std::isnan(v) || std::isinf(v) || v < 0)
                return "autograd: invalid optimizer moment " + std::to_string(i) + "/" + std::to_string(j);
        }
    }
    return "";
}

std::string AdamW::LoadState(const OptimizerState& state) {
    std::string e = validateState(state);
    if (!e.empty()) return e;
    for (size_t i = 0; i < Params.size(); i++) {
        size_t n = (size_t)Params[i].Value->Numel();
        if (n == 0) continue;
        int rc;
        if ((rc = oe_memcpy_h2d(device_, mGPU_[i], state.Moments[i].M.data(), n * 4, Engine.Stream)) != 0 ||
            (rc = oe_memcpy_h2d(device_, vGPU_[i], state.Moments[i].V.data(), n * 4, Engine.Stream)) != 0)
            return engine_error("oe_memcpy_h2d", rc);
    }
    int rc = oe_stream_sync(device_, Engine.Stream);
    if (rc != 0) return engine_error("oe_stream_sync", rc);
    StepCount = state.StepCount;
    LR = state.LR;
    WeightDecay = state.WeightDecay;
    Beta1 = state.Beta1;
    Beta2 = state.Beta2;
    Eps = state.Eps;
    std::vector<std::string> names;
    for (const Parameter& p : Params) names.push_back(p.Name);
    std::vector<ParameterGroup> groups;
    if (!(e = validateGroupStates(groups_, names, state.Groups, state.WeightDecay, &groups)).empty()) return e;
    groups_ = groups;
    groupOf_.assign(Params.size(), 0);
    for (size_t g = 0; g < groups_.size(); g++)
        for (int index : groups_[g].Indexes) groupOf_[index] = (int)g;
    WeightDecay = groups_[0].WeightDecay;
    if (graphStep_ != 0) return PrepareGraph();
    return "";
}

std::string AdamW::SaveSafeTensors(const std::string& path) {
    OptimizerState s;
    std::string e = State(&s);
    if (!e.empty()) return e;
    EntryMap entries;
    Metadata metadata;
    if (!(e = optimizerEntries(std::move(s), &entries, &metadata)).empty()) return e;
    return write_safetensors(path, entries, &metadata);
}

std::string AdamW::LoadSafeTensors(const std::string& path) {
    EntryMap entries;
    Metadata metadata;
    std::string e = read_safetensors(path, &entries, &metadata);
    if (!e.empty()) return e;
    OptimizerState s;
    if (!(e = optimizerStateFromEntries(entries, metadata, (int)Params.size(), &s)).empty()) return e;
    return LoadState(s);
}

std::string AdamW::Snapshot(OptimizerSnapshot* out) {
    auto s = std::make_shared<OptimizerState>();
    std::string e = State(s.get());
    if (!e.empty()) return e;
    out->Version = 1;
    out->Kind = "adamw";
    out->AdamW = s;
    out->SGD.reset();
    return "";
}

std::string AdamW::ValidateSnapshot(const OptimizerSnapshot& s) {
    if (s.Version != 1 || s.Kind != "adamw" || !s.AdamW || s.SGD) return "autograd: incompatible AdamW snapshot";
    return validateState(*s.AdamW);
}

std::string AdamW::LoadSnapshot(const OptimizerSnapshot& s) {
    std::string e = ValidateSnapshot(s);
    if (!e.empty()) return e;
    return LoadState(*s.AdamW);
}

}  // namespace autograd
