// Tensors, parameter groups, clip state and the OneCycle schedule of the host mirror.
#include <cmath>
#include <cstring>
#include <mutex>
#include <set>
#include <thread>

#include "autograd.hpp"

namespace autograd {

namespace {
std::string engine_error(const char* op, int rc) {
    return std::string("cuda: ") + op + " failed (" + std::to_string(rc) + "): " + oe_last_error();
}
bool bad_float(float v) { return std::isnan(v) || std::isinf(v); }
}  // namespace

#define GG_TRY(call, op)                          \
    do {                                          \
        int gg_rc_ = (call);                      \
        if (gg_rc_ != 0) return engine_error(op, gg_rc_); \
    } while (0)

// -------------------------------------------------------------------------------------
// Tensor
// -------------------------------------------------------------------------------------
std::string Tensor::New(const std::vector<float>& values, const std::vector<int>& shape, int device,
                        bool requiresGrad, std::shared_ptr<Tensor>* out) {
    long long n = 1;
    for (int d : shape) {
        if (d < 0) return "autograd: negative dimension";
        n *= d;
    }
    if (n != (long long)values.size()) return "autograd: value count does not match the shape";
    GG_TRY(oe_init(device), "oe_init");
    auto t = std::make_shared<Tensor>();
    t->Shape = shape;
    t->Device = device;
    t->RequiresGrad = requiresGrad;
    if (n > 0) {
        GG_TRY(oe_mem_alloc(device, (uint64_t)n * 4, &t->buf), "oe_mem_alloc");
        GG_TRY(oe_memcpy_h2d(device, t->buf, values.data(), (uint64_t)n * 4, 0), "oe_memcpy_h2d");
        GG_TRY(oe_stream_sync(device, 0), "oe_stream_sync");
    }
    *out = t;
    return "";
}

Tensor::~Tensor() { Close(); }

int Tensor::Numel() const {
    long long n = 1;
    for (int d : Shape) n *= d;
    return (int)n;
}

void Tensor::Close() {
    if (closed_) return;
    closed_ = true;
    oe_mem_free(Device, buf);
    oe_mem_free(Device, gradBuf);
    oe_mem_free(Device, bf16Buf);
    for (auto& r : retired_) oe_mem_free(Device, r.first);
    retired_.clear();
    buf = gradBuf = bf16Buf = 0;
}

std::string Tensor::ToHost(std::vector<float>* out) const {
    out->assign((size_t)Numel(), 0.f);
    if (out->empty()) return "";
    GG_TRY(oe_memcpy_d2h(Device, out->data(), buf, out->size() * 4, 0), "oe_memcpy_d2h");
    GG_TRY(oe_stream_sync(Device, 0), "oe_stream_sync");
    return "";
}

std::string Tensor::GradToHost(std::vector<float>* out) const {
    if (gradBuf == 0) return "autograd: tensor has no gradient";
    out->assign((size_t)Numel(), 0.f);
    GG_TRY(oe_memcpy_d2h(Device, out->data(), gradBuf, out->size() * 4, 0), "oe_memcpy_d2h");
    GG_TRY(oe_stream_sync(Device, 0), "oe_stream_sync");
    return "";
}

std::string Tensor::CopyFromHost(const std::vector<float>& values) {
    if ((int)values.size() != Numel()) return "autograd: value count does not match the tensor";
    if (values.empty()) return "";
    GG_TRY(oe_memcpy_h2d(Device, buf, values.data(), values.size() * 4, 0), "oe_memcpy_h2d");
    GG_TRY(oe_stream_sync(Device, 0), "oe_stream_sync");
    version++;  // a write through the tensor invalidates its shadow (autograd/cuda_autocast.go:30-33)
    return "";
}

std::string Tensor::EnsureGrad() {
    if (gradBuf != 0 || Numel() == 0) return "";
    GG_TRY(oe_mem_alloc(Device, (uint64_t)Numel() * 4, &gradBuf), "oe_mem_alloc");
    GG_TRY(oe_memset_u32(Device, gradBuf, 0, (uint64_t)Numel(), 0), "oe_memset_u32");
    gradKnownZero = true;
    return "";
}

std::string Tensor::SetGrad(const std::vector<float>& values) {
    if ((int)values.size() != Numel()) return "autograd: gradient count does not match the tensor";
    std::string e = EnsureGrad();
    if (!e.empty()) return e;
    if (values.empty()) return "";
    gradKnownZero = false;
    GG_TRY(oe_memcpy_h2d(Device, gradBuf, values.data(), values.size() * 4, 0), "oe_memcpy_h2d");
    GG_TRY(oe_stream_sync(Device, 0), "oe_stream_sync");
    return "";
}

void Tensor::FreeGrad() {
    oe_mem_free(Device, gradBuf);
    gradBuf = 0;
    gradKnownZero = false;
}

std::string Tensor::ZeroGrad() {
    if (gradBuf == 0) return "";
    GG_TRY(oe_memset_u32(Device, gradBuf, 0, (uint64_t)Numel(), 0), "oe_memset_u32");
    gradKnownZero = true;
    return "";
}

std::string Tensor::EnsureShadow() {
    if (bf16Buf != 0 || Numel() == 0) return "";
    GG_TRY(oe_mem_alloc(Device, (uint64_t)Numel() * 2, &bf16Buf), "oe_mem_alloc");
    return "";
}

uint64_t Tensor::AcquireShadowLease() {
    if (bf16Buf == 0) return 0;
    leases_++;
    return bf16Buf;
}

void Tensor::ReleaseShadowLease(uint64_t address) {
    if (address == 0) return;
    if (address == bf16Buf && leases_ > 0) {
        leases_--;
        return;
    }
    for (size_t i = 0; i < retired_.size(); i++) {
        if (retired_[i].first != address) continue;
        if (--retired_[i].second <= 0) {
            oe_mem_free(Device, address);  // the last reader is gone
            retired_.erase(retired_.begin() + (long)i);
        }
        return;
    }
}

std::string Tensor::ShadowForWriting() {
    if (bf16Buf != 0 && leases_ > 0) {
        // Someone still reads the current shadow: keep it alive for them and write elsewhere.
        retired_.push_back({bf16Buf, leases_});
        bf16Buf = 0;
        leases_ = 0;
    }
    return EnsureShadow();
}

std::string Tensor::ShadowToHost(std::vector<uint16_t>* out) const {
    if (bf16Buf == 0) return "autograd: tensor has no bf16 shadow";
    out->assign((size_t)Numel(), 0);
    GG_TRY(oe_memcpy_d2h(Device, out->data(), bf16Buf, out->size() * 2, 0), "oe_memcpy_d2h");
    GG_TRY(oe_stream_sync(Device, 0), "oe_stream_sync");
    return "";
}

// -------------------------------------------------------------------------------------
// parameter groups (autograd/param_groups.go)
// -------------------------------------------------------------------------------------
std::string normalizeLRScale(float scale, float* out) {
    if (bad_float(scale) || scale < 0) return "autograd: invalid parameter group learning-rate scale";
    *out = scale == 0 ? 1.0f : scale;
    return "";
}

std::string validateGroupDecay(float decay) {
    if (decay < 0 || bad_float(decay)) return "autograd: invalid parameter group weight decay";
    return "";
}

std::string validateLearningRate(float lr) {
    if (lr < 0 || bad_float(lr)) return "autograd: invalid learning rate";
    return "";
}

std::string PartitionParameters(const std::vector<Parameter>& params, const std::vector<std::string>& labels,
                                std::vector<ParameterGroupSpec>* specs) {
    // labels[i] is what the reference's assign(name) callback returns for params[i]
    // (autograd/param_groups.go:63-102).
    if (labels.size() != params.size()) return "autograd: nil parameter group assignment";
    std::vector<std::string> order;
    std::map<std::string, std::vector<Parameter>> grouped;
    std::set<std::string> seen;
    for (size_t i = 0; i < params.size(); i++) {
        const Parameter& p = params[i];
        if (!p.Value) return "autograd: partition needs parameter values";
        if (seen.count(p.Name)) return "autograd: duplicate parameter name \"" + p.Name + "\"";
        seen.insert(p.Name);
        if (labels[i].empty()) return "autograd: parameter \"" + p.Name + "\" is not assigned to a group";
        if (!grouped.count(labels[i])) order.push_back(labels[i]);
        grouped[labels[i]].push_back(p);
    }
    if (order.empty()) return "autograd: no parameters to partition";
    specs->clear();
    for (const std::string& name : order) {
        ParameterGroupSpec s;
        s.Name = name;
        s.Params = grouped[name];
        specs->push_back(s);
    }
    return "";
}

std::string resolveParameterGroups(const std::vector<Parameter>& params, const std::vector<ParameterGroupSpec>& specs,
                                   std::vector<ParameterGroup>* groups, std::vector<int>* owner) {
    groups->clear();
    if (specs.empty()) {
        ParameterGroup g;
        g.Name = DefaultParameterGroupName;
        for (size_t i = 0; i < params.size(); i++) g.Indexes.push_back((int)i);
        g.LRScale = 1;
        groups->push_back(g);
        owner->assign(params.size(), 0);
        return "";
    }
    owner->assign(params.size(), -1);
    std::map<const Tensor*, int> lookup;  // by tensor identity, as the reference does
    for (size_t i = 0; i < params.size(); i++)
        if (params[i].Value) lookup[params[i].Value.get()] = (int)i;
    std::set<std::string> names;
    std::vector<std::string> specNames(specs.size());
    for (size_t index = 0; index < specs.size(); index++) {
        const ParameterGroupSpec& spec = specs[index];
        if (spec.Name.empty()) return "autograd: parameter group " + std::to_string(index) + " has no name";
        if (names.count(spec.Name)) return "autograd: duplicate parameter group \"" + spec.Name + "\"";
        names.insert(spec.Name);
        specNames[index] = spec.Name;
        float scale = 0;
        std::string e = normalizeLRScale(spec.LRScale, &scale);
        if (!e.empty()) return e;
        if (!(e = validateGroupDecay(spec.WeightDecay)).empty()) return e;
        if (spec.Params.empty() && !params.empty()) return "autograd: parameter group \"" + spec.Name + "\" has no parameters";
        ParameterGroup group;
        group.Name = spec.Name;
        group.LRScale = scale;
        group.WeightDecay = spec.WeightDecay;
        for (const Parameter& p : spec.Params) {
            if (!p.Value) return "autograd: group \"" + spec.Name + "\" has a parameter without a value";
            auto it = lookup.find(p.Value.get());
            if (it == lookup.end()) return "autograd: parameter \"" + p.Name + "\" is not part of this optimizer";
            int found = it->second;
            if (params[found].Name != p.Name) return "autograd: parameter \"" + p.Name + "\" is renamed inside group \"" + spec.Name + "\"";
            if ((*owner)[found] >= 0)
                return "autograd: parameter \"" + p.Name + "\" appears in groups \"" + specNames[(*owner)[found]] + "\" and \"" + spec.Name + "\"";
            (*owner)[found] = (int)index;
            group.Indexes.push_back(found);
        }
        groups->push_back(group);
    }
    for (size_t i = 0; i < owner->size(); i++)
        if ((*owner)[i] < 0) return "autograd: parameter \"" + params[i].Name + "\" is not in any group";
    return "";
}

std::vector<OptimizerGroupState> groupStates(const std::vector<ParameterGroup>& groups, const std::vector<std::string>& names) {
    std::vector<OptimizerGroupState> states;
    for (const ParameterGroup& g : groups) {
        OptimizerGroupState s;
        s.Name = g.Name;
        for (int index : g.Indexes) s.Names.push_back(names[index]);
        s.LRScale = g.LRScale;
        s.WeightDecay = g.WeightDecay;
        states.push_back(s);
    }
    return states;
}

std::string validateGroupStates(const std::vector<ParameterGroup>& live, const std::vector<std::string>& names,
                                const std::vector<OptimizerGroupState>& states, float baseDecay,
                                std::vector<ParameterGroup>* resolved) {
    resolved->clear();
    if (states.empty()) {  // legacy single-group layout (autograd/param_groups.go:209-223)
        if (live.size() != 1) return "autograd: saved state has no parameter groups for " + std::to_string(live.size()) + " groups";
        ParameterGroup group = live[0];
        if (group.LRScale != 1) return "autograd: saved state cannot express the learning-rate scale of group \"" + group.Name + "\"";
        std::string e = validateGroupDecay(baseDecay);
        if (!e.empty()) return e;
        group.WeightDecay = baseDecay;
        resolved->push_back(group);
        return "";
    }
    if (states.size() != live.size())
        return "autograd: saved state has " + std::to_string(states.size()) + " parameter groups, live optimizer has " + std::to_string(live.size());
    for (size_t index = 0; index < states.size(); index++) {
        const OptimizerGroupState& state = states[index];
        const ParameterGroup& group = live[index];
        if (state.Name != group.Name)
            return "autograd: parameter group " + std::to_string(index) + " is \"" + group.Name + "\", saved state is \"" + state.Name + "\"";
        if (state.Names.size() != group.Indexes.size())
            return "autograd: parameter group \"" + group.Name + "\" holds " + std::to_string(group.Indexes.size()) + " parameters, saved state has " + std::to_string(state.Names.size());
        for (size_t position = 0; position < group.Indexes.size(); position++)
            if (state.Names[position] != names[group.Indexes[position]])
                return "autograd: parameter group \"" + group.Name + "\" expects \"" + names[group.Indexes[position]] + "\", saved state has \"" + state.Names[position] + "\"";
        float scale = 0;
        std::string e = normalizeLRScale(state.LRScale, &scale);
        if (!e.empty()) return e;
        if (!(e = validateGroupDecay(state.WeightDecay)).empty()) return e;
        ParameterGroup r;
        r.Name = group.Name;
        r.Indexes = group.Indexes;
        r.LRScale = scale;
        r.WeightDecay = state.WeightDecay;
        resolved->push_back(r);
    }
    return "";
}

// -------------------------------------------------------------------------------------
// ClipGradNorm on the device, state per (thread, device) (autograd/cuda_clip.go:25-134)
// -------------------------------------------------------------------------------------
namespace {
struct ClipState {
    oe_plan* plan = nullptr;
    int device = 0;
};
std::mutex g_clip_mu;
std::map<std::pair<std::thread::id, int>, ClipState> g_clip;
thread_local int t_last_clip_device = -1;
}  // namespace

float ClipGradNorm(const std::vector<Parameter>& params, float maxNorm) {
    if (params.empty() || !params[0].Value) return 0.0f;
    int device = params[0].Value->Device;
    std::vector<oe_tensor_desc> descs;
    for (const Parameter& p : params) {
        // Clipping observes gradients, it must not create them (autograd/cuda_clip.go:70-76).
        if (!p.Value || p.Value->Numel() == 0) continue;
        if (p.Value->Device != device) throw std::runtime_error("autograd: ClipGradNorm parameters must use one device");
        oe_tensor_desc d;
        memset(&d, 0, sizeof d);
        d.param = p.Value->buf;
        d.grad = p.Value->gradBuf;
        d.numel = (uint64_t)p.Value->Numel();
        d.lr_scale = 1;
        descs.push_back(d);
    }
    ClipState* state;
    {
        std::lock_guard<std::mutex> lock(g_clip_mu);
        state = &g_clip[{std::this_thread::get_id(), device}];
    }
    int rc;
    if (state->plan == nullptr) {
        rc = oe_plan_create(device, descs.data(), (uint32_t)descs.size(), 0, &state->plan);
        state->device = device;
    } else {
        // The plan compares addresses and sizes and re-uploads only when something changed.
        rc = oe_plan_update(state->plan, descs.data(), (uint32_t)descs.size(), 0);
    }
    if (rc != 0) throw std::runtime_error(engine_error("clip plan", rc));
    rc = oe_clip_grad_norm(state->plan, &maxNorm, 0, 0);
    if (rc != 0) throw std::runtime_error(engine_error("oe_clip_grad_norm", rc));
    t_last_clip_device = device;
    return std::nanf("");  // the norm stays on the device (autograd/nn.go:314-317)
}

float GradientNormToHost() {
    if (t_last_clip_device < 0) return 0.0f;
    ClipState state;
    {
        std::lock_guard<std::mutex> lock(g_clip_mu);
        auto it = g_clip.find({std::this_thread::get_id(), t_last_clip_device});
        if (it == g_clip.end() || it->second.plan == nullptr) return 0.0f;
        state = it->second;
    }
    float norm = 0;
    int rc = oe_read_norm(state.plan, &norm, nullptr, 0);
    if (rc != 0) throw std::runtime_error(engine_error("oe_read_norm", rc));
    return norm;
}

void ReleaseClipState() {
    std::lock_guard<std::mutex> lock(g_clip_mu);
    for (auto it = g_clip.begin(); it != g_clip.end();) {
        if (it->first.first == std::this_thread::get_id()) {
            oe_plan_destroy(it->second.plan);
            it = g_clip.erase(it);
        } else {
            ++it;
        }
    }
    t_last_clip_device = -1;
}

// -------------------------------------------------------------------------------------
// GradAccumulator bookkeeping (autograd/accumulate.go:21-71)
// -------------------------------------------------------------------------------------
std::string GradAccumulator::New(int groups, GradAccumulator* out) {
    if (groups < 1) return "autograd: gradient accumulation needs at least one micro-batch";
    out->groups = groups;
    out->pending = 0;
    return "";
}

std::string GradAccumulator::MicroBatch(float* seed, bool* complete) {
    if (groups < 1) return "autograd: invalid gradient accumulator";
    if (seed) *seed = 1.0f / (float)groups;  // what Backward seeds differentiation with
    pending++;
    bool done = pending >= groups;
    if (done) pending = 0;
    if (complete) *complete = done;
    return "";
}

// -------------------------------------------------------------------------------------
// OneCycle (autograd/nn.go:539-571)
// -------------------------------------------------------------------------------------
OneCycle OneCycle::New(double maxLR, int total, double pctStart) {
    if (total < 2 || pctStart <= 0 || pctStart >= 1 || maxLR <= 0 || std::isnan(maxLR) || std::isinf(maxLR))
        throw std::runtime_error("autograd: invalid OneCycle configuration");
    OneCycle c;
    c.MaxLR = maxLR;
    c.Total = total;
    c.PctStart = pctStart;
    return c;
}

double OneCycle::LR() const {
    const double pi = 3.14159265358979323846;
    double initial = MaxLR / DivFactor, final_ = initial / FinalDivFactor, step = (double)StepCount;
    double warm = std::max(PctStart * (double)Total - 1, 0.0);
    double start, end, p = 0;
    if (step <= warm) {
        start = initial;
        end = MaxLR;
        if (warm > 0) p = step / warm;
    } else {
        start = MaxLR;
        end = final_;
        p = (step - warm) / ((double)(Total - 1) - warm);
    }
    return end + (start - end) * (1 + std::cos(pi * p)) / 2;
}

void OneCycle::Step(CheckpointOptimizer& o) {
    StepCount++;
    o.SetLearningRate((float)LR());
}

std::string validateOneCycle(const OneCycle& c) {
    for (double v : {c.MaxLR, c.PctStart, c.DivFactor, c.FinalDivFactor})
        if (std::isnan(v) || std::isinf(v)) return "autograd: non-finite OneCycle configuration";
    if (c.Total < 2 || c.StepCount < 0 || c.StepCount > c.Total || c.MaxLR <= 0 || c.PctStart <= 0 || c.PctStart >= 1 ||
        c.DivFactor <= 0 || c.FinalDivFactor <= 0)
        return "autograd: invalid OneCycle state";
    return "";
}

}  // namespace autograd
