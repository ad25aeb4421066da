// Flat C handle API (include/gograd_host.h) over the C++ host mirror. Exceptions — the
// mirror's counterpart of a Go panic — are turned into error codes here.
#include <climits>
#include <cmath>
#include <cstring>
#include <functional>
#include <memory>

#include "../../../include/gograd_host.h"
#include "autograd.hpp"

using namespace autograd;

struct gg_tensor {
    std::shared_ptr<Tensor> t;
};

struct gg_optimizer {
    std::unique_ptr<AdamW> adamw;
    std::unique_ptr<SGD> sgd;
    CheckpointOptimizer* base() { return adamw ? (CheckpointOptimizer*)adamw.get() : (CheckpointOptimizer*)sgd.get(); }
    const CheckpointOptimizer* base() const {
        return adamw ? (const CheckpointOptimizer*)adamw.get() : (const CheckpointOptimizer*)sgd.get();
    }
};

namespace {
thread_local std::string t_err;

int fail(const std::string& message) {
    t_err = message;
    return 1;
}

int guarded(const std::function<std::string()>& fn) {
    try {
        std::string e = fn();
        if (e.empty()) return 0;
        return fail(e);
    } catch (const std::exception& ex) {
        return fail(ex.what());
    }
}

std::vector<Parameter> make_params(const char* const* names, gg_tensor* const* tensors, int32_t n) {
    std::vector<Parameter> params;
    for (int32_t i = 0; i < n; i++) {
        Parameter p;
        p.Name = names && names[i] ? names[i] : "";
        p.Value = tensors && tensors[i] ? tensors[i]->t : nullptr;
        params.push_back(p);
    }
    return params;
}

std::vector<ParameterGroupSpec> make_specs(const std::vector<Parameter>& params, const gg_groups* g) {
    std::vector<ParameterGroupSpec> specs;
    if (!g) return specs;
    for (int32_t i = 0; i < g->n_groups; i++) {
        ParameterGroupSpec s;
        s.Name = g->group_names[i] ? g->group_names[i] : "";
        for (int32_t k = g->offsets[i]; k < g->offsets[i + 1]; k++) {
            int32_t index = g->members[k];
            if (index >= 0 && index < (int32_t)params.size()) {
                s.Params.push_back(params[(size_t)index]);
            } else {
                Parameter stranger;  // a parameter the optimizer does not own
                stranger.Name = "?";
                stranger.Value = std::make_shared<Tensor>();
                s.Params.push_back(stranger);
            }
        }
        s.LRScale = g->lr_scales[i];
        s.WeightDecay = g->decays[i];
        specs.push_back(s);
    }
    return specs;
}
}  // namespace

extern "C" {

const char* gg_last_error(void) { return t_err.c_str(); }

int gg_tensor_new(const float* values, const int32_t* shape, int32_t rank, int32_t device, int32_t requires_grad,
                  gg_tensor** out) {
    if (!out) return fail("out is NULL");
    *out = nullptr;
    return guarded([&]() -> std::string {
        std::vector<int> s(shape, shape + rank);
        long long n = 1;
        for (int d : s) n *= d;
        if (n < 0) return "autograd: negative dimension";
        std::vector<float> v(values, values + n);
        auto h = new gg_tensor();
        std::string e = Tensor::New(v, s, device, requires_grad != 0, &h->t);
        if (!e.empty()) {
            delete h;
            return e;
        }
        *out = h;
        return "";
    });
}

void gg_tensor_free(gg_tensor* t) { delete t; }
int64_t gg_tensor_numel(const gg_tensor* t) { return t ? t->t->Numel() : -1; }

int gg_tensor_to_host(const gg_tensor* t, float* out) {
    return guarded([&]() -> std::string {
        std::vector<float> v;
        std::string e = t->t->ToHost(&v);
        if (e.empty() && !v.empty()) memcpy(out, v.data(), v.size() * 4);
        return e;
    });
}

int gg_tensor_copy_from_host(gg_tensor* t, const float* values) {
    return guarded([&]() { return t->t->CopyFromHost(std::vector<float>(values, values + t->t->Numel())); });
}

int gg_tensor_has_grad(const gg_tensor* t) { return t && t->t->gradBuf != 0 ? 1 : 0; }

int gg_tensor_set_grad(gg_tensor* t, const float* values) {
    return guarded([&]() -> std::string {
        if (!values) {
            t->t->FreeGrad();
            return "";
        }
        return t->t->SetGrad(std::vector<float>(values, values + t->t->Numel()));
    });
}

int gg_tensor_ensure_grad(gg_tensor* t) {
    return guarded([&]() { return t->t->EnsureGrad(); });
}

int gg_tensor_grad_to_host(const gg_tensor* t, float* out) {
    return guarded([&]() -> std::string {
        std::vector<float> v;
        std::string e = t->t->GradToHost(&v);
        if (e.empty() && !v.empty()) memcpy(out, v.data(), v.size() * 4);
        return e;
    });
}

int gg_tensor_shadow_to_host(const gg_tensor* t, uint16_t* out) {
    return guarded([&]() -> std::string {
        std::vector<uint16_t> v;
        std::string e = t->t->ShadowToHost(&v);
        if (e.empty() && !v.empty()) memcpy(out, v.data(), v.size() * 2);
        return e;
    });
}

int gg_tensor_shadow_current(const gg_tensor* t) { return t && t->t->ShadowCurrent() ? 1 : 0; }

uint64_t gg_tensor_address(const gg_tensor* t, int32_t which) {
    if (!t) return 0;
    if (which == 1) t->t->MarkGradWritten();  // whoever asks for the raw gradient address may write through it
    return which == 0 ? t->t->buf : which == 1 ? t->t->gradBuf : t->t->bf16Buf;
}

int gg_tensor_grad_known_zero(const gg_tensor* t) { return t && t->t->gradBuf != 0 && t->t->gradKnownZero ? 1 : 0; }

uint64_t gg_tensor_shadow_lease(gg_tensor* t) { return t ? t->t->AcquireShadowLease() : 0; }
void gg_tensor_shadow_release(gg_tensor* t, uint64_t address) {
    if (t) t->t->ReleaseShadowLease(address);
}
int gg_tensor_leased_shadows(const gg_tensor* t) { return t ? t->t->LeasedShadowBuffers() : 0; }

int gg_adamw_new(const char* const* names, gg_tensor* const* tensors, int32_t n, const float* lr, const float* decay,
                 gg_optimizer** out) {
    if (!out || !lr || !decay) return fail("NULL argument");
    *out = nullptr;
    return guarded([&]() -> std::string {
        auto h = new gg_optimizer();
        std::string e = AdamW::New(make_params(names, tensors, n), *lr, *decay, &h->adamw);
        if (!e.empty()) {
            delete h;
            return e;
        }
        *out = h;
        return "";
    });
}

int gg_adamw_new_groups(const char* const* names, gg_tensor* const* tensors, int32_t n, const float* lr,
                        const gg_groups* groups, gg_optimizer** out) {
    if (!out || !lr) return fail("NULL argument");
    *out = nullptr;
    return guarded([&]() -> std::string {
        auto params = make_params(names, tensors, n);
        auto h = new gg_optimizer();
        std::string e = AdamW::NewGroups(params, *lr, make_specs(params, groups), &h->adamw);
        if (!e.empty()) {
            delete h;
            return e;
        }
        *out = h;
        return "";
    });
}

int gg_adamw_set_config(gg_optimizer* o, const float* beta1, const float* beta2, const float* eps) {
    if (!o || !o->adamw) return fail("not an AdamW optimizer");
    if (beta1) o->adamw->Beta1 = *beta1;
    if (beta2) o->adamw->Beta2 = *beta2;
    if (eps) o->adamw->Eps = *eps;
    return 0;
}

static SGDOptions to_options(const gg_sgd_options* x) {
    SGDOptions o;
    o.LR = x->lr;
    o.Momentum = x->momentum;
    o.Dampening = x->dampening;
    o.WeightDecay = x->weight_decay;
    o.Nesterov = x->nesterov != 0;
    o.Maximize = x->maximize != 0;
    return o;
}

int gg_sgd_new(const char* const* names, gg_tensor* const* tensors, int32_t n, const gg_sgd_options* options,
               gg_optimizer** out) {
    if (!out || !options) return fail("NULL argument");
    *out = nullptr;
    return guarded([&]() -> std::string {
        auto h = new gg_optimizer();
        std::string e = SGD::New(make_params(names, tensors, n), to_options(options), &h->sgd);
        if (!e.empty()) {
            delete h;
            return e;
        }
        *out = h;
        return "";
    });
}

int gg_sgd_new_groups(const char* const* names, gg_tensor* const* tensors, int32_t n, const gg_sgd_options* options,
                      const gg_groups* groups, gg_optimizer** out) {
    if (!out || !options) return fail("NULL argument");
    *out = nullptr;
    return guarded([&]() -> std::string {
        auto params = make_params(names, tensors, n);
        auto specs = make_specs(params, groups);
        if (specs.empty()) return "autograd: NewSGDGroups needs at least one parameter group";
        auto h = new gg_optimizer();
        std::string e = SGD::NewGroups(params, to_options(options), specs, &h->sgd);
        if (!e.empty()) {
            delete h;
            return e;
        }
        *out = h;
        return "";
    });
}

int gg_opt_set_engine(gg_optimizer* o, int32_t write_shadow, int32_t clip_devform) {
    if (!o) return fail("optimizer is NULL");
    EngineOptions& e = o->adamw ? o->adamw->Engine : o->sgd->Engine;
    e.WriteShadow = write_shadow != 0;
    e.ClipDevForm = clip_devform != 0;
    return 0;
}

int gg_opt_set_zero_grad_in_step(gg_optimizer* o, int32_t on) {
    if (!o) return fail("optimizer is NULL");
    // For SGD the option only holds once the optimizer is prepared for graphs, where ZeroGrad zeroes
    // instead of releasing; Step checks that.
    (o->adamw ? o->adamw->Engine : o->sgd->Engine).ZeroGradInStep = on != 0;
    return 0;
}

int gg_opt_set_grad_scale(gg_optimizer* o, const float* scale) {
    if (!o || !scale) return fail("optimizer or scale is NULL");
    if (!std::isfinite(*scale) || !(*scale > 0)) return fail("autograd: invalid gradient scale");
    (o->adamw ? o->adamw->Engine : o->sgd->Engine).GradScale = *scale;
    return 0;
}

int gg_opt_step(gg_optimizer* o) {
    return guarded([&]() -> std::string {
        o->base()->Step();
        return "";
    });
}

int gg_opt_step_clipped(gg_optimizer* o, const float* max_norm) {
    return guarded([&]() -> std::string {
        if (o->adamw)
            o->adamw->StepClipped(*max_norm);
        else
            o->sgd->StepClipped(*max_norm);
        return "";
    });
}

int gg_opt_last_norm(gg_optimizer* o, float* out) {
    return guarded([&]() -> std::string {
        if (!o->adamw) return "only AdamW keeps the norm of its last clipped step";
        *out = o->adamw->LastGradNorm();
        return "";
    });
}

int gg_opt_zero_grad(gg_optimizer* o) {
    return guarded([&]() -> std::string {
        o->base()->ZeroGrad();
        return "";
    });
}

int gg_opt_get_lr(const gg_optimizer* o, float* out) {
    *out = o->base()->LearningRate();
    return 0;
}

int gg_opt_set_lr(gg_optimizer* o, const float* lr) {
    return guarded([&]() -> std::string {
        o->base()->SetLearningRate(*lr);
        return "";
    });
}

int64_t gg_opt_step_count(const gg_optimizer* o) { return o->adamw ? o->adamw->StepCount : o->sgd->StepCount; }

int gg_opt_close(gg_optimizer* o) {
    return guarded([&]() -> std::string {
        o->base()->Close();
        return "";
    });
}

void gg_opt_free(gg_optimizer* o) { delete o; }

int gg_opt_state(gg_optimizer* o, int32_t index, int32_t which, float* out, int32_t* initialized) {
    return guarded([&]() -> std::string {
        if (o->adamw) {
            OptimizerState s;
            std::string e = o->adamw->State(&s);
            if (!e.empty()) return e;
            if (index < 0 || index >= (int32_t)s.Moments.size() || which < 0 || which > 1) return "state index out of range";
            const std::vector<float>& v = which == 0 ? s.Moments[(size_t)index].M : s.Moments[(size_t)index].V;
            if (out && !v.empty()) memcpy(out, v.data(), v.size() * 4);
            if (initialized) *initialized = 1;
            return "";
        }
        SGDState s;
        std::string e = o->sgd->State(&s);
        if (!e.empty()) return e;
        if (index < 0 || index >= (int32_t)s.Buffers.size() || which != 2) return "state index out of range";
        if (initialized) *initialized = s.Initialized[(size_t)index] ? 1 : 0;
        if (out && !s.Buffers[(size_t)index].empty()) memcpy(out, s.Buffers[(size_t)index].data(), s.Buffers[(size_t)index].size() * 4);
        return "";
    });
}

int gg_opt_group_scale(const gg_optimizer* o, int32_t index, float* step_size, float* decay) {
    if (o->adamw)
        o->adamw->groupScale(index, step_size, decay);
    else
        o->sgd->groupScale(index, step_size, decay);
    return 0;
}

int gg_opt_save(gg_optimizer* o, const char* path) {
    return guarded([&]() { return o->adamw ? o->adamw->SaveSafeTensors(path) : o->sgd->SaveSafeTensors(path); });
}

int gg_opt_load(gg_optimizer* o, const char* path) {
    return guarded([&]() { return o->adamw ? o->adamw->LoadSafeTensors(path) : o->sgd->LoadSafeTensors(path); });
}

int gg_opt_prepare_graph(gg_optimizer* o) {
    return guarded([&]() -> std::string {
        if (!o) return "optimizer is NULL";
        return o->adamw ? o->adamw->PrepareGraph() : o->sgd->PrepareGraph();
    });
}

int gg_opt_step_captured(gg_optimizer* o) {
    return guarded([&]() -> std::string {
        if (!o) return "optimizer is NULL";
        if (o->adamw)
            o->adamw->StepCaptured();
        else
            o->sgd->StepCaptured();
        return "";
    });
}

int gg_opt_graph_step_count(gg_optimizer* o, int32_t* out) {
    return guarded([&]() -> std::string {
        if (!o || !out) return "NULL argument";
        int step = 0;
        std::string e = o->adamw ? o->adamw->GraphStepCount(&step) : o->sgd->GraphStepCount(&step);
        *out = step;
        return e;
    });
}

int gg_adamw_prepare_graph(gg_optimizer* o) {
    if (!o || !o->adamw) return fail("not an AdamW optimizer");
    return gg_opt_prepare_graph(o);
}

int gg_adamw_step_captured(gg_optimizer* o) {
    if (!o || !o->adamw) return fail("not an AdamW optimizer");
    return gg_opt_step_captured(o);
}

int gg_adamw_graph_step_count(gg_optimizer* o, int32_t* out) {
    if (!o || !o->adamw) return fail("not an AdamW optimizer");
    return gg_opt_graph_step_count(o, out);
}

int gg_partition_parameters(const char* const* names, gg_tensor* const* tensors, const char* const* labels, int32_t n,
                            char* out, int32_t capacity) {
    return guarded([&]() -> std::string {
        std::vector<std::string> l;
        for (int32_t i = 0; i < n; i++) l.push_back(labels && labels[i] ? labels[i] : "");
        std::vector<ParameterGroupSpec> specs;
        std::string e = PartitionParameters(make_params(names, tensors, n), l, &specs);
        if (!e.empty()) return e;
        std::string j = "[";
        for (size_t g = 0; g < specs.size(); g++) {
            j += std::string(g ? "," : "") + "{\"Name\":" + ggjson::quote(specs[g].Name) + ",\"Params\":[";
            for (size_t k = 0; k < specs[g].Params.size(); k++) j += (k ? "," : "") + ggjson::quote(specs[g].Params[k].Name);
            j += "]}";
        }
        j += "]";
        if ((int32_t)j.size() + 1 > capacity) return "partition does not fit the buffer";
        memcpy(out, j.c_str(), j.size() + 1);
        return "";
    });
}

int gg_clip_grad_norm(gg_tensor* const* tensors, int32_t n, const float* max_norm) {
    return guarded([&]() -> std::string {
        std::vector<Parameter> params;
        for (int32_t i = 0; i < n; i++) params.push_back(Parameter{"p" + std::to_string(i), tensors[i]->t});
        ClipGradNorm(params, *max_norm);
        return "";
    });
}

int gg_gradient_norm_to_host(float* out) {
    return guarded([&]() -> std::string {
        *out = GradientNormToHost();
        return "";
    });
}

void gg_release_clip_state(void) { ReleaseClipState(); }

static OneCycle to_cycle(const gg_onecycle* c) {
    OneCycle o;
    o.MaxLR = c->max_lr;
    o.PctStart = c->pct_start;
    o.DivFactor = c->div_factor;
    o.FinalDivFactor = c->final_div_factor;
    o.Total = c->total;
    o.StepCount = c->step_count;
    return o;
}

static void from_cycle(const OneCycle& o, gg_onecycle* c) {
    c->max_lr = o.MaxLR;
    c->pct_start = o.PctStart;
    c->div_factor = o.DivFactor;
    c->final_div_factor = o.FinalDivFactor;
    c->total = o.Total;
    c->step_count = o.StepCount;
}

namespace {
thread_local std::string t_loop_error;  // what a loop callback left with gg_loop_set_error
std::string take_loop_error(const char* fallback) {
    std::string e = t_loop_error.empty() ? fallback : t_loop_error;
    t_loop_error.clear();
    return e;
}
}  // namespace

void gg_loop_set_error(const char* message) { t_loop_error = message ? message : ""; }

int gg_training_loop_run(gg_training_loop* c) {
    if (!c) return fail("loop is NULL");
    TrainingLoop loop;
    if (c->next)
        loop.Next = [c](std::string* err) {
            int status = c->next(c->user);
            if (status != 0) *err = take_loop_error(status == GG_LOOP_CANCELLED ? "context canceled" : "autograd: the reader failed");
            return status;
        };
    if (c->next_epoch)
        loop.NextEpoch = [c]() -> std::string { return c->next_epoch(c->user) == 0 ? "" : take_loop_error("autograd: the reader could not start an epoch"); };
    if (c->position)
        loop.Position = [c](std::string* payload) -> std::string {
            std::vector<char> buf(1 << 16);
            int32_t length = 0;
            if (c->position(c->user, buf.data(), (int32_t)buf.size(), &length) != 0 || length < 0 || length > (int32_t)buf.size())
                return take_loop_error("autograd: the sampler could not save its position");
            payload->assign(buf.data(), (size_t)length);
            return "";
        };
    if (c->step)
        loop.Step = [c](float seed, double* loss, std::string* err) {
            int status = c->step(c->user, &seed, loss);
            if (status != 0) *err = take_loop_error(status == GG_LOOP_CANCELLED ? "context canceled" : "autograd: the step failed");
            return status;
        };
    if (c->report) loop.Report = [c](int update, double loss) { c->report(c->user, update, &loss); };
    if (c->save)
        loop.Save = [c](const std::string* savepoint) -> std::string {
            int rc = savepoint ? c->save(c->user, savepoint->data(), (int32_t)savepoint->size()) : c->save(c->user, nullptr, 0);
            return rc == 0 ? "" : take_loop_error("autograd: saving failed");
        };
    loop.Optimizer = c->optimizer ? c->optimizer->base() : nullptr;
    OneCycle cycle;
    if (c->schedule) {
        cycle = to_cycle(c->schedule);
        loop.Schedule = &cycle;
    }
    loop.Updates = c->updates;
    loop.Applied = c->applied;
    loop.Accumulate = c->accumulate;
    loop.LogEvery = c->log_every;
    bool cancelled = false;
    std::string e;
    try {
        e = loop.Run(&cancelled);
    } catch (const std::exception& ex) {
        e = ex.what();
    }
    c->applied = loop.Applied;
    if (c->schedule) from_cycle(cycle, c->schedule);
    if (e.empty()) return 0;
    fail(e);
    return cancelled ? GG_LOOP_CANCELLED : 1;
}

int gg_accumulator_new(int32_t groups, gg_accumulator* out) {
    if (!out) return fail("accumulator is NULL");
    GradAccumulator a;
    std::string e = GradAccumulator::New(groups, &a);
    if (!e.empty()) return fail(e);
    out->groups = a.groups;
    out->pending = a.pending;
    return 0;
}

int gg_accumulator_micro_batch(gg_accumulator* a, float* seed_out, int32_t* complete_out) {
    if (!a) return fail("autograd: invalid gradient accumulator");
    GradAccumulator acc;
    acc.groups = a->groups;
    acc.pending = a->pending;
    bool complete = false;
    std::string e = acc.MicroBatch(seed_out, &complete);
    if (!e.empty()) return fail(e);
    a->pending = acc.pending;
    if (complete_out) *complete_out = complete ? 1 : 0;
    return 0;
}

void gg_accumulator_reset(gg_accumulator* a) {
    if (a) a->pending = 0;
}

int gg_onecycle_new(const double* max_lr, int32_t total, const double* pct_start, gg_onecycle* out) {
    return guarded([&]() -> std::string {
        from_cycle(OneCycle::New(*max_lr, total, *pct_start), out);
        return "";
    });
}

int gg_onecycle_lr(const gg_onecycle* c, double* out) {
    *out = to_cycle(c).LR();
    return 0;
}

int gg_onecycle_step(gg_onecycle* c, gg_optimizer* o) {
    return guarded([&]() -> std::string {
        OneCycle cyc = to_cycle(c);
        cyc.Step(*o->base());
        from_cycle(cyc, c);
        return "";
    });
}

int gg_save_training_checkpoint(const char* path, const char* const* names, gg_tensor* const* tensors, int32_t n,
                                gg_optimizer* o, const gg_onecycle* scheduler, const char* const* user_keys,
                                const char* const* user_values, int32_t n_user) {
    return guarded([&]() -> std::string {
        if (!o || !scheduler) return "autograd: model, optimizer and scheduler are required";
        std::map<std::string, std::string> user;
        for (int32_t i = 0; i < n_user; i++) user[user_keys[i]] = user_values[i];
        OneCycle c = to_cycle(scheduler);
        return SaveTrainingCheckpoint(path, make_params(names, tensors, n), o->base(), &c, user);
    });
}

int gg_load_training_checkpoint(const char* path, const char* const* names, gg_tensor* const* tensors, int32_t n,
                                gg_optimizer* o, gg_onecycle* scheduler, char* user_json, int32_t capacity) {
    return guarded([&]() -> std::string {
        if (!o || !scheduler) return "autograd: model, optimizer and scheduler are required";
        OneCycle c = to_cycle(scheduler);
        std::map<std::string, std::string> user;
        std::string e = LoadTrainingCheckpoint(path, make_params(names, tensors, n), o->base(), &c, &user);
        if (!e.empty()) return e;
        from_cycle(c, scheduler);
        if (user_json && capacity > 0) {
            std::string j = "{";
            bool first = true;
            for (const auto& kv : user) {
                j += (first ? "" : ",") + ggjson::quote(kv.first) + ":" + ggjson::quote(kv.second);
                first = false;
            }
            j += "}";
            strncpy(user_json, j.c_str(), (size_t)capacity - 1);
            user_json[capacity - 1] = 0;
        }
        return "";
    });
}

int gg_safetensors_write(const char* path, const char* const* names, const float* const* data, const int32_t* shapes,
                         const int32_t* shape_offsets, int32_t n, const char* const* meta_keys,
                         const char* const* meta_values, int32_t n_meta) {
    return guarded([&]() -> std::string {
        EntryMap entries;
        for (int32_t i = 0; i < n; i++) {
            SafeTensorEntry e;
            long long count = 1;
            for (int32_t k = shape_offsets[i]; k < shape_offsets[i + 1]; k++) {
                e.Shape.push_back(shapes[k]);
                count *= shapes[k];
            }
            if (count > 0) e.Values.assign(data[i], data[i] + count);
            entries[names[i]] = std::move(e);
        }
        Metadata metadata;
        for (int32_t i = 0; i < n_meta; i++) metadata[meta_keys[i]] = meta_values[i];
        return write_safetensors(path, entries, n_meta >= 0 ? &metadata : nullptr);
    });
}

namespace {
// Names, shapes, configuration and groups of an AdamW state from the flat C arguments; the moments
// stay with the caller.
std::string state_from_c(int32_t n, const char* const* names, const int32_t* shapes, const int32_t* shape_offsets,
                         const gg_adamw_config* config, const gg_groups* groups, OptimizerState* out) {
    if (!config || !groups || (n > 0 && (!names || !shapes || !shape_offsets))) return "NULL argument";
    OptimizerState s;
    s.StepCount = config->step_count;
    s.LR = config->lr;
    s.WeightDecay = config->weight_decay;
    s.Beta1 = config->beta1;
    s.Beta2 = config->beta2;
    s.Eps = config->eps;
    for (int32_t i = 0; i < n; i++) {
        s.Names.push_back(names[i]);
        s.Shapes.push_back(std::vector<int>(shapes + shape_offsets[i], shapes + shape_offsets[i + 1]));
    }
    for (int32_t g = 0; g < groups->n_groups; g++) {
        OptimizerGroupState gs;
        gs.Name = groups->group_names[g];
        for (int32_t k = groups->offsets[g]; k < groups->offsets[g + 1]; k++) {
            int32_t index = groups->members[k];
            if (index < 0 || index >= n) return "autograd: group member out of range";
            gs.Names.push_back(names[index]);
        }
        float scale = 0;
        std::string e = normalizeLRScale(groups->lr_scales[g], &scale);
        if (!e.empty()) return e;
        gs.LRScale = scale;
        gs.WeightDecay = groups->decays[g];
        s.Groups.push_back(gs);
    }
    *out = std::move(s);
    return "";
}
}  // namespace

int gg_adamw_state_write(const char* path, int32_t n, const char* const* names, const int32_t* shapes,
                         const int32_t* shape_offsets, const float* const* m, const float* const* v,
                         const gg_adamw_config* config, const gg_groups* groups) {
    return guarded([&]() -> std::string {
        OptimizerState s;
        std::string e = state_from_c(n, names, shapes, shape_offsets, config, groups, &s);
        if (!e.empty()) return e;
        s.Moments.resize((size_t)n);
        for (int32_t i = 0; i < n; i++) {
            long long count = 1;
            for (int d : s.Shapes[(size_t)i]) count *= d;
            s.Moments[(size_t)i].M.assign(m[i], m[i] + count);
            s.Moments[(size_t)i].V.assign(v[i], v[i] + count);
        }
        EntryMap entries;
        Metadata metadata;
        e = optimizerEntries(std::move(s), &entries, &metadata);
        if (!e.empty()) return e;
        return write_safetensors(path, entries, &metadata);
    });
}

struct gg_state_stream {
    SafeTensorStream stream;
};

int gg_adamw_state_stream_begin(const char* path, int32_t n, const char* const* names, const int32_t* shapes,
                                const int32_t* shape_offsets, const gg_adamw_config* config, const gg_groups* groups,
                                gg_state_stream** out) {
    return guarded([&]() -> std::string {
        if (!path || !out) return "NULL argument";
        OptimizerState s;
        std::string e = state_from_c(n, names, shapes, shape_offsets, config, groups, &s);
        if (!e.empty()) return e;
        std::map<std::string, std::vector<int>> entry_shapes;
        for (int32_t i = 0; i < n; i++) {
            long long count = 0;
            if (!safe_numel(s.Shapes[(size_t)i], INT32_MAX, &count)) return "autograd: invalid shape of " + s.Names[(size_t)i];
            entry_shapes["m." + std::to_string(i)] = {(int)count};
            entry_shapes["v." + std::to_string(i)] = {(int)count};
        }
        Metadata metadata;
        optimizerMetadata(s, &metadata);
        std::unique_ptr<gg_state_stream> h(new gg_state_stream());
        e = h->stream.Begin(path, entry_shapes, &metadata);
        if (!e.empty()) return e;
        *out = h.release();
        return "";
    });
}

int gg_sgd_state_stream_begin(const char* path, int32_t n, const char* const* names, const int32_t* shapes,
                              const int32_t* shape_offsets, const gg_sgd_config* config, const uint8_t* initialized,
                              const gg_groups* groups, gg_state_stream** out) {
    return guarded([&]() -> std::string {
        if (!path || !out || !config || (n > 0 && !initialized)) return "NULL argument";
        // names, shapes and groups arrive in the flat form the AdamW writer takes
        gg_adamw_config unused = {config->step_count, config->lr, config->weight_decay, 0.0f, 0.0f, 0.0f};
        OptimizerState base;
        std::string e = state_from_c(n, names, shapes, shape_offsets, &unused, groups, &base);
        if (!e.empty()) return e;
        SGDState s;
        s.StepCount = config->step_count;
        s.Names = base.Names;
        s.Shapes = base.Shapes;
        s.Groups = base.Groups;
        s.Options.LR = config->lr;
        s.Options.Momentum = config->momentum;
        s.Options.Dampening = config->dampening;
        s.Options.WeightDecay = config->weight_decay;
        s.Options.Nesterov = config->nesterov != 0;
        s.Options.Maximize = config->maximize != 0;
        if (!(e = s.Options.validate()).empty()) return e;
        std::map<std::string, std::vector<int>> entry_shapes;
        for (int32_t i = 0; i < n; i++) {
            s.Initialized.push_back(initialized[i] != 0);
            if (!initialized[i]) continue;  // only initialised parameters have a buffer entry (autograd/sgd_state.go:150-164)
            if (!(s.Options.Momentum > 0) || s.StepCount == 0) return "autograd: invalid SGD momentum buffer " + std::to_string(i);
            long long count = 0;
            if (!safe_numel(s.Shapes[(size_t)i], INT32_MAX, &count)) return "autograd: invalid shape of " + s.Names[(size_t)i];
            entry_shapes["buffer." + std::to_string(i)] = {(int)count};
        }
        Metadata metadata;
        sgdMetadata(s, &metadata);
        std::unique_ptr<gg_state_stream> h(new gg_state_stream());
        e = h->stream.Begin(path, entry_shapes, &metadata);
        if (!e.empty()) return e;
        *out = h.release();
        return "";
    });
}

int gg_state_stream_next(const gg_state_stream* s, char* name_out, int32_t capacity, int64_t* remaining_out) {
    if (!s || !name_out || !remaining_out || capacity < 1) return fail("NULL argument");
    std::string name;
    long long remaining = 0;
    if (!s->stream.Next(&name, &remaining)) {
        name_out[0] = 0;
        *remaining_out = 0;
        return 0;
    }
    if ((size_t)capacity <= name.size()) return fail("name buffer too small");
    memcpy(name_out, name.c_str(), name.size() + 1);
    *remaining_out = remaining;
    return 0;
}

int gg_state_stream_append(gg_state_stream* s, const char* entry, const float* values, int64_t count) {
    return guarded([&]() -> std::string {
        if (!s || !entry || (count > 0 && !values)) return "NULL argument";
        return s->stream.Append(entry, values, count);
    });
}

int gg_state_stream_finish(gg_state_stream* s) {
    if (!s) return fail("NULL argument");
    std::string e = s->stream.Finish();
    delete s;
    return e.empty() ? 0 : fail(e);
}

void gg_state_stream_abort(gg_state_stream* s) {
    if (!s) return;
    s->stream.Abort();
    delete s;
}

int gg_safetensors_describe(const char* path, char* out, int32_t capacity) {
    return guarded([&]() -> std::string {
        EntryMap entries;
        Metadata metadata;
        std::string e = read_safetensors(path, &entries, &metadata);
        if (!e.empty()) return e;
        std::string j = "{\"entries\":{";
        bool first = true;
        for (const auto& kv : entries) {
            double sum = 0;
            for (float v : kv.second.Values) sum += v;
            j += (first ? "" : ",") + ggjson::quote(kv.first) + ":{\"shape\":[";
            for (size_t i = 0; i < kv.second.Shape.size(); i++) j += (i ? "," : "") + std::to_string(kv.second.Shape[i]);
            j += "],\"sum\":" + ggjson::number_text(sum, false) + "}";
            first = false;
        }
        j += "},\"metadata\":{";
        first = true;
        for (const auto& kv : metadata) {
            j += (first ? "" : ",") + ggjson::quote(kv.first) + ":" + ggjson::quote(kv.second);
            first = false;
        }
        j += "}}";
        if ((int32_t)j.size() + 1 > capacity) return "description does not fit the buffer";
        memcpy(out, j.c_str(), j.size() + 1);
        return "";
    });
}

}  // extern "C"
