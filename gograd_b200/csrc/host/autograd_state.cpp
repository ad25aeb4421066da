// Checkpoint layout of the host mirror: optimizer state <-> safetensors entries + metadata,
// and the "gograd-training-1" training checkpoint. Field names, entry names and metadata
// keys are the reference's (autograd/optimizer_state.go:18-32,142-226, autograd/sgd_state.go:13-194,
// autograd/optimizer.go:85-120, autograd/training_checkpoint.go:13-132); the JSON documents use Go's
// default struct-field keys in declaration order.
#include <cmath>

#include "autograd.hpp"

namespace autograd {

namespace {
using ggjson::number_text;
using ggjson::quote;

std::string f32(float v) { return number_text((double)v, true); }
std::string f64(double v) { return number_text(v, false); }

std::string string_list(const std::vector<std::string>& v, bool null_when_empty) {
    if (v.empty() && null_when_empty) return "null";
    std::string s = "[";
    for (size_t i = 0; i < v.size(); i++) s += (i ? "," : "") + quote(v[i]);
    return s + "]";
}

std::string shapes_json(const std::vector<std::vector<int>>& shapes) {
    if (shapes.empty()) return "null";
    std::string s = "[";
    for (size_t i = 0; i < shapes.size(); i++) {
        s += i ? ",[" : "[";
        for (size_t j = 0; j < shapes[i].size(); j++) s += (j ? "," : "") + std::to_string(shapes[i][j]);
        s += "]";
    }
    return s + "]";
}

std::string groups_json(const std::vector<OptimizerGroupState>& groups) {
    std::string s = "[";
    for (size_t i = 0; i < groups.size(); i++) {
        const OptimizerGroupState& g = groups[i];
        s += std::string(i ? "," : "") + "{\"Name\":" + quote(g.Name) + ",\"Names\":" + string_list(g.Names, false) +
             ",\"LRScale\":" + f32(g.LRScale) + ",\"WeightDecay\":" + f32(g.WeightDecay) + "}";
    }
    return s + "]";
}

bool get_int(const ggjson::Value* v, int* out) {
    if (!v || !v->is(ggjson::Value::Number) || v->num != std::floor(v->num) || std::fabs(v->num) > 2147483647.0) return false;
    *out = (int)v->num;
    return true;
}
bool get_f32(const ggjson::Value* v, float* out) {
    if (!v || !v->is(ggjson::Value::Number)) return false;
    *out = (float)v->num;
    return true;
}
bool get_f64(const ggjson::Value* v, double* out) {
    if (!v || !v->is(ggjson::Value::Number)) return false;
    *out = v->num;
    return true;
}
bool get_bool(const ggjson::Value* v, bool* out) {
    if (!v || !v->is(ggjson::Value::Bool)) return false;
    *out = v->b;
    return true;
}
bool get_strings(const ggjson::Value* v, std::vector<std::string>* out) {
    out->clear();
    if (!v || v->is(ggjson::Value::Null)) return true;
    if (!v->is(ggjson::Value::Arr)) return false;
    for (const auto& x : *v->arr) {
        if (!x.is(ggjson::Value::String)) return false;
        out->push_back(x.raw);
    }
    return true;
}
bool get_shapes(const ggjson::Value* v, std::vector<std::vector<int>>* out) {
    out->clear();
    if (!v || v->is(ggjson::Value::Null)) return true;
    if (!v->is(ggjson::Value::Arr)) return false;
    for (const auto& s : *v->arr) {
        std::vector<int> shape;
        if (s.is(ggjson::Value::Arr)) {
            for (const auto& d : *s.arr) {
                int x;
                if (!get_int(&d, &x)) return false;
                shape.push_back(x);
            }
        } else if (!s.is(ggjson::Value::Null)) {
            return false;
        }
        out->push_back(shape);
    }
    return true;
}
bool get_groups(const ggjson::Value* v, std::vector<OptimizerGroupState>* out) {
    out->clear();
    if (!v || v->is(ggjson::Value::Null)) return true;  // legacy state without groups
    if (!v->is(ggjson::Value::Arr)) return false;
    for (const auto& g : *v->arr) {
        if (!g.is(ggjson::Value::Obj)) return false;
        OptimizerGroupState s;
        const ggjson::Value* name = g.get("Name");
        if (!name || !name->is(ggjson::Value::String)) return false;
        s.Name = name->raw;
        if (!get_strings(g.get("Names"), &s.Names) || !get_f32(g.get("LRScale"), &s.LRScale) ||
            !get_f32(g.get("WeightDecay"), &s.WeightDecay))
            return false;
        out->push_back(s);
    }
    return true;
}

bool parse_int_text(const std::string& s, int* out) {  // strconv.Atoi
    if (s.empty()) return false;
    size_t i = (s[0] == '-' || s[0] == '+') ? 1 : 0;
    if (i == s.size()) return false;
    long long v = 0;
    for (; i < s.size(); i++) {
        if (s[i] < '0' || s[i] > '9') return false;
        v = v * 10 + (s[i] - '0');
        if (v > 2147483647LL) return false;
    }
    *out = (int)(s[0] == '-' ? -v : v);
    return true;
}

std::string meta(const Metadata& m, const char* key) {
    auto it = m.find(key);
    return it == m.end() ? "" : it->second;
}
}  // namespace

// ---- AdamW ------------------------------------------------------------------------------
std::string optimizerEntries(OptimizerState state, EntryMap* entries, Metadata* metadata) {
    entries->clear();
    for (size_t i = 0; i < state.Moments.size(); i++) {
        SafeTensorEntry m, v;
        m.Values = std::move(state.Moments[i].M);
        m.Shape = {(int)m.Values.size()};
        v.Values = std::move(state.Moments[i].V);
        v.Shape = {(int)v.Values.size()};
        (*entries)["m." + std::to_string(i)] = std::move(m);
        (*entries)["v." + std::to_string(i)] = std::move(v);
    }
    optimizerMetadata(state, metadata);
    return "";
}

// The metadata document of a "gograd-adamw" file: everything but the moments themselves
// (autograd/optimizer_state.go:142-160).
void optimizerMetadata(const OptimizerState& state, Metadata* metadata) {
    std::string config = "{\"StepCount\":" + std::to_string(state.StepCount) + ",\"Moments\":null,\"Names\":" +
                         string_list(state.Names, true) + ",\"Shapes\":" + shapes_json(state.Shapes) + ",\"LR\":" +
                         f32(state.LR) + ",\"WeightDecay\":" + f32(state.WeightDecay) + ",\"Beta1\":" + f32(state.Beta1) +
                         ",\"Beta2\":" + f32(state.Beta2) + ",\"Eps\":" + f32(state.Eps) + ",\"Groups\":" +
                         groups_json(state.Groups) + "}";
    *metadata = {{"format", "gograd-adamw"}, {"version", "1"}, {"step_count", std::to_string(state.StepCount)},
                 {"optimizer", config}};
}

std::string optimizerStateFromEntries(const EntryMap& entries, const Metadata& metadata, int count, OptimizerState* out) {
    if (meta(metadata, "format") != "gograd-adamw") return "autograd: not an optimizer state";
    int version = 0;
    if (!parse_int_text(meta(metadata, "version"), &version) || version != 1)
        return "autograd: unsupported optimizer state version \"" + meta(metadata, "version") + "\"";
    int stepCount = 0;
    if (!parse_int_text(meta(metadata, "step_count"), &stepCount) || stepCount < 0)
        return "autograd: invalid optimizer step count \"" + meta(metadata, "step_count") + "\"";
    ggjson::Value root;
    std::string err;
    if (!ggjson::Parser(meta(metadata, "optimizer")).parse(&root, &err) || !root.is(ggjson::Value::Obj))
        return "autograd: invalid optimizer configuration: " + err;
    OptimizerState s;
    if (!get_int(root.get("StepCount"), &s.StepCount) || !get_strings(root.get("Names"), &s.Names) ||
        !get_shapes(root.get("Shapes"), &s.Shapes) || !get_f32(root.get("LR"), &s.LR) ||
        !get_f32(root.get("WeightDecay"), &s.WeightDecay) || !get_f32(root.get("Beta1"), &s.Beta1) ||
        !get_f32(root.get("Beta2"), &s.Beta2) || !get_f32(root.get("Eps"), &s.Eps) || !get_groups(root.get("Groups"), &s.Groups))
        return "autograd: invalid optimizer configuration: wrong field type";
    if (s.StepCount != stepCount || (int)entries.size() != count * 2) return "autograd: optimizer state count or step mismatch";
    s.Moments.resize((size_t)count);
    for (int i = 0; i < count; i++) {
        auto m = entries.find("m." + std::to_string(i)), v = entries.find("v." + std::to_string(i));
        if (m == entries.end() || v == entries.end()) return "autograd: optimizer state is missing parameter " + std::to_string(i);
        if (m->second.Shape != std::vector<int>{(int)m->second.Values.size()} ||
            v->second.Shape != std::vector<int>{(int)v->second.Values.size()})
            return "autograd: optimizer moment shape mismatch " + std::to_string(i);
        s.Moments[(size_t)i].M = m->second.Values;
        s.Moments[(size_t)i].V = v->second.Values;
    }
    *out = std::move(s);
    return "";
}

// ---- SGD --------------------------------------------------------------------------------
// Metadata of a "gograd-sgd" file: it depends on names, shapes, options, flags and groups, never
// on the buffer values, so a streamed writer can lay the file out before any value arrives.
void sgdMetadata(const SGDState& s, Metadata* metadata) {
    std::string init = s.Initialized.empty() ? "[]" : "[";
    for (size_t i = 0; i < s.Initialized.size(); i++) init += std::string(i ? "," : "") + (s.Initialized[i] ? "true" : "false");
    if (!s.Initialized.empty()) init += "]";
    const SGDOptions& o = s.Options;
    std::string config = "{\"StepCount\":" + std::to_string(s.StepCount) + ",\"Names\":" + string_list(s.Names, true) +
                         ",\"Shapes\":" + shapes_json(s.Shapes) + ",\"Options\":{\"LR\":" + f32(o.LR) + ",\"Momentum\":" +
                         f32(o.Momentum) + ",\"Dampening\":" + f32(o.Dampening) + ",\"WeightDecay\":" + f32(o.WeightDecay) +
                         ",\"Nesterov\":" + (o.Nesterov ? "true" : "false") + ",\"Maximize\":" + (o.Maximize ? "true" : "false") +
                         "},\"Initialized\":" + init + ",\"Buffers\":null,\"Groups\":" + groups_json(s.Groups) + "}";
    *metadata = {{"format", "gograd-sgd"}, {"version", "1"}, {"step_count", std::to_string(s.StepCount)}, {"optimizer", config}};
}

std::string sgdEntries(SGDState s, EntryMap* entries, Metadata* metadata) {
    entries->clear();
    sgdMetadata(s, metadata);
    for (size_t i = 0; i < s.Initialized.size(); i++) {
        if (!s.Initialized[i]) continue;  // only initialised parameters have a buffer entry
        SafeTensorEntry b;
        b.Values = std::move(s.Buffers[i]);
        b.Shape = {(int)b.Values.size()};
        (*entries)["buffer." + std::to_string(i)] = std::move(b);
    }
    return "";
}

std::string sgdStateFromEntries(const EntryMap& entries, const Metadata& metadata, SGDState* out) {
    if (meta(metadata, "format") != "gograd-sgd" || meta(metadata, "version") != "1") return "autograd: unsupported SGD state format";
    ggjson::Value root;
    std::string err;
    if (!ggjson::Parser(meta(metadata, "optimizer")).parse(&root, &err) || !root.is(ggjson::Value::Obj))
        return "autograd: invalid SGD configuration: " + err;
    SGDState s;
    const ggjson::Value* o = root.get("Options");
    if (!get_int(root.get("StepCount"), &s.StepCount) || !get_strings(root.get("Names"), &s.Names) ||
        !get_shapes(root.get("Shapes"), &s.Shapes) || !o || !o->is(ggjson::Value::Obj) || !get_f32(o->get("LR"), &s.Options.LR) ||
        !get_f32(o->get("Momentum"), &s.Options.Momentum) || !get_f32(o->get("Dampening"), &s.Options.Dampening) ||
        !get_f32(o->get("WeightDecay"), &s.Options.WeightDecay) || !get_bool(o->get("Nesterov"), &s.Options.Nesterov) ||
        !get_bool(o->get("Maximize"), &s.Options.Maximize) || !get_groups(root.get("Groups"), &s.Groups))
        return "autograd: invalid SGD configuration: wrong field type";
    const ggjson::Value* init = root.get("Initialized");
    if (init && init->is(ggjson::Value::Arr)) {
        for (const auto& b : *init->arr) {
            bool flag = false;
            if (!get_bool(&b, &flag)) return "autograd: invalid SGD configuration: wrong field type";
            s.Initialized.push_back(flag);
        }
    }
    int step = 0;
    if (!parse_int_text(meta(metadata, "step_count"), &step) || step != s.StepCount || step < 0 ||
        s.Initialized.size() != s.Names.size())
        return "autograd: invalid SGD state metadata";
    s.Buffers.resize(s.Names.size());
    size_t expected = 0;
    for (size_t i = 0; i < s.Initialized.size(); i++) {
        if (!s.Initialized[i]) continue;
        expected++;
        auto it = entries.find("buffer." + std::to_string(i));
        if (it == entries.end() || it->second.Shape != std::vector<int>{(int)it->second.Values.size()})
            return "autograd: missing or invalid SGD buffer " + std::to_string(i);
        s.Buffers[i] = it->second.Values;
    }
    if (entries.size() != expected) return "autograd: unexpected SGD state entries";
    *out = std::move(s);
    return "";
}

// ---- snapshots --------------------------------------------------------------------------
static int snapshotStep(const OptimizerSnapshot& s) {
    if (s.Kind == "adamw" && s.AdamW) return s.AdamW->StepCount;
    if (s.Kind == "sgd" && s.SGD) return s.SGD->StepCount;
    return -1;
}

std::string snapshotEntries(const OptimizerSnapshot& s, EntryMap* entries, Metadata* metadata) {
    if (s.Kind == "adamw" && s.AdamW) return optimizerEntries(*s.AdamW, entries, metadata);
    if (s.Kind == "sgd" && s.SGD) return sgdEntries(*s.SGD, entries, metadata);
    return "autograd: unknown optimizer snapshot";
}

std::string snapshotFromEntries(const EntryMap& entries, Metadata metadata, OptimizerSnapshot* out) {
    std::string kind = meta(metadata, "optimizer_kind");
    if (kind.empty()) kind = "adamw";  // legacy training-1 files (autograd/optimizer.go:94-98)
    out->Version = 1;
    out->Kind = kind;
    if (kind == "sgd") {
        metadata["format"] = "gograd-sgd";
        auto s = std::make_shared<SGDState>();
        std::string e = sgdStateFromEntries(entries, metadata, s.get());
        if (!e.empty()) return e;
        out->SGD = s;
        out->AdamW.reset();
        return "";
    }
    if (kind != "adamw") return "autograd: unknown optimizer kind \"" + kind + "\"";
    ggjson::Value root;
    std::string err;
    if (!ggjson::Parser(meta(metadata, "optimizer")).parse(&root, &err) || !root.is(ggjson::Value::Obj))
        return "autograd: invalid optimizer configuration: " + err;
    std::vector<std::string> names;
    if (!get_strings(root.get("Names"), &names)) return "autograd: invalid optimizer configuration: wrong field type";
    metadata["format"] = "gograd-adamw";
    auto s = std::make_shared<OptimizerState>();
    std::string e = optimizerStateFromEntries(entries, metadata, (int)names.size(), s.get());
    if (!e.empty()) return e;
    out->AdamW = s;
    out->SGD.reset();
    return "";
}

// ---- training checkpoint ----------------------------------------------------------------
static std::string scheduler_json(const OneCycle& c) {
    return "{\"MaxLR\":" + f64(c.MaxLR) + ",\"PctStart\":" + f64(c.PctStart) + ",\"DivFactor\":" + f64(c.DivFactor) +
           ",\"FinalDivFactor\":" + f64(c.FinalDivFactor) + ",\"Total\":" + std::to_string(c.Total) + ",\"StepCount\":" +
           std::to_string(c.StepCount) + "}";
}

static std::string parse_scheduler(const std::string& text, OneCycle* c) {
    ggjson::Value root;
    std::string err;
    if (!ggjson::Parser(text).parse(&root, &err) || !root.is(ggjson::Value::Obj)) return "autograd: invalid scheduler state: " + err;
    if (!get_f64(root.get("MaxLR"), &c->MaxLR) || !get_f64(root.get("PctStart"), &c->PctStart) ||
        !get_f64(root.get("DivFactor"), &c->DivFactor) || !get_f64(root.get("FinalDivFactor"), &c->FinalDivFactor) ||
        !get_int(root.get("Total"), &c->Total) || !get_int(root.get("StepCount"), &c->StepCount))
        return "autograd: invalid scheduler state: wrong field type";
    return "";
}

static std::string parse_user(const std::string& text, std::map<std::string, std::string>* user) {
    user->clear();
    ggjson::Value root;
    std::string err;
    if (!ggjson::Parser(text).parse(&root, &err)) return "autograd: invalid user metadata: " + err;
    if (root.is(ggjson::Value::Null)) return "";
    if (!root.is(ggjson::Value::Obj)) return "autograd: invalid user metadata";
    for (const auto& kv : *root.obj) {
        if (!kv.second.is(ggjson::Value::String)) return "autograd: invalid user metadata";
        (*user)[kv.first] = kv.second.raw;
    }
    return "";
}

std::string SaveTrainingCheckpoint(const std::string& path, const std::vector<Parameter>& model,
                                   CheckpointOptimizer* optimizer, const OneCycle* scheduler,
                                   const std::map<std::string, std::string>& user) {
    if (!optimizer || !scheduler) return "autograd: model, optimizer and scheduler are required";
    OptimizerSnapshot state;
    std::string e = optimizer->Snapshot(&state);
    if (!e.empty()) return e;
    if (!(e = optimizer->ValidateSnapshot(state)).empty()) return e;
    if (!(e = validateOneCycle(*scheduler)).empty()) return e;
    if (scheduler->StepCount != snapshotStep(state)) return "autograd: optimizer/scheduler step mismatch";
    EntryMap entries, opt;
    Metadata meta_out;
    if (!(e = snapshotEntries(state, &opt, &meta_out)).empty()) return e;
    for (const Parameter& p : model) {
        if (!p.Value || p.Name.empty()) return "autograd: model entries need names and values";
        SafeTensorEntry entry;
        if (!(e = p.Value->ToHost(&entry.Values)).empty()) return e;
        entry.Shape = p.Value->Shape;
        if (entries.count("model." + p.Name)) return "autograd: duplicate model entry " + p.Name;
        entries["model." + p.Name] = std::move(entry);
    }
    for (auto& kv : opt) entries["optimizer." + kv.first] = std::move(kv.second);
    std::string user_json = "{";
    bool first = true;
    for (const auto& kv : user) {
        user_json += (first ? "" : ",") + quote(kv.first) + ":" + quote(kv.second);
        first = false;
    }
    user_json += "}";
    meta_out["format"] = "gograd-training-1";
    meta_out["optimizer_kind"] = state.Kind;
    meta_out["scheduler"] = scheduler_json(*scheduler);
    meta_out["user"] = user_json;
    return write_safetensors(path, entries, &meta_out);
}

std::string TrainingCheckpointMetadata(const std::string& path, std::map<std::string, std::string>* user) {
    EntryMap entries;
    Metadata metadata;
    std::string e = read_safetensors(path, &entries, &metadata);
    if (!e.empty()) return e;
    if (meta(metadata, "format") != "gograd-training-1") return "autograd: not a training checkpoint";
    return parse_user(meta(metadata, "user"), user);
}

std::string LoadTrainingCheckpoint(const std::string& path, const std::vector<Parameter>& model,
                                   CheckpointOptimizer* optimizer, OneCycle* scheduler,
                                   std::map<std::string, std::string>* user) {
    if (!optimizer || !scheduler) return "autograd: model, optimizer and scheduler are required";
    EntryMap entries;
    Metadata metadata;
    std::string e = read_safetensors(path, &entries, &metadata);
    if (!e.empty()) return e;
    if (meta(metadata, "format") != "gograd-training-1") return "autograd: not a training checkpoint";
    EntryMap model_entries, opt;
    for (auto& kv : entries) {
        if (kv.first.rfind("model.", 0) == 0)
            model_entries[kv.first.substr(6)] = std::move(kv.second);
        else if (kv.first.rfind("optimizer.", 0) == 0)
            opt[kv.first.substr(10)] = std::move(kv.second);
        else
            return "autograd: unknown checkpoint entry \"" + kv.first + "\"";
    }
    // Everything is validated before anything is copied (autograd/training_checkpoint.go:79-132).
    if (model_entries.size() != model.size()) return "autograd: checkpoint has " + std::to_string(model_entries.size()) + " model entries, module has " + std::to_string(model.size());
    for (const Parameter& p : model) {
        auto it = model_entries.find(p.Name);
        if (it == model_entries.end()) return "autograd: missing tensor " + p.Name;
        if (it->second.Shape != p.Value->Shape) return "autograd: shape mismatch for " + p.Name;
    }
    OptimizerSnapshot state;
    if (!(e = snapshotFromEntries(opt, metadata, &state)).empty()) return e;
    if (!(e = optimizer->ValidateSnapshot(state)).empty()) return e;
    OneCycle schedule;
    if (!(e = parse_scheduler(meta(metadata, "scheduler"), &schedule)).empty()) return e;
    if (!(e = validateOneCycle(schedule)).empty()) return e;
    if (schedule.StepCount != snapshotStep(state)) return "autograd: optimizer/scheduler step mismatch";
    std::map<std::string, std::string> parsed_user;
    if (!(e = parse_user(meta(metadata, "user"), &parsed_user)).empty()) return e;
    for (const Parameter& p : model)
        if (!(e = p.Value->CopyFromHost(model_entries[p.Name].Values)).empty()) return e;
    if (!(e = optimizer->LoadSnapshot(state)).empty()) return e;
    *scheduler = schedule;
    if (user) *user = parsed_user;
    return "";
}

}  // namespace autograd
