// Adapter ingest and the adapter registry (host only): PEFT adapter_config.json rules, safetensors -> BF16, PEFT key
// classification, the load-time audit, slot packing, routing tables and slot lifecycle.
//
// Follows, by behaviour (names of the rejections included, so that a caller's log reads like the reference's):
//   parse_peft_adapter_config     crates/atlas-core/src/config/parsers/lora.rs:121-262
//   load_adapter_safetensors      crates/spark-runtime/src/weights/adapter.rs:62-105   (F16 / F32 -> BF16 on the host)
//   classify_key, adapter_id_hash crates/spark-model/src/lora/key.rs:33-113
//   validate_peft_config          crates/spark-model/src/lora/env.rs:59-77
//   audit_adapter, pack_slot,
//   load_lora_adapters_multi,
//   pack_store_into_slot          crates/spark-model/src/lora/loading.rs:48-459
//   LoraWeights lifecycle         crates/spark-model/src/lora/types.rs:268-413
// The registry never touches a GPU: it is told the pool's device base address, hands back host images (one slot's
// bytes; the pointer / scale / rank tables) and the caller uploads them.
#include "atlas_b200.h"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "json_min.hpp"

namespace atlas {
namespace {

const char* const kModuleNames[ATLAS_B200_NUM_MODULES] = {"q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"};
const char* const kModulePaths[ATLAS_B200_NUM_MODULES] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                                                          "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"};

void put_err(char* err, size_t cap, const std::string& msg) {
    if (!err || cap == 0) return;
    const size_t n = msg.size() < cap - 1 ? msg.size() : cap - 1;
    std::memcpy(err, msg.data(), n);
    err[n] = 0;
}

struct Reject {
    std::string msg;
};

std::string leaf_of(const std::string& entry) {
    const size_t dot = entry.rfind('.');
    return dot == std::string::npos ? entry : entry.substr(dot + 1);
}

int module_by_name(const std::string& leaf) {
    for (int m = 0; m < ATLAS_B200_NUM_MODULES; ++m)
        if (leaf == kModuleNames[m]) return m;
    return -1;
}

// ---------------------------------------------------------------------------------------------------
// PEFT config
// ---------------------------------------------------------------------------------------------------
struct PeftConfig {
    size_t r = 0;
    double lora_alpha = 0.0;
    bool use_rslora = false;
    std::vector<std::string> target_modules;
    bool has_layers = false;
    std::vector<size_t> layers_to_transform;
    float scaling() const {
        if (r == 0) return 0.0f;
        return use_rslora ? float(lora_alpha / std::sqrt(double(r))) : float(lora_alpha / double(r));
    }
};

bool nonempty_object(const json::Value* v) { return v && v->kind == json::Value::Object && !v->members.empty(); }

// returns 0, ATLAS_B200_ERR_REJECT (msg = named reason) or ATLAS_B200_ERR_DIMS (msg = what is malformed)
int parse_peft(const char* text, size_t len, PeftConfig& out, std::string& msg) {
    json::Value doc;
    {
        json::Parser ps(text, len);
        std::string e;
        if (!ps.parse(doc, e) || doc.kind != json::Value::Object) {
            msg = "Parsing PEFT adapter_config.json (r / lora_alpha / target_modules required): " + (e.empty() ? std::string("not an object") : e);
            return ATLAS_B200_ERR_DIMS;
        }
    }
    const json::Value* r = doc.get("r");
    const json::Value* alpha = doc.get("lora_alpha");
    const json::Value* targets = doc.get("target_modules");
    if (!r || !r->is_integer() || r->text[0] == '-' || !alpha || alpha->kind != json::Value::Number || !targets) {
        msg = "Parsing PEFT adapter_config.json (r / lora_alpha / target_modules required)";
        return ATLAS_B200_ERR_DIMS;
    }
    auto reject = [&](const std::string& m) { msg = m; return ATLAS_B200_ERR_REJECT; };
    if (const json::Value* pt = doc.get("peft_type"); pt && pt->kind == json::Value::String) {
        std::string up = pt->text;
        for (char& c : up) c = char(std::toupper(static_cast<unsigned char>(c)));
        if (up != "LORA") return reject("REJECT(peft_type): adapter declares peft_type='" + pt->text + "'; only LORA is supported");
    }
    if (const json::Value* v = doc.get("use_dora"); v && v->kind == json::Value::Bool && v->b)
        return reject("REJECT(use_dora): DoRA adapters are unsupported (magnitude decomposition has no runtime-delta form)");
    if (const json::Value* v = doc.get("bias"); v && v->kind == json::Value::String && v->text != "none")
        return reject("REJECT(bias): bias='" + v->text + "' ships trained bias deltas; only bias='none' is supported");
    if (nonempty_object(doc.get("rank_pattern")))
        return reject("REJECT(rank_pattern): per-module rank overrides are unsupported in v0 (uniform r only)");
    if (nonempty_object(doc.get("alpha_pattern")))
        return reject("REJECT(alpha_pattern): per-module alpha overrides are unsupported in v0 (uniform lora_alpha only)");
    if (const json::Value* v = doc.get("modules_to_save"); v && v->kind == json::Value::Array && !v->items.empty())
        return reject("REJECT(modules_to_save): adapter saves full modules " + v->dump() + "; full-weight replacement is unsupported");
    const json::Value* rs = doc.get("use_rslora");
    if (!rs || rs->kind != json::Value::Bool)
        return reject("REJECT(use_rslora): field absent — scaling inputs are never defaulted (PEFT <0.7 config; re-export the adapter with peft>=0.7)");
    out.use_rslora = rs->b;
    if (const json::Value* lt = doc.get("layers_to_transform"); lt && lt->kind != json::Value::Null) {
        if (lt->kind != json::Value::Array)
            return reject("REJECT(layers_to_transform): expected null or an array of layer indices, got " + lt->dump());
        out.has_layers = true;
        for (const json::Value& e : lt->items) {
            if (!e.is_integer() || e.text[0] == '-') return reject("REJECT(layers_to_transform): entries must be non-negative integers");
            out.layers_to_transform.push_back(size_t(e.as_u64()));
        }
    }
    out.r = size_t(r->as_u64());
    if (out.r == 0) return reject("REJECT(r): LoRA rank must be > 0");
    out.lora_alpha = alpha->as_double();
    if (!(std::isfinite(out.lora_alpha) && out.lora_alpha > 0.0))
        return reject("REJECT(lora_alpha): must be a finite positive number, got " + alpha->text);
    if (targets->kind == json::Value::String)
        return reject("REJECT(target_modules): string form '" + targets->text + "' (e.g. 'all-linear') is unsupported — re-export the adapter with an explicit module list");
    if (targets->kind != json::Value::Array) return reject("REJECT(target_modules): expected an array of module names, got " + targets->dump());
    for (const json::Value& e : targets->items) {
        if (e.kind != json::Value::String) return reject("REJECT(target_modules): entries must be strings");
        out.target_modules.push_back(e.text);
    }
    if (out.target_modules.empty()) return reject("REJECT(target_modules): empty list — adapter targets nothing");
    for (const std::string& entry : out.target_modules) {
        const std::string leaf = leaf_of(entry);
        static const char* const gdn[] = {"in_proj_qkvz", "in_proj_ba", "in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b", "out_proj", "conv1d"};
        for (const char* g : gdn)
            if (leaf == g)
                return reject("REJECT(gdn): target module '" + leaf + "' is a GDN/linear-attention projection; GDN layers are unsupported in v0 (full-attention layers only)");
        if (leaf == "embed_tokens" || leaf == "lm_head") return reject("REJECT(embedding): target module '" + leaf + "' is unsupported in v0");
        if (module_by_name(leaf) < 0)
            return reject("REJECT(unknown_module): target module '" + leaf + "' is not in the v0 allow-list [q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj]");
    }
    return ATLAS_B200_OK;
}

// ---------------------------------------------------------------------------------------------------
// BF16 conversion
// ---------------------------------------------------------------------------------------------------
inline uint16_t f32_bits_to_bf16(uint32_t bits) {
    if ((bits & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((bits >> 16) | 0x0040u);      // NaN: quieted, sign and payload top bits kept
    return uint16_t((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}

inline uint32_t f16_bits_to_f32_bits(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return sign;
        int e = -1;                                       // subnormal half: normalise
        do { man <<= 1; ++e; } while (!(man & 0x400u));
        return sign | uint32_t(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
    if (exp == 31) return sign | 0x7F800000u | (man << 13);
    return sign | (exp + 112u) << 23 | man << 13;
}

int convert_to_bf16(const std::string& dtype, const void* src, size_t n, void* dst) {
    auto* out = static_cast<uint16_t*>(dst);
    const auto* in = static_cast<const unsigned char*>(src);
    if (dtype == "BF16") { std::memcpy(dst, src, n * 2); return ATLAS_B200_OK; }
    if (dtype == "F16") {
        for (size_t i = 0; i < n; ++i) out[i] = f32_bits_to_bf16(f16_bits_to_f32_bits(uint16_t(in[2 * i] | (in[2 * i + 1] << 8))));
        return ATLAS_B200_OK;
    }
    if (dtype == "F32") {
        for (size_t i = 0; i < n; ++i) {
            const uint32_t b = uint32_t(in[4 * i]) | uint32_t(in[4 * i + 1]) << 8 | uint32_t(in[4 * i + 2]) << 16 | uint32_t(in[4 * i + 3]) << 24;
            out[i] = f32_bits_to_bf16(b);
        }
        return ATLAS_B200_OK;
    }
    return ATLAS_B200_ERR_DIMS;
}

// ---------------------------------------------------------------------------------------------------
// safetensors: 8-byte little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, then the bytes
// ---------------------------------------------------------------------------------------------------
struct TensorView {
    std::string dtype;
    std::vector<size_t> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
    size_t elems() const { size_t n = 1; for (size_t d : shape) n *= d; return n; }
};

int read_safetensors(const void* file, size_t len, std::map<std::string, TensorView>& out, std::string& msg) {
    const auto* p = static_cast<const unsigned char*>(file);
    if (len < 8) { msg = "safetensors: file shorter than its length prefix"; return ATLAS_B200_ERR_DIMS; }
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | p[i];
    if (hlen > len - 8) { msg = "safetensors: header length exceeds the file"; return ATLAS_B200_ERR_DIMS; }
    json::Value hdr;
    {
        json::Parser ps(reinterpret_cast<const char*>(p + 8), size_t(hlen));
        std::string e;
        if (!ps.parse(hdr, e) || hdr.kind != json::Value::Object) { msg = "safetensors: malformed header (" + e + ")"; return ATLAS_B200_ERR_DIMS; }
    }
    const unsigned char* data0 = p + 8 + hlen;
    const size_t data_len = len - 8 - size_t(hlen);
    for (const auto& m : hdr.members) {
        if (m.first == "__metadata__") continue;
        const json::Value* dt = m.second.get("dtype");
        const json::Value* sh = m.second.get("shape");
        const json::Value* off = m.second.get("data_offsets");
        if (!dt || dt->kind != json::Value::String || !sh || sh->kind != json::Value::Array || !off || off->kind != json::Value::Array ||
            off->items.size() != 2) { msg = "safetensors: tensor '" + m.first + "' lacks dtype / shape / data_offsets"; return ATLAS_B200_ERR_DIMS; }
        TensorView t;
        t.dtype = dt->text;
        for (const json::Value& d : sh->items) {
            if (!d.is_integer()) { msg = "safetensors: tensor '" + m.first + "' has a malformed shape"; return ATLAS_B200_ERR_DIMS; }
            t.shape.push_back(size_t(d.as_u64()));
        }
        const uint64_t b = off->items[0].as_u64(), e = off->items[1].as_u64();
        if (e < b || e > data_len) { msg = "safetensors: tensor '" + m.first + "' lies outside the file"; return ATLAS_B200_ERR_DIMS; }
        t.data = data0 + b;
        t.bytes = size_t(e - b);
        out[m.first] = t;
    }
    return ATLAS_B200_OK;
}

// ---------------------------------------------------------------------------------------------------
// key classification
// ---------------------------------------------------------------------------------------------------
bool ends_with(const std::string& s, const char* suffix) {
    const size_t n = std::strlen(suffix);
    return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

int classify_key(const std::string& key, uint32_t num_hidden_layers, const uint8_t* full_attention, uint32_t& layer, int& module,
                 int& ab, std::string& msg) {
    auto reject = [&](const std::string& m) { msg = m; return ATLAS_B200_ERR_REJECT; };
    static const std::string prefix = "base_model.model.";
    if (key.compare(0, prefix.size(), prefix) != 0) return reject("REJECT[not-peft-key]: '" + key + "' lacks the 'base_model.model.' PEFT prefix");
    std::string stripped = key.substr(prefix.size());
    if (stripped.find("lora_embedding_") != std::string::npos)
        return reject("REJECT[embedding-lora]: '" + key + "' — embed_tokens/lm_head LoRA is out of v0 scope");
    std::string module_path;
    if (ends_with(stripped, ".lora_A.weight")) { module_path = stripped.substr(0, stripped.size() - 14); ab = 0; }
    else if (ends_with(stripped, ".lora_B.weight")) { module_path = stripped.substr(0, stripped.size() - 14); ab = 1; }
    else
        return reject("REJECT[unrecognized-tensor]: '" + key + "' is not a lora_A/lora_B weight (modules_to_save exports and old '.lora_A.<adapter>.weight' layouts are not supported in v0)");
    const size_t at = module_path.find(".layers.");
    if (at == std::string::npos) return reject("REJECT[non-layer-module]: '" + key + "' targets '" + module_path + "' outside the layer stack");
    const std::string rest = module_path.substr(at + 8);
    const size_t dot = rest.find('.');
    if (dot == std::string::npos) return reject("REJECT[malformed-key]: '" + key + "'");
    const std::string idx = rest.substr(0, dot), tail = rest.substr(dot + 1);
    if (idx.empty() || idx.size() > 9) return reject("REJECT[malformed-layer-index]: '" + key + "'");
    for (char c : idx)
        if (c < '0' || c > '9') return reject("REJECT[malformed-layer-index]: '" + key + "'");
    layer = uint32_t(std::strtoul(idx.c_str(), nullptr, 10));
    if (layer >= num_hidden_layers)
        return reject("REJECT[layer-out-of-range]: '" + key + "' targets layer " + idx + " (model has " + std::to_string(num_hidden_layers) + ")");
    module = -1;
    for (int m = 0; m < ATLAS_B200_NUM_MODULES; ++m)
        if (tail == kModulePaths[m]) module = m;
    if (module < 0) {
        if (tail.compare(0, 12, "linear_attn.") == 0)
            return reject("REJECT[gdn-target]: '" + key + "' — GDN/linear-attention projections (in_proj_qkv / in_proj_z / in_proj_a / in_proj_b / out_proj) are rejected until an exact-replay parity harness exists");
        return reject("REJECT[unsupported-module]: '" + key + "' targets '" + tail + "'");
    }
    if (full_attention && !full_attention[layer])
        return reject("REJECT[non-full-attention-layer]: '" + key + "' targets layer " + idx + "; v0 applies LoRA only on the full-attention layers");
    return ATLAS_B200_OK;
}

uint64_t adapter_id_hash(const char* name, uint64_t generation) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (const unsigned char* c = reinterpret_cast<const unsigned char*>(name); *c; ++c) { h ^= *c; h *= 0x100000001b3ull; }
    if (generation != 0)
        for (int i = 0; i < 8; ++i) { h ^= (generation >> (8 * i)) & 0xFFu; h *= 0x100000001b3ull; }
    return h == 0 ? 1 : h;
}

}  // namespace
}  // namespace atlas

// =====================================================================================================
// the registry object
// =====================================================================================================
struct atlas_b200_registry {
    atlas_b200_model_dims cfg{};
    uint32_t num_hidden_layers = 0;
    std::vector<int32_t> ordinal_of_layer;        // global layer -> pool ordinal, -1 = carries no LoRA
    std::vector<uint8_t> full_attention;          // [num_hidden_layers]
    size_t max_loras = 0, max_rank = 0, slot_bytes = 0;
    uint64_t pool_base = 0;
    struct Slot {
        std::string name;                         // empty = placeholder (never filled)
        atlas::PeftConfig peft;
        float scale = 0.0f;
        uint32_t rank = 0;
        uint64_t generation = 0;
        std::vector<uint8_t> present;             // [ordinals * modules]: the adapter carries this (layer, module)
    };
    std::vector<Slot> slots;
    size_t active = 0, pinned = 0;
    std::vector<std::atomic<size_t>> ref_counts;
    std::vector<std::atomic<uint64_t>> last_used;
    std::atomic<uint64_t> lru_tick{0};
    std::mutex mu;                                // guards slots / active / pinned (loads and swaps)

    atlas_b200_registry(size_t n) : ref_counts(n), last_used(n) {
        for (auto& r : ref_counts) r.store(0);
        for (auto& l : last_used) l.store(0);
    }
};

using namespace atlas;

extern "C" {

int atlas_b200_peft_parse(const char* json_text, size_t len, atlas_b200_peft_config* out, char* err, size_t err_cap) {
    if (!json_text || !out) return ATLAS_B200_ERR_NULL;
    PeftConfig c;
    std::string msg;
    const int rc = parse_peft(json_text, len, c, msg);
    if (rc) { put_err(err, err_cap, msg); return rc; }
    if (c.target_modules.size() > ATLAS_B200_PEFT_MAX_TARGETS || c.layers_to_transform.size() > ATLAS_B200_PEFT_MAX_LAYERS) return ATLAS_B200_ERR_LIMIT;
    std::memset(out, 0, sizeof(*out));
    out->r = c.r;
    out->lora_alpha = c.lora_alpha;
    out->use_rslora = c.use_rslora ? 1 : 0;
    out->n_target_modules = uint32_t(c.target_modules.size());
    for (size_t i = 0; i < c.target_modules.size(); ++i) {
        if (c.target_modules[i].size() >= sizeof(out->target_modules[0])) return ATLAS_B200_ERR_LIMIT;
        std::memcpy(out->target_modules[i], c.target_modules[i].c_str(), c.target_modules[i].size() + 1);
    }
    out->has_layers_to_transform = c.has_layers ? 1 : 0;
    out->n_layers_to_transform = uint32_t(c.layers_to_transform.size());
    for (size_t i = 0; i < c.layers_to_transform.size(); ++i) out->layers_to_transform[i] = uint32_t(c.layers_to_transform[i]);
    return ATLAS_B200_OK;
}

float atlas_b200_peft_config_scaling(const atlas_b200_peft_config* cfg) {
    if (!cfg || cfg->r == 0) return 0.0f;
    return cfg->use_rslora ? float(cfg->lora_alpha / std::sqrt(double(cfg->r))) : float(cfg->lora_alpha / double(cfg->r));
}

int atlas_b200_classify_key(const char* key, uint32_t num_hidden_layers, const uint8_t* full_attention, uint32_t* layer, int* module,
                            int* ab, char* err, size_t err_cap) {
    if (!key || !layer || !module || !ab) return ATLAS_B200_ERR_NULL;
    std::string msg;
    const int rc = classify_key(key, num_hidden_layers, full_attention, *layer, *module, *ab, msg);
    if (rc) put_err(err, err_cap, msg);
    return rc;
}

uint64_t atlas_b200_adapter_id_hash(const char* name, uint64_t generation) { return name ? adapter_id_hash(name, generation) : 0; }

int atlas_b200_convert_to_bf16(const char* dtype, const void* src, size_t n_elems, void* dst_bf16) {
    if (!dtype || (!src && n_elems) || (!dst_bf16 && n_elems)) return ATLAS_B200_ERR_NULL;
    return convert_to_bf16(dtype, src, n_elems, dst_bf16);
}

int atlas_b200_registry_create(const atlas_b200_model_dims* cfg, uint32_t num_hidden_layers, const uint8_t* full_attention,
                               size_t max_loras, size_t max_rank, uint64_t pool_device_base, atlas_b200_registry** out) {
    if (!cfg || !out) return ATLAS_B200_ERR_NULL;
    if (max_loras == 0 || max_rank == 0 || num_hidden_layers == 0) return ATLAS_B200_ERR_DIMS;
    auto* reg = new atlas_b200_registry(max_loras);
    reg->cfg = *cfg;
    reg->num_hidden_layers = num_hidden_layers;
    reg->full_attention.assign(num_hidden_layers, 1);
    if (full_attention) reg->full_attention.assign(full_attention, full_attention + num_hidden_layers);
    reg->ordinal_of_layer.assign(num_hidden_layers, -1);
    int32_t ord = 0;
    for (uint32_t l = 0; l < num_hidden_layers; ++l)
        if (reg->full_attention[l]) reg->ordinal_of_layer[l] = ord++;
    if (uint32_t(ord) != cfg->num_full_attention_layers) { delete reg; return ATLAS_B200_ERR_DIMS; }
    reg->max_loras = max_loras;
    reg->max_rank = max_rank;
    reg->slot_bytes = atlas_b200_pool_slot_bytes(cfg, max_rank);
    reg->pool_base = pool_device_base;
    reg->slots.resize(max_loras);
    for (auto& s : reg->slots) s.present.assign(size_t(ord) * ATLAS_B200_NUM_MODULES, 0);
    *out = reg;
    return ATLAS_B200_OK;
}

void atlas_b200_registry_destroy(atlas_b200_registry* reg) { delete reg; }
size_t atlas_b200_registry_slot_bytes(const atlas_b200_registry* reg) { return reg ? reg->slot_bytes : 0; }
size_t atlas_b200_registry_pool_bytes(const atlas_b200_registry* reg) { return reg ? reg->slot_bytes * reg->max_loras : 0; }

int atlas_b200_registry_load_adapter(atlas_b200_registry* reg, size_t slot, const char* name, const char* config_json, size_t config_len,
                                     const void* safetensors, size_t st_len, void* slot_image, char* err, size_t err_cap) {
    if (!reg || !name || !config_json || !safetensors || !slot_image) return ATLAS_B200_ERR_NULL;
    if (slot >= reg->max_loras) { put_err(err, err_cap, "LoRA disk swap: slot " + std::to_string(slot) + " >= max_loras " + std::to_string(reg->max_loras)); return ATLAS_B200_ERR_LIMIT; }
    std::lock_guard<std::mutex> lock(reg->mu);
    // a filled slot is only replaced while idle, and before anything destructive happens
    const bool refill = !reg->slots[slot].name.empty();
    if (refill) {
        const size_t busy = reg->ref_counts[slot].load(std::memory_order_acquire);
        if (busy > 0) {
            put_err(err, err_cap, "LoRA disk swap REFUSED: slot " + std::to_string(slot) + " has " + std::to_string(busy) +
                                  " in-flight sequence(s) (ref_count>0); cannot replace an adapter mid-decode");
            return ATLAS_B200_ERR_BUSY;
        }
    }
    std::string msg;
    PeftConfig peft;
    int rc = parse_peft(config_json, config_len, peft, msg);
    if (rc) { put_err(err, err_cap, msg); return rc; }
    auto reject = [&](const std::string& m) { put_err(err, err_cap, m); return ATLAS_B200_ERR_REJECT; };
    // validate_peft_config
    if (peft.r > reg->max_rank) return reject("REJECT[rank-exceeds-pool]: r=" + std::to_string(peft.r) + " > --max-lora-rank=" + std::to_string(reg->max_rank));
    for (const std::string& t : peft.target_modules)
        if (module_by_name(leaf_of(t)) < 0)
            return reject("REJECT[unsupported-target]: target_modules entry '" + t + "' (allowed: q_proj k_proj v_proj o_proj gate_proj up_proj down_proj)");
    std::map<std::string, TensorView> tensors;
    rc = read_safetensors(safetensors, st_len, tensors, msg);
    if (rc) { put_err(err, err_cap, msg); return rc; }
    // 1) every tensor must classify; duplicates are fatal
    struct Pair { const TensorView* ab[2] = {nullptr, nullptr}; std::string key[2]; };
    std::map<std::pair<uint32_t, int>, Pair> found;
    for (const auto& kv : tensors) {
        uint32_t layer = 0;
        int module = 0, ab = 0;
        rc = classify_key(kv.first, reg->num_hidden_layers, reg->full_attention.data(), layer, module, ab, msg);
        if (rc) { put_err(err, err_cap, msg); return rc; }
        Pair& pr = found[{layer, module}];
        if (pr.ab[ab]) return reject("REJECT[duplicate-tensor]: two tensors map to layer " + std::to_string(layer) + " " + kModuleNames[module] + " lora_" + (ab ? "B" : "A"));
        pr.ab[ab] = &kv.second;
        pr.key[ab] = kv.first;
    }
    if (found.empty()) return reject("REJECT[empty-adapter]: no lora_A/lora_B tensors in adapter");
    // 2) pairs complete, shapes A = [r, in], B = [out, r], dtypes convertible
    for (const auto& kv : found) {
        const Pair& pr = kv.second;
        if (!pr.ab[0] || !pr.ab[1])
            return reject("REJECT[unpaired-tensor]: layer " + std::to_string(kv.first.first) + " " + kModuleNames[kv.first.second] + " has only one of lora_A/lora_B");
        size_t out_dim = 0, in_dim = 0;
        atlas_b200_module_dims(&reg->cfg, kv.first.second, &out_dim, &in_dim);
        auto shape_text = [](const TensorView& t) { std::string s = "["; for (size_t i = 0; i < t.shape.size(); ++i) s += (i ? ", " : "") + std::to_string(t.shape[i]); return s + "]"; };
        if (pr.ab[0]->shape != std::vector<size_t>{peft.r, in_dim})
            return reject("REJECT[shape-mismatch]: '" + pr.key[0] + "' is " + shape_text(*pr.ab[0]) + ", expected [" + std::to_string(peft.r) + ", " + std::to_string(in_dim) + "] (r, in_dim)");
        if (pr.ab[1]->shape != std::vector<size_t>{out_dim, peft.r})
            return reject("REJECT[shape-mismatch]: '" + pr.key[1] + "' is " + shape_text(*pr.ab[1]) + ", expected [" + std::to_string(out_dim) + ", " + std::to_string(peft.r) + "] (out_dim, r)");
        for (int ab = 0; ab < 2; ++ab) {
            const TensorView& t = *pr.ab[ab];
            const size_t esz = t.dtype == "F32" ? 4 : (t.dtype == "F16" || t.dtype == "BF16") ? 2 : 0;
            if (esz == 0) return reject("REJECT[dtype]: LoRA adapter tensor '" + pr.key[ab] + "' has dtype " + t.dtype + " (F16, F32 and BF16 are supported)");
            if (t.bytes != t.elems() * esz) { put_err(err, err_cap, "safetensors: tensor '" + pr.key[ab] + "' has " + std::to_string(t.bytes) + " bytes for its shape"); return ATLAS_B200_ERR_DIMS; }
        }
    }
    // 3) every target_modules entry matched at least one pair
    for (const std::string& t : peft.target_modules) {
        const int m = module_by_name(leaf_of(t));
        bool any = false;
        for (const auto& kv : found) any = any || kv.first.second == m;
        if (!any) return reject("REJECT[unmatched-target]: target_modules entry '" + t + "' matched no adapter tensor on any full-attention layer");
    }
    // pack: the slot's image is zeroed first (pads and omitted modules stay zero), then A contiguous, B row-repacked
    std::memset(slot_image, 0, reg->slot_bytes);
    atlas_b200_registry::Slot& s = reg->slots[slot];
    std::fill(s.present.begin(), s.present.end(), uint8_t(0));
    std::vector<uint16_t> a_bf, b_bf;
    for (const auto& kv : found) {
        const int32_t ord = reg->ordinal_of_layer[kv.first.first];
        const Pair& pr = kv.second;
        a_bf.resize(pr.ab[0]->elems());
        b_bf.resize(pr.ab[1]->elems());
        convert_to_bf16(pr.ab[0]->dtype, pr.ab[0]->data, a_bf.size(), a_bf.data());
        convert_to_bf16(pr.ab[1]->dtype, pr.ab[1]->data, b_bf.size(), b_bf.data());
        rc = atlas_b200_pack_module(&reg->cfg, reg->max_rank, size_t(ord), kv.first.second, a_bf.data(), b_bf.data(), peft.r, slot_image);
        if (rc) return rc;
        s.present[size_t(ord) * ATLAS_B200_NUM_MODULES + kv.first.second] = 1;
    }
    s.name = name;
    s.scale = peft.scaling();
    s.rank = uint32_t(peft.r);
    s.peft = std::move(peft);
    if (refill) s.generation += 1;             // contents replaced: a fresh adapter identity for the same name
    return ATLAS_B200_OK;
}

int atlas_b200_registry_set_pinned(atlas_b200_registry* reg, size_t pinned) {
    if (!reg) return ATLAS_B200_ERR_NULL;
    if (pinned > reg->max_loras) return ATLAS_B200_ERR_DIMS;
    std::lock_guard<std::mutex> lock(reg->mu);
    reg->pinned = pinned;
    return ATLAS_B200_OK;
}

int atlas_b200_registry_set_active(atlas_b200_registry* reg, size_t slot) {
    if (!reg) return ATLAS_B200_ERR_NULL;
    std::lock_guard<std::mutex> lock(reg->mu);
    if (slot >= reg->max_loras || reg->slots[slot].name.empty()) return ATLAS_B200_ERR_DIMS;
    reg->active = slot;
    return ATLAS_B200_OK;
}

int atlas_b200_registry_route_tables(const atlas_b200_registry* reg, uint32_t layer, int module, uint64_t* a_table, uint64_t* b_table) {
    if (!reg || !a_table || !b_table) return ATLAS_B200_ERR_NULL;
    if (layer >= reg->num_hidden_layers || reg->ordinal_of_layer[layer] < 0 || module < 0 || module >= ATLAS_B200_NUM_MODULES) return ATLAS_B200_ERR_DIMS;
    const size_t ord = size_t(reg->ordinal_of_layer[layer]);
    std::vector<uint8_t> present(reg->max_loras);
    for (size_t k = 0; k < reg->max_loras; ++k) present[k] = reg->slots[k].present[ord * ATLAS_B200_NUM_MODULES + module];
    return atlas_b200_build_route_tables(&reg->cfg, reg->max_rank, ord, module, reg->pool_base, reg->max_loras, present.data(), a_table, b_table);
}

int atlas_b200_registry_scale_table(const atlas_b200_registry* reg, float* out) {
    if (!reg || !out) return ATLAS_B200_ERR_NULL;
    for (size_t k = 0; k < reg->max_loras; ++k) out[k] = reg->slots[k].name.empty() ? 0.0f : reg->slots[k].scale;
    return ATLAS_B200_OK;
}

int atlas_b200_registry_rank_table(const atlas_b200_registry* reg, uint32_t* out) {
    if (!reg || !out) return ATLAS_B200_ERR_NULL;
    for (size_t k = 0; k < reg->max_loras; ++k) out[k] = reg->slots[k].name.empty() ? 0u : reg->slots[k].rank;
    return ATLAS_B200_OK;
}

int32_t atlas_b200_registry_acquire_slot(atlas_b200_registry* reg, int32_t slot) {
    if (!reg) return -1;
    const size_t resolved = slot >= 0 ? size_t(slot) : reg->active;
    if (resolved >= reg->max_loras) return -1;
    reg->ref_counts[resolved].fetch_add(1, std::memory_order_acq_rel);
    reg->last_used[resolved].store(reg->lru_tick.fetch_add(1, std::memory_order_relaxed) + 1, std::memory_order_relaxed);
    return int32_t(resolved);
}

void atlas_b200_registry_release_slot(atlas_b200_registry* reg, int32_t resolved) {
    if (!reg || resolved < 0 || size_t(resolved) >= reg->max_loras) return;
    size_t v = reg->ref_counts[size_t(resolved)].load(std::memory_order_acquire);
    while (v > 0 && !reg->ref_counts[size_t(resolved)].compare_exchange_weak(v, v - 1, std::memory_order_release, std::memory_order_acquire)) {}
}

void atlas_b200_registry_touch_slot(atlas_b200_registry* reg, size_t slot) {
    if (!reg || slot >= reg->max_loras) return;
    reg->last_used[slot].store(reg->lru_tick.fetch_add(1, std::memory_order_relaxed) + 1, std::memory_order_relaxed);
}

size_t atlas_b200_registry_slot_ref_count(const atlas_b200_registry* reg, size_t slot) {
    return (reg && slot < reg->max_loras) ? reg->ref_counts[slot].load(std::memory_order_acquire) : 0;
}
uint64_t atlas_b200_registry_slot_last_used(const atlas_b200_registry* reg, size_t slot) {
    return (reg && slot < reg->max_loras) ? reg->last_used[slot].load(std::memory_order_relaxed) : 0;
}
uint64_t atlas_b200_registry_slot_generation(const atlas_b200_registry* reg, size_t slot) {
    return (reg && slot < reg->max_loras) ? reg->slots[slot].generation : 0;
}

int32_t atlas_b200_registry_slot_of(const atlas_b200_registry* reg, const char* name) {
    if (!reg || !name || !*name) return -1;
    for (size_t k = 0; k < reg->max_loras; ++k)
        if (reg->slots[k].name == name) return int32_t(k);
    return -1;
}

uint64_t atlas_b200_registry_adapter_id_for_slot(const atlas_b200_registry* reg, int32_t slot) {
    if (!reg) return 0;
    const size_t resolved = slot >= 0 ? size_t(slot) : reg->active;
    if (resolved >= reg->max_loras || reg->slots[resolved].name.empty()) return 0;
    return adapter_id_hash(reg->slots[resolved].name.c_str(), reg->slots[resolved].generation);
}

int32_t atlas_b200_registry_select_victim(const atlas_b200_registry* reg) {
    if (!reg) return -1;
    std::vector<size_t> idx, ref;
    std::vector<uint8_t> filled;
    std::vector<uint64_t> lru;
    for (size_t k = reg->pinned; k < reg->max_loras; ++k) {
        idx.push_back(k);
        filled.push_back(reg->slots[k].name.empty() ? 0 : 1);
        ref.push_back(reg->ref_counts[k].load(std::memory_order_acquire));
        lru.push_back(reg->last_used[k].load(std::memory_order_relaxed));
    }
    return atlas_b200_select_victim_slot(idx.data(), filled.data(), ref.data(), lru.data(), idx.size());
}

}  // extern "C"
