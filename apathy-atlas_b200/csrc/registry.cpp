// LoRA registry: slot math and the fixed-address rank-padded pool layout (host only).
//
// Mirrors crates/spark-model/src/lora/slot_math.rs and the packing walk of
// crates/spark-model/src/lora/loading.rs:128-230.  A slot is one adapter's byte image;
// slot k sits at k * pool_slot_bytes.  Inside a slot the walk is
// (adapted layer ascending) x (q,k,v,o,gate,up,down) x (A then B):
// A as [max_rank, in] with real rows first, B as [out, max_rank] with real columns first,
// both zero padded, so kernels may contract over max_rank.
#include "atlas_b200.h"

#include <cmath>
#include <cstring>

namespace atlas {

static bool module_dims(const atlas_b200_model_dims& c, int module, size_t& out_dim, size_t& in_dim) {
    const size_t h = c.hidden_size;
    const size_t q = size_t(c.num_attention_heads) * c.head_dim;
    const size_t kv = size_t(c.num_key_value_heads) * c.head_dim;
    switch (module) {
        case ATLAS_B200_Q: out_dim = (c.attn_gated ? 2 : 1) * q; in_dim = h; return true;
        case ATLAS_B200_K:
        case ATLAS_B200_V: out_dim = kv; in_dim = h; return true;
        case ATLAS_B200_O: out_dim = h; in_dim = q; return true;
        case ATLAS_B200_GATE:
        case ATLAS_B200_UP: out_dim = c.intermediate_size; in_dim = h; return true;
        case ATLAS_B200_DOWN: out_dim = h; in_dim = c.intermediate_size; return true;
        default: return false;
    }
}

static size_t layer_bytes(const atlas_b200_model_dims& c, size_t max_rank) {
    size_t total = 0;
    for (int m = 0; m < ATLAS_B200_NUM_MODULES; ++m) {
        size_t o = 0, i = 0;
        module_dims(c, m, o, i);
        total += (max_rank * i + o * max_rank) * 2;
    }
    return total;
}

}  // namespace atlas

extern "C" {

int atlas_b200_build_seq_slot(const int32_t* adapter_slots, size_t n, size_t padded_n, int32_t active, int32_t* out) {
    if ((!adapter_slots && n) || !out) return ATLAS_B200_ERR_NULL;
    if (padded_n < n) return ATLAS_B200_ERR_DIMS;
    for (size_t i = 0; i < padded_n; ++i) {
        if (i < n) {
            const int32_t s = adapter_slots[i];
            out[i] = s >= 0 ? s : active;   // a request without an adapter defers to the active slot
        } else {
            out[i] = -1;                    // pad row: no delta
        }
    }
    return ATLAS_B200_OK;
}

int32_t atlas_b200_routed_prefill_slot_of(int32_t adapter_slot, size_t active, size_t num_slots) {
    const size_t resolved = adapter_slot >= 0 ? size_t(adapter_slot) : active;
    return (resolved != active && resolved < num_slots) ? int32_t(resolved) : -1;
}

float atlas_b200_peft_scaling(double lora_alpha, size_t r, int use_rslora) {
    if (r == 0) return 0.0f;
    return use_rslora ? float(lora_alpha / std::sqrt(double(r))) : float(lora_alpha / double(r));
}

int atlas_b200_module_dims(const atlas_b200_model_dims* cfg, int module, size_t* out_dim, size_t* in_dim) {
    if (!cfg || !out_dim || !in_dim) return ATLAS_B200_ERR_NULL;
    return atlas::module_dims(*cfg, module, *out_dim, *in_dim) ? ATLAS_B200_OK : ATLAS_B200_ERR_DIMS;
}

size_t atlas_b200_pool_slot_bytes(const atlas_b200_model_dims* cfg, size_t max_rank) {
    if (!cfg) return 0;
    return atlas::layer_bytes(*cfg, max_rank) * cfg->num_full_attention_layers;
}

size_t atlas_b200_slot_base_offset(size_t slot, const atlas_b200_model_dims* cfg, size_t max_rank) {
    return slot * atlas_b200_pool_slot_bytes(cfg, max_rank);
}

int atlas_b200_module_slot_offsets(const atlas_b200_model_dims* cfg, size_t max_rank, size_t layer_ordinal,
                                   int module, size_t* a_off, size_t* b_off) {
    if (!cfg || !a_off || !b_off) return ATLAS_B200_ERR_NULL;
    if (layer_ordinal >= cfg->num_full_attention_layers || module < 0 || module >= ATLAS_B200_NUM_MODULES)
        return ATLAS_B200_ERR_DIMS;
    size_t off = layer_ordinal * atlas::layer_bytes(*cfg, max_rank);
    for (int m = 0; m < module; ++m) {
        size_t o = 0, i = 0;
        atlas::module_dims(*cfg, m, o, i);
        off += (max_rank * i + o * max_rank) * 2;
    }
    size_t o = 0, i = 0;
    atlas::module_dims(*cfg, module, o, i);
    *a_off = off;
    *b_off = off + max_rank * i * 2;
    return ATLAS_B200_OK;
}

int atlas_b200_pack_module(const atlas_b200_model_dims* cfg, size_t max_rank, size_t layer_ordinal, int module,
                           const void* a_bf16, const void* b_bf16, size_t r, void* slot_image) {
    if (!cfg || !a_bf16 || !b_bf16 || !slot_image) return ATLAS_B200_ERR_NULL;
    if (r == 0 || r > max_rank) return ATLAS_B200_ERR_LIMIT;
    size_t a_off = 0, b_off = 0;
    const int st = atlas_b200_module_slot_offsets(cfg, max_rank, layer_ordinal, module, &a_off, &b_off);
    if (st != ATLAS_B200_OK) return st;
    size_t out_dim = 0, in_dim = 0;
    atlas::module_dims(*cfg, module, out_dim, in_dim);
    auto* img = static_cast<unsigned char*>(slot_image);
    std::memset(img + a_off, 0, max_rank * in_dim * 2);
    std::memcpy(img + a_off, a_bf16, r * in_dim * 2);
    std::memset(img + b_off, 0, out_dim * max_rank * 2);
    const auto* bsrc = static_cast<const unsigned char*>(b_bf16);
    for (size_t row = 0; row < out_dim; ++row)
        std::memcpy(img + b_off + row * max_rank * 2, bsrc + row * r * 2, r * 2);
    return ATLAS_B200_OK;
}

int atlas_b200_build_route_tables(const atlas_b200_model_dims* cfg, size_t max_rank, size_t layer_ordinal, int module,
                                  uint64_t pool_base, size_t max_loras, const uint8_t* present,
                                  uint64_t* a_table, uint64_t* b_table) {
    if (!cfg || !a_table || !b_table) return ATLAS_B200_ERR_NULL;
    size_t a_off = 0, b_off = 0;
    const int st = atlas_b200_module_slot_offsets(cfg, max_rank, layer_ordinal, module, &a_off, &b_off);
    if (st != ATLAS_B200_OK) return st;
    const size_t slot_bytes = atlas_b200_pool_slot_bytes(cfg, max_rank);
    for (size_t s = 0; s < max_loras; ++s) {
        const bool on = pool_base != 0 && (!present || present[s]);
        a_table[s] = on ? pool_base + s * slot_bytes + a_off : 0;     // 0 = base only for this slot
        b_table[s] = on ? pool_base + s * slot_bytes + b_off : 0;
    }
    return ATLAS_B200_OK;
}

int atlas_b200_select_victim_slot(const size_t* slot_index, const uint8_t* filled, const size_t* ref_count,
                                  const uint64_t* last_used, size_t count) {
    if (count && (!slot_index || !filled || !ref_count || !last_used)) return ATLAS_B200_ERR_NULL;
    for (size_t i = 0; i < count; ++i)
        if (!filled[i]) return int(slot_index[i]);          // a never-filled slot costs no eviction
    long best = -1;
    for (size_t i = 0; i < count; ++i) {
        if (ref_count[i] != 0) continue;                     // busy slots are never victims
        if (best < 0 || last_used[i] < last_used[size_t(best)]) best = long(i);
    }
    return best < 0 ? -1 : int(slot_index[size_t(best)]);
}

int atlas_b200_column_shard(uint32_t n, uint32_t tp, uint32_t rank, uint32_t* row_begin, uint32_t* row_count) {
    if (!row_begin || !row_count) return ATLAS_B200_ERR_NULL;
    if (tp == 0 || rank >= tp || n % tp != 0) return ATLAS_B200_ERR_DIMS;
    *row_count = n / tp;
    *row_begin = rank * (n / tp);
    return ATLAS_B200_OK;
}

}  // extern "C"
