// C ABI of the B200 NVFP4 + multi-LoRA linear path: argument validation, variant dispatch and
// kernel launches.  Single translation unit (the kernels share one device status word).
//
// Host-side operator layer (namespace atlas::ops) mirrors the reference's launch wrappers:
//   ops::apply_lora_bgmv   <- crates/spark-model/src/layers/ops/lora_delta.rs:269-314
//   ops::apply_lora_delta  <- crates/spark-model/src/layers/ops/lora_delta.rs:145-235
//   ops::w4a16_gemm        <- crates/spark-model/src/layers/ops/gemm_dense.rs:258-281
//   ops::nvfp4_lora_linear    (fused; new)
// Like them it only launches: no allocation, no synchronisation, no host read of device data.
#include "atlas_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernel_tc.cuh"
#include "kernel_tc_persist.cuh"
#include "kernel_dense_tc.cuh"
#include "kernels_simt.cuh"
#include "kernel_shrink_mma.cuh"
#include "kernel_shrink_tc.cuh"
#include "kernels_mlp_glue.cuh"
#include "kernel_push.cuh"
#include "kernel_kv_epilogue.cuh"

namespace atlas {

static thread_local int t_last_variant = ATLAS_B200_VARIANT_NONE;
static thread_local uint32_t t_last_shape[6] = {0, 0, 0, 0, 0, 0};
static unsigned long long* g_profile_buf = nullptr;   // device buffer for per-CTA cycle counters (diagnostics)
static size_t g_profile_words = 0;

static inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? ATLAS_B200_OK : ATLAS_B200_ERR_CUDA_BASE - int(e); }
static inline int launch_status() { return cuda_status(cudaGetLastError()); }
static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------------------------------------
// device capability and the tensor-map encoder (resolved from the driver at first use; the
// library does not link libcuda)
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// What the launcher learns about a device and the per-device settings it has applied.  Function attributes
// (opt-in shared memory, carve-out) and occupancy answers belong to a device, so everything here is kept per
// device ordinal and created under a lock the first time that device is current in a call.
constexpr int kMaxDevices = 64;
constexpr int kPersistKernels = 3;
struct DeviceState {
    bool ready = false;
    bool sm100 = false;
    int sm_count = 148;
    bool tc_attr_set[20] = {};        // token tiles 16..256 x {A16, A4} x {single CTA, CTA pair}
    int known_clusters[20][9] = {};   // resident clusters per kernel instance and K split; 0 = not asked yet
    bool persist_attr_set[kPersistKernels] = {};
    int persist_clusters[kPersistKernels] = {};
    bool carveout_set = false;
    bool shrink_tc_attr_set = false;
    bool push_attr_set = false;
    bool dense_attr_set[5] = {};      // token tiles 16, 32, 64, 128, 256 of the dense-BF16 kernel
};
static DeviceState g_dev[kMaxDevices];
static std::mutex g_dev_mutex;
static EncodeTiledFn g_encode = nullptr;

// state of the current device; nullptr when there is none (no driver, ordinal out of range)
static DeviceState* device_state() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { (void)cudaGetLastError(); return nullptr; }
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        int major = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        st.sm100 = (major == 10);
        cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (st.sm_count <= 0) st.sm_count = 148;
        if (!g_encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
                q == cudaDriverEntryPointSuccess)
                g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
        st.ready = true;
    }
    return &st;
}

static int rt_sm_count() { DeviceState* st = device_state(); return st ? st->sm_count : 148; }

// Encoded tensor maps are a pure function of (address, shape, strides, box, type, swizzle): a serving loop calls with the
// same tensors step after step, so the most recent encodings are kept per host thread (direct-mapped, 64 entries) and a
// repeated call costs a compare instead of a driver call per map.
struct MapKey {
    const void* base;
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    int32_t rank, dtype, swizzle;
};
struct MapEntry {
    MapKey key;
    CUtensorMap map;
    bool valid;
};
static thread_local MapEntry t_map_cache[64];

static bool encode_tiled(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base, const uint64_t* dims,
                         const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swz,
                         CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    MapKey key;
    std::memset(&key, 0, sizeof(key));
    key.base = base; key.rank = int32_t(rank); key.dtype = int32_t(dt); key.swizzle = int32_t(swz) | (int32_t(promo) << 8);
    for (uint32_t i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    for (uint32_t i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
    uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
    h ^= (key.dims[0] * 31 + key.dims[1]) * 0xBF58476D1CE4E5B9ull + key.box[0] * 131 + key.box[1] * 17 + uint64_t(key.swizzle);
    MapEntry& e = t_map_cache[(h >> 32) & 63u];
    if (e.valid && std::memcmp(&e.key, &key, sizeof(key)) == 0) { *map = e.map; return true; }
    cuuint64_t gd[3], gs[2];
    cuuint32_t bx[3], es[3] = {1, 1, 1};
    for (uint32_t i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; }
    for (uint32_t i = 0; i + 1 < rank; ++i) gs[i] = strides[i];
    if (g_encode(map, dt, rank, const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                 promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    e.key = key; e.map = *map; e.valid = true;
    return true;
}

static bool encode_2d(CUtensorMap* map, CUtensorMapDataType dt, size_t elem, const void* base, uint64_t inner,
                      uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                      CUtensorMapSwizzle swz, CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    (void)elem;
    const uint64_t dims[2] = {inner, outer}, strides[1] = {row_stride_bytes};
    const uint32_t box[2] = {box_inner, box_outer};
    return encode_tiled(map, dt, 2, base, dims, strides, box, swz, promo);
}

// ---------------------------------------------------------------------------------------------
// launches
// ---------------------------------------------------------------------------------------------
namespace ops {

// tensor-core shrink where rows can be read with aligned 128-bit loads in whole 32-element chunks
static bool shrink_takes_mma_path(const ShrinkParams& p) {
    return (p.k_in % 32 == 0) && (p.x_row_stride % 8 == 0) && aligned(p.x, 16) && (p.seq_slot || aligned(p.a_uniform, 4));
}

static int launch_shrink(ShrinkParams p, uint32_t n_slots, cudaStream_t st, bool release_dependents = false,
                         bool dependent_leaves_sms_free = false) {
    p.release_dependents = release_dependents ? 1u : 0u;
    p.profile = nullptr;
    if (p.M == 0 || p.max_rank == 0) return ATLAS_B200_OK;
    // Same shared-memory carve-out as the tcgen05 kernel, so that kernel's CTAs can become resident
    // next to this grid's instead of waiting for the SMs to drain and be reconfigured.
    DeviceState* dst = device_state();
    if (dst && !dst->carveout_set) {
        cudaFuncSetAttribute(lora_shrink_grouped_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(lora_shrink_mma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        dst->carveout_set = true;
    }
    const bool mma_ok = shrink_takes_mma_path(p);
    if (p.tile_out && !mma_ok) return ATLAS_B200_ERR_DIMS;      // tile output exists in the tensor-core shrink only
    const void* a_base = p.seq_slot ? p.a_pool_base : static_cast<const void*>(p.a_uniform);
    const size_t a_stride = p.seq_slot ? p.a_slot_stride : size_t(p.max_rank) * p.k_in * 2;
    if (mma_ok && p.M >= 1024 && !release_dependents && p.k_in % SHT_KSTAGE == 0 && p.max_rank % 16 == 0 && p.max_rank <= 256 &&
        n_slots <= 4096 && dst && dst->sm100 && g_encode && a_base && aligned(a_base, 16) && a_stride % 16 == 0 &&
        (!p.tile_out || (p.part_rows && p.chunk % p.part_rows == 0))) {
        // a prefill batch: one cluster per 128 tokens and all ranks of all their adapters on the tcgen05 tensor cores,
        // x read once (kernel_shrink_tc.cuh)
        if (!dst->shrink_tc_attr_set) {
            cudaError_t e = cudaFuncSetAttribute(lora_shrink_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SHT_SMEM_BYTES);
            if (e != cudaSuccess) return cuda_status(e);
            dst->shrink_tc_attr_set = true;
        }
        CUtensorMap map_x, map_a;
        if (!encode_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.x, p.k_in, p.M, uint64_t(p.x_row_stride) * 2, SHT_KSTAGE, SHT_ROWS,
                       CU_TENSOR_MAP_SWIZZLE_128B))
            return ATLAS_B200_ERR_DIMS;
        {
            const uint64_t dims[3] = {p.k_in, p.max_rank, p.seq_slot ? n_slots : 1u};
            const uint64_t strides[2] = {uint64_t(p.k_in) * 2, uint64_t(a_stride)};
            const uint32_t box[3] = {SHT_KSTAGE, p.max_rank, 1};
            if (!encode_tiled(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a_base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
                return ATLAS_B200_ERR_DIMS;
        }
        p.a_pool_base = nullptr;      // host-side fields: not part of what the kernel reads
        if (p.m_begin % 64 != 0 || p.m_begin >= p.M) return ATLAS_B200_ERR_DIMS;
        if (p.tile_out && p.chunk && p.chunk < uint32_t(SHT_ROWS)) return ATLAS_B200_ERR_DIMS;   // a cluster's rows lie in at most two token tiles
        const uint32_t rows = p.m_count ? std::min(p.m_count, p.M - p.m_begin) : p.M - p.m_begin;
        // two CTAs per 128 rows, each contracting half of K: fixed by K alone, so that a row's result does not depend on
        // how the batch is cut into launches
        p.ksplit = (p.k_in / SHT_KSTAGE >= 2) ? 2u : 1u;
        const uint32_t n_ctas = p.ksplit * ((rows + SHT_ROWS - 1) / SHT_ROWS);
        p.profile = (g_profile_buf && size_t(n_ctas) * 16 <= g_profile_words) ? g_profile_buf : nullptr;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n_ctas);
        cfg.blockDim = dim3(SHT_THREADS);
        cfg.dynamicSmemBytes = SHT_SMEM_BYTES;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = p.ksplit;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return cuda_status(cudaLaunchKernelEx(&cfg, lora_shrink_tc_kernel, map_x, map_a, p));
    }
    if (p.m_begin || p.m_count || p.n_tile_dest > 1) return ATLAS_B200_ERR_DIMS;      // a row range / several destinations: that kernel only
    if (mma_ok) {
        const uint32_t chunk = p.chunk ? p.chunk : uint32_t(SHM_CHUNK);
        // CTAs per (slot, granule, chunk) sharing K: 8 for the sake of loads in flight; fewer when the dependent kernel
        // runs beside this grid on a part of the machine only (a decode batch) and this grid would otherwise be so
        // large that the dependent's CTAs find no room until it has drained
        const size_t items = size_t(n_slots) * ((p.max_rank + SHM_RANKS - 1) / SHM_RANKS) * ((p.M + chunk - 1) / chunk);
        uint32_t ksplit = SHM_KSPLIT;
        while (release_dependents && dependent_leaves_sms_free && ksplit > 2 && items * ksplit > size_t(rt_sm_count()) * 4) ksplit >>= 1;
        p.ksplit = ksplit;
        dim3 grid(n_slots * ksplit, (p.max_rank + SHM_RANKS - 1) / SHM_RANKS, (p.M + chunk - 1) / chunk);
        if (grid.y > 65535 || grid.z > 65535) return ATLAS_B200_ERR_LIMIT;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(SHM_THREADS);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;      // SHM_KSPLIT CTAs along x share one (slot, ranks, chunk)
        attr[0].val.clusterDim.x = ksplit;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return cuda_status(cudaLaunchKernelEx(&cfg, lora_shrink_mma_kernel, p));
    }
    dim3 grid(n_slots, (p.max_rank + SHRINK_RT - 1) / SHRINK_RT, (p.M + SHRINK_TC - 1) / SHRINK_TC);
    if (grid.y > 65535 || grid.z > 65535) return ATLAS_B200_ERR_LIMIT;
    lora_shrink_grouped_kernel<<<grid, SHRINK_THREADS, 0, st>>>(p);
    return launch_status();
}

static int launch_expand(const ExpandParams& p, cudaStream_t st) {
    if (p.M == 0 || p.n_out == 0) return ATLAS_B200_OK;
    if (p.max_rank > EXPAND_MAX_RANK) return ATLAS_B200_ERR_LIMIT;
    // rows per CTA: 32 for large batches (a CTA re-uses its B rows out of L1 while neighbouring rows share an adapter),
    // fewer while the grid would otherwise leave SMs without a CTA (a decode batch)
    ExpandParams q = p;
    const uint32_t col_blocks = (p.n_out + EXPAND_OUTS - 1) / EXPAND_OUTS;
    uint32_t rpc = EXPAND_ROWS;
    while (rpc > 1 && col_blocks * ((p.M + rpc - 1) / rpc) < 2u * uint32_t(rt_sm_count())) rpc >>= 1;
    q.rows_per_cta = rpc;
    dim3 grid(col_blocks, (p.M + rpc - 1) / rpc);
    if (grid.y > 65535) return ATLAS_B200_ERR_LIMIT;
    lora_expand_fold_kernel<<<grid, EXPAND_OUTS, 0, st>>>(q);
    return launch_status();
}

int apply_lora_bgmv(const void* x, const int32_t* seq_slot, const uint64_t* a_table, const uint64_t* b_table,
                    const float* scale_table, void* base_out, void* lora_xa, uint32_t n, uint32_t k_in,
                    uint32_t n_out, uint32_t max_rank, uint32_t x_row_stride, uint32_t out_row_stride,
                    uint32_t max_loras, cudaStream_t st) {
    if (n == 0) return ATLAS_B200_OK;
    if (!x || !seq_slot || !a_table || !b_table || !scale_table || !base_out || !lora_xa) return ATLAS_B200_ERR_NULL;
    if (k_in == 0 || n_out == 0 || max_rank == 0 || max_loras == 0) return ATLAS_B200_ERR_DIMS;
    if (x_row_stride < k_in || out_row_stride < n_out) return ATLAS_B200_ERR_DIMS;
    if (max_loras > 65535 || max_rank > EXPAND_MAX_RANK) return ATLAS_B200_ERR_LIMIT;
    if (!aligned(x, 2) || !aligned(base_out, 2) || !aligned(lora_xa, 2)) return ATLAS_B200_ERR_ALIGN;

    ShrinkParams sp{};
    sp.x = static_cast<const uint16_t*>(x);
    sp.seq_slot = seq_slot;
    sp.a_table = a_table;
    sp.b_table = nullptr;            // the reference's shrink looks at the A entry only (lora_bgmv.cu:63-65)
    sp.out = static_cast<uint16_t*>(lora_xa);
    sp.M = n; sp.k_in = k_in; sp.max_rank = max_rank; sp.x_row_stride = x_row_stride; sp.max_loras = max_loras;
    sp.post = 0.0f;
    int rc = launch_shrink(sp, max_loras, st);
    if (rc) return rc;

    ExpandParams ep{};
    ep.xa = static_cast<const uint16_t*>(lora_xa);
    ep.seq_slot = seq_slot;
    ep.a_table = a_table;            // a row whose shrink was skipped has no valid xa: skip its expand too
    ep.b_table = b_table;
    ep.scale_table = scale_table;
    ep.out = static_cast<uint16_t*>(base_out);
    ep.M = n; ep.n_out = n_out; ep.max_rank = max_rank; ep.out_row_stride = out_row_stride; ep.max_loras = max_loras;
    return launch_expand(ep, st);
}

int apply_lora_delta(const void* x, const void* a, const void* b, float scale, void* base_out, void* lora_xa,
                     void* lora_delta, uint32_t m, uint32_t k_in, uint32_t n_out, uint32_t max_rank, cudaStream_t st) {
    if (m == 0) return ATLAS_B200_OK;
    if (!x || !a || !b || !base_out || !lora_xa) return ATLAS_B200_ERR_NULL;
    if (k_in == 0 || n_out == 0 || max_rank == 0) return ATLAS_B200_ERR_DIMS;
    if (max_rank > EXPAND_MAX_RANK) return ATLAS_B200_ERR_LIMIT;

    ShrinkParams sp{};
    sp.x = static_cast<const uint16_t*>(x);
    sp.a_uniform = static_cast<const uint16_t*>(a);
    sp.out = static_cast<uint16_t*>(lora_xa);
    sp.M = m; sp.k_in = k_in; sp.max_rank = max_rank; sp.x_row_stride = k_in; sp.max_loras = 1;
    int rc = launch_shrink(sp, 1, st);
    if (rc) return rc;

    ExpandParams ep{};
    ep.xa = static_cast<const uint16_t*>(lora_xa);
    ep.b_uniform = static_cast<const uint16_t*>(b);
    ep.scale_uniform = scale;
    ep.out = static_cast<uint16_t*>(base_out);
    ep.delta_out = static_cast<uint16_t*>(lora_delta);
    ep.M = m; ep.n_out = n_out; ep.max_rank = max_rank; ep.out_row_stride = n_out; ep.max_loras = 1;
    return launch_expand(ep, st);
}

static int launch_simt_linear(const atlas_b200_linear_desc& d, cudaStream_t st) {
    SimtLinearParams p{};
    p.x = static_cast<const uint16_t*>(d.x);
    p.w_packed = static_cast<const uint8_t*>(d.w_packed);
    p.w_scale = static_cast<const uint8_t*>(d.w_scale);
    p.w_bf16 = static_cast<const uint16_t*>(d.w_bf16);
    p.y = static_cast<uint16_t*>(d.y);
    p.M = d.m; p.N = d.n; p.K = d.k; p.x_row_stride = d.x_row_stride; p.out_row_stride = d.out_row_stride;
    p.scale2 = d.w_bf16 ? 1.0f : d.scale2;
    dim3 grid((d.n + SIMT_TF - 1) / SIMT_TF, (d.m + SIMT_TM - 1) / SIMT_TM);
    if (grid.y > 65535) return ATLAS_B200_ERR_LIMIT;
    linear_simt_kernel<<<grid, 256, 0, st>>>(p);
    return launch_status();
}

// Shapes the tcgen05 path takes.  Everything here is a property of host-visible arguments.
static bool tc_eligible(const atlas_b200_linear_desc& d) {
    DeviceState* dst = device_state();
    if (!dst || !dst->sm100 || !g_encode) return false;
    if (d.w_bf16) return false;                                   // dense base: CUDA-core path
    if (d.k % tc::KRAW != 0) return false;                        // TMA row strides of codes and scales: 16-byte multiples
    if (d.x_row_stride % 8 != 0) return false;
    if (!aligned(d.x, 16) || !aligned(d.w_packed, 16) || !aligned(d.w_scale, 16)) return false;
    if (d.seq_slot) {
        if (d.max_rank > tc::MAX_RANK_TC || d.max_rank % 8 != 0) return false;
        if (d.max_loras > tc::MAX_LORAS_TC) return false;
        if (!aligned(d.lora_t, 16)) return false;
    }
    if (!(d.scale2 != 0.0f) || !std::isfinite(d.scale2)) return false;
    return true;
}

// Bytes of `ws` the FP4-activation mode needs: packed codes [m, k/2] then scale bytes [m, k/16],
// the second at a 256-byte boundary.
static size_t act_fp4_codes_bytes(const atlas_b200_linear_desc& d) { return (size_t(d.m) * (d.k / 2) + 255) / 256 * 256; }
static size_t act_fp4_ws_bytes(const atlas_b200_linear_desc& d) { return act_fp4_codes_bytes(d) + size_t(d.m) * (d.k / 16); }

// The B side of the adapter pool can be described as one 3-D tensor [max_loras][n][max_rank]
static bool b_pool_is_strided(const atlas_b200_linear_desc& d) {
    return d.seq_slot && d.b_pool_base && d.b_slot_stride && d.b_slot_stride % 16 == 0 && aligned(d.b_pool_base, 16) &&
           d.max_rank % 8 == 0;
}

// Where the shrink's masked-t tiles live in `ws` (tiles == nullptr: the fused kernel builds them itself from lora_t)
struct TTiles {
    uint16_t* tiles = nullptr;
    uint32_t cap = 0;          // blocks reserved per token tile (per half of one, for CTA pairs)
    uint32_t part_rows = 0;    // rows of a block: the token tile, or half of it for CTA pairs
};

// The six tensor maps of a tcgen05 launch.  `xrows` = token rows of an activation tile one CTA stages, `mt` = token
// tile, `l_gran_t` = bytes of one masked-t block as the shrink writes it ([part_rows x 16] BF16).
struct TcMaps { CUtensorMap x, w, s, b, xs, t; };

static int encode_tc_maps(const atlas_b200_linear_desc& d, bool a4, uint32_t xrows, uint32_t mt, uint32_t l_gran_t,
                          const TTiles& tt, TcMaps& m) {
    if (a4) {
        // the quantised activations in `ws`, in the weights' own layout
        const uint8_t* codes = static_cast<const uint8_t*>(d.ws);
        if (!encode_2d(&m.x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, d.k / 2, d.m, d.k / 2, tc::KRAW / 2, xrows,
                       CU_TENSOR_MAP_SWIZZLE_128B))
            return ATLAS_B200_ERR_DIMS;
        if (!encode_2d(&m.xs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes + act_fp4_codes_bytes(d), d.k / 16, d.m, d.k / 16,
                       tc::KRAW / 16, mt, CU_TENSOR_MAP_SWIZZLE_NONE))
            return ATLAS_B200_ERR_DIMS;
    } else if (!encode_2d(&m.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d.x, d.k, d.m, uint64_t(d.x_row_stride) * 2, tc::KB, xrows,
                          CU_TENSOR_MAP_SWIZZLE_128B))
        return ATLAS_B200_ERR_DIMS;
    if (!encode_2d(&m.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d.w_packed, d.k / 2, d.n, d.k / 2, tc::KRAW / 2, tc::FT,
                   CU_TENSOR_MAP_SWIZZLE_128B))
        return ATLAS_B200_ERR_DIMS;
    if (!encode_2d(&m.s, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d.w_scale, d.k / 16, d.n, d.k / 16, tc::KRAW / 16, tc::FT,
                   CU_TENSOR_MAP_SWIZZLE_NONE))
        return ATLAS_B200_ERR_DIMS;

    // B side of the adapter pool as one 3-D tensor [max_loras][n][max_rank]: box = one granule of one slot
    if (b_pool_is_strided(d)) {
        const uint64_t dims[3] = {d.max_rank, d.n, d.max_loras};
        const uint64_t strides[2] = {uint64_t(d.max_rank) * 2, uint64_t(d.b_slot_stride)};
        const uint32_t box[3] = {16, tc::FT, 1};
        if (!encode_tiled(&m.b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d.b_pool_base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B))
            return ATLAS_B200_ERR_DIMS;
    } else {
        m.b = m.s;   // never dereferenced
    }
    if (!a4) m.xs = m.s;   // never dereferenced
    if (tt.tiles) {
        // the masked-t blocks are shared-memory images already: plain bytes, 256 to a row, one block per copy
        const uint64_t rows = uint64_t((d.m + mt - 1) / mt) * tt.cap * mt * 32 / 256;
        if (l_gran_t % 256 != 0 ||
            !encode_2d(&m.t, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, tt.tiles, 256, rows, 256, 256, l_gran_t / 256, CU_TENSOR_MAP_SWIZZLE_NONE))
            return ATLAS_B200_ERR_DIMS;
    } else {
        m.t = m.s;         // never dereferenced
    }
    return ATLAS_B200_OK;
}

// the launch constants both tcgen05 kernels share
static int fill_tc_params(const atlas_b200_linear_desc& d, bool a4, bool b_strided, const TTiles& tt, tc::Params& p) {
    p.b_pool_strided = b_strided ? 1u : 0u;
    p.t_tile_cap = tt.tiles ? tt.cap : 0u;
    p.seq_slot = d.seq_slot;
    p.a_table = d.a_table;
    p.b_table = d.b_table;
    p.rank_table = d.rank_table;
    p.t = static_cast<const uint16_t*>(d.lora_t);
    p.y = static_cast<uint16_t*>(d.y);
    p.n_dest = d.n_dest ? d.n_dest : 1u;
    p.y_col0 = d.n_dest ? d.y_col_offset : 0u;
    bool rows_16b = d.out_row_stride % 8 == 0 && p.y_col0 % 8 == 0;
    for (uint32_t r = 0; r < p.n_dest; ++r) {
        p.y_dest[r] = static_cast<uint16_t*>(d.n_dest ? d.y_dest[r] : d.y);
        rows_16b = rows_16b && aligned(p.y_dest[r], 16);
    }
    if (d.n_dest && !rows_16b) return ATLAS_B200_ERR_ALIGN;
    p.staged_epilogue = rows_16b ? 1u : 0u;
    p.M = d.m; p.N = d.n; p.K = d.k; p.out_row_stride = d.out_row_stride;
    p.max_loras = d.max_loras; p.max_rank = d.max_rank;
    p.out_scale = a4 ? d.scale2 : d.scale2 * kWeightPreScale;
    p.k_split = 1;
    return ATLAS_B200_OK;
}

// How many clusters of (PAIR ? 2 : 1) x 1 x k_split CTAs of one kernel instance can be resident at once.  Clusters live
// inside one GPC, so fewer fit than the SM count suggests.  An occupancy query, answered by the runtime without touching
// the device; asked once per shape.  -1: the query failed.
template <int MT, bool A4, bool PAIR>
static int tc_active_clusters(int slot_idx, uint32_t k_split) {
    using C = tc::Cfg<MT, A4, PAIR>;
    DeviceState* dst = device_state();
    if (!dst) return -1;
    slot_idx += (A4 ? 5 : 0) + (PAIR ? 10 : 0);
    int (&known)[20][9] = dst->known_clusters;
    if (k_split > 8) return -1;
    if (known[slot_idx][k_split] == 0) {
        if (!dst->tc_attr_set[slot_idx]) {
            if (cudaFuncSetAttribute(tc::nvfp4_lora_linear_tc_kernel<MT, A4, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     C::SMEM_BYTES) != cudaSuccess) {
                (void)cudaGetLastError();
                return -1;
            }
            dst->tc_attr_set[slot_idx] = true;
        }
        cudaLaunchConfig_t q{};
        q.gridDim = dim3(PAIR ? 2 : 1, 1, k_split);
        q.blockDim = dim3(tc::NUM_THREADS);
        q.dynamicSmemBytes = C::SMEM_BYTES;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = PAIR ? 2 : 1;
        qa[0].val.clusterDim.y = 1;
        qa[0].val.clusterDim.z = k_split;
        q.attrs = qa;
        q.numAttrs = 1;
        int n = 0;
        known[slot_idx][k_split] =
            cudaOccupancyMaxActiveClusters(&n, tc::nvfp4_lora_linear_tc_kernel<MT, A4, PAIR>, &q) == cudaSuccess && n > 0 ? n : -1;
        (void)cudaGetLastError();
    }
    return known[slot_idx][k_split];
}

static int tc_active_clusters_of(uint32_t mt, bool a4, bool pair, uint32_t k_split) {
#define ATLAS_OCC(MT_, I_) \
    if (mt == MT_) return a4 ? (pair ? tc_active_clusters<MT_, true, (MT_ >= 128)>(I_, k_split) : tc_active_clusters<MT_, true, false>(I_, k_split)) \
                             : (pair ? tc_active_clusters<MT_, false, (MT_ >= 128)>(I_, k_split) : tc_active_clusters<MT_, false, false>(I_, k_split));
    ATLAS_OCC(16, 0) ATLAS_OCC(32, 1) ATLAS_OCC(64, 2) ATLAS_OCC(128, 3) ATLAS_OCC(256, 4)
#undef ATLAS_OCC
    return -1;
}

template <int MT, bool A4, bool PAIR>
static int launch_tc(const atlas_b200_linear_desc& d, int slot_idx, const ShrinkParams* shrink, const TTiles& tt,
                     uint32_t k_split, cudaStream_t st) {
    const bool after_shrink = shrink != nullptr;     // the shrink is launched from here, once the launch shape is final
    using C = tc::Cfg<MT, A4, PAIR>;
    DeviceState* dst = device_state();
    if (!dst) return ATLAS_B200_ERR_ARCH;
    slot_idx += (A4 ? 5 : 0) + (PAIR ? 10 : 0);
    if (!dst->tc_attr_set[slot_idx]) {
        cudaError_t e = cudaFuncSetAttribute(tc::nvfp4_lora_linear_tc_kernel<MT, A4, PAIR>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return cuda_status(e);
        dst->tc_attr_set[slot_idx] = true;
    }
    TcMaps maps;
    const bool b_strided = b_pool_is_strided(d);
    {
        const int rc = encode_tc_maps(d, A4, C::XROWS, MT, C::L_GRAN_T, tt, maps);
        if (rc) return rc;
    }
    const CUtensorMap &map_x = maps.x, &map_w = maps.w, &map_s = maps.s, &map_b = maps.b, &map_xs = maps.xs, &map_t = maps.t;

    tc::Params p{};
    {
        const int rc = fill_tc_params(d, A4, b_strided, tt, p);
        if (rc) return rc;
    }
    dim3 grid((d.n + tc::FT - 1) / tc::FT, (d.m + MT - 1) / MT);
    if (PAIR) grid.x = (grid.x + 1u) & ~1u;      // whole pairs: a CTA past the last feature loads zeros and stores nothing
    // split K: k_split CTAs along z form a cluster (times two for pairs), share one tile and exchange partial sums;
    // the receive area is ceil(chunks / k_split) 8 KB blocks from each of them
    if (k_split > 1 && (k_split * (PAIR ? 2u : 1u) > 8u ||
                        size_t(k_split) * ((MT / 16 + k_split - 1) / k_split) * 8192 > size_t(C::STAGING_BYTES)))
        return ATLAS_B200_ERR_LIMIT;
    grid.z = k_split;
    p.k_split = k_split;
    t_last_shape[0] = MT; t_last_shape[1] = PAIR ? 1u : 0u; t_last_shape[2] = k_split; t_last_shape[3] = tt.tiles ? 1u : 0u;
    t_last_shape[4] = 0u; t_last_shape[5] = 0u;
    if (shrink) {
        // A small batch: let this kernel start under the shrink.  A large one: the shrink is a sizeable grid that
        // should have the whole machine first; this kernel then follows it.
        const uint32_t main_ctas = grid.x * grid.y * grid.z;
        const int rc = launch_shrink(*shrink, d.max_loras, st, d.m <= 1024, main_ctas * 3 <= uint32_t(rt_sm_count()) * 2);
        if (rc) return rc;
    }
    p.profile = (g_profile_buf && size_t(grid.x) * grid.y * tc::PROFILE_WORDS <= g_profile_words) ? g_profile_buf : nullptr;
    if (grid.y > 65535) return ATLAS_B200_ERR_LIMIT;
    // Launched as a programmatic dependent of the shrink that precedes it in the stream: its CTAs
    // may start while the shrink still runs (the shrink releases them as soon as it is resident) and
    // wait for the shrink's completion only where they first read t, after the base K loop.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(tc::NUM_THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    if (PAIR || k_split > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = PAIR ? 2 : 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = k_split;
        ++n_attr;
    }
    if (after_shrink) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    p.wait_for_shrink = after_shrink ? 1u : 0u;
    return cuda_status(cudaLaunchKernelEx(&cfg, tc::nvfp4_lora_linear_tc_kernel<MT, A4, PAIR>, map_x, map_w, map_s, map_b, map_xs, map_t, p));
}

// ---- the persistent form (kernel_tc_persist.cuh): one cluster of two CTAs per pair of SMs, a static tile loop ----
// instance index: 0 = <256, 1, A16>, 1 = <256, 1, A4>, 2 = <192, 2, A16>
template <int MT, int G, bool A4>
static int persist_resident_clusters(int idx) {
    using C = tc::PCfg<MT, G, A4>;
    DeviceState* dst = device_state();
    if (!dst) return -1;
    if (dst->persist_clusters[idx] == 0) {
        if (!dst->persist_attr_set[idx]) {
            if (cudaFuncSetAttribute(tc::nvfp4_lora_linear_tc_persistent_kernel<MT, G, A4>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) {
                (void)cudaGetLastError();
                return -1;
            }
            dst->persist_attr_set[idx] = true;
        }
        cudaLaunchConfig_t q{};
        q.gridDim = dim3(2, 1, 1);
        q.blockDim = dim3(tc::P_NUM_THREADS);
        q.dynamicSmemBytes = C::SMEM_BYTES;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = 2;
        qa[0].val.clusterDim.y = 1;
        qa[0].val.clusterDim.z = 1;
        q.attrs = qa;
        q.numAttrs = 1;
        int n = 0;
        dst->persist_clusters[idx] =
            cudaOccupancyMaxActiveClusters(&n, tc::nvfp4_lora_linear_tc_persistent_kernel<MT, G, A4>, &q) == cudaSuccess && n > 0 ? n : -1;
        (void)cudaGetLastError();
    }
    return dst->persist_clusters[idx];
}

// tiles of one launch: pairs of feature tiles x token passes
template <int MT, int G>
static uint32_t persist_tiles(const atlas_b200_linear_desc& d) {
    const uint32_t n_fpairs = ((d.n + tc::FT - 1) / tc::FT + 1) / 2;
    const uint32_t n_passes = (d.m + MT * G - 1) / (MT * G);
    return n_fpairs * n_passes;
}

template <int MT, int G, bool A4>
static int launch_tc_persist(const atlas_b200_linear_desc& d, int idx, const ShrinkParams* shrink, const TTiles& tt, cudaStream_t st) {
    using C = tc::PCfg<MT, G, A4>;
    const int clusters = persist_resident_clusters<MT, G, A4>(idx);
    if (clusters <= 0) return ATLAS_B200_ERR_DIMS;
    TcMaps maps;
    {
        const int rc = encode_tc_maps(d, A4, C::XROWS, MT, C::L_GRAN_T, tt, maps);
        if (rc) return rc;
    }
    tc::Params p{};
    {
        const int rc = fill_tc_params(d, A4, b_pool_is_strided(d), tt, p);
        if (rc) return rc;
    }
    if (!p.staged_epilogue) return ATLAS_B200_ERR_ALIGN;
    tc::PParams pp{};
    pp.n_fpairs = ((d.n + tc::FT - 1) / tc::FT + 1) / 2;
    pp.n_passes = (d.m + MT * G - 1) / (MT * G);
    pp.n_tiles = pp.n_fpairs * pp.n_passes;
    const uint32_t pairs = std::min<uint32_t>(uint32_t(clusters), pp.n_tiles);
    t_last_shape[0] = MT; t_last_shape[1] = 1u; t_last_shape[2] = 1u; t_last_shape[3] = tt.tiles ? 1u : 0u;
    t_last_shape[4] = uint32_t(G); t_last_shape[5] = pairs;
    if (shrink) {
        const int rc = launch_shrink(*shrink, d.max_loras, st, d.m <= 1024, false);
        if (rc) return rc;
    }
    p.profile = (g_profile_buf && size_t(pairs) * 2 * tc::PROFILE_WORDS <= g_profile_words) ? g_profile_buf : nullptr;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pairs * 2, 1, 1);
    cfg.blockDim = dim3(tc::P_NUM_THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
    if (shrink) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    p.wait_for_shrink = shrink ? 1u : 0u;
    return cuda_status(cudaLaunchKernelEx(&cfg, tc::nvfp4_lora_linear_tc_persistent_kernel<MT, G, A4>, maps.x, maps.w, maps.s, maps.b,
                                          maps.xs, maps.t, p, pp));
}

// ---- dense-BF16 base on the tensor cores (kernel_dense_tc.cuh) ----
static bool dense_tc_eligible(const atlas_b200_linear_desc& d) {
    DeviceState* dst = device_state();
    return dst && dst->sm100 && g_encode && d.w_bf16 && d.k % tc::KB == 0 && d.x_row_stride % 8 == 0 && aligned(d.x, 16) &&
           aligned(d.w_bf16, 16) && !d.n_dest;
}

template <int MT>
static int launch_dense_tc_mt(const atlas_b200_linear_desc& d, int idx, uint32_t k_split, cudaStream_t st) {
    using C = tc::DCfg<MT>;
    DeviceState* dst = device_state();
    if (!dst->dense_attr_set[idx]) {
        cudaError_t e = cudaFuncSetAttribute(tc::dense_bf16_linear_tc_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return cuda_status(e);
        dst->dense_attr_set[idx] = true;
    }
    CUtensorMap map_x, map_w;
    if (!encode_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d.x, d.k, d.m, uint64_t(d.x_row_stride) * 2, tc::KB, MT, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d.w_bf16, d.k, d.n, uint64_t(d.k) * 2, tc::KB, tc::FT, CU_TENSOR_MAP_SWIZZLE_128B))
        return ATLAS_B200_ERR_DIMS;
    tc::DParams p{};
    p.y = static_cast<uint16_t*>(d.y);
    p.M = d.m; p.N = d.n; p.K = d.k; p.out_row_stride = d.out_row_stride; p.k_split = k_split;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((d.n + tc::FT - 1) / tc::FT, (d.m + MT - 1) / MT, k_split);
    if (cfg.gridDim.y > 65535) return ATLAS_B200_ERR_LIMIT;
    cfg.blockDim = dim3(tc::D_THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = k_split;
    cfg.attrs = attr;
    cfg.numAttrs = k_split > 1 ? 1 : 0;
    return cuda_status(cudaLaunchKernelEx(&cfg, tc::dense_bf16_linear_tc_kernel<MT>, map_x, map_w, p));
}

static int launch_dense_tc(const atlas_b200_linear_desc& d, cudaStream_t st) {
    uint32_t mt = 16;
    while (mt < 128 && mt < d.m) mt <<= 1;
    // few output tiles (a decode batch): CTAs along z share a tile's K so that every SM streams weights
    const uint32_t tiles = ((d.n + tc::FT - 1) / tc::FT) * ((d.m + mt - 1) / mt);
    uint32_t k_split = std::max(1u, std::min(std::min(uint32_t(rt_sm_count()) / std::max(tiles, 1u), 8u), d.k / uint32_t(tc::KB)));
    while (k_split & (k_split - 1)) --k_split;           // a power of two: clusters of 1, 2, 4 or 8
    t_last_shape[0] = mt; t_last_shape[1] = 0u; t_last_shape[2] = k_split; t_last_shape[3] = 0u; t_last_shape[4] = 0u; t_last_shape[5] = 0u;
    if (mt == 16) return launch_dense_tc_mt<16>(d, 0, k_split, st);
    if (mt == 32) return launch_dense_tc_mt<32>(d, 1, k_split, st);
    if (mt == 64) return launch_dense_tc_mt<64>(d, 2, k_split, st);
    return launch_dense_tc_mt<128>(d, 3, k_split, st);
}

static int validate_linear(const atlas_b200_linear_desc& d) {
    if (!d.x || (!d.y && !d.n_dest)) return ATLAS_B200_ERR_NULL;
    if (d.n_dest > uint32_t(tc::MAX_DEST)) return ATLAS_B200_ERR_LIMIT;
    for (uint32_t r = 0; r < d.n_dest; ++r)
        if (!d.y_dest[r]) return ATLAS_B200_ERR_NULL;
    if (d.n_dest && uint64_t(d.y_col_offset) + d.n > d.out_row_stride) return ATLAS_B200_ERR_DIMS;
    if (!d.w_bf16 && (!d.w_packed || !d.w_scale)) return ATLAS_B200_ERR_NULL;
    if (d.k == 0 || d.n == 0) return ATLAS_B200_ERR_DIMS;
    if (!d.w_bf16 && d.k % 16 != 0) return ATLAS_B200_ERR_DIMS;   // NVFP4 scale groups are 16 wide
    if (d.x_row_stride < d.k || d.out_row_stride < d.n) return ATLAS_B200_ERR_DIMS;
    if (d.seq_slot) {
        if (!d.a_table || !d.b_table || !d.scale_table || !d.lora_t) return ATLAS_B200_ERR_NULL;
        if (d.max_loras == 0 || d.max_rank == 0) return ATLAS_B200_ERR_DIMS;
        if (d.max_loras > 65535 || d.max_rank > EXPAND_MAX_RANK) return ATLAS_B200_ERR_LIMIT;
    }
    if ((d.flags & ATLAS_B200_FLAG_FORCE_SIMT) && (d.flags & ATLAS_B200_FLAG_FORCE_TCGEN05)) return ATLAS_B200_ERR_DIMS;
    return ATLAS_B200_OK;
}

// A call that stops after the shrink: rows [row_begin, row_begin + row_count) of the batch, masked-t tiles written into
// n_dest scratch buffers laid out like d.ws (see atlas_b200_lora_shrink_tiles).
struct ShrinkOnly {
    uint32_t row_begin, row_count, n_dest;
    void* const* ws_dest;
};

int nvfp4_lora_linear(const atlas_b200_linear_desc& d, cudaStream_t st, const ShrinkOnly* shrink_only = nullptr) {
    int rc = validate_linear(d);
    if (rc) return rc;
    t_last_variant = ATLAS_B200_VARIANT_NONE;
    if (d.m == 0) return ATLAS_B200_OK;

    const bool staged = (d.flags & ATLAS_B200_FLAG_STAGED_LORA) != 0;
    bool use_tc = !(d.flags & ATLAS_B200_FLAG_FORCE_SIMT) && !staged && tc_eligible(d);
    if (!use_tc && shrink_only) return ATLAS_B200_ERR_DIMS;
    if (!use_tc && (d.flags & ATLAS_B200_FLAG_FORCE_TCGEN05) && !(d.w_bf16 && !staged && dense_tc_eligible(d))) return ATLAS_B200_ERR_DIMS;
    if (!use_tc && d.n_dest) return ATLAS_B200_ERR_DIMS;          // placement into several buffers is the tcgen05 epilogue's

    const bool act_fp4 = (d.flags & ATLAS_B200_FLAG_ACT_FP4) != 0;
    if (act_fp4) {
        // FP4 activations exist on the tensor-core path only: no other path is substituted for it
        if (!use_tc) return ATLAS_B200_ERR_DIMS;
        if (!d.ws || !aligned(d.ws, 256)) return d.ws ? ATLAS_B200_ERR_ALIGN : ATLAS_B200_ERR_NULL;
        if (d.ws_bytes < act_fp4_ws_bytes(d)) return ATLAS_B200_ERR_WORKSPACE;
        // x -> NVFP4 with a tensor scale of one (scale byte = E4M3 of group max / 6), the activation side
        // of crates/spark-model/src/layers/ops/gemm_fp4.rs:20-40 — unless the caller says they are in place already
        uint8_t* codes = static_cast<uint8_t*>(d.ws);
        if (!(d.flags & ATLAS_B200_FLAG_ACT_FP4_READY) && !shrink_only) {
        const size_t groups = size_t(d.m) * (d.k / 16);
        const unsigned blocks = unsigned(std::min<size_t>((groups + 255) / 256, size_t(rt_sm_count()) * 16));
        quantize_nvfp4_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(d.x), codes, codes + act_fp4_codes_bytes(d),
                                                      1.0f, d.m, d.k, d.x_row_stride, 1u);
        rc = launch_status();
        if (rc) return rc;
        }
    }
    if (use_tc) {
        // Token tile: the smallest power of two that covers m, at most 256 — then halved (down to 64)
        // while the grid would leave more than a quarter of the SMs without a CTA, e.g. for a
        // column shard of a wide layer: more, lighter CTAs finish sooner than few heavy ones.
        uint32_t mt = 16;
        while (mt < 256 && mt < d.m) mt <<= 1;
        const uint32_t f_tiles = (d.n + tc::FT - 1) / tc::FT;
        // Fewer tiles than half the SMs (a decode batch, a column shard): several CTAs share a tile, each
        // contracting a share of K, rather than leaving SMs idle — a CTA's time is set by the weights it has
        // to expand, which only a K split divides.  Clusters of at most 8 CTAs; whole 256-element stages.
        uint32_t k_split = 1;
        bool pair = mt >= 128 && !(d.flags & ATLAS_B200_FLAG_NO_CTA_PAIR);    // pairs of CTAs issue their MMAs together (see tc::Cfg)
        if (!(d.flags & ATLAS_B200_FLAG_NO_K_SPLIT)) {
            const uint32_t m_tiles = (d.m + mt - 1) / mt;
            const uint32_t fit = uint32_t(rt_sm_count()) / (f_tiles * m_tiles);
            k_split = std::max(1u, std::min(std::min(fit, 8u), d.k / uint32_t(tc::KRAW)));
            // ... but only as many as still lets every cluster be resident at once (a second wave would cost more than the
            // split saves), preferring the shape with pairs, then the one without, then a smaller split
            const bool may_pair = pair;
            for (; k_split > 1; --k_split) {
                if (may_pair && k_split <= 4 &&
                    tc_active_clusters_of(mt, act_fp4, true, k_split) >= int(((f_tiles + 1) / 2) * m_tiles)) { pair = true; break; }
                if (tc_active_clusters_of(mt, act_fp4, false, k_split) >= int(f_tiles * m_tiles)) { pair = false; break; }
            }
            if (k_split == 1) pair = may_pair;
        }
        if (k_split == 1) {
            while (mt > 64 && f_tiles * ((d.m + mt - 1) / mt) * 4 < uint32_t(rt_sm_count()) * 3) mt >>= 1;
            pair = mt >= 128 && !(d.flags & ATLAS_B200_FLAG_NO_CTA_PAIR);
        }

        ShrinkParams sp{};
        sp.x = static_cast<const uint16_t*>(d.x);
        sp.seq_slot = d.seq_slot;
        sp.a_table = d.a_table;
        sp.b_table = d.b_table;
        sp.scale_table = d.scale_table;
        sp.rank_table = d.rank_table;
        sp.out = static_cast<uint16_t*>(d.lora_t);
        sp.M = d.m; sp.k_in = d.k; sp.max_rank = d.max_rank; sp.x_row_stride = d.x_row_stride; sp.max_loras = d.max_loras;
        sp.a_pool_base = d.a_pool_base; sp.a_slot_stride = d.a_slot_stride;
        // t = scale_s / (scale2 * 2^8) * (A_s x), the unit of the MMA accumulator (no 2^8 with FP4 activations)
        sp.post = act_fp4 ? 1.0f / d.scale2 : 1.0f / (d.scale2 * kWeightPreScale);

        // Masked-t tiles: with scratch to put them in, the shrink writes the activation operand of every LoRA
        // K-step once, in the layout the MMA reads, and the fused kernel's CTAs fetch it by TMA — instead of
        // each CTA rebuilding the same tiles from lora_t.  Needs the strided pool (the TMA producer then feeds
        // both LoRA operands) and the tensor-core shrink; otherwise the in-kernel build stays in use.
        TTiles tt;
        if (d.seq_slot && d.ws && b_pool_is_strided(d) && shrink_takes_mma_path(sp)) {
            const size_t off = act_fp4 ? (act_fp4_ws_bytes(d) + 255) / 256 * 256 : 0;
            const uint32_t cap = std::min(mt, d.max_loras) * ((d.max_rank + 15u) / 16u);
            const size_t bytes = size_t((d.m + mt - 1) / mt) * cap * mt * 32;
            if (aligned(d.ws, 256) && d.ws_bytes >= off + bytes && size_t((d.m + mt - 1) / mt) * cap * mt < (1ull << 31)) {
                tt.tiles = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(d.ws) + off);
                tt.cap = cap;
                sp.tile_out = tt.tiles;
                sp.tile_cap = cap;
                sp.chunk = mt;
                sp.part_rows = tt.part_rows = pair ? mt / 2 : mt;
            }
        }
        // Many tiles per SM pair (a prefill batch): the persistent form, whose operand rings run across tile
        // boundaries and whose row stores overlap the next tile's K loop.  It takes 256-token tiles of CTA pairs
        // without a K split, 16-byte aligned destination rows, and LoRA operands that both come by TMA.
        bool persistent = mt == 256 && pair && k_split == 1 && !(d.flags & ATLAS_B200_FLAG_NO_PERSISTENT) &&
                          (!d.seq_slot || b_pool_is_strided(d)) && d.out_row_stride % 8 == 0 &&
                          (d.n_dest ? d.y_col_offset % 8 == 0 : aligned(d.y, 16));
        for (uint32_t r = 0; persistent && r < d.n_dest; ++r) persistent = aligned(d.y_dest[r], 16);
        // two token tiles of 192 per pass (the expanded weight operand is used twice) where the batch has several passes
        bool two_tiles = persistent && !act_fp4 && !(d.flags & ATLAS_B200_FLAG_ONE_TILE_PASS) && d.m >= 768;
        if (two_tiles) {
            // ... unless whole waves say otherwise: a pass of two 192-token tiles takes about 977 cycles per K block, a pass
            // of one 256-token tile about 725 (measured), and the last wave costs a full pass however few CTA pairs it holds
            // (a 1024-feature projection over 8192 tokens: 88 two-tile passes or 128 one-tile passes on 74 pairs, two waves each)
            const int c2 = persist_resident_clusters<192, 2, false>(2), c1 = persist_resident_clusters<256, 1, false>(0);
            if (c1 > 0 && c2 > 0) {
                const uint64_t w2 = (persist_tiles<192, 2>(d) + uint32_t(c2) - 1) / uint32_t(c2);
                const uint64_t w1 = (persist_tiles<256, 1>(d) + uint32_t(c1) - 1) / uint32_t(c1);
                if (w1 * 725 < w2 * 977) two_tiles = false;
            }
        }
        if (persistent) {
            const int clusters = act_fp4 ? persist_resident_clusters<256, 1, true>(1)
                                         : (two_tiles ? persist_resident_clusters<192, 2, false>(2) : persist_resident_clusters<256, 1, false>(0));
            const uint32_t tiles = two_tiles ? persist_tiles<192, 2>(d) : persist_tiles<256, 1>(d);
            persistent = clusters > 0 && tiles > uint32_t(clusters);
        }
        const uint32_t mt_tiles = (persistent && two_tiles) ? 192u : mt;     // token tile of the shrink's masked-t blocks
        if (persistent && d.seq_slot) {
            TTiles t2;
            ShrinkParams sp2 = sp;
            sp2.tile_out = nullptr;
            if (d.ws && shrink_takes_mma_path(sp)) {
                const size_t off = act_fp4 ? (act_fp4_ws_bytes(d) + 255) / 256 * 256 : 0;
                const uint32_t cap = std::min(mt_tiles, d.max_loras) * ((d.max_rank + 15u) / 16u);
                const size_t n_t = (d.m + mt_tiles - 1) / mt_tiles;
                const size_t bytes = n_t * cap * mt_tiles * 32;
                if (aligned(d.ws, 256) && d.ws_bytes >= off + bytes && n_t * cap * mt_tiles < (1ull << 31)) {
                    t2.tiles = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(d.ws) + off);
                    t2.cap = cap;
                    sp2.tile_out = t2.tiles;
                    sp2.tile_cap = cap;
                    sp2.chunk = mt_tiles;
                    sp2.part_rows = t2.part_rows = mt_tiles / 2;
                }
            }
            if (t2.tiles) { tt = t2; sp = sp2; } else persistent = false;
        }
        if (shrink_only) {
            // the shrink alone, for a row range, into several copies of the scratch: the launch shape decided above fixes
            // the tile layout, exactly as the call that later consumes the tiles (ATLAS_B200_FLAG_REUSE_SHRINK) decides it
            if (!d.seq_slot || !tt.tiles || shrink_only->n_dest == 0 || shrink_only->n_dest > 8) return ATLAS_B200_ERR_DIMS;
            const size_t off = size_t(reinterpret_cast<uint8_t*>(tt.tiles) - static_cast<uint8_t*>(d.ws));
            for (uint32_t i = 0; i < shrink_only->n_dest; ++i)
                if (!shrink_only->ws_dest[i] || !aligned(shrink_only->ws_dest[i], 256)) return ATLAS_B200_ERR_ALIGN;
            sp.tile_out = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(shrink_only->ws_dest[0]) + off);
            for (uint32_t i = 1; i < shrink_only->n_dest; ++i)
                sp.tile_out_more[i - 1] = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(shrink_only->ws_dest[i]) + off);
            sp.n_tile_dest = shrink_only->n_dest;
            sp.m_begin = shrink_only->row_begin;
            sp.m_count = shrink_only->row_count;
            rc = launch_shrink(sp, d.max_loras, st);
            if (rc == ATLAS_B200_OK) t_last_variant = ATLAS_B200_VARIANT_TCGEN05;
            return rc;
        }
        const ShrinkParams* shrink = (d.seq_slot && !(d.flags & ATLAS_B200_FLAG_REUSE_SHRINK)) ? &sp : nullptr;
        if (persistent) {
            if (act_fp4) rc = launch_tc_persist<256, 1, true>(d, 1, shrink, tt, st);
            else if (two_tiles) rc = launch_tc_persist<192, 2, false>(d, 2, shrink, tt, st);
            else rc = launch_tc_persist<256, 1, false>(d, 0, shrink, tt, st);
            if (rc == ATLAS_B200_OK) t_last_variant = ATLAS_B200_VARIANT_TCGEN05;
            return rc;
        }
        if (act_fp4) {
            if (mt == 16) rc = launch_tc<16, true, false>(d, 0, shrink, tt, k_split, st);
            else if (mt == 32) rc = launch_tc<32, true, false>(d, 1, shrink, tt, k_split, st);
            else if (mt == 64) rc = launch_tc<64, true, false>(d, 2, shrink, tt, k_split, st);
            else if (mt == 128) rc = pair ? launch_tc<128, true, true>(d, 3, shrink, tt, k_split, st) : launch_tc<128, true, false>(d, 3, shrink, tt, k_split, st);
            else rc = pair ? launch_tc<256, true, true>(d, 4, shrink, tt, k_split, st) : launch_tc<256, true, false>(d, 4, shrink, tt, k_split, st);
        } else if (mt == 16) rc = launch_tc<16, false, false>(d, 0, shrink, tt, k_split, st);
        else if (mt == 32) rc = launch_tc<32, false, false>(d, 1, shrink, tt, k_split, st);
        else if (mt == 64) rc = launch_tc<64, false, false>(d, 2, shrink, tt, k_split, st);
        else if (mt == 128) rc = pair ? launch_tc<128, false, true>(d, 3, shrink, tt, k_split, st) : launch_tc<128, false, false>(d, 3, shrink, tt, k_split, st);
        else rc = pair ? launch_tc<256, false, true>(d, 4, shrink, tt, k_split, st) : launch_tc<256, false, false>(d, 4, shrink, tt, k_split, st);
        if (rc == ATLAS_B200_OK) t_last_variant = ATLAS_B200_VARIANT_TCGEN05;
        return rc;
    }

    // Base linear — a dense BF16 weight on the tensor cores where the shape allows, everything else on CUDA cores —
    // then the reference's two-stage LoRA in place
    const bool dense_tc = !(d.flags & ATLAS_B200_FLAG_FORCE_SIMT) && !staged && dense_tc_eligible(d);
    rc = dense_tc ? launch_dense_tc(d, st) : launch_simt_linear(d, st);
    if (rc) return rc;
    if (d.seq_slot) {
        ShrinkParams sp{};
        sp.x = static_cast<const uint16_t*>(d.x);
        sp.seq_slot = d.seq_slot;
        sp.a_table = d.a_table;
        sp.b_table = d.b_table;
        sp.rank_table = d.rank_table;
        sp.out = static_cast<uint16_t*>(d.lora_t);
        sp.M = d.m; sp.k_in = d.k; sp.max_rank = d.max_rank; sp.x_row_stride = d.x_row_stride; sp.max_loras = d.max_loras;
        sp.post = 0.0f;
        rc = launch_shrink(sp, d.max_loras, st);
        if (rc) return rc;
        ExpandParams ep{};
        ep.xa = static_cast<const uint16_t*>(d.lora_t);
        ep.seq_slot = d.seq_slot;
        ep.a_table = d.a_table;
        ep.b_table = d.b_table;
        ep.scale_table = d.scale_table;
        ep.out = static_cast<uint16_t*>(d.y);
        ep.M = d.m; ep.n_out = d.n; ep.max_rank = d.max_rank; ep.out_row_stride = d.out_row_stride; ep.max_loras = d.max_loras;
        rc = launch_expand(ep, st);
        if (rc) return rc;
    }
    t_last_variant = dense_tc ? ATLAS_B200_VARIANT_TCGEN05 : ATLAS_B200_VARIANT_SIMT;
    return ATLAS_B200_OK;
}

}  // namespace ops
}  // namespace atlas

// =============================================================================================
// extern "C"
// =============================================================================================
using namespace atlas;

extern "C" {

int atlas_b200_lora_bgmv(const void* x, const int32_t* seq_slot, const uint64_t* a_table, const uint64_t* b_table,
                         const float* scale_table, void* base_out, void* lora_xa, uint32_t n, uint32_t k_in,
                         uint32_t n_out, uint32_t max_rank, uint32_t x_row_stride, uint32_t out_row_stride,
                         uint32_t max_loras, void* stream) {
    return ops::apply_lora_bgmv(x, seq_slot, a_table, b_table, scale_table, base_out, lora_xa, n, k_in, n_out, max_rank,
                                x_row_stride, out_row_stride, max_loras, static_cast<cudaStream_t>(stream));
}

int atlas_b200_lora_delta(const void* x, const void* a, const void* b, float scale, void* base_out, void* lora_xa,
                          void* lora_delta, uint32_t m, uint32_t k_in, uint32_t n_out, uint32_t max_rank, void* stream) {
    return ops::apply_lora_delta(x, a, b, scale, base_out, lora_xa, lora_delta, m, k_in, n_out, max_rank,
                                 static_cast<cudaStream_t>(stream));
}

int atlas_b200_w4a16_gemm(const void* a_bf16, const void* b_packed, const void* b_scale, float scale2, void* c_bf16,
                          uint32_t m, uint32_t n, uint32_t k, void* ws, size_t ws_bytes, void* stream) {
    (void)ws; (void)ws_bytes;
    atlas_b200_linear_desc d;
    std::memset(&d, 0, sizeof(d));
    d.x = a_bf16; d.m = m; d.k = k; d.x_row_stride = k;
    d.n = n; d.w_packed = b_packed; d.w_scale = b_scale; d.scale2 = scale2;
    d.y = c_bf16; d.out_row_stride = n;
    return ops::nvfp4_lora_linear(d, static_cast<cudaStream_t>(stream));
}

int atlas_b200_dequant_nvfp4_to_bf16(const void* packed, const void* scales, void* out_bf16, float combined_global,
                                     uint32_t n, uint32_t k, void* stream) {
    if (n == 0 || k == 0) return ATLAS_B200_OK;
    if (!packed || !scales || !out_bf16) return ATLAS_B200_ERR_NULL;
    if (k % 16 != 0) return ATLAS_B200_ERR_DIMS;
    if (!aligned(out_bf16, 4)) return ATLAS_B200_ERR_ALIGN;
    dequant_nvfp4_kernel<<<n, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(packed), static_cast<const uint8_t*>(scales), static_cast<uint16_t*>(out_bf16),
        combined_global, n, k);
    return launch_status();
}

int atlas_b200_quantize_bf16_to_nvfp4(const void* in_bf16, void* packed, void* scales, float scale2, uint32_t n,
                                      uint32_t k, void* stream) {
    if (n == 0 || k == 0) return ATLAS_B200_OK;
    if (!in_bf16 || !packed || !scales) return ATLAS_B200_ERR_NULL;
    if (k % 16 != 0) return ATLAS_B200_ERR_DIMS;
    const size_t groups = size_t(n) * (k / 16);
    const unsigned blocks = unsigned(std::min<size_t>((groups + 255) / 256, size_t(rt_sm_count()) * 16));
    const uint32_t vec = aligned(in_bf16, 16) && aligned(packed, 8) && k % 16 == 0;
    quantize_nvfp4_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(in_bf16), static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scales), scale2, n, k, k, vec);
    return launch_status();
}

int atlas_b200_nvfp4_global_absmax(const void* in_bf16, float* global_max_dev, size_t total, void* stream) {
    if (total == 0) return ATLAS_B200_OK;
    if (!in_bf16 || !global_max_dev) return ATLAS_B200_ERR_NULL;
    if (!aligned(in_bf16, 2) || !aligned(global_max_dev, 4)) return ATLAS_B200_ERR_ALIGN;
    const unsigned blocks = unsigned(std::min<size_t>((total / 8 + 255) / 256 + 1, size_t(rt_sm_count()) * 8));
    nvfp4_global_absmax_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint16_t*>(in_bf16), global_max_dev, total);
    return launch_status();
}

float atlas_b200_nvfp4_scale2_from_absmax(float global_max) { return global_max / (6.0f * 448.0f); }

float atlas_b200_nvfp4_combined_global_scale(float stored_scale, int is_reciprocal) {
    if (!is_reciprocal) return stored_scale;
    return stored_scale != 0.0f ? 1.0f / stored_scale : 0.0f;
}

int atlas_b200_push_columns(const void* src, uint32_t src_row_stride, void* const* dest, uint32_t n_dest, uint32_t dst_row_stride,
                            uint32_t m, uint32_t n_cols, void* stream) {
    if (!src || (!dest && n_dest)) return ATLAS_B200_ERR_NULL;
    if (n_dest > uint32_t(PUSH_MAX_DEST)) return ATLAS_B200_ERR_LIMIT;
    if (m == 0 || n_cols == 0 || n_dest == 0) return ATLAS_B200_OK;
    if (n_cols > src_row_stride || n_cols > dst_row_stride) return ATLAS_B200_ERR_DIMS;
    if (n_cols % 8 || src_row_stride % 8 || dst_row_stride % 8 || !aligned(src, 16)) return ATLAS_B200_ERR_ALIGN;
    PushParams p{};
    p.src = static_cast<const uint4*>(src);
    for (uint32_t d = 0; d < n_dest; ++d) {
        if (!dest[d]) return ATLAS_B200_ERR_NULL;
        if (!aligned(dest[d], 16)) return ATLAS_B200_ERR_ALIGN;
        p.dst[d] = static_cast<uint4*>(dest[d]);
    }
    p.n_dest = n_dest;
    p.m = m;
    p.chunks_per_row = n_cols / 8;
    p.src_row_chunks = src_row_stride / 8;
    p.dst_row_chunks = dst_row_stride / 8;
    const uint64_t total = uint64_t(m) * p.chunks_per_row;
    const uint64_t want = (total + uint64_t(PUSH_THREADS) * 4 - 1) / (uint64_t(PUSH_THREADS) * 4);
    const uint32_t grid = uint32_t(std::min<uint64_t>(std::max<uint64_t>(want, 1), uint64_t(rt_sm_count()) * 2));
    // same shared-memory carve-out as the tcgen05 kernels: an SM must not have to drain and be reconfigured before it can
    // take one of these CTAs next to theirs
    DeviceState* dst_state = device_state();
    if (dst_state && !dst_state->push_attr_set) {
        cudaFuncSetAttribute(push_columns_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        dst_state->push_attr_set = true;
    }
    push_columns_kernel<<<grid, PUSH_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return launch_status();
}

static int kv_norm_rope_cache_write(const void* k_in, const void* v_in, uint32_t in_row_stride, const void* k_norm_weight,
                                    const uint32_t* positions, const uint32_t* positions_h, const uint32_t* positions_w, const long long* slot_mapping, void* k_cache, void* v_cache,
                                        uint32_t tokens, uint32_t kv_heads, uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size,
                                        float rms_eps, float theta, void* stream, float fp8_inv_scale = 0.0f) {
    if (!k_in || !k_norm_weight || !positions || !slot_mapping || !k_cache || (v_in && !v_cache)) return ATLAS_B200_ERR_NULL;
    if (tokens == 0 || kv_heads == 0) return ATLAS_B200_OK;
    if (head_dim == 0 || head_dim % 32 || head_dim > uint32_t(KVE_MAX_HEAD_DIM) || rotary_dim > head_dim || rotary_dim % 64 ||
        block_size == 0 || in_row_stride < kv_heads * head_dim)
        return ATLAS_B200_ERR_DIMS;
    KvEpilogueParams p{};
    p.k_in = static_cast<const uint16_t*>(k_in);
    p.v_in = static_cast<const uint16_t*>(v_in);
    p.k_norm_w = static_cast<const uint16_t*>(k_norm_weight);
    p.positions = positions;
    p.positions_h = positions_h;
    p.positions_w = positions_w;
    p.slot_mapping = slot_mapping;
    p.k_cache = static_cast<uint16_t*>(k_cache);
    p.v_cache = static_cast<uint16_t*>(v_cache);
    p.tokens = tokens; p.kv_heads = kv_heads; p.head_dim = head_dim; p.rotary_dim = rotary_dim; p.block_size = block_size;
    p.in_row_stride = in_row_stride; p.rms_eps = rms_eps; p.theta = theta; p.fp8_inv_scale = fp8_inv_scale;
    const dim3 grid((tokens + KVE_TOKENS - 1) / KVE_TOKENS), block(KVE_WARPS * 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool exact = rotary_dim == 64 && fp8_inv_scale == 0.0f && (head_dim == 64 || head_dim == 128 || head_dim == 256);
    if (head_dim <= 64) exact ? kv_norm_rope_cache_kernel<2, true><<<grid, block, 0, st>>>(p) : kv_norm_rope_cache_kernel<2, false><<<grid, block, 0, st>>>(p);
    else if (head_dim <= 128) exact ? kv_norm_rope_cache_kernel<4, true><<<grid, block, 0, st>>>(p) : kv_norm_rope_cache_kernel<4, false><<<grid, block, 0, st>>>(p);
    else exact ? kv_norm_rope_cache_kernel<8, true><<<grid, block, 0, st>>>(p) : kv_norm_rope_cache_kernel<8, false><<<grid, block, 0, st>>>(p);
    return launch_status();
}

int atlas_b200_kv_norm_rope_cache_write(const void* k_in, const void* v_in, uint32_t in_row_stride, const void* k_norm_weight,
                                        const uint32_t* positions, const long long* slot_mapping, void* k_cache, void* v_cache,
                                        uint32_t tokens, uint32_t kv_heads, uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size,
                                        float rms_eps, float theta, void* stream) {
    return kv_norm_rope_cache_write(k_in, v_in, in_row_stride, k_norm_weight, positions, nullptr, nullptr, slot_mapping, k_cache, v_cache, tokens,
                                    kv_heads, head_dim, rotary_dim, block_size, rms_eps, theta, stream);
}

int atlas_b200_k_norm_rope_cache_write_fp8(const void* k_in, uint32_t in_row_stride, const void* k_norm_weight, const uint32_t* positions,
                                           const long long* slot_mapping, void* k_cache_fp8, uint32_t tokens, uint32_t kv_heads,
                                           uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size, float rms_eps, float theta,
                                           float inv_scale, void* stream) {
    if (!(inv_scale > 0.0f)) return ATLAS_B200_ERR_DIMS;
    return kv_norm_rope_cache_write(k_in, nullptr, in_row_stride, k_norm_weight, positions, nullptr, nullptr, slot_mapping, k_cache_fp8, nullptr,
                                    tokens, kv_heads, head_dim, rotary_dim, block_size, rms_eps, theta, stream, inv_scale);
}

int atlas_b200_kv_norm_mrope_cache_write(const void* k_in, const void* v_in, uint32_t in_row_stride, const void* k_norm_weight,
                                         const uint32_t* pos_t, const uint32_t* pos_h, const uint32_t* pos_w, const long long* slot_mapping,
                                         void* k_cache, void* v_cache, uint32_t tokens, uint32_t kv_heads, uint32_t head_dim,
                                         uint32_t rotary_dim, uint32_t block_size, float rms_eps, float theta, void* stream) {
    if (!pos_h || !pos_w) return ATLAS_B200_ERR_NULL;
    return kv_norm_rope_cache_write(k_in, v_in, in_row_stride, k_norm_weight, pos_t, pos_h, pos_w, slot_mapping, k_cache, v_cache, tokens,
                                    kv_heads, head_dim, rotary_dim, block_size, rms_eps, theta, stream);
}

int atlas_b200_qkv_norm_rope_cache_write(void* q, const void* k_in, const void* v_in, uint32_t q_row_stride, uint32_t kv_row_stride,
                                         const void* q_norm_weight, const void* k_norm_weight, const uint32_t* positions,
                                         const float* inv_freq, const long long* slot_mapping, void* k_cache, void* v_cache,
                                         uint32_t tokens, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t rotary_dim,
                                         uint32_t block_size, float rms_eps, float attention_factor, int norm_offset_one, void* stream) {
    if (!q || !k_in || !v_in || !q_norm_weight || !k_norm_weight || !positions || !slot_mapping || !k_cache || !v_cache ||
        (rotary_dim && !inv_freq))
        return ATLAS_B200_ERR_NULL;
    if (tokens == 0 || q_heads + kv_heads == 0) return ATLAS_B200_OK;
    if (head_dim == 0 || head_dim % 2 || head_dim > uint32_t(KVE_MAX_HEAD_DIM) || rotary_dim > head_dim || rotary_dim % 2 ||
        block_size == 0 || q_row_stride < q_heads * head_dim || kv_row_stride < kv_heads * head_dim)
        return ATLAS_B200_ERR_DIMS;
    // packed pairs are read as 32-bit words
    if (!aligned(q, 4) || !aligned(k_in, 4) || !aligned(v_in, 4) || !aligned(v_cache, 4) || !aligned(q_norm_weight, 4) ||
        !aligned(k_norm_weight, 4) || q_row_stride % 2 || kv_row_stride % 2)
        return ATLAS_B200_ERR_ALIGN;
    QkvEpilogueParams p{};
    p.q = static_cast<uint16_t*>(q);
    p.k_in = static_cast<const uint16_t*>(k_in);
    p.v_in = static_cast<const uint16_t*>(v_in);
    p.q_norm_w = static_cast<const uint16_t*>(q_norm_weight);
    p.k_norm_w = static_cast<const uint16_t*>(k_norm_weight);
    p.positions = positions; p.inv_freq = inv_freq; p.slot_mapping = slot_mapping;
    p.k_cache = static_cast<uint16_t*>(k_cache);
    p.v_cache = static_cast<uint16_t*>(v_cache);
    p.tokens = tokens; p.q_heads = q_heads; p.kv_heads = kv_heads; p.head_dim = head_dim; p.rotary_dim = rotary_dim;
    p.block_size = block_size; p.q_row_stride = q_row_stride; p.kv_row_stride = kv_row_stride;
    p.rms_eps = rms_eps; p.attention_factor = attention_factor; p.norm_offset_one = norm_offset_one ? 1u : 0u;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool exact = rotary_dim == 64 && (head_dim == 64 || head_dim == 128 || head_dim == 256);
    if (head_dim <= 64) exact ? qkv_norm_rope_cache_kernel<1, true><<<tokens, KVE_WARPS * 32, 0, st>>>(p)
                              : qkv_norm_rope_cache_kernel<1, false><<<tokens, KVE_WARPS * 32, 0, st>>>(p);
    else if (head_dim <= 128) exact ? qkv_norm_rope_cache_kernel<2, true><<<tokens, KVE_WARPS * 32, 0, st>>>(p)
                                    : qkv_norm_rope_cache_kernel<2, false><<<tokens, KVE_WARPS * 32, 0, st>>>(p);
    else exact ? qkv_norm_rope_cache_kernel<4, true><<<tokens, KVE_WARPS * 32, 0, st>>>(p)
               : qkv_norm_rope_cache_kernel<4, false><<<tokens, KVE_WARPS * 32, 0, st>>>(p);
    return launch_status();
}

int atlas_b200_copy_columns(const void* src, uint32_t src_row_stride, void* const* dest, uint32_t n_dest, uint32_t dst_row_stride,
                            uint32_t m, uint32_t n_cols, void* stream) {
    if (!src || (!dest && n_dest)) return ATLAS_B200_ERR_NULL;
    if (m == 0 || n_cols == 0 || n_dest == 0) return ATLAS_B200_OK;
    if (n_cols > src_row_stride || n_cols > dst_row_stride) return ATLAS_B200_ERR_DIMS;
    for (uint32_t d = 0; d < n_dest; ++d) {
        if (!dest[d]) return ATLAS_B200_ERR_NULL;
        // one strided copy per destination, carried by the copy engines
        cudaError_t e = cudaMemcpy2DAsync(dest[d], size_t(dst_row_stride) * 2, src, size_t(src_row_stride) * 2, size_t(n_cols) * 2, m,
                                          cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return cuda_status(e);
    }
    return ATLAS_B200_OK;
}

int atlas_b200_silu_mul(const void* gate_bf16, const void* up_bf16, void* out_bf16, float gate_scale, float up_scale, float swiglu_limit,
                        uint32_t m, uint32_t k, uint32_t in_row_stride, uint32_t out_row_stride, void* stream) {
    if (m == 0 || k == 0) return ATLAS_B200_OK;
    if (!gate_bf16 || !up_bf16 || !out_bf16) return ATLAS_B200_ERR_NULL;
    if (k % 8 != 0 || in_row_stride < k || out_row_stride < k) return ATLAS_B200_ERR_DIMS;
    if (in_row_stride % 8 != 0 || out_row_stride % 8 != 0 || !aligned(gate_bf16, 16) || !aligned(up_bf16, 16) || !aligned(out_bf16, 16))
        return ATLAS_B200_ERR_ALIGN;
    const size_t vecs = size_t(m) * (k / 8);
    const unsigned blocks = unsigned(std::min<size_t>((vecs + 255) / 256, size_t(rt_sm_count()) * 16));
    silu_mul_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(gate_bf16), static_cast<const uint16_t*>(up_bf16), static_cast<uint16_t*>(out_bf16), gate_scale,
        up_scale, swiglu_limit, m, k, in_row_stride, out_row_stride);
    return launch_status();
}

int atlas_b200_silu_mul_quant_nvfp4(const void* gate_bf16, const void* up_bf16, void* ws, size_t ws_bytes, float gate_scale, float up_scale,
                                    float swiglu_limit, uint32_t m, uint32_t k, uint32_t in_row_stride, void* stream) {
    if (m == 0 || k == 0) return ATLAS_B200_OK;
    if (!gate_bf16 || !up_bf16 || !ws) return ATLAS_B200_ERR_NULL;
    if (k % 16 != 0 || in_row_stride < k) return ATLAS_B200_ERR_DIMS;
    if (in_row_stride % 8 != 0 || !aligned(gate_bf16, 16) || !aligned(up_bf16, 16) || !aligned(ws, 256)) return ATLAS_B200_ERR_ALIGN;
    const size_t codes_bytes = (size_t(m) * (k / 2) + 255) / 256 * 256;
    if (ws_bytes < codes_bytes + size_t(m) * (k / 16)) return ATLAS_B200_ERR_WORKSPACE;
    const size_t groups = size_t(m) * (k / 16);
    const unsigned blocks = unsigned(std::min<size_t>((groups + 255) / 256, size_t(rt_sm_count()) * 16));
    uint8_t* codes = static_cast<uint8_t*>(ws);
    silu_mul_quant_nvfp4_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(gate_bf16), static_cast<const uint16_t*>(up_bf16), codes, codes + codes_bytes, gate_scale, up_scale,
        swiglu_limit, m, k, in_row_stride);
    return launch_status();
}

int atlas_b200_nvfp4_lora_linear(const atlas_b200_linear_desc* desc, void* stream) {
    if (!desc) return ATLAS_B200_ERR_NULL;
    return ops::nvfp4_lora_linear(*desc, static_cast<cudaStream_t>(stream));
}

int atlas_b200_lora_shrink_tiles(const atlas_b200_linear_desc* desc, uint32_t row_begin, uint32_t row_count,
                                 void* const* ws_dest, uint32_t n_dest, void* stream) {
    if (!desc || !ws_dest) return ATLAS_B200_ERR_NULL;
    ops::ShrinkOnly so{row_begin, row_count, n_dest, ws_dest};
    return ops::nvfp4_lora_linear(*desc, static_cast<cudaStream_t>(stream), &so);
}

// ---------------------------------------------------------------------------------------------
// Fused layer for callers that cannot allocate device memory.
//
// Some hosts of this library may launch kernels but may not call cudaMalloc: a plug-in that is
// handed tensors by an engine which owns every byte of device memory, or code running inside a
// region (a captured serving step, a real-time loop) where the allocator must not be entered.
// Such a caller has nowhere to get the shrink scratch `lora_t` from.  This entry point keeps that
// scratch in a fixed array inside the library image instead, so the caller passes inputs and the
// output only.
//
// The array holds ATLAS_B200_STATIC_SCRATCH_ELEMS BF16 values (1 MiB) on every GPU that loads the
// library, for the life of the process.  A call needs m * max_rank of them; more is refused.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) uint16_t g_static_lora_t[ATLAS_B200_STATIC_SCRATCH_ELEMS];

namespace atlas {
// In host code `g_static_lora_t` names a host-side shadow of the symbol, not device memory, so the
// device address is asked for once per device, with that device current, and cached.
static void* g_static_scratch_addr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

static int static_scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e);
    if (dev < 0 || dev >= kMaxDevices) return ATLAS_B200_ERR_LIMIT;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_addr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_lora_t);
        if (e != cudaSuccess) return cuda_status(e);
        if (!ptr) return ATLAS_B200_ERR_NULL;
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return ATLAS_B200_OK;
}
}  // namespace atlas

extern "C" int atlas_b200_nvfp4_lora_linear_noalloc(const atlas_b200_linear_desc* desc, void* stream) {
    if (!desc) return ATLAS_B200_ERR_NULL;
    atlas_b200_linear_desc d = *desc;
    if (d.seq_slot) {
        // validate the size before anything else so that an oversized call never touches the array
        if (d.max_rank == 0 || d.max_loras == 0) return ATLAS_B200_ERR_DIMS;
        if (uint64_t(d.m) * uint64_t(d.max_rank) > uint64_t(ATLAS_B200_STATIC_SCRATCH_ELEMS)) return ATLAS_B200_ERR_LIMIT;
        void* scratch = nullptr;
        const int rc = static_scratch_for_current_device(&scratch);
        if (rc) return rc;
        // Nothing in the scratch has to start at zero: the shrink writes every element of every routed
        // row (pad ranks as zeros) and un-routed rows are never read, so leftovers of an earlier call
        // are harmless and no clearing pass is launched.
        d.lora_t = scratch;
    }
    return ops::nvfp4_lora_linear(d, static_cast<cudaStream_t>(stream));
}

int atlas_b200_device_status(uint32_t* out_word, int clear) {
    if (!out_word) return ATLAS_B200_ERR_NULL;
    cudaError_t e = cudaMemcpyFromSymbol(out_word, g_status_word, sizeof(uint32_t));
    if (e != cudaSuccess) return cuda_status(e);
    if (clear) {
        const uint32_t zero = 0;
        e = cudaMemcpyToSymbol(g_status_word, &zero, sizeof(uint32_t));
    }
    return cuda_status(e);
}

int atlas_b200_selftest_bounded_wait(uint64_t limit_ns, uint32_t out_host[3]) {
    if (!out_host) return ATLAS_B200_ERR_NULL;
    if (limit_ns == 0 || limit_ns > 100000000ull) return ATLAS_B200_ERR_LIMIT;        // at most 0.1 s: this is a test of giving up
    uint32_t* out_dev = nullptr;
    cudaError_t e = cudaMalloc(&out_dev, 3 * sizeof(uint32_t));
    if (e != cudaSuccess) return cuda_status(e);
    cudaMemset(out_dev, 0xFF, 3 * sizeof(uint32_t));
    tc::bounded_wait_selftest_kernel<<<1, 64>>>(limit_ns, uint32_t(STATUS_WAIT_EXPIRED_PRODUCER), out_dev);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpy(out_host, out_dev, 3 * sizeof(uint32_t), cudaMemcpyDeviceToHost);
    cudaFree(out_dev);
    return cuda_status(e);
}

int atlas_b200_last_variant(void) { return t_last_variant; }

int atlas_b200_last_launch_shape(uint32_t out[4]) {
    if (!out) return ATLAS_B200_ERR_NULL;
    for (int i = 0; i < 4; ++i) out[i] = t_last_shape[i];
    return ATLAS_B200_OK;
}

int atlas_b200_last_persistent_shape(uint32_t out[2]) {
    if (!out) return ATLAS_B200_ERR_NULL;
    out[0] = t_last_shape[4];
    out[1] = t_last_shape[5];
    return ATLAS_B200_OK;
}

int atlas_b200_set_profile_buffer(void* device_buffer, size_t n_words) {
    g_profile_buf = static_cast<unsigned long long*>(device_buffer);
    g_profile_words = device_buffer ? n_words : 0;
    return ATLAS_B200_OK;
}

const char* atlas_b200_version(void) { return "atlas_b200 0.1 (sm_100a)"; }

}  // extern "C"
