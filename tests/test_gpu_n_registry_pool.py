"""The adapter pool as the reference lays it out, end to end: PEFT adapters (config + safetensors) go through the
library's ingest into a 2-layer x 7-module x 4-slot slot-major pool on the GPU, the per-(layer, module) tables come from
the registry, and the kernels are fed slot 0's B of the module plus pool_slot_bytes as the slot stride.  The fused
layer (TMA path over the strided pool) and the routed LoRA op are checked against the oracle."""
import json

import numpy as np
import pytest

from gpu_util import ATOL, RTOL, assert_close, bits_from_dev, to_dev
from test_adapter_ingest import base_json, write_safetensors

pytestmark = pytest.mark.gpu

DIMS = dict(hidden_size=512, intermediate_size=1024, num_attention_heads=4, num_key_value_heads=2, head_dim=128)
N_LAYERS, FULL = 4, [1, 3]
MODS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
PATH = {"q_proj": "self_attn", "k_proj": "self_attn", "v_proj": "self_attn", "o_proj": "self_attn", "gate_proj": "mlp", "up_proj": "mlp", "down_proj": "mlp"}


def _adapter(atlas, cfg, seed, r, modules, dtype):
    rng = np.random.default_rng(seed)
    np_dt = {"F32": np.float32, "F16": np.float16}[dtype]
    t = {}
    for l in FULL:
        for m in modules:
            out_dim, in_dim = atlas.module_dims(cfg, MODS.index(m))
            key = f"base_model.model.model.layers.{l}.{PATH[m]}.{m}"
            t[key + ".lora_A.weight"] = (dtype, (rng.uniform(-1, 1, (r, in_dim)) / np.sqrt(in_dim)).astype(np_dt))
            t[key + ".lora_B.weight"] = (dtype, (rng.standard_normal((out_dim, r)) * 0.1).astype(np_dt))
    cj = json.dumps(base_json(r=r, lora_alpha=2 * r, target_modules=list(modules), layers_to_transform=FULL))
    return cj, t


@pytest.mark.parametrize("layer,module,M", [(3, 1, 48), (1, 6, 48), (3, 4, 1100)])
def test_slot_major_pool_feeds_the_kernels(cuda, atlas, oracle, layer, module, M):
    from atlas_b200 import adapters, registry, synth
    cfg = registry.model_dims(**DIMS, num_full_attention_layers=len(FULL))
    fa = [1 if i in FULL else 0 for i in range(N_LAYERS)]
    max_loras, max_rank = 4, 16
    slot_bytes = atlas.pool_slot_bytes(cfg, max_rank)
    pool = cuda.zeros(slot_bytes * max_loras, dtype=cuda.uint8, device="cuda")
    reg = adapters.AdapterRegistry(cfg, N_LAYERS, fa, max_loras, max_rank, device_pool=pool)
    # slot 0: every module, r = 16, F32; slot 1: attention only, r = 8, F16; slot 2: empty; slot 3: MLP only, r = 16
    specs = {0: (16, MODS, "F32"), 1: (8, MODS[:4], "F16"), 3: (16, MODS[4:], "F32")}
    tensors = {}
    for s, (r, mods, dt) in specs.items():
        cj, t = _adapter(atlas, cfg, 10 + s, r, mods, dt)
        reg.load_adapter(s, f"adapter{s}", cj, write_safetensors(t))
        tensors[s] = t
    route = reg.route(layer, module)
    assert route.b_slot_stride == slot_bytes and route.a_slot_stride == slot_bytes
    out_dim, in_dim = atlas.module_dims(cfg, module)
    # host-side pool for the oracle: the same adapters, BF16 as the ingest converts them
    hp = oracle.HostPool(in_dim, out_dim, max_rank, max_loras)
    for s, (r, mods, dt) in specs.items():
        if MODS[module] not in mods:
            continue
        key = f"base_model.model.model.layers.{layer}.{PATH[MODS[module]]}.{MODS[module]}"
        a = adapters.convert_to_bf16(dt, tensors[s][key + ".lora_A.weight"][1])
        b = adapters.convert_to_bf16(dt, tensors[s][key + ".lora_B.weight"][1])
        hp.pack(s, a, b, 2.0)
    # a batch that uses every slot, the empty one and "no adapter" included
    base = synth.make_case("pool", M=M, K=in_dim, N=out_dim, ranks=[4], max_rank=max_rank, max_loras=max_loras, scale2=0.02, seed=layer * 10 + module)
    slots = (np.arange(M) % 5 - 1).astype(np.int32)                  # -1, 0, 1, 2, 3, ...
    x, packed, scales = to_dev(cuda, base.x), to_dev(cuda, base.packed), to_dev(cuda, base.scales)
    seq = to_dev(cuda, slots)
    y = cuda.full((M, out_dim), 0x7FC0, dtype=cuda.int16, device="cuda")
    lora_t = cuda.zeros((M, max_rank), dtype=cuda.int16, device="cuda")
    ws = cuda.empty(atlas.lora_ws_bytes(M, max_loras, max_rank), dtype=cuda.uint8, device="cuda")
    d = atlas.make_linear_desc(x=x, m=M, k=in_dim, n=out_dim, y=y, w_packed=packed, w_scale=scales, scale2=base.scale2,
                               seq_slot=seq, route=route, lora_t=lora_t, ws=ws, ws_bytes=ws.numel(), flags=atlas.FLAG_FORCE_TCGEN05)
    atlas.nvfp4_lora_linear(d)
    cuda.cuda.synchronize()
    assert atlas.last_launch_shape()["lora_tiles_from_shrink"]       # both LoRA operands came by TMA out of the strided pool
    want = oracle.fused_linear_f32(base.x, M, out_dim, in_dim, packed=base.packed, scales=base.scales, scale2=base.scale2,
                                   seq_slot=slots, pool=hp)
    assert_close(oracle, bits_from_dev(y), want, "fused layer over the slot-major pool")
    # rows whose slot does not carry the module are the base result, bit for bit
    yb = cuda.full((M, out_dim), 0x7FC0, dtype=cuda.int16, device="cuda")
    atlas.w4a16_gemm(x, packed, scales, base.scale2, yb, M, out_dim, in_dim)
    cuda.cuda.synchronize()
    carried = np.array([s >= 0 and hp.a[s] is not None for s in slots])
    assert carried.any() and (~carried).any()
    assert np.array_equal(bits_from_dev(y)[~carried], bits_from_dev(yb)[~carried])
    # the routed LoRA op on top of the base result, against the staged oracle.  Both sides keep the reference's rounding
    # boundaries (base -> BF16, xa -> BF16, delta -> BF16, fold -> BF16), so where base and delta cancel they may differ by
    # one BF16 ulp (2^-8) of the larger term on top of the path's rtol / atol.
    xa = cuda.zeros((M, max_rank), dtype=cuda.int16, device="cuda")
    base_gpu = oracle.bf16_to_f32(bits_from_dev(yb))
    atlas.apply_lora_bgmv(route, x, yb, seq, M, in_dim, out_dim, xa)
    cuda.cuda.synchronize()
    base_bits = oracle.w4a16_gemm_bf16w(base.x, base.packed, base.scales, base.scale2, M, out_dim, in_dim)
    base_ref = oracle.bf16_to_f32(base_bits.copy())
    oracle.lora_bgmv_staged(base.x, slots, hp, base_bits, M)
    got, exp = oracle.bf16_to_f32(bits_from_dev(yb)), oracle.bf16_to_f32(base_bits)
    lim = ATOL + RTOL * np.abs(exp) + 2.0 ** -8 * (np.abs(base_ref) + np.abs(exp - base_ref))
    bad = ~(np.abs(got - exp) <= lim)
    assert np.isfinite(got).all() and not bad.any(), (int(bad.sum()), got[bad][:4], exp[bad][:4], base_ref[bad][:4])
    assert np.array_equal(got[~carried], base_gpu[~carried])            # rows without the module: untouched by the op
    assert atlas.device_status() == 0
