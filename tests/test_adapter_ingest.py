"""Adapter ingest and registry (host only): PEFT config rules with every named rejection, safetensors -> BF16, key
classification, the load-time audit, slot packing against a numpy restatement of the pool layout, routing tables,
slot lifecycle — and, where a checkout of the reference sits beside this repository, its own adapter fixture
(72 tensors, r = 8, alpha 16) against the committed per-pair digests of delta = scaling * B @ A."""
import json
import os
import struct

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
HOLO_LAYERS, HOLO_FULL = 24, [3, 7, 11, 15, 19, 23]


@pytest.fixture(scope="module")
def ad(atlas):
    from atlas_b200 import adapters
    return adapters


def base_json(**over):
    d = {"peft_type": "LORA", "r": 16, "lora_alpha": 32, "use_rslora": False, "bias": "none",
         "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj"], "lora_dropout": 0.05,
         "task_type": "CAUSAL_LM", "rank_pattern": {}, "alpha_pattern": {}, "modules_to_save": None}
    d.update(over)
    return {k: v for k, v in d.items() if v is not ...}


# ---- PEFT config ------------------------------------------------------------------------------------
def test_peft_happy_paths(ad):
    c = ad.parse_peft_adapter_config(json.dumps(base_json()))
    assert c["r"] == 16 and c["lora_alpha"] == 32.0 and not c["use_rslora"] and c["scaling"] == 2.0 and len(c["target_modules"]) == 6
    assert ad.parse_peft_adapter_config(json.dumps(base_json(use_rslora=True)))["scaling"] == 8.0          # 32 / sqrt(16)
    assert ad.parse_peft_adapter_config(json.dumps(base_json(lora_alpha=16.5)))["lora_alpha"] == 16.5
    c = ad.parse_peft_adapter_config(json.dumps(base_json(layers_to_transform=HOLO_FULL)))
    assert c["layers_to_transform"] == HOLO_FULL
    assert ad.parse_peft_adapter_config(json.dumps(base_json(layers_to_transform=None)))["layers_to_transform"] is None
    c = ad.parse_peft_adapter_config(json.dumps(base_json(target_modules=["model.layers.3.self_attn.k_proj"])))
    assert c["target_modules"] == ["model.layers.3.self_attn.k_proj"]                                  # validated on its leaf, kept verbatim


@pytest.mark.parametrize("over,tag", [
    (dict(use_rslora=...), "REJECT(use_rslora)"),
    (dict(use_dora=True), "REJECT(use_dora)"),
    (dict(bias="lora_only"), "REJECT(bias)"),
    (dict(rank_pattern={"k_proj": 8}), "REJECT(rank_pattern)"),
    (dict(alpha_pattern={"k_proj": 8}), "REJECT(alpha_pattern)"),
    (dict(modules_to_save=["lm_head"]), "REJECT(modules_to_save)"),
    (dict(peft_type="ADALORA"), "REJECT(peft_type)"),
    (dict(target_modules="all-linear"), "REJECT(target_modules)"),
    (dict(target_modules=[]), "REJECT(target_modules)"),
    (dict(target_modules=[3]), "REJECT(target_modules)"),
    (dict(target_modules=["lm_head"]), "REJECT(embedding)"),
    (dict(target_modules=["fc1"]), "REJECT(unknown_module)"),
    (dict(layers_to_transform="3"), "REJECT(layers_to_transform)"),
    (dict(layers_to_transform=[-1]), "REJECT(layers_to_transform)"),
    (dict(r=0), "REJECT(r)"),
    (dict(lora_alpha=0), "REJECT(lora_alpha)"),
    (dict(lora_alpha=-4.0), "REJECT(lora_alpha)"),
])
def test_peft_named_rejections(ad, over, tag):
    with pytest.raises(ad.AdapterRejected) as e:
        ad.parse_peft_adapter_config(json.dumps(base_json(**over)))
    assert e.value.status == ad.ERR_REJECT and tag in e.value.reason, e.value.reason


@pytest.mark.parametrize("m", ["in_proj_qkvz", "in_proj_ba", "in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b", "out_proj", "conv1d"])
def test_peft_gdn_modules_rejected(ad, m):
    with pytest.raises(ad.AdapterRejected) as e:
        ad.parse_peft_adapter_config(json.dumps(base_json(target_modules=["k_proj", m])))
    assert "REJECT(gdn)" in e.value.reason


def test_peft_malformed_documents(ad):
    for text in ("", "[1, 2]", "{\"r\": 8", json.dumps({"lora_alpha": 8, "target_modules": ["k_proj"], "use_rslora": False})):
        with pytest.raises(ad.AdapterRejected) as e:
            ad.parse_peft_adapter_config(text)
        assert e.value.status == -1


# ---- keys and identities ----------------------------------------------------------------------------
def test_classify_key(ad):
    fa = [1 if i in HOLO_FULL else 0 for i in range(HOLO_LAYERS)]
    ok = {"base_model.model.model.language_model.layers.3.self_attn.k_proj.lora_A.weight": (3, 1, 0),
          "base_model.model.model.layers.7.self_attn.o_proj.lora_B.weight": (7, 3, 1),
          "base_model.model.model.layers.23.mlp.down_proj.lora_B.weight": (23, 6, 1),
          "base_model.model.model.layers.11.self_attn.q_proj.lora_A.weight": (11, 0, 0),
          "base_model.model.model.layers.15.mlp.gate_proj.lora_A.weight": (15, 4, 0)}
    for k, want in ok.items():
        assert ad.classify_key(k, HOLO_LAYERS, fa) == want
    bad = {"model.layers.3.self_attn.k_proj.weight": "REJECT[not-peft-key]",
           "base_model.model.model.embed_tokens.lora_embedding_A": "REJECT[embedding-lora]",
           "base_model.model.model.layers.3.self_attn.k_proj.lora_A.default.weight": "REJECT[unrecognized-tensor]",
           "base_model.model.lm_head.lora_A.weight": "REJECT[non-layer-module]",
           "base_model.model.model.layers.x3.self_attn.k_proj.lora_A.weight": "REJECT[malformed-layer-index]",
           "base_model.model.model.layers.99.self_attn.k_proj.lora_A.weight": "REJECT[layer-out-of-range]",
           "base_model.model.model.layers.3.linear_attn.in_proj_qkv.lora_A.weight": "REJECT[gdn-target]",
           "base_model.model.model.layers.3.self_attn.rotary.lora_A.weight": "REJECT[unsupported-module]",
           "base_model.model.model.layers.4.mlp.down_proj.lora_A.weight": "REJECT[non-full-attention-layer]"}
    for k, tag in bad.items():
        with pytest.raises(ad.AdapterRejected) as e:
            ad.classify_key(k, HOLO_LAYERS, fa)
        assert tag in e.value.reason, (k, e.value.reason)
    assert ad.classify_key("base_model.model.model.layers.4.mlp.down_proj.lora_A.weight", HOLO_LAYERS, None) == (4, 6, 0)


def _fnv(name, gen):
    h = 0xcbf29ce484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    if gen:
        for b in struct.pack("<Q", gen):
            h = ((h ^ b) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return h or 1


def test_adapter_id_hash(ad):
    for name in ("sparky", "vega", "", "anything"):
        for gen in (0, 1, 2, 1 << 40):
            assert ad.adapter_id_hash(name, gen) == _fnv(name, gen) != 0
    assert ad.adapter_id_hash("sparky", 0) != ad.adapter_id_hash("vega", 0)
    assert len({ad.adapter_id_hash("sol", g) for g in range(3)}) == 3


def test_convert_to_bf16_matches_round_to_nearest_even(ad, oracle):
    rng = np.random.default_rng(5)
    f32 = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 3,
                          np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, np.inf, -np.inf, 1e-40, 3.3e38, np.nan], np.float32)])
    want = np.array([oracle.lib().orc_f32_to_bf16(float(v)) for v in f32], dtype=np.uint16)
    got = ad.convert_to_bf16("F32", f32)
    fin = ~np.isnan(f32)
    assert np.array_equal(got[fin], want[fin]) and (got[~fin] & 0x7FC0 == 0x7FC0).all()
    f16 = np.concatenate([rng.standard_normal(4096).astype(np.float16), np.array([6e-8, 6.1e-5, 65504, -0.0, np.inf], np.float16)])
    got16 = ad.convert_to_bf16("F16", f16)
    want16 = np.array([oracle.lib().orc_f32_to_bf16(float(v)) for v in f16.astype(np.float32)], dtype=np.uint16)
    assert np.array_equal(got16, want16)
    bf = rng.integers(0, 1 << 16, 100).astype(np.uint16)
    assert np.array_equal(ad.convert_to_bf16("BF16", bf), bf)


# ---- a synthetic PEFT adapter -------------------------------------------------------------------------
def write_safetensors(tensors):
    """{name: (dtype string, numpy array)} -> file bytes."""
    header, blobs, off = {}, [], 0
    for name, (dt, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw); off += len(raw)
    header["__metadata__"] = {"format": "pt"}
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    return struct.pack("<Q", len(h)) + h + b"".join(blobs)


DIMS = dict(hidden_size=64, intermediate_size=160, num_attention_heads=4, num_key_value_heads=2, head_dim=16)
N_LAYERS, FULL = 6, [1, 4]


def tiny_adapter(seed, r, dtype="F32", modules=("k_proj", "v_proj", "o_proj", "down_proj"), layers=FULL, prefix="model.language_model"):
    rng = np.random.default_rng(seed)
    shape = {"q_proj": (64, 64), "k_proj": (32, 64), "v_proj": (32, 64), "o_proj": (64, 64), "gate_proj": (160, 64),
             "up_proj": (160, 64), "down_proj": (64, 160)}
    path = {"q_proj": "self_attn", "k_proj": "self_attn", "v_proj": "self_attn", "o_proj": "self_attn",
            "gate_proj": "mlp", "up_proj": "mlp", "down_proj": "mlp"}
    np_dt = {"F32": np.float32, "F16": np.float16}[dtype]
    t = {}
    for l in layers:
        for m in modules:
            out_dim, in_dim = shape[m]
            key = f"base_model.model.{prefix}.layers.{l}.{path[m]}.{m}"
            t[key + ".lora_A.weight"] = (dtype, (rng.standard_normal((r, in_dim)) * 0.1).astype(np_dt))
            t[key + ".lora_B.weight"] = (dtype, (rng.standard_normal((out_dim, r)) * 0.1).astype(np_dt))
    cfg = base_json(r=r, lora_alpha=2 * r, target_modules=list(modules), layers_to_transform=list(layers))
    return json.dumps(cfg), t


def make_registry(atlas, ad, max_loras=4, max_rank=16, pool_base=0x7000_0000_0000):
    from atlas_b200 import registry
    cfg = registry.model_dims(**DIMS, num_full_attention_layers=len(FULL))
    fa = [1 if i in FULL else 0 for i in range(N_LAYERS)]
    return ad.AdapterRegistry(cfg, N_LAYERS, fa, max_loras, max_rank, pool_base=pool_base), cfg


@pytest.mark.parametrize("dtype", ["F32", "F16"])
def test_load_packs_the_slot_as_the_pool_layout_says(atlas, ad, dtype):
    reg, cfg = make_registry(atlas, ad)
    cj, tens = tiny_adapter(1, r=8, dtype=dtype)
    image = reg.load_adapter(2, "alpha", cj, write_safetensors(tens))
    assert image.size == reg.slot_bytes == atlas.pool_slot_bytes(cfg, 16)
    want = np.zeros_like(image)
    mods = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
    for name, (dt, arr) in tens.items():
        layer, module, ab = ad.classify_key(name, N_LAYERS, [1 if i in FULL else 0 for i in range(N_LAYERS)])
        a_off, b_off = atlas.module_slot_offsets(cfg, 16, FULL.index(layer), module)
        out_dim, in_dim = atlas.module_dims(cfg, module)
        bits = ad.convert_to_bf16(dt, arr)
        if ab == 0:
            want[a_off:a_off + 8 * in_dim * 2] = bits.view(np.uint8).reshape(-1)
        else:
            blk = np.zeros((out_dim, 16), dtype=np.uint16)
            blk[:, :8] = bits
            want[b_off:b_off + out_dim * 16 * 2] = blk.view(np.uint8).reshape(-1)
    assert np.array_equal(image, want)
    # tables: slot 2 present for the four modules it carries on both adapted layers, null elsewhere
    for layer in FULL:
        for module in range(7):
            a, b = reg.route_tables(layer, module)
            carried = mods[module] in ("k_proj", "v_proj", "o_proj", "down_proj")
            a_off, b_off = atlas.module_slot_offsets(cfg, 16, FULL.index(layer), module)
            assert a[2] == (reg.pool_base + 2 * reg.slot_bytes + a_off if carried else 0)
            assert b[2] == (reg.pool_base + 2 * reg.slot_bytes + b_off if carried else 0)
            assert not a[[0, 1, 3]].any() and not b[[0, 1, 3]].any()
    assert list(reg.scale_table()) == [0.0, 0.0, 2.0, 0.0] and list(reg.rank_table()) == [0, 0, 8, 0]
    with pytest.raises(atlas.AtlasError):
        reg.route_tables(0, 1)                      # layer 0 carries no LoRA
    assert reg.slot_of("alpha") == 2 and reg.slot_of("nobody") is None


def test_load_time_audit_rejections(atlas, ad):
    reg, _ = make_registry(atlas, ad)

    def rejected(cj, tens, tag):
        with pytest.raises(ad.AdapterRejected) as e:
            reg.load_adapter(0, "x", cj, write_safetensors(tens))
        assert tag in e.value.reason, e.value.reason
    cj, tens = tiny_adapter(2, r=32)
    rejected(cj, tens, "REJECT[rank-exceeds-pool]")
    cj, tens = tiny_adapter(2, r=8)
    t2 = dict(tens); t2.pop(next(k for k in t2 if k.endswith("lora_B.weight")))
    rejected(cj, t2, "REJECT[unpaired-tensor]")
    t2 = dict(tens); k = next(k for k in t2 if k.endswith("k_proj.lora_A.weight")); t2[k] = ("F32", np.zeros((8, 48), np.float32))
    rejected(cj, t2, "REJECT[shape-mismatch]")
    t2 = dict(tens); k = next(k for k in t2 if k.endswith("k_proj.lora_B.weight")); t2[k] = ("F32", np.zeros((32, 4), np.float32))
    rejected(cj, t2, "REJECT[shape-mismatch]")
    rejected(cj, {}, "REJECT[empty-adapter]")
    t2 = dict(tens); t2["base_model.model.model.layers.2.mlp.down_proj.lora_A.weight"] = ("F32", np.zeros((8, 160), np.float32))
    rejected(cj, t2, "REJECT[non-full-attention-layer]")
    t2 = dict(tens); t2["base_model.model.model.norm.weight"] = ("F32", np.zeros(64, np.float32))
    rejected(cj, t2, "REJECT[unrecognized-tensor]")
    cfg_more = json.dumps({**json.loads(cj), "target_modules": ["k_proj", "v_proj", "o_proj", "down_proj", "gate_proj"]})
    rejected(cfg_more, tens, "REJECT[unmatched-target]")
    # the same (layer, module, A) under two key prefixes
    t2 = dict(tens); k = next(k for k in t2 if k.endswith("layers.1.self_attn.k_proj.lora_A.weight"))
    t2[k.replace("model.language_model", "model")] = t2[k]
    rejected(cj, t2, "REJECT[duplicate-tensor]")
    t2 = dict(tens); k = next(iter(t2)); t2[k] = ("I32", np.zeros(t2[k][1].shape, np.int32))
    rejected(cj, t2, "REJECT[dtype]")
    assert reg.slot_of("x") is None                   # nothing was installed by any of the refused loads


def test_lifecycle_reference_vectors(atlas, ad):
    """The acquire / release / generation vectors of the reference's registry tests, on a registry with two adapters."""
    reg, _ = make_registry(atlas, ad)
    cj, tens = tiny_adapter(3, r=8)
    raw = write_safetensors(tens)
    reg.load_adapters([("alpha", cj, raw), ("beta", cj, raw)])
    assert reg.slot_of("beta") == 1 and reg.slot_of("missing") is None
    ida, idb = ad.adapter_id_hash("alpha", 0), ad.adapter_id_hash("beta", 0)
    assert ida != idb and ida != 0
    assert reg.adapter_id_for_slot(0) == ida and reg.adapter_id_for_slot(1) == idb and reg.adapter_id_for_slot(-1) == ida
    assert reg.adapter_id_for_slot(99) == 0 and reg.adapter_id_for_slot(3) == 0          # out of range / placeholder
    reg.set_active(1)
    assert reg.acquire_slot(0) == 0 and reg.slot_ref_count(0) == 1 and reg.slot_ref_count(1) == 0
    assert reg.acquire_slot(-1) == 1 and reg.slot_ref_count(1) == 1                      # -1 resolves to the active slot
    assert reg.acquire_slot(0) == 0 and reg.slot_ref_count(0) == 2
    assert reg.slot_last_used(0) == 3 and reg.slot_last_used(1) == 2                     # strictly increasing ticks
    # a busy slot refuses a swap, and nothing about it changes
    with pytest.raises(ad.AdapterRejected) as e:
        reg.load_adapter(0, "gamma", cj, raw)
    assert e.value.status == ad.ERR_BUSY and "REFUSED" in e.value.reason and reg.slot_of("alpha") == 0 and reg.slot_generation(0) == 0
    reg.release_slot(0); assert reg.slot_ref_count(0) == 1
    reg.release_slot(0); assert reg.slot_ref_count(0) == 0
    reg.release_slot(1); assert reg.slot_ref_count(1) == 0
    reg.release_slot(0); assert reg.slot_ref_count(0) == 0                               # saturating
    assert reg.acquire_slot(99) == -1
    reg.release_slot(-1)
    assert reg.slot_ref_count(99) == 0
    # an idle slot takes the swap: same name, new contents, fresh identity
    reg.load_adapter(0, "alpha", cj, raw)
    assert reg.slot_generation(0) == 1 and reg.adapter_id_for_slot(0) == ad.adapter_id_hash("alpha", 1) != ida


def test_victim_selection_over_the_cache_region(atlas, ad):
    reg, _ = make_registry(atlas, ad, max_loras=4)
    cj, tens = tiny_adapter(4, r=8)
    raw = write_safetensors(tens)
    reg.load_adapters([("pinned0", cj, raw)])                  # slot 0 pinned; 1..3 are the cache
    assert reg.select_victim() == 1                            # a never-filled slot first
    for k, n in ((1, "c1"), (2, "c2"), (3, "c3")):
        reg.load_adapter(k, n, cj, raw)
        reg.touch_slot(k)
    assert reg.select_victim() == 1                            # least recently used idle slot
    reg.touch_slot(1)
    assert reg.select_victim() == 2
    r2 = reg.acquire_slot(2)
    assert reg.select_victim() == 3
    reg.acquire_slot(3); reg.acquire_slot(1)
    assert reg.select_victim() is None                         # every cache slot busy: pool full, retry later
    reg.release_slot(r2)
    assert reg.select_victim() == 2


# ---- the reference's own adapter fixture, where its checkout is present ---------------------------------
def _reference_dir():
    d = os.environ.get("ATLAS_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    return d if os.path.isdir(os.path.join(d, "test_data", "lora-holo-tiny")) else None


@pytest.mark.skipif(_reference_dir() is None, reason="needs a checkout of the reference beside the repository (its adapter fixture is not copied)")
def test_reference_adapter_fixture_all_pairs(atlas, ad, oracle):
    from atlas_b200 import registry
    g = np.load(os.path.join(GOLDEN, "peft_holo_tiny_pairs.npz"))
    cfg = registry.model_dims(hidden_size=1024, intermediate_size=3584, num_attention_heads=8, num_key_value_heads=2, head_dim=256,
                              attn_gated=1, num_full_attention_layers=len(HOLO_FULL))
    fa = [1 if i in HOLO_FULL else 0 for i in range(HOLO_LAYERS)]
    reg = ad.AdapterRegistry(cfg, HOLO_LAYERS, fa, 2, 16, pool_base=1 << 40)
    image = reg.load_adapter_dir(0, "holo-tiny", os.path.join(_reference_dir(), "test_data", "lora-holo-tiny"))
    assert int(g["n_tensors"]) == 72 and reg.scale_table()[0] == 2.0 == float(g["scaling"]) and reg.rank_table()[0] == 8
    img16 = image.view(np.uint16)
    for key, total, abs_total, corner, shape in zip(g["keys"], g["sums"], g["abs_sums"], g["corners"], g["shapes"]):
        layer, module, _ = ad.classify_key(str(key) + ".lora_A.weight", HOLO_LAYERS, fa)
        out_dim, in_dim = atlas.module_dims(cfg, module)
        assert [out_dim, in_dim, 8] == list(shape)
        a_off, b_off = atlas.module_slot_offsets(cfg, 16, HOLO_FULL.index(layer), module)
        a = oracle.bf16_to_f32(img16[a_off // 2: a_off // 2 + 16 * in_dim].reshape(16, in_dim)).astype(np.float64)
        b = oracle.bf16_to_f32(img16[b_off // 2: b_off // 2 + out_dim * 16].reshape(out_dim, 16)).astype(np.float64)
        assert not a[8:].any() and not b[:, 8:].any()                      # pads are zero
        delta = 2.0 * (b @ a)
        assert np.isclose(delta.sum(), total, rtol=1e-9, atol=1e-9) and np.isclose(np.abs(delta).sum(), abs_total, rtol=1e-9)
        assert np.allclose(delta[:4, :4], corner, rtol=1e-12, atol=0)
