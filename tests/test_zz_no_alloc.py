"""The allocation-free entry point against the regular one.

`atlas_b200_nvfp4_lora_linear_noalloc` exists for callers that can launch kernels but cannot obtain
device memory themselves — a plug-in inside an engine that owns all device memory, or a call site where
the CUDA allocator must not be entered.  It takes the shrink scratch from a fixed array inside the
library instead of from the caller.  Here it is driven through the C ABI twice in a row (the second
call finds the first call's leftovers in the shared array) and must reproduce the regular entry
point's output, which the other test files have already checked against the oracle.

This file sorts last on purpose: a run that stops at the first failure has then executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

from gpu_util import ATOL, RTOL, DeviceCase, assert_close, bits_from_dev, ideal

pytestmark = pytest.mark.gpu


def _run_noalloc(torch, atlas, dc, fill):
    c = dc.case
    y = torch.full((c.M, c.N), int(np.uint16(fill).view(np.int16)), dtype=torch.int16, device="cuda")
    d = atlas.make_linear_desc(x=dc.x, m=c.M, k=c.K, n=c.N, y=y, w_packed=dc.packed, w_scale=dc.scales,
                               scale2=c.scale2, seq_slot=dc.seq_slot, route=dc.pool.route(), lora_t=None)
    assert not d.lora_t                                    # the caller hands over no scratch at all
    variant = atlas.nvfp4_lora_linear_noalloc(d)
    torch.cuda.synchronize()
    return bits_from_dev(y), variant


def test_noalloc_entry_matches_regular_entry_twice(cuda, atlas, oracle):
    torch = cuda
    from atlas_b200 import synth
    # two different problems back to back: the second call sees the first call's data in the shared array
    cases = [
        synth.make_case("na1", M=200, K=512, N=384, ranks=[32] * 6, max_rank=32, max_loras=8,
                        none_frac=0.15, scale2=0.02, b_std=0.1, seed=11),
        synth.make_case("na2", M=72, K=256, N=256, ranks=[8, 16, 4], max_rank=16, max_loras=4,
                        none_frac=0.3, scale2=0.02, b_std=0.1, seed=12),
    ]
    for rep, case in enumerate(cases):
        dc = DeviceCase(torch, atlas, case)
        want_bits, want_variant = dc.run()                 # regular entry, caller-owned scratch
        got_bits, variant = _run_noalloc(torch, atlas, dc, fill=0x7FC0)
        assert variant == want_variant == atlas.VARIANT_TCGEN05
        assert_close(oracle, got_bits, oracle.bf16_to_f32(want_bits), f"call {rep}: no-alloc vs regular entry")
        assert np.array_equal(got_bits, want_bits), f"call {rep}: same kernels, same inputs: bits must match"
        assert_close(oracle, got_bits, ideal(oracle, case), f"call {rep}: no-alloc vs oracle")
    assert atlas.device_status() == 0


def test_noalloc_entry_at_the_limit_and_on_the_cuda_core_path(cuda, atlas, oracle):
    """Both consumers of the built-in array: the tensor-core path with m * max_rank exactly at its capacity, and the
    CUDA-core path (K not a multiple of 256), each against the regular entry point."""
    torch = cuda
    from atlas_b200 import synth
    m_full = atlas.STATIC_SCRATCH_ELEMS // 64                          # 8192 rows x rank 64 = every element of the array
    cases = [
        synth.make_case("na_full", M=m_full, K=256, N=128, ranks=[64, 32], max_rank=64, max_loras=2, ids="segments", segments=9,
                        none_frac=0.1, scale2=0.02, b_std=0.1, seed=13),
        synth.make_case("na_simt", M=40, K=272, N=136, ranks=[8, 16], max_rank=16, max_loras=3, none_frac=0.2, scale2=0.02,
                        b_std=0.1, seed=14),
    ]
    for case, want_variant in zip(cases, (atlas.VARIANT_TCGEN05, atlas.VARIANT_SIMT)):
        dc = DeviceCase(torch, atlas, case)
        want_bits, variant = dc.run()
        assert variant == want_variant
        got_bits, variant = _run_noalloc(torch, atlas, dc, fill=0x7FC0)
        assert variant == want_variant
        assert np.array_equal(got_bits, want_bits)
    assert atlas.device_status() == 0


def test_noalloc_entry_rejects_oversized_scratch(cuda, atlas):
    torch = cuda
    d = atlas.LinearDesc()
    buf = torch.zeros(64, dtype=torch.int16, device="cuda")
    ptr = buf.data_ptr()
    d.x = d.y = d.w_packed = d.w_scale = d.seq_slot = d.a_table = d.b_table = d.scale_table = ptr
    d.k = d.x_row_stride = 256
    d.n = d.out_row_stride = 128
    d.max_loras, d.max_rank = 4, 64
    d.m = atlas.STATIC_SCRATCH_ELEMS // 64 + 1             # one row more than the array can hold
    rc = atlas.lib().atlas_b200_nvfp4_lora_linear_noalloc(C.byref(d), None)
    assert rc == -5                                        # refused before anything is launched
    torch.cuda.synchronize()
    assert atlas.lib().atlas_b200_nvfp4_lora_linear_noalloc(None, None) == -4
