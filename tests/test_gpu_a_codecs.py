"""NVFP4 codecs on the GPU, bit-exact against the oracle."""
import numpy as np
import pytest

from gpu_util import bits_from_dev, to_dev

pytestmark = pytest.mark.gpu


def test_dequant_every_scale_byte_and_code(cuda, atlas, oracle):
    torch = cuda
    N, K = 256, 32
    scales = np.repeat(np.arange(256, dtype=np.uint8)[:, None], K // 16, axis=1)
    packed = np.tile((np.arange(16, dtype=np.uint8) | (np.arange(16, dtype=np.uint8)[::-1] << 4)), (N, 1))
    for g in (1.0, 0.37, 2.0 ** -14):
        out = torch.zeros((N, K), dtype=torch.int16, device="cuda")
        atlas.dequant_nvfp4_to_bf16(to_dev(torch, packed), to_dev(torch, scales), out, g, N, K)
        torch.cuda.synchronize()
        want = oracle.dequant_nvfp4_to_bf16(packed, scales, g, N, K)
        assert np.array_equal(bits_from_dev(out), want), f"global={g}"


def test_dequant_random_tensor(cuda, atlas, oracle):
    torch = cuda
    from atlas_b200 import synth
    N, K = 300, 1024
    packed, scales = synth.make_nvfp4_weight(11, N, K)
    out = torch.zeros((N, K), dtype=torch.int16, device="cuda")
    atlas.dequant_nvfp4_to_bf16(to_dev(torch, packed), to_dev(torch, scales), out, 1.0, N, K)
    torch.cuda.synchronize()
    assert np.array_equal(bits_from_dev(out), oracle.dequant_nvfp4_to_bf16(packed, scales, 1.0, N, K))


def test_quantiser_bit_exact(cuda, atlas, oracle):
    torch = cuda
    from atlas_b200 import synth
    N, K = 64, 512
    w = synth.normal(5, N * K, 0.02).reshape(N, K)
    w[3] = 0.0                                  # an all-zero row: scale byte 0, codes 0
    w[4, :16] = 1e-8                            # a group far below the smallest scale
    w[5, 7] = 1e4                               # an outlier that saturates the scale
    wb = oracle.f32_to_bf16(w)
    gmax = oracle.lib().orc_nvfp4_global_absmax(wb.ctypes.data, wb.size)
    for scale2 in (gmax / (6.0 * 448.0), 1.0):
        packed = torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda")
        scales = torch.zeros((N, K // 16), dtype=torch.uint8, device="cuda")
        atlas.quantize_bf16_to_nvfp4(to_dev(torch, wb), packed, scales, float(np.float32(scale2)), N, K)
        torch.cuda.synchronize()
        wp, ws = oracle.quantize_bf16_to_nvfp4(wb, float(np.float32(scale2)), N, K)
        assert np.array_equal(scales.cpu().numpy(), ws)
        assert np.array_equal(packed.cpu().numpy(), wp)
