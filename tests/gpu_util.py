"""Helpers shared by the GPU parity tests: move a synthetic case to the device, call the C ABI, compare."""
import ctypes as C
import os

import numpy as np

RTOL, ATOL = 2e-2, 1e-2      # the tolerance the path's specification states for BF16 outputs


def to_dev(torch, a: np.ndarray):
    """numpy -> device tensor with the same bytes (uint16 travels as int16)."""
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits_from_dev(t) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def host_pool(oracle, case):
    pool = oracle.HostPool(case.K, case.N, case.max_rank, case.max_loras)
    for s, ad in enumerate(case.adapters):
        if ad is not None:
            pool.pack(s, ad.a, ad.b, ad.scale)
    return pool


def device_pool(torch, atlas, case):
    pool = atlas.LoraPool(case.K, case.N, case.max_rank, case.max_loras)
    for s, ad in enumerate(case.adapters):
        if ad is None:
            continue
        r = ad.rank
        pool.a_pool[s].zero_(); pool.b_pool[s].zero_()
        pool.a_pool[s, :r].copy_(to_dev(torch, ad.a).view(torch.bfloat16))
        pool.b_pool[s, :, :r].copy_(to_dev(torch, ad.b).view(torch.bfloat16))
        pool._a_host[s] = pool.a_pool[s].data_ptr()
        pool._b_host[s] = pool.b_pool[s].data_ptr()
        pool._scale_host[s] = ad.scale
        pool._rank_host[s] = r
    pool.refresh_tables()
    return pool


class DeviceCase:
    def __init__(self, torch, atlas, case, x_row_stride=None, out_row_stride=None):
        self.case = case
        xs = x_row_stride or case.K
        self.x_row_stride = xs
        self.out_row_stride = out_row_stride or case.N
        xh = np.zeros((case.M, xs), dtype=np.uint16)
        xh[:, :case.K] = case.x
        self.x = to_dev(torch, xh)
        self.packed = to_dev(torch, case.packed) if case.packed is not None else None
        self.scales = to_dev(torch, case.scales) if case.scales is not None else None
        self.w_bf16 = to_dev(torch, case.w_bf16) if case.w_bf16 is not None else None
        self.seq_slot = to_dev(torch, case.seq_slot.astype(np.int32))
        self.pool = device_pool(torch, atlas, case)
        self.lora_t = torch.zeros((case.M, case.max_rank), dtype=torch.int16, device="cuda")
        self.torch, self.atlas = torch, atlas

    def run(self, *, lora=True, with_ranks=True, flags=0, fill=0x7FC0, strided=True, lora_ws=False):
        """Returns (y bits [M, out_row_stride], variant). y is pre-filled with a NaN pattern."""
        torch, atlas, c = self.torch, self.atlas, self.case
        y = torch.full((c.M, self.out_row_stride), np.int16(np.uint16(fill).view(np.int16)), dtype=torch.int16, device="cuda")
        ws, ws_bytes = None, 0
        if flags & atlas.FLAG_ACT_FP4:
            ws_bytes = atlas.act_fp4_ws_bytes(c.M, c.K)
        if lora_ws:                                        # room for the shrink's activation tiles (after the FP4 region)
            ws_bytes = (ws_bytes + 255) // 256 * 256 + atlas.lora_ws_bytes(c.M, c.max_loras, c.max_rank)
        if ws_bytes:
            ws = self.ws = torch.full((ws_bytes,), 0xA5, dtype=torch.uint8, device="cuda")
        d = atlas.make_linear_desc(ws=ws, ws_bytes=ws_bytes,
            x=self.x, m=c.M, k=c.K, n=c.N, y=y, w_packed=self.packed, w_scale=self.scales, scale2=c.scale2,
            w_bf16=self.w_bf16, x_row_stride=self.x_row_stride, out_row_stride=self.out_row_stride,
            seq_slot=self.seq_slot if lora else None, route=self.pool.route(with_ranks, strided) if lora else None,
            lora_t=self.lora_t if lora else None, flags=flags)
        variant = atlas.nvfp4_lora_linear(d)
        torch.cuda.synchronize()
        return bits_from_dev(y), variant


def ideal(oracle, case, rows=None, cols=None, lora=True, use_ranks=True, act_fp4=False):
    kw = dict(packed=case.packed, scales=case.scales, scale2=case.scale2, w_bf16=case.w_bf16, act_fp4=act_fp4)
    if lora:
        kw.update(seq_slot=case.seq_slot, pool=host_pool(oracle, case), use_ranks=use_ranks)
    return oracle.fused_linear_f32(case.x, case.M, case.N, case.K, rows=rows, cols=cols, **kw)


def assert_close(oracle, got_bits, want_f32, what=""):
    got = oracle.bf16_to_f32(np.ascontiguousarray(got_bits))
    assert np.isfinite(got).all(), f"{what}: non-finite output (unwritten or corrupt elements)"
    err = np.abs(got - want_f32)
    lim = ATOL + RTOL * np.abs(want_f32)
    bad = err > lim
    if bad.any():
        i = np.unravel_index(np.argmax(err - lim), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} outside rtol {RTOL} / atol {ATOL}; worst at {i}: "
                             f"got {got[i]} want {want_f32[i]}")


# ---- launching the reference's own kernels (compiled to cubins under oracle/_ref) -----------------
class RefModule:
    def __init__(self, name):
        import oracle.oracle_ctypes as oc
        path = os.path.join(oc.REF_DIR, name + ".cubin")
        self.cu = C.CDLL("libcuda.so.1")
        self.mod = C.c_void_p()
        data = open(path, "rb").read()
        rc = self.cu.cuModuleLoadData(C.byref(self.mod), data)
        assert rc == 0, f"cuModuleLoadData({name}) -> {rc}"

    def launch(self, func, grid, block, args, stream=0):
        fn = C.c_void_p()
        rc = self.cu.cuModuleGetFunction(C.byref(fn), self.mod, func.encode())
        assert rc == 0, f"cuModuleGetFunction({func}) -> {rc}"
        holders = []
        for a in args:
            if isinstance(a, float):
                holders.append(C.c_float(a))
            elif isinstance(a, tuple):                     # ("u32", v)
                holders.append(C.c_uint32(a[1]))
            else:
                holders.append(C.c_uint64(a))              # device address
        arr = (C.c_void_p * len(holders))(*[C.cast(C.byref(h), C.c_void_p) for h in holders])
        rc = self.cu.cuLaunchKernel(fn, grid[0], grid[1], grid[2], block[0], block[1], block[2], 0,
                                    C.c_void_p(stream), arr, None)
        assert rc == 0, f"cuLaunchKernel({func}) -> {rc}"


def ref_available():
    import oracle.oracle_ctypes as oc
    return os.path.exists(os.path.join(oc.REF_DIR, "lora_bgmv.cubin"))
