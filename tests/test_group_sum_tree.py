"""The QKV consumer kernels sum a head's squares with fewer shuffles than the two-level butterfly of the reference kernels
(kernels/gb10/common/fused_k_norm_rope_cache.cu, fused_verify_elemwise.cu: a butterfly per group of lanes, then a butterfly
over the group sums held by lanes 0 .. N-1).  Their claim is that the result has the same bits, because only commutativity of
the FP32 addition is used.  This test replays both schedules lane by lane in numpy float32 and compares bits; the GPU parity
tests then compare the kernels themselves with the reference's."""
import numpy as np
import pytest

F = np.float32
LANES = np.arange(32)


def _butterfly(v):
    v = v.copy()
    for o in (16, 8, 4, 2, 1):
        v = (v + v[LANES ^ o]).astype(F)
    return v


def two_level(s):
    """s[g, lane]: per-lane partial of group g.  A butterfly per group; the group sums in lanes 0 .. N-1 of a zero-filled
    warp; one more butterfly."""
    mine = np.zeros(32, F)
    for g in range(s.shape[0]):
        mine[g] = _butterfly(s[g])[0]
    return _butterfly(mine)


def shared_shuffles(s):
    """The kernels' schedule: at offsets 16, 8, 4 a lane keeps one of two values and hands the other one to its partner (as
    long as more than one value is held), the remaining offsets are a plain butterfly, and the group sums — now spread over
    the lanes by the bits 16, 8, 4 — are combined highest index bit first."""
    n = s.shape[0]
    vals = [x.copy() for x in s]
    o, held = 16, n
    while held > 1:
        up = (LANES & o) != 0
        for k in range(held // 2):
            keep = np.where(up, vals[2 * k + 1], vals[2 * k])
            send = np.where(up, vals[2 * k], vals[2 * k + 1])
            vals[k] = (keep + send[LANES ^ o]).astype(F)
        held //= 2
        o //= 2
    v = vals[0]
    while o > 0:
        v = (v + v[LANES ^ o]).astype(F)
        o //= 2
    for groups, off in ((8, 4), (4, 8), (2, 16)):
        if n >= groups:
            v = (v + v[LANES ^ off]).astype(F)
    return v


@pytest.mark.parametrize("n_groups", [1, 2, 4, 8])
def test_shared_shuffle_sum_has_the_bits_of_the_two_level_butterfly(n_groups):
    rng = np.random.default_rng(n_groups)
    for trial in range(400):
        scale = rng.choice([1e-6, 1e-3, 1.0, 1e3, 1e6])
        s = (rng.standard_normal((n_groups, 32)) ** 2 * scale).astype(F)
        if n_groups > 1 and trial % 3 == 0:
            s[rng.integers(1, n_groups):] = 0            # a head narrower than the register array: absent groups are zero
        want, got = two_level(s), shared_shuffles(s)
        assert (want.view(np.uint32) == want.view(np.uint32)[0]).all()      # every lane ends with the same sum
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_mean_by_reciprocal_is_exact_for_power_of_two_heads():
    """total / head_dim and total * (1 / head_dim) round to the same float when head_dim is a power of two."""
    rng = np.random.default_rng(7)
    totals = np.concatenate([(rng.standard_normal(20000) ** 2 * 10.0 ** rng.integers(-30, 30, 20000)).astype(F),
                             np.array([0.0, 1e-45, 1e-40, 3e38], F)])
    for head_dim in (32, 64, 128, 256):
        assert np.array_equal((totals / F(head_dim)).view(np.uint32), (totals * F(1.0 / head_dim)).view(np.uint32))
