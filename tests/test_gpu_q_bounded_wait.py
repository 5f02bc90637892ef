"""The bounded wait that every kernel of the library is built on, made to run out in the safe form: a one-CTA
self-test kernel waits on a barrier that nothing arrives on, with a 2 ms limit, gives up, records the status code and
returns normally — no trap, no endless loop, and the context stays usable afterwards."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_wait_gives_up_records_the_status_and_the_context_survives(cuda, atlas, oracle):
    torch = cuda
    assert atlas.device_status() == 0
    first, second, waited_ns = atlas.selftest_bounded_wait(2_000_000)
    assert first == 1                      # the waiter's limit expired and its wait returned false
    assert second == 1                     # the other waiter left through the CTA's abort flag
    assert 2_000_000 <= waited_ns < 100_000_000
    assert atlas.device_status() == 0x100  # STATUS_WAIT_EXPIRED_PRODUCER, as the tcgen05 kernels would record it
    assert atlas.device_status() == 0      # reading clears the word
    # the context is alive: an ordinary call of the library still runs and is right
    from atlas_b200 import synth
    from gpu_util import DeviceCase, assert_close, ideal
    case = synth.make_case("after", M=64, K=512, N=256, ranks=[8, 16], max_rank=16, scale2=0.02, seed=3)
    y, variant = DeviceCase(torch, atlas, case).run()
    assert_close(oracle, y, ideal(oracle, case), "call after the expired wait")
    assert atlas.device_status() == 0


def test_selftest_refuses_long_limits(atlas, cuda):
    with pytest.raises(atlas.AtlasError):
        atlas.selftest_bounded_wait(10_000_000_000)
