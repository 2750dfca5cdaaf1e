"""The give-up path of the kernels' bounded waits, exercised without hanging or faulting
anything: with the wait limit lowered to a few milliseconds, one tiny single-CTA GEMM is
launched whose producer announces but never issues the loads of one k-block (the library's
test aid). The consumer's wait on that stage must run out, the kernel must return through its
normal teardown (tensor memory freed), difb200_poll_status must report status 5 with the place,
and the next ordinary call must be bit-exact. The reference has no counterpart (its kernels
use unbounded barriers); its host-side error contract is DIF_BACKEND_EXECUTION_ERROR with text
(reference include/dif/backend/abi.h:22-30)."""
import numpy as np
import pytest

import oracle_bridge as ob
from helpers import bf16_normal, from_torch_bf16

pytestmark = pytest.mark.gpu


def _operands(rng, M, N, K):
    import torch
    x8 = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    w8 = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    xs = (rng.random(M, dtype=np.float32) * 1e-2 + 1e-3).astype(np.float32)
    ws = (rng.random(N, dtype=np.float32) * 1e-2 + 1e-3).astype(np.float32)
    t = lambda a: torch.from_numpy(a).cuda()
    return (x8, w8, xs, ws), (t(x8), t(w8), t(xs), t(ws))


@pytest.mark.parametrize("k_block", [0, 1])
def test_gemm_wait_runs_out_is_reported_and_recovered(k_block):
    import torch
    from diffusion_compiler_b200 import _lib, ops
    lib = _lib.lib()
    rng = np.random.default_rng(5)
    M, N, K = 128, 256, 384  # one 128x256 tile, three k-blocks, single-CTA form
    host, dev = _operands(rng, M, N, K)
    ops.linear_int8_scaled(*dev)  # a plain call first: one-time set-up is behind us
    ops.poll_status()
    lib.difb200_set_wait_limit_ns(5_000_000)  # 5 ms instead of 1.5 s
    try:
        lib.difb200_test_withhold_gemm_load(k_block)
        ops.linear_int8_scaled(*dev)      # result undefined; must return by itself
        torch.cuda.synchronize()          # no fault: the context stays usable
        with pytest.raises(_lib.Difb200Error) as info:
            ops.poll_status()
        assert info.value.status == 5 and "bounded device-side wait ran out" in str(info.value)
        assert "kernel 2" in str(info.value)
    finally:
        lib.difb200_set_wait_limit_ns(0)
    ops.poll_status()  # the words were cleared by the failing poll
    got = from_torch_bf16(ops.linear_int8_scaled(*dev))
    ops.poll_status()
    want = ob.orc().linear_int8_scaled(host[0], host[1], host[2], host[3])
    assert np.array_equal(got, want), "the call after a timed-out one is not bit-exact"


def test_exchange_flag_wait_runs_out_is_reported_and_recovered():
    """The one-CTA kernel that orders an attention launch behind the slices pushed by other ranks
    (direct exchange): with the flag set beforehand it returns at once; with a flag that nothing
    sets it gives up after its limit (10 ms here), which the status poll reports as status 5 with the
    place (kernel 5), and the device goes on working."""
    import torch
    from diffusion_compiler_b200 import _lib, ops
    lib = _lib.lib()
    assert lib.difb200_world_selftest_flags(10_000_000, 1) == 0, lib.difb200_last_error().decode()
    assert lib.difb200_world_selftest_flags(10_000_000, 0) == 5
    text = lib.difb200_last_error().decode()
    assert "bounded device-side wait ran out" in text and "kernel 5" in text
    ops.poll_status()  # cleared by the failing poll
    assert lib.difb200_world_selftest_flags(10_000_000, 1) == 0
    x = torch.arange(8, device="cuda")
    assert int(x.sum().item()) == 28
