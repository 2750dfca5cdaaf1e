"""difb200_w8a8_linear_static, the W8A8 linear for hosts that must not allocate device memory
(a runtime with a pre-planned arena, a serving loop that cannot afford the device
synchronisation an allocation implies). It keeps codes, row scales and status words in a fixed
array inside libdifb200.so. This test calls it through the C-ABI twice in a row -- the second
time on a smaller problem, so the array still holds the first call's bytes -- and requires the
outputs to equal difb200_w8a8_linear's (caller scratch) bit for bit, the bar of the other
linear tests. The file is named to be collected last."""
import ctypes as C

import numpy as np
import pytest

from helpers import activations, bf16_normal, to_torch_bf16

pytestmark = pytest.mark.gpu


def _call_static(lib, x, w8, ws, bias, gelu, out, check_previous):
    import torch
    M, K = x.shape
    N = w8.shape[0]
    flags = (1 if bias is not None else 0) | (2 if gelu else 0)
    p = lambda t: C.c_void_p(0 if t is None else t.data_ptr())
    return lib.difb200_w8a8_linear_static(p(x), p(w8), p(ws), p(bias), flags, 2, 1.0, M, N, K, p(out),
                                          check_previous, C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_linear_matches_caller_scratch_twice():
    import torch
    from diffusion_compiler_b200 import _lib, ops
    lib = _lib.lib()
    rng = np.random.default_rng(11)
    for call, (M, K, N, gelu) in enumerate([(1536, 3072, 1024, True), (200, 1024, 520, False)]):
        x = to_torch_bf16(activations(rng, M, K))
        wf = to_torch_bf16(bf16_normal(rng, (N, K), 0.02))
        w8, ws = ops.quantize_int8_rows([wf], 2)
        bias = to_torch_bf16(bf16_normal(rng, (N,), 0.01))
        want = ops.w8a8_linear(x, w8, ws, bias=bias, gelu=gelu)
        got = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call_static(lib, x, w8, ws, bias, gelu, got, check_previous=call)
        assert rc == 0, lib.difb200_last_error().decode()
        torch.cuda.synchronize()
        if call > 0:  # the array's address is resolved by now: a call must not change free memory
            assert torch.cuda.mem_get_info()[0] == free_before, "the static entry point allocated device memory"
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "call %d differs" % call
    # M = 0 with check_previous is the poll of this entry point: nothing is launched, 0 is returned
    empty = torch.empty(0, 1024, dtype=torch.bfloat16, device="cuda")
    assert _call_static(lib, empty, w8, ws, None, False, empty, check_previous=1) == 0


def test_static_scratch_rejects_oversize():
    import torch
    from diffusion_compiler_b200 import _lib
    lib = _lib.lib()
    M, K, N = 9216, 12288, 256  # 113 MB of codes: beyond the 40 MiB array
    x = torch.empty(1, dtype=torch.bfloat16, device="cuda")  # never touched: the call is rejected first
    rc = lib.difb200_w8a8_linear_static(C.c_void_p(x.data_ptr()), C.c_void_p(x.data_ptr()), C.c_void_p(x.data_ptr()),
                                        None, 0, 2, 1.0, M, N, K, C.c_void_p(x.data_ptr()), 0, None)
    assert rc == 2
    assert b"static array holds" in lib.difb200_last_error()
