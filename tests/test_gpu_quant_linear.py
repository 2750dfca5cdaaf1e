"""GPU parity of the W8A8 linear path (QuantizeInt8Rows + LinearInt8Scaled) against the CPU
oracle, through the C-ABI of libdifb200.so. INT8 codes, F32 scales and INT32 accumulators must
be bit-exact; bf16 outputs bit-exact without GELU and within rel-L2 <= 2e-3 with it."""
import numpy as np
import pytest

import oracle_bridge as ob
from helpers import activations, bf16_normal, cosine, from_torch_bf16, rel_l2, to_torch_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import torch
    from diffusion_compiler_b200 import ops as _ops
    assert torch.cuda.is_available()
    return _ops


def _quant_case(ops, rng, impl, rows, K, clip, residual, parts=None):
    import torch
    x = activations(rng, rows, K)
    x[rows // 2] = 0  # an all-zero row exercises the guarded scale
    if parts is None:
        parts = [K]
    cuts = np.cumsum([0] + list(parts))
    xs = [np.ascontiguousarray(x[:, cuts[i]:cuts[i + 1]]) for i in range(len(parts))]
    want = ob.orc().quantize_int8_rows(xs, impl, clip, residual)
    got = ops.quantize_int8_rows([to_torch_bf16(a) for a in xs], impl, clip, residual=residual)
    torch.cuda.synchronize()
    names = ["codes", "scales", "rcodes", "rscales"]
    for name, w, g in zip(names, want, got):
        g = g.cpu().numpy().reshape(w.shape)
        assert np.array_equal(w.view(np.uint8), g.view(np.uint8)), \
            "%s differ: impl=%d rows=%d K=%d (%d mismatches)" % (
                name, impl, rows, K, int(np.sum(w.view(np.uint8) != g.view(np.uint8))))


@pytest.mark.parametrize("impl", [1, 2, 3, 5, 6])
@pytest.mark.parametrize("rows,K", [(1, 256), (37, 768), (64, 3072), (5, 12288)])
def test_quantize_h256_bit_exact(ops, impl, rows, K):
    rng = np.random.default_rng(100 + impl)
    _quant_case(ops, rng, impl, rows, K, 1.0, False)
    _quant_case(ops, rng, impl, rows, K, 0.9995, True)


@pytest.mark.parametrize("impl", [4, 7])
@pytest.mark.parametrize("rows,K", [(3, 4096), (9, 12288)])
def test_quantize_h4096_bit_exact(ops, impl, rows, K):
    rng = np.random.default_rng(200 + impl)
    _quant_case(ops, rng, impl, rows, K, 1.0, False)
    _quant_case(ops, rng, impl, rows, K, 0.97, True)


@pytest.mark.parametrize("impl", [1, 2, 6])
def test_quantize_concatenated_inputs(ops, impl):
    rng = np.random.default_rng(7)
    _quant_case(ops, rng, impl, 19, 1024, 1.0, False, parts=[256, 512, 256])


def test_quantize_direct_per_token_head(ops):
    """Direct on [B,S,H,128]: the per-token-per-head quantisation of attention Q/K."""
    rng = np.random.default_rng(8)
    _quant_case(ops, rng, 1, 2 * 33 * 4, 128, 1.0, False)
    _quant_case(ops, rng, 1, 11, 100, 1.0, True)  # odd width: scalar path


@pytest.mark.parametrize("impl", [2, 3, 5, 6])
@pytest.mark.parametrize("N,K", [(5, 256), (40, 768), (64, 3072), (6, 12288)])
def test_weight_rows_with_mse_scale_bit_exact(ops, impl, N, K):
    """Weight-side packing (offline packer's encoder, reference tools/difflux2sample.cpp:2994-3059)
    with and without the MSE scale search (:1225-1259) against the CPU restatement."""
    import torch
    rng = np.random.default_rng(1000 * impl + K)
    w = ob.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    w[N // 2] = 0
    dw = torch.from_numpy(w.view(np.int16)).cuda().view(torch.bfloat16)
    for mse in (False, True):
        want_codes, want_scales = ob.orc().quantize_weight_rows(w, impl, mse=mse)
        codes, scales = ops.quantize_weight_rows(dw, impl, mse_scale=mse)
        torch.cuda.synchronize()
        assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_scales.view(np.uint32)), mse
        assert np.array_equal(codes.cpu().numpy(), want_codes), mse
    ops.poll_status()


@pytest.mark.parametrize("impl,mse", [(2, False), (3, True), (5, True), (6, False)])
def test_weight_rows_with_input_equalization(ops, impl, mse):
    """Input equalisation of the offline packer (reference tools/difflux2sample.cpp:2967-2990 for
    the vector, :3005-3014 for its use): codes and scales bit-exact given the same vector; the
    vector computed on the GPU within one bf16 ulp of the CPU restatement (libm's logf against
    CUDA's)."""
    import torch
    rng = np.random.default_rng(77 + impl)
    N, K = 48, 768
    gains = np.exp(rng.standard_normal(K) * 0.8).astype(np.float32)  # uneven column magnitudes
    w = ob.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32) * gains)
    eq = ob.orc().weight_equalization(w)
    dw = torch.from_numpy(w.view(np.int16)).cuda().view(torch.bfloat16)
    got_eq = ops.weight_equalization(dw)
    diff = np.abs(got_eq.view(torch.int16).cpu().numpy().astype(np.int32) - eq.view(np.int16).astype(np.int32))
    assert diff.max() <= 1 and np.count_nonzero(diff) <= K // 50
    assert ob.bf16_to_f32(eq).min() >= 0.5 and ob.bf16_to_f32(eq).max() <= 2.0 and len(np.unique(eq)) > 8
    deq = torch.from_numpy(eq.view(np.int16)).cuda().view(torch.bfloat16)
    want_codes, want_scales = ob.orc().quantize_weight_rows(w, impl, mse=mse, equalise=eq)
    codes, scales = ops.quantize_weight_rows(dw, impl, mse_scale=mse, input_scale=deq)
    torch.cuda.synchronize()
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_scales.view(np.uint32))
    assert np.array_equal(codes.cpu().numpy(), want_codes)
    plain_codes, _ = ob.orc().quantize_weight_rows(w, impl, mse=mse)
    assert not np.array_equal(plain_codes, want_codes)  # the vector does change the packing
    ops.poll_status()


def _weights(rng, N, K, impl):
    wf = bf16_normal(rng, (N, K), 0.02)
    return ob.orc().quantize_int8_rows([wf], impl, 1.0)


@pytest.fixture(params=["1", "2"], ids=["single-cta", "cta-pair"])
def gemm_form(request, monkeypatch):
    """Runs a test with the 128x256 single-CTA tiles and with the 256x256 CTA-pair (cta_group::2)
    tiles of the GEMM kernel."""
    monkeypatch.setenv("DIFB200_GEMM_CTAS", request.param)
    return request.param


@pytest.mark.parametrize("M,K,N", [(128, 256, 256), (100, 512, 200), (300, 1024, 520), (1024, 3072, 3072),
                                   (2000, 768, 1800)])
def test_linear_int8_scaled_bit_exact(ops, gemm_form, M, K, N):
    import torch
    rng = np.random.default_rng(M + N)
    ob.orc().lib.orc_set_threads(8)
    x = activations(rng, M, K)
    w8, ws = _weights(rng, N, K, 2)
    x8, xs = ob.orc().quantize_int8_rows([x], 2, 1.0)
    bias = bf16_normal(rng, (N,), 0.01)
    want, want_acc = ob.orc().linear_int8_scaled(x8, w8, xs, ws, want_acc=True)
    t = lambda a: torch.from_numpy(a).cuda()
    got, acc = ops.linear_int8_scaled(t(x8), t(w8), t(xs), t(ws), want_acc=True)
    torch.cuda.synchronize()
    assert np.array_equal(acc.cpu().numpy(), want_acc), "INT32 accumulators differ"
    assert np.array_equal(from_torch_bf16(got), want), "bf16 dequantised outputs differ"
    # + BiasAdd keeps the intermediate bf16 rounding of the two-op program
    want_b = ob.orc().bias_add(want, bias)
    got_b = ops.linear_int8_scaled(t(x8), t(w8), t(xs), t(ws), bias=to_torch_bf16(bias))
    assert np.array_equal(from_torch_bf16(got_b), want_b), "bias epilogue differs"
    # + Gelu(tanh): libm tanhf vs device tanhf, tolerance from the north star
    want_g = ob.orc().gelu_tanh(want_b)
    got_g = from_torch_bf16(ops.linear_int8_scaled(t(x8), t(w8), t(xs), t(ws), bias=to_torch_bf16(bias), gelu=True))
    a, b = ob.bf16_to_f32(got_g), ob.bf16_to_f32(want_g)
    assert rel_l2(a, b) <= 2e-3 and cosine(a, b) >= 0.9999
    assert np.mean(got_g != want_g) < 5e-3  # last-bit differences of tanh only
    ops.poll_status()


def test_w8a8_linear_end_to_end_single_layer(ops):
    """The single-layer benchmark case (M=1024, K=N=3072, H256ConvRot activations, bias): GPU quant + GEMM chained."""
    import torch
    rng = np.random.default_rng(0)
    ob.orc().lib.orc_set_threads(8)
    M, K, N = 1024, 3072, 3072
    x = activations(rng, M, K)
    w8, ws = _weights(rng, N, K, 2)
    bias = bf16_normal(rng, (N,), 0.01)
    x8, xs = ob.orc().quantize_int8_rows([x], 2, 1.0)
    want = ob.orc().bias_add(ob.orc().linear_int8_scaled(x8, w8, xs, ws), bias)
    codes, scales = ops.quantize_int8_rows([to_torch_bf16(x)], 2)
    got = ops.linear_int8_scaled(codes, torch.from_numpy(w8).cuda(), scales, torch.from_numpy(ws).cuda(),
                                 bias=to_torch_bf16(bias))
    torch.cuda.synchronize()
    assert np.array_equal(codes.cpu().numpy(), x8)
    assert np.array_equal(from_torch_bf16(got), want)
    ops.poll_status()


def test_w8a8_linear_single_call_matches_two_calls(ops):
    """difb200_w8a8_linear (caller scratch) == quantize + linear through their own entry points."""
    import torch
    rng = np.random.default_rng(3)
    M, K, N = 640, 1024, 768
    x = to_torch_bf16(activations(rng, M, K))
    w8, ws = _weights(rng, N, K, 2)
    w8, ws = torch.from_numpy(w8).cuda(), torch.from_numpy(ws).cuda()
    bias = to_torch_bf16(bf16_normal(rng, (N,), 0.01))
    codes, scales = ops.quantize_int8_rows([x], 2)
    want = ops.linear_int8_scaled(codes, w8, scales, ws, bias=bias, gelu=True)
    got = ops.w8a8_linear(x, w8, ws, bias=bias, gelu=True)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    ops.poll_status()


def test_weight_rows_equal_the_reference_packers_own_files(ops):
    """The GPU weight quantiser against whole runs of the reference's own offline packer
    (rewrite_named_linear_w8a8 of reference tools/difflux2sample.cpp; its cache tensors are the
    committed fixture tests/golden/packer_mse_scale.npz): given the packer's input-equalisation
    vector, the codes and scales are the packer's, bit for bit, with and without the MSE search."""
    import os
    import torch
    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "packer_mse_scale.npz"))
    keys = sorted({k.split("/")[0] for k in data.files if k.startswith("pack_")})
    assert len(keys) == 6
    for key in keys:
        impl = int(key.split("_")[1][4:])
        equalise, mse = key.split("_")[2] == "eq1", key.split("_")[3] == "mse1"
        w = np.ascontiguousarray(data[key + "/weight"])
        dw = torch.from_numpy(w.view(np.int16)).cuda().view(torch.bfloat16)
        deq = None
        if equalise:
            eq = np.ascontiguousarray(data[key + "/input_scale"]).reshape(-1)
            deq = torch.from_numpy(eq.view(np.int16)).cuda().view(torch.bfloat16)
        if impl in (4, 7) and (equalise or mse):
            # the 4096-wide variants are packed here without the two options only: refused, not approximated
            from diffusion_compiler_b200 import _lib
            with pytest.raises(_lib.Difb200Error) as info:
                ops.quantize_weight_rows(dw, impl, mse_scale=mse, input_scale=deq)
            assert info.value.status == 2
            continue
        codes, scales = ops.quantize_weight_rows(dw, impl, mse_scale=mse, input_scale=deq)
        torch.cuda.synchronize()
        assert np.array_equal(scales.cpu().numpy().view(np.uint32), data[key + "/scale_bits"]), key
        assert np.array_equal(codes.cpu().numpy(), data[key + "/codes"]), key
    ops.poll_status()
