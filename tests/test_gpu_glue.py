"""GPU parity of the block glue operators, one DiffIR op at a time through the plugin C-ABI, against
the reference CPU executor (oracle/_ref).

Elementwise operators (ResidualGate, SwiGlu, Gelu, BiasAdd, Add, Multiply) must give the
reference's bits, and so must the normalisations on bf16 rows (RmsNorm, RmsNormModulate,
LayerNormModulate, QkNormPartialRope, also fused with the ConvRot quantiser): their row statistic
is computed in the reference's sequential fp32 order (reference src/runtime/cpu_executor.cpp:
1051-1075, 1108-1148, 1200-1265, 1741-1837). With DIFB200_EXACT_NORM=0 the statistic is a parallel
sum whose last bit can differ: then at most 0.2 % of the outputs may differ, by about one bf16 ulp
of their terms, inside the bf16 bar of the path (rel-L2 <= 2e-3, cosine >= 0.9999)."""
import numpy as np
import pytest

import oracle_bridge as ob
from helpers import cosine, rel_l2

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")]

S, HIDDEN = 300, 3072


def _bf(rng, shape, std=1.0):
    return ob.f32_to_bf16((rng.standard_normal(shape) * std).astype(np.float32))


def _run(p, consts, inputs):
    from diffusion_compiler_b200 import plugin
    want, _ = ob.ref().run(p, {**consts, **inputs})
    ex = plugin.PluginExecutor(0)
    got, _ = ex.prepare(p, consts).run(inputs)
    ex.close()
    return got, want


def _exact(got, want, out):
    assert np.array_equal(got[out], want[out])


def _one_ulp(got, want, out):
    a, b = got[out].astype(np.int32), want[out].astype(np.int32)
    differing = np.count_nonzero(a != b)
    assert differing <= 0.002 * a.size, differing
    fa, fb = ob.bf16_to_f32(got[out]), ob.bf16_to_f32(want[out])
    # a last-bit difference of the row statistic moves a result by about one bf16 ulp of the terms
    # that were added to form it
    assert np.abs(fa - fb).max() <= 0.01 * np.abs(fb).max()
    assert rel_l2(fa, fb) <= 2e-3 and cosine(fa, fb) >= 0.9999


def _program():
    from diffusion_compiler_b200 import diffir
    return diffir, diffir.Program()


def test_rms_norm():
    d, p = _program()
    rng = np.random.default_rng(1)
    x = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Input)
    w = p.add_tensor(d.DType.BF16, [HIDDEN], d.Role.Constant)
    o = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Output)
    p.add_op(d.Opcode.RmsNorm, [x, w], [o], [d.Attribute.f64(d.AttrKey.Epsilon, 1e-6)])
    got, want = _run(p, {w: _bf(rng, [HIDDEN])}, {x: _bf(rng, [S, HIDDEN])})
    _exact(got, want, o)


@pytest.mark.parametrize("exact", [True, False])
def test_rms_norm_modulate(monkeypatch, exact):
    monkeypatch.setenv("DIFB200_EXACT_NORM", "1" if exact else "0")
    d, p = _program()
    rng = np.random.default_rng(2)
    x = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Input)
    w = p.add_tensor(d.DType.BF16, [HIDDEN], d.Role.Constant)
    a = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Input)
    b = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Input)
    o = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Output)
    p.add_op(d.Opcode.RmsNormModulate, [x, w, a, b], [o],
             [d.Attribute.f64(d.AttrKey.Epsilon, 1e-5), d.Attribute.u64(d.AttrKey.BlockSize, 128)])
    got, want = _run(p, {w: _bf(rng, [HIDDEN])},
                     {x: _bf(rng, [S, HIDDEN]), a: _bf(rng, [S, HIDDEN], 0.1), b: _bf(rng, [S, HIDDEN], 0.1)})
    (_exact if exact else _one_ulp)(got, want, o)


def test_layer_norm_modulate():
    d, p = _program()
    rng = np.random.default_rng(3)
    x = p.add_tensor(d.DType.BF16, [2, S, HIDDEN], d.Role.Input)
    w = p.add_tensor(d.DType.BF16, [HIDDEN], d.Role.Constant)
    bias = p.add_tensor(d.DType.BF16, [HIDDEN], d.Role.Constant)
    scale = p.add_tensor(d.DType.BF16, [2, 1, HIDDEN], d.Role.Input)
    shift = p.add_tensor(d.DType.BF16, [2, 1, HIDDEN], d.Role.Input)
    o = p.add_tensor(d.DType.BF16, [2, S, HIDDEN], d.Role.Output)
    p.add_op(d.Opcode.LayerNormModulate, [x, w, bias, scale, shift], [o],
             [d.Attribute.f64(d.AttrKey.Epsilon, 1e-6), d.Attribute.u64(d.AttrKey.BlockSize, 128)])
    got, want = _run(p, {w: _bf(rng, [HIDDEN]), bias: _bf(rng, [HIDDEN], 0.1)},
                     {x: _bf(rng, [2, S, HIDDEN]), scale: _bf(rng, [2, 1, HIDDEN], 0.1),
                      shift: _bf(rng, [2, 1, HIDDEN], 0.1)})
    _exact(got, want, o)


def test_layer_norm_modulate_quant_fused_in_the_plugin(monkeypatch):
    """LayerNormModulate -> QuantizeInt8Rows, which the plugin's planner runs as one kernel, against
    the reference executor's two ops and against the plugin's own two kernels: codes and scales are
    the reference's bit for bit either way (the row statistic follows the reference's order)."""
    from diffusion_compiler_b200 import plugin
    d, p = _program()
    rng = np.random.default_rng(31)
    x = p.add_tensor(d.DType.BF16, [2, S, HIDDEN], d.Role.Input)
    w = p.add_tensor(d.DType.BF16, [HIDDEN], d.Role.Constant)
    bias = p.add_tensor(d.DType.BF16, [HIDDEN], d.Role.Constant)
    scale = p.add_tensor(d.DType.BF16, [2, 1, HIDDEN], d.Role.Input)
    shift = p.add_tensor(d.DType.BF16, [2, 1, HIDDEN], d.Role.Input)
    h = p.add_tensor(d.DType.BF16, [2, S, HIDDEN])
    codes = p.add_tensor(d.DType.I8, [2, S, HIDDEN], d.Role.Output)
    scales = p.add_tensor(d.DType.F32, [2 * S], d.Role.Output)
    p.add_op(d.Opcode.LayerNormModulate, [x, w, bias, scale, shift], [h],
             [d.Attribute.f64(d.AttrKey.Epsilon, 1e-6), d.Attribute.u64(d.AttrKey.BlockSize, 128)])
    p.add_op(d.Opcode.QuantizeInt8Rows, [h], [codes, scales],
             [d.Attribute.u64(d.AttrKey.BlockSize, 256), d.Attribute.u64(d.AttrKey.Implementation, 2)])
    consts = {w: _bf(rng, [HIDDEN]), bias: _bf(rng, [HIDDEN], 0.1)}
    inputs = {x: _bf(rng, [2, S, HIDDEN]), scale: _bf(rng, [2, 1, HIDDEN], 0.1), shift: _bf(rng, [2, 1, HIDDEN], 0.1)}
    want, _ = ob.ref().run(p, {**consts, **inputs})
    runs, resident = [], []
    monkeypatch.setenv("DIFB200_BUFFER_REUSE", "0")  # residency per tensor, so that the saved tensor shows
    for fusion in ("1", "0"):
        monkeypatch.setenv("DIFB200_NORM_FUSION", fusion)
        ex = plugin.PluginExecutor(0)
        prepared = ex.prepare(p, consts)
        got, _ = prepared.run(inputs)
        resident.append(int(prepared.compile_telemetry.resident_bytes))
        ex.close()
        runs.append(got)
    assert resident[1] - resident[0] >= 2 * S * HIDDEN * 2  # the normalised tensor is not resident when fused
    for got in runs:
        assert np.array_equal(got[codes], want[codes])
        assert np.array_equal(got[scales].view(np.uint32), want[scales].view(np.uint32))


def test_qk_norm_partial_rope():
    d, p = _program()
    rng = np.random.default_rng(4)
    heads, dim, rotary = 4, 128, 96
    x = p.add_tensor(d.DType.BF16, [S, heads, dim], d.Role.Input)
    w = p.add_tensor(d.DType.BF16, [dim], d.Role.Constant)
    c = p.add_tensor(d.DType.BF16, [S, rotary], d.Role.Constant)
    s = p.add_tensor(d.DType.BF16, [S, rotary], d.Role.Constant)
    o = p.add_tensor(d.DType.BF16, [S, heads, dim], d.Role.Output)
    p.add_op(d.Opcode.QkNormPartialRope, [x, w, c, s], [o],
             [d.Attribute.f64(d.AttrKey.Epsilon, 1e-5), d.Attribute.u64(d.AttrKey.RotaryDim, rotary),
              d.Attribute.u64(d.AttrKey.BlockSize, 128)])
    angle = rng.uniform(0, 6.28, [S, rotary]).astype(np.float32)
    got, want = _run(p, {w: _bf(rng, [dim]), c: ob.f32_to_bf16(np.cos(angle)), s: ob.f32_to_bf16(np.sin(angle))},
                     {x: _bf(rng, [S, heads, dim])})
    _exact(got, want, o)


@pytest.mark.parametrize("interleaved,rotary,table_f32", [(False, 96, False), (True, 128, True), (False, 64, False)])
def test_qk_norm_rope_quant_matches_the_two_reference_ops(interleaved, rotary, table_f32):
    """difb200_qk_norm_rope_quant (one kernel) against the reference executor running
    QkNormPartialRope and then QuantizeInt8Rows(Direct) on its output: codes and scales bit for bit,
    written into the tail of a longer destination (the in-place slice and concat forms of the
    kernel are exercised by the MMDiT block tests)."""
    import ctypes as C
    import torch
    from diffusion_compiler_b200 import _lib
    d, p = _program()
    rng = np.random.default_rng(7)
    tokens, heads, dim = 70, 3, 128
    x = p.add_tensor(d.DType.BF16, [tokens, heads, dim], d.Role.Input)
    w = p.add_tensor(d.DType.BF16, [dim], d.Role.Constant)
    width = rotary // 2 if interleaved else rotary
    tdt = d.DType.F32 if table_f32 else d.DType.BF16
    c = p.add_tensor(tdt, [tokens, width], d.Role.Constant)
    s = p.add_tensor(tdt, [tokens, width], d.Role.Constant)
    r = p.add_tensor(d.DType.BF16, [tokens, heads, dim])
    codes = p.add_tensor(d.DType.I8, [tokens, heads, dim], d.Role.Output)
    scales = p.add_tensor(d.DType.F32, [tokens * heads], d.Role.Output)
    attrs = [d.Attribute.f64(d.AttrKey.Epsilon, 1e-5), d.Attribute.u64(d.AttrKey.RotaryDim, rotary),
             d.Attribute.u64(d.AttrKey.BlockSize, 128)]
    if interleaved:
        attrs += [d.Attribute.u64(d.AttrKey.Implementation, 2), d.Attribute.u64(d.AttrKey.RotaryLayout, 1)]
    p.add_op(d.Opcode.QkNormPartialRope, [x, w, c, s], [r], attrs)
    p.add_op(d.Opcode.QuantizeInt8Rows, [r], [codes, scales],
             [d.Attribute.u64(d.AttrKey.BlockSize, 256), d.Attribute.u64(d.AttrKey.Implementation, 1)])
    angle = rng.uniform(0, 6.28, [tokens, width]).astype(np.float32)
    cos_t, sin_t = np.cos(angle), np.sin(angle)
    if not table_f32:
        cos_t, sin_t = ob.f32_to_bf16(cos_t), ob.f32_to_bf16(sin_t)
    xv, wv = _bf(rng, [tokens, heads, dim]), _bf(rng, [dim])
    want, _ = ob.ref().run(p, {w: wv, c: cos_t, s: sin_t, x: xv})
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    dense, dw = t(xv.view(np.int16)), t(wv.view(np.int16))
    dc, ds = t(cos_t if table_f32 else cos_t.view(np.int16)), t(sin_t if table_f32 else sin_t.view(np.int16))
    lead = 5  # destination starts 5 tokens into a longer sequence
    out_codes = torch.zeros((tokens + lead, heads, dim), dtype=torch.int8, device="cuda")
    out_scales = torch.zeros((tokens + lead) * heads, dtype=torch.float32, device="cuda")
    L = _lib.lib()
    ptr = lambda tensor: C.c_void_p(tensor.data_ptr())
    _lib.check(L.difb200_qk_norm_rope_quant(ptr(dense), ptr(dw), ptr(dc), ptr(ds), None, ptr(out_codes[lead:]),
                                            ptr(out_scales[lead * heads:]), 1 if table_f32 else 2, tokens, heads,
                                            rotary, width, tokens, tokens, 0, 1e-5, 1 if interleaved else 0, None))
    torch.cuda.synchronize()
    assert np.array_equal(out_codes[lead:].cpu().numpy(), want[codes])
    assert np.array_equal(out_scales[lead * heads:].cpu().numpy().view(np.uint32), want[scales].view(np.uint32))
    assert torch.count_nonzero(out_codes[:lead]) == 0


@pytest.mark.parametrize("impl,weighted", [(2, True), (3, False)])
def test_rms_norm_modulate_quant_against_the_two_reference_ops(impl, weighted):
    """difb200_rms_norm_modulate_quant (the row statistic in the reference's order, then one kernel
    that normalises, modulates, rotates and quantises) against the reference executor running
    RmsNormModulate and QuantizeInt8Rows: codes and scales bit for bit."""
    import torch
    from diffusion_compiler_b200 import ops
    d, p = _program()
    rng = np.random.default_rng(9 + impl)
    rows, cols = 200, 1536
    x = p.add_tensor(d.DType.BF16, [rows, cols], d.Role.Input)
    ins = [x]
    consts = {}
    if weighted:
        w = p.add_tensor(d.DType.BF16, [cols], d.Role.Constant)
        ins.append(w)
        consts[w] = _bf(rng, [cols])
    a = p.add_tensor(d.DType.BF16, [rows, cols], d.Role.Input)
    b = p.add_tensor(d.DType.BF16, [rows, cols], d.Role.Input)
    h = p.add_tensor(d.DType.BF16, [rows, cols])
    codes = p.add_tensor(d.DType.I8, [rows, cols], d.Role.Output)
    scales = p.add_tensor(d.DType.F32, [rows], d.Role.Output)
    p.add_op(d.Opcode.RmsNormModulate, ins + [a, b], [h],
             [d.Attribute.f64(d.AttrKey.Epsilon, 1e-5), d.Attribute.u64(d.AttrKey.BlockSize, 128)])
    p.add_op(d.Opcode.QuantizeInt8Rows, [h], [codes, scales],
             [d.Attribute.u64(d.AttrKey.BlockSize, 256), d.Attribute.u64(d.AttrKey.Implementation, impl)])
    xv, av, bv = _bf(rng, [rows, cols]), _bf(rng, [rows, cols], 0.1), _bf(rng, [rows, cols], 0.1)
    want, _ = ob.ref().run(p, {**consts, x: xv, a: av, b: bv})
    t = lambda arr: torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).cuda().view(torch.bfloat16)
    got_codes, got_scales = ops.rms_norm_modulate_quant(t(xv), t(consts[ins[1]]) if weighted else None, t(av), t(bv),
                                                        1e-5, impl)
    torch.cuda.synchronize()
    ops.poll_status()
    gc, gs = got_codes.cpu().numpy().astype(np.int32), got_scales.cpu().numpy()
    wc, ws = want[codes].astype(np.int32), want[scales]
    assert np.array_equal(gc, wc), (np.abs(gc - wc).max(), np.mean(gc != wc))
    assert np.array_equal(gs.view(np.uint32), ws.view(np.uint32))


def test_residual_gate_swiglu_gelu_bits():
    d, p = _program()
    rng = np.random.default_rng(5)
    x = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Input)
    y = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Input)
    g = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Input)
    wide = p.add_tensor(d.DType.BF16, [S, 2 * HIDDEN], d.Role.Input)
    gated = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Output)
    act = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Output)
    gelu = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Output)
    total = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Output)
    product = p.add_tensor(d.DType.BF16, [S, HIDDEN], d.Role.Output)
    p.add_op(d.Opcode.ResidualGate, [x, y, g], [gated])
    p.add_op(d.Opcode.SwiGlu, [wide], [act])
    p.add_op(d.Opcode.Gelu, [x], [gelu], [d.Attribute.u64(d.AttrKey.Approximation, 1)])
    p.add_op(d.Opcode.Add, [x, y], [total])
    p.add_op(d.Opcode.Multiply, [x, y], [product])
    got, want = _run(p, {}, {x: _bf(rng, [S, HIDDEN], 2.0), y: _bf(rng, [S, HIDDEN]), g: _bf(rng, [S, HIDDEN], 0.3),
                             wide: _bf(rng, [S, 2 * HIDDEN])})
    for out in (gated, act, gelu, total, product):
        _exact(got, want, out)
