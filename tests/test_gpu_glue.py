"""GPU parity of the block glue operators, one DiffIR op at a time through the plugin C-ABI, against
the reference CPU executor (oracle/_ref).

Elementwise operators (ResidualGate, SwiGlu, Gelu, BiasAdd, Add, Multiply) must give the
reference's bits. The normalisations (RmsNorm, RmsNormModulate, LayerNormModulate,
QkNormPartialRope) sum a row in a different order than the reference's sequential fp32 loop
(reference src/runtime/cpu_executor.cpp:1051-1075, 1108-1148, 1200-1265, 1741-1837), so their
statistic can differ in the last bit: at most 0.2 % of the outputs may differ, by about one bf16
ulp of their terms, inside the bf16 bar of the path (rel-L2 <= 2e-3, cosine >= 0.9999)."""
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
    _one_ulp(got, want, o)


def test_rms_norm_modulate():
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
    _one_ulp(got, want, o)


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
    _one_ulp(got, want, o)


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
    _one_ulp(got, want, o)


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
