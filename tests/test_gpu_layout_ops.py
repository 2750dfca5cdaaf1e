"""GPU parity of the rotary, mask and layout operators of a DiT block, one program through the
plugin C-ABI, bit for bit against the reference CPU executor (oracle/_ref) and against the
known answers the reference's own unit test holds for them.

The first test restates the program and the input data of the reference's
test_krea2_rotary_layout_mask_and_broadcast_oracle (reference tests/dif_tests.cpp:1468-1613:
RotaryFrequency with three position axes, interleaved RotaryApply, BooleanMaskToBias in both
forms, Slice -> Reshape -> BroadcastTo -> Sigmoid, Concat) without its Permute, which is outside
this backend's operator subset. The expected cosine table and rotary bits are the creator
values that test compares with. The second test runs the same operators, plus AffineLastDim,
Cast and Fill (verifier rules reference src/ir/verify.cpp:245-265, 521-527, 562-570), on shapes
large enough to leave a single CTA, with odd tails."""
import numpy as np
import pytest

import oracle_bridge as ob

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")]

CREATOR_COSINE = np.array([
    1.0, 1.0, 1.0, 1.0, 1.0, 0.5403022766113281, -0.416146844625473, 0.9980006814002991, 1.0,
    -0.416146844625473, -0.9899924993515015, 0.9955033659934998, 1.0, -0.9899924993515015,
    -0.6536436080932617, 0.9920106530189514], np.float32)
CREATOR_ROTARY_BITS = np.array([
    16000, 48896, 16192, 49024, 16288, 49088, 16352, 49152, 15821, 15949, 16026, 16077, 16128, 16154, 16179,
    16205, 15949, 48794, 16163, 15753, 16069, 16215, 16219, 48985, 16230, 48973, 16226, 16007, 15904, 16159,
    16032, 48697, 48589, 15949, 48757, 48865, 16082, 48939, 48966, 16187, 16205, 16179, 48948, 16046, 48865,
    48759, 15938, 15859, 16256, 16128, 15761, 16125, 48887, 16350, 49110, 49199, 48717, 48589, 48231, 48587,
    15814, 48818, 16043, 16140], np.uint16)


def _bf(values, shape):
    return ob.f32_to_bf16(np.asarray(values, np.float32).reshape(shape))


def _run(p, consts, inputs):
    from diffusion_compiler_b200 import plugin
    want, _ = ob.ref().run(p, {**consts, **inputs})
    ex = plugin.PluginExecutor(0)
    prepared = ex.prepare(p, consts)
    got, _ = prepared.run(inputs)
    prepared.close()
    ex.close()
    return got, want


def test_reference_rotary_mask_layout_case_and_its_known_answers():
    from diffusion_compiler_b200 import diffir as d
    p = d.Program()
    F32, BF16, I32, BOOL = d.DType.F32, d.DType.BF16, d.DType.I32, d.DType.Bool
    IN, OUT, CONST = d.Role.Input, d.Role.Output, d.Role.Constant
    pos = p.add_tensor(F32, [1, 4, 3], IN)
    pair_axes = p.add_tensor(I32, [4], CONST)
    pair_idx = p.add_tensor(I32, [4], CONST)
    axis_dims = p.add_tensor(I32, [3], CONST)
    cos = p.add_tensor(F32, [1, 4, 4], OUT)
    sin = p.add_tensor(F32, [1, 4, 4], OUT)
    x = p.add_tensor(BF16, [1, 4, 2, 8], IN)
    rot = p.add_tensor(BF16, [1, 4, 2, 8], OUT)
    valid = p.add_tensor(BOOL, [1, 4], IN)
    bias = p.add_tensor(BF16, [1, 1, 4, 4], OUT)
    row = p.add_tensor(BF16, [1, 12], IN)
    sl = p.add_tensor(BF16, [1, 4], OUT)
    rs = p.add_tensor(BF16, [1, 1, 4], OUT)
    bc = p.add_tensor(BF16, [1, 4, 4], OUT)
    sg = p.add_tensor(BF16, [1, 4, 4], OUT)
    c_a = p.add_tensor(BF16, [2, 1, 3], IN)
    c_b = p.add_tensor(BF16, [2, 2, 3], IN)
    cat = p.add_tensor(BF16, [2, 3, 3], OUT)
    key_bias = p.add_tensor(BF16, [1, 1, 4, 4], OUT)
    p.add_op(d.Opcode.RotaryFrequency, [pos, pair_axes, pair_idx, axis_dims], [cos, sin],
             [d.Attribute.f64(d.AttrKey.Theta, 1000.0), d.Attribute.f64(d.AttrKey.Ntk, 1.0)])
    p.add_op(d.Opcode.RotaryApply, [x, cos, sin], [rot], [d.Attribute.u64(d.AttrKey.RotaryLayout, 1)])
    p.add_op(d.Opcode.BooleanMaskToBias, [valid], [bias])
    p.add_op(d.Opcode.Slice, [row], [sl], [d.Attribute.u64(d.AttrKey.Axis, 1), d.Attribute.u64(d.AttrKey.Start, 4)])
    p.add_op(d.Opcode.Reshape, [sl], [rs])
    p.add_op(d.Opcode.BroadcastTo, [rs], [bc])
    p.add_op(d.Opcode.Sigmoid, [bc], [sg])
    p.add_op(d.Opcode.Concat, [c_a, c_b], [cat], [d.Attribute.u64(d.AttrKey.Axis, 1)])
    p.add_op(d.Opcode.BooleanMaskToBias, [valid], [key_bias], [d.Attribute.boolean(d.AttrKey.MaskQueries, False)])
    consts = {pair_axes: np.array([0, 1, 2, 2], np.int32), pair_idx: np.array([0, 0, 0, 1], np.int32),
              axis_dims: np.array([2, 2, 4], np.int32)}
    inputs = {
        pos: np.array([0, 0, 0, 0, 1, 2, 0, 2, 3, 0, 3, 4], np.float32).reshape(1, 4, 3),
        x: _bf([.25, -.5, .75, -1., 1.25, -1.5, 1.75, -2., .1, .2, .3, .4, .5, .6, .7, .8,
                .2, -.3, .4, -.5, .6, -.7, .8, -.9, .9, -.8, .7, -.6, .5, -.4, .3, -.2,
                -.1, .2, -.3, .4, -.5, .6, -.7, .8, .8, .7, .6, .5, .4, .3, .2, .1,
                1., .5, 0., -.5, -1., -1.5, -2., -2.5, -.2, -.1, 0., .1, .2, .3, .4, .5], [1, 4, 2, 8]),
        valid: np.array([[1, 1, 0, 1]], np.uint8),
        row: _bf(np.arange(-4, 8), [1, 12]),
        c_a: _bf([1, 2, 3, 10, 11, 12], [2, 1, 3]),
        c_b: _bf([4, 5, 6, 7, 8, 9, 13, 14, 15, 16, 17, 18], [2, 2, 3]),
    }
    got, want = _run(p, consts, inputs)
    # the reference executor reproduces its own test's known answers here ...
    assert np.array_equal(want[cos].ravel(), CREATOR_COSINE)
    assert np.array_equal(want[rot].ravel(), CREATOR_ROTARY_BITS)
    # ... and the GPU path gives the same bytes for every output
    for tid in (cos, sin, rot, bias, sl, rs, bc, sg, cat, key_bias):
        assert np.array_equal(got[tid], want[tid]), "output tensor %d differs from the reference" % tid
    assert np.array_equal(got[cos].ravel(), CREATOR_COSINE)
    assert np.array_equal(got[rot].ravel(), CREATOR_ROTARY_BITS)
    assert np.array_equal(ob.bf16_to_f32(got[cat]).ravel(), np.arange(1, 19, dtype=np.float32))


def test_rotary_mask_layout_and_elementwise_ops_at_block_shapes():
    """Two position axes over a 14 x 19 image grid plus 37 text tokens, 6 heads of 128 (the
    producer chain of the attention benchmark case), a padded-text key mask in both bias forms,
    and the layout / elementwise operators on 303-token tensors: all bit-exact."""
    from diffusion_compiler_b200 import diffir as d
    rng = np.random.default_rng(9)
    B, S, H, D = 2, 37 + 14 * 19, 6, 128
    pairs = D // 2
    p = d.Program()
    F32, BF16, I32, BOOL, F16 = d.DType.F32, d.DType.BF16, d.DType.I32, d.DType.Bool, d.DType.F16
    IN, OUT, CONST = d.Role.Input, d.Role.Output, d.Role.Constant
    pos = p.add_tensor(F32, [B, S, 2], IN)
    pair_axes = p.add_tensor(I32, [pairs], CONST)
    pair_idx = p.add_tensor(I32, [pairs], CONST)
    axis_dims = p.add_tensor(I32, [2], CONST)
    cos = p.add_tensor(F32, [B, S, pairs], OUT)
    sin = p.add_tensor(F32, [B, S, pairs], OUT)
    x = p.add_tensor(BF16, [B, S, H, D], IN)
    rot = p.add_tensor(BF16, [B, S, H, D], OUT)
    valid = p.add_tensor(BOOL, [B, S], IN)
    bias_full = p.add_tensor(BF16, [B, 1, S, S], OUT)
    bias_keys = p.add_tensor(BF16, [B, 1, S, S], OUT)
    wide = p.add_tensor(BF16, [S, 3 * 384], IN)
    mid = p.add_tensor(BF16, [S, 384], OUT)
    tok = p.add_tensor(BF16, [B, S, 384], IN)
    head = p.add_tensor(BF16, [B, 37, 384], OUT)
    joined = p.add_tensor(BF16, [B, S + 37, 384], OUT)
    vec = p.add_tensor(BF16, [B, 1, 384], IN)
    spread = p.add_tensor(BF16, [B, S, 384], OUT)
    a_scale = p.add_tensor(BF16, [384], CONST)
    a_bias = p.add_tensor(BF16, [384], CONST)
    affine = p.add_tensor(BF16, [B, S, 384], OUT)
    as_f32 = p.add_tensor(F32, [B, S, 384], OUT)
    as_f16 = p.add_tensor(F16, [B, S, 384], OUT)
    back = p.add_tensor(BF16, [B, S, 384], OUT)
    filled = p.add_tensor(BF16, [S, 77], OUT)
    summed = p.add_tensor(BF16, [B, S, 384], OUT)
    p.add_op(d.Opcode.RotaryFrequency, [pos, pair_axes, pair_idx, axis_dims], [cos, sin],
             [d.Attribute.f64(d.AttrKey.Theta, 10000.0), d.Attribute.f64(d.AttrKey.Ntk, 1.0)])
    p.add_op(d.Opcode.RotaryApply, [x, cos, sin], [rot], [d.Attribute.u64(d.AttrKey.RotaryLayout, 1)])
    p.add_op(d.Opcode.BooleanMaskToBias, [valid], [bias_full])
    p.add_op(d.Opcode.BooleanMaskToBias, [valid], [bias_keys], [d.Attribute.boolean(d.AttrKey.MaskQueries, False)])
    p.add_op(d.Opcode.Slice, [wide], [mid], [d.Attribute.u64(d.AttrKey.Axis, 1), d.Attribute.u64(d.AttrKey.Start, 384)])
    p.add_op(d.Opcode.Slice, [tok], [head], [d.Attribute.u64(d.AttrKey.Axis, 1), d.Attribute.u64(d.AttrKey.Start, 5)])
    p.add_op(d.Opcode.Concat, [head, tok], [joined], [d.Attribute.u64(d.AttrKey.Axis, 1)])
    p.add_op(d.Opcode.BroadcastTo, [vec], [spread])
    p.add_op(d.Opcode.AffineLastDim, [tok, a_scale, a_bias], [affine])
    p.add_op(d.Opcode.Cast, [affine], [as_f32])
    p.add_op(d.Opcode.Cast, [as_f32], [as_f16])
    p.add_op(d.Opcode.Cast, [as_f16], [back])
    p.add_op(d.Opcode.Fill, [], [filled], [d.Attribute.f64(d.AttrKey.Value, -0.3337)])
    p.add_op(d.Opcode.Add, [spread, back], [summed])
    # 32 pairs per axis; text tokens sit at (0, 0), image tokens at (row, column)
    positions = np.zeros((B, S, 2), np.float32)
    grid = np.stack(np.meshgrid(np.arange(14), np.arange(19), indexing="ij"), -1).reshape(-1, 2)
    positions[:, 37:, :] = grid
    consts = {pair_axes: np.repeat(np.arange(2, dtype=np.int32), pairs // 2),
              pair_idx: np.tile(np.arange(pairs // 2, dtype=np.int32), 2),
              axis_dims: np.array([D // 2, D // 2], np.int32),
              a_scale: ob.f32_to_bf16(rng.standard_normal(384).astype(np.float32)),
              a_bias: ob.f32_to_bf16(rng.standard_normal(384).astype(np.float32))}
    mask = np.ones((B, S), np.uint8)
    mask[:, 30:37] = 0  # padded text
    mask[1, 100] = 0
    bf = lambda shape: ob.f32_to_bf16(rng.standard_normal(shape).astype(np.float32))
    inputs = {pos: positions, x: bf([B, S, H, D]), valid: mask, wide: bf([S, 3 * 384]), tok: bf([B, S, 384]),
              vec: bf([B, 1, 384])}
    got, want = _run(p, consts, inputs)
    for name, tid in (("cos", cos), ("sin", sin), ("RotaryApply", rot), ("mask bias", bias_full),
                      ("key mask bias", bias_keys), ("Slice last axis", mid), ("Slice tokens", head),
                      ("Concat", joined), ("BroadcastTo", spread), ("AffineLastDim", affine), ("Cast f32", as_f32),
                      ("Cast f16", as_f16), ("Cast bf16", back), ("Fill", filled), ("Add", summed)):
        assert np.array_equal(got[tid], want[tid]), "%s differs from the reference executor" % name
