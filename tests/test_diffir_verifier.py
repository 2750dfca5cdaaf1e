"""CPU: the library's host-side DiffIR decoder and verifier (difb200_program_check, the front door of
the plugin's compile) against the reference's own decoder (reference src/ir/codec.cpp:407-476,
src/ir/verify.cpp; run through oracle/_ref). The drop-in must refuse what the reference refuses:

  * programs with every operator this backend runs are accepted by both;
  * targeted malformed programs -- one per rule of the reference verifier for those operators --
    are invalid (status 1) here and rejected by the reference;
  * seeded random mutations of valid programs, re-sealed with a correct SHA-256 so that they reach
    the decoder and the verifier: whatever this library accepts the reference accepts, whatever it
    calls invalid the reference rejects, and nothing crashes."""
import ctypes as C
import hashlib
import random
import struct

import numpy as np
import pytest

import oracle_bridge as ob
from diffusion_compiler_b200 import blocks
from diffusion_compiler_b200 import diffir as d

needs_ref = pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")

F32, BF16, F16, I8, I32, BOOL = d.DType.F32, d.DType.BF16, d.DType.F16, d.DType.I8, d.DType.I32, d.DType.Bool
IN, OUT, CONST = d.Role.Input, d.Role.Output, d.Role.Constant
A, K, OP = d.Attribute, d.AttrKey, d.Opcode


def _lib():
    from diffusion_compiler_b200 import _lib, build
    build.build()
    return _lib.lib()


def check(data: bytes):
    lib = _lib()
    rc = lib.difb200_program_check(data, len(data))
    return rc, (lib.difb200_last_error().decode() if rc else "")


def ref_accepts(data: bytes):
    ref = C.CDLL(ob.REF_PATH)
    err = C.create_string_buffer(512)
    return ref.difref_encode_check(data, C.c_size_t(len(data)), err, C.c_size_t(512)) == 0, err.value.decode()


def seal(payload: bytes) -> bytes:
    return payload + hashlib.sha256(payload).digest()


def zoo_program() -> d.Program:
    """The operators the two block programs do not use, on small shapes."""
    p = d.Program()
    B, S, H, D = 2, 8, 2, 128
    pairs = D // 2
    pos = p.add_tensor(F32, [B, S, 2], IN)
    pair_axes, pair_idx, axis_dims = (p.add_tensor(I32, [n], CONST) for n in (pairs, pairs, 2))
    cos, sin = p.add_tensor(F32, [B, S, pairs], OUT), p.add_tensor(F32, [B, S, pairs], OUT)
    x = p.add_tensor(BF16, [B, S, H, D], IN)
    rot = p.add_tensor(BF16, [B, S, H, D], OUT)
    valid = p.add_tensor(BOOL, [B, S], IN)
    bias = p.add_tensor(BF16, [B, 1, S, S], d.Role.Internal)
    attn = p.add_tensor(BF16, [B, S, H, D], OUT)
    tok = p.add_tensor(BF16, [B, S, 256], IN)
    vec = p.add_tensor(BF16, [B, 1, 256], IN)
    spread = p.add_tensor(BF16, [B, S, 256], OUT)
    a_scale, a_bias, n_w = (p.add_tensor(BF16, [256], CONST) for _ in range(3))
    affine, normed, acted, gated, mult, summed = (p.add_tensor(BF16, [B, S, 256], OUT) for _ in range(6))
    as_f32 = p.add_tensor(F32, [B, S, 256], OUT)
    w = p.add_tensor(BF16, [64, 256], CONST)
    lin_b = p.add_tensor(BF16, [64], CONST)
    lin = p.add_tensor(BF16, [B * S, 64], OUT)
    flat = p.add_tensor(BF16, [B * S, 256], d.Role.Internal)
    codes, rcodes = p.add_tensor(I8, [B * S, 256], OUT), p.add_tensor(I8, [B * S, 256], OUT)
    scales, rscales = p.add_tensor(F32, [B * S], OUT), p.add_tensor(F32, [B * S], OUT)
    clip = p.add_tensor(F32, [1], IN)
    p.add_op(OP.RotaryFrequency, [pos, pair_axes, pair_idx, axis_dims], [cos, sin],
             [A.f64(K.Theta, 10000.0), A.f64(K.Ntk, 1.0)])
    p.add_op(OP.RotaryApply, [x, cos, sin], [rot], [A.u64(K.RotaryLayout, 1)])
    p.add_op(OP.BooleanMaskToBias, [valid], [bias], [A.boolean(K.MaskQueries, False)])
    p.add_op(OP.Attention, [rot, rot, x, bias], [attn], [A.u64(K.Implementation, 2)])
    p.add_op(OP.BroadcastTo, [vec], [spread])
    p.add_op(OP.AffineLastDim, [tok, a_scale, a_bias], [affine])
    p.add_op(OP.RmsNorm, [affine, n_w], [normed], [A.f64(K.Epsilon, 1e-6)])
    p.add_op(OP.SiLU, [normed], [acted])
    p.add_op(OP.Sigmoid, [acted], [gated])
    p.add_op(OP.Multiply, [gated, spread], [mult])
    p.add_op(OP.Add, [mult, tok], [summed])
    p.add_op(OP.Cast, [summed], [as_f32])
    p.add_op(OP.Reshape, [summed], [flat])
    p.add_op(OP.Linear, [flat, w, lin_b], [lin])
    p.add_op(OP.QuantizeInt8Rows, [flat, clip], [codes, scales, rcodes, rscales], [A.u64(K.Implementation, 5)])
    return p


def seed_programs():
    rng = np.random.default_rng(0)
    quantize = lambda w: ob.orc().quantize_int8_rows([w], 2)
    video = blocks.synth_video_block(rng, 64, 512, 4, 128, 1024, 96, quantize)[0]
    mmdit = blocks.synth_mmdit_block(rng, batch=1, grid=(4, 4), text_tokens=8, hidden=512, heads=4, mlp=1024,
                                     quantize=quantize)[0]
    return [d.encode(video), d.encode(mmdit), d.encode(zoo_program())]


def test_every_operator_of_the_backend_is_covered_and_accepted():
    programs = seed_programs()
    seen = set()
    for data in programs:
        assert check(data) == (0, "")
        seen |= {int(op.opcode) for op in d.decode(data).operations}
    names = {OP(o).name for o in seen}
    assert names == {"Add", "Multiply", "RmsNormModulate", "SwiGlu", "ResidualGate", "Linear", "QkNormPartialRope",
                     "Attention", "BiasAdd", "SiLU", "RmsNorm", "Fill", "Cast", "AffineLastDim", "Gelu", "Sigmoid",
                     "Reshape", "BroadcastTo", "Slice", "RotaryFrequency", "RotaryApply", "BooleanMaskToBias",
                     "Concat", "QuantizeInt8Rows", "LinearInt8Scaled", "LayerNormModulate"}, names


@needs_ref
def test_reference_accepts_the_same_programs():
    for data in seed_programs():
        assert ref_accepts(data) == (True, "")


def _simple(build):
    p = d.Program()
    build(p)
    return d.encode(p)


def _cases():
    """(name, program bytes): each breaks one rule of the reference verifier."""
    out = []

    def add(name, build):
        out.append((name, _simple(build)))

    def slice_case(axis=1, start=4, out_cols=4, kinds=(1, 1), drop=None):
        def build(p):
            a = p.add_tensor(BF16, [3, 16], IN)
            o = p.add_tensor(BF16, [3, out_cols], OUT)
            attrs = [A(int(K.Axis), kinds[0], axis), A(int(K.Start), kinds[1], start)]
            if drop is not None:
                attrs.pop(drop)
            p.add_op(OP.Slice, [a], [o], attrs)
        return build
    add("slice window past the end", slice_case(start=14, out_cols=4))
    add("slice start past the axis", slice_case(start=17, out_cols=0 + 1))
    add("slice without Start", slice_case(drop=1))
    add("slice Axis of the wrong kind", slice_case(kinds=(3, 1)))
    add("slice axis out of range", slice_case(axis=2))

    def concat_case(n=2, axis_attr=True, out_rows=6, axis=0):
        def build(p):
            parts = [p.add_tensor(BF16, [3, 8], IN) for _ in range(n)]
            o = p.add_tensor(BF16, [out_rows, 8], OUT)
            p.add_op(OP.Concat, parts, [o], [A.u64(K.Axis, axis)] if axis_attr else [])
        return build
    add("concat of one input", concat_case(n=1, out_rows=3))
    add("concat without Axis", concat_case(axis_attr=False))
    add("concat output of the wrong extent", concat_case(out_rows=7))
    add("concat axis out of range", concat_case(axis=2))

    def norm_case(opcode, attrs):
        def build(p):
            x = p.add_tensor(BF16, [4, 256], IN)
            o = p.add_tensor(BF16, [4, 256], OUT)
            if opcode == OP.RmsNorm:
                w = p.add_tensor(BF16, [256], CONST)
                p.add_op(opcode, [x, w], [o], attrs)
            elif opcode == OP.RmsNormModulate:
                s, t = p.add_tensor(BF16, [4, 256], IN), p.add_tensor(BF16, [4, 256], IN)
                p.add_op(opcode, [x, s, t], [o], attrs)
            else:
                w, b = p.add_tensor(BF16, [256], CONST), p.add_tensor(BF16, [256], CONST)
                s, t = p.add_tensor(BF16, [2, 256], IN), p.add_tensor(BF16, [2, 256], IN)
                p.add_op(opcode, [x, w, b, s, t], [o], attrs)
        return build
    for opcode in (OP.RmsNorm, OP.RmsNormModulate, OP.LayerNormModulate):
        add("%s BlockSize 48" % OP(opcode).name, norm_case(opcode, [A.u64(K.BlockSize, 48)]))
        add("%s BlockSize 2048" % OP(opcode).name, norm_case(opcode, [A.u64(K.BlockSize, 2048)]))
        add("%s Epsilon 0" % OP(opcode).name, norm_case(opcode, [A.f64(K.Epsilon, 0.0)]))
        add("%s Epsilon as u64" % OP(opcode).name, norm_case(opcode, [A.u64(K.Epsilon, 1)]))
    add("RmsNorm Implementation 3", norm_case(OP.RmsNorm, [A.u64(K.Implementation, 3)]))
    add("RmsNorm Implementation 2 at width 256", norm_case(OP.RmsNorm, [A.u64(K.Implementation, 2)]))
    add("RmsNorm reduction tile 4096", norm_case(OP.RmsNorm, [A.u64(K.ReductionTileSize, 4096)]))
    add("RmsNorm reduction tile at width 256", norm_case(OP.RmsNorm, [A.u64(K.ReductionTileSize, 2048),
                                                                          A.u64(K.BlockSize, 512)]))
    add("RmsNormModulate layout 3", norm_case(OP.RmsNormModulate, [A.u64(K.ModulationLayout, 3)]))

    def rope_case(attrs, table=(8, 48), weight=128):
        def build(p):
            x = p.add_tensor(BF16, [8, 2, 128], IN)
            w = p.add_tensor(BF16, [weight], CONST)
            c, s = p.add_tensor(F32, list(table), CONST), p.add_tensor(F32, list(table), CONST)
            o = p.add_tensor(BF16, [8, 2, 128], OUT)
            p.add_op(OP.QkNormPartialRope, [x, w, c, s], [o], attrs)
        return build
    add("rope BlockSize 100", rope_case([A.u64(K.BlockSize, 100)]))
    add("rope Heads disagrees", rope_case([A.u64(K.Heads, 3)]))
    add("rope HeadDim disagrees", rope_case([A.u64(K.HeadDim, 64)]))
    add("rope RotaryDim odd", rope_case([A.u64(K.RotaryDim, 95)]))
    add("rope RotaryDim zero", rope_case([A.u64(K.RotaryDim, 0)]))
    add("rope RotaryDim does not fit the tables", rope_case([A.u64(K.RotaryDim, 64)]))
    add("rope RotaryDim above the head", rope_case([A.u64(K.RotaryDim, 192)], table=(8, 96)))
    add("rope Start past the tables", rope_case([A.u64(K.Start, 1)]))
    add("rope weight of the wrong width", rope_case([], weight=64))
    add("rope rank-3 table with batch 2 for an unbatched input", rope_case([], table=(2, 8, 48)))

    def rotary_apply_case(attrs):
        def build(p):
            x = p.add_tensor(BF16, [1, 4, 2, 128], IN)
            c, s = p.add_tensor(F32, [1, 4, 64], IN), p.add_tensor(F32, [1, 4, 64], IN)
            o = p.add_tensor(BF16, [1, 4, 2, 128], OUT)
            p.add_op(OP.RotaryApply, [x, c, s], [o], attrs)
        return build
    add("rotary apply without a layout", rotary_apply_case([]))
    add("rotary apply half-split layout", rotary_apply_case([A.u64(K.RotaryLayout, 2)]))

    def frequency_case(attrs):
        def build(p):
            pos = p.add_tensor(F32, [1, 4, 2], IN)
            a, i, n = p.add_tensor(I32, [8], CONST), p.add_tensor(I32, [8], CONST), p.add_tensor(I32, [2], CONST)
            c, s = p.add_tensor(F32, [1, 4, 8], OUT), p.add_tensor(F32, [1, 4, 8], OUT)
            p.add_op(OP.RotaryFrequency, [pos, a, i, n], [c, s], attrs)
        return build
    add("rotary frequency Theta 0", frequency_case([A.f64(K.Theta, 0.0)]))
    add("rotary frequency Ntk negative", frequency_case([A.f64(K.Ntk, -1.0)]))
    add("rotary frequency Theta as u64", frequency_case([A.u64(K.Theta, 10000)]))

    def attention_case(attrs, dtype=BF16, dims=(1, 8, 2, 128), kv=None, biased=False):
        def build(p):
            q = p.add_tensor(dtype, list(dims), IN)
            kd = list(dims)
            if kv is not None:
                kd[-2] = kv
            k, v = p.add_tensor(dtype, kd, IN), p.add_tensor(dtype, kd, IN)
            o = p.add_tensor(dtype, list(dims), OUT)
            ins = [q, k, v]
            if biased:
                ins.append(p.add_tensor(dtype, [dims[0], 1, dims[-3], dims[-3]], IN))
            p.add_op(OP.Attention, ins, [o], attrs)
        return build
    add("attention Implementation 6", attention_case([A.u64(K.Implementation, 6)]))
    add("attention Implementation 1 batched", attention_case([]))
    add("attention Implementation 2 in f32", attention_case([A.u64(K.Implementation, 2)], dtype=F32))
    add("attention Implementation 4 causal", attention_case([A.u64(K.Implementation, 4), A.boolean(K.Causal, True)]))
    add("attention Implementation 4 biased", attention_case([A.u64(K.Implementation, 4)], biased=True))
    add("attention Implementation 5 with GQA", attention_case([A.u64(K.Implementation, 5), A.u64(K.KvHeads, 1)], kv=1))
    add("attention Implementation 3 in bf16", attention_case([A.u64(K.Implementation, 3)], dims=(8, 1, 128)))
    add("attention BlockSize 16", attention_case([A.u64(K.Implementation, 2), A.u64(K.BlockSize, 16)]))
    add("attention KvHeads does not divide", attention_case([A.u64(K.Implementation, 2), A.u64(K.KvHeads, 3)], dims=(1, 8, 4, 128), kv=3))
    add("attention KvHeads as bool", attention_case([A.u64(K.Implementation, 2), A.boolean(K.KvHeads, True)]))

    def linear_case(attrs, dtype=BF16, bias=False):
        def build(p):
            x, w = p.add_tensor(dtype, [4, 32], IN), p.add_tensor(dtype, [8, 32], CONST)
            o = p.add_tensor(dtype, [4, 8], OUT)
            ins = [x, w] + ([p.add_tensor(dtype, [8], CONST)] if bias else [])
            p.add_op(OP.Linear, ins, [o], attrs)
        return build
    add("linear bias mode 3", linear_case([A.u64(K.LinearBiasMode, 3)], bias=True))
    add("linear addmm without a bias", linear_case([A.u64(K.LinearBiasMode, 2)]))
    add("linear workspace limit 0", linear_case([A.u64(K.WorkspaceLimitBytes, 0)]))
    add("linear Implementation 4", linear_case([A.u64(K.Implementation, 4)]))
    add("linear tf32 on bf16", linear_case([A.u64(K.Implementation, 2)]))

    def gelu_case(attrs):
        def build(p):
            x, o = p.add_tensor(BF16, [4, 32], IN), p.add_tensor(BF16, [4, 32], OUT)
            p.add_op(OP.Gelu, [x], [o], attrs)
        return build
    add("gelu without an approximation", gelu_case([]))
    add("gelu approximation 3", gelu_case([A.u64(K.Approximation, 3)]))
    add("gelu approximation as f64", gelu_case([A.f64(K.Approximation, 1.0)]))

    def cast_same(p):
        x, o = p.add_tensor(BF16, [4, 32], IN), p.add_tensor(BF16, [4, 32], OUT)
        p.add_op(OP.Cast, [x], [o])
    add("cast to the same dtype", cast_same)

    def swiglu_case(start):
        def build(p):
            x, o = p.add_tensor(BF16, [4, 64], IN), p.add_tensor(BF16, [4, 32], OUT)
            p.add_op(OP.SwiGlu, [x], [o], [A.u64(K.Start, start)])
        return build
    add("swiglu window past the end", swiglu_case(1))
    add("swiglu window that overflows", swiglu_case(2 ** 64 - 8))

    def quant_case(attrs, width=256):
        def build(p):
            x = p.add_tensor(BF16, [4, width], IN)
            c, s = p.add_tensor(I8, [4, width], OUT), p.add_tensor(F32, [4], OUT)
            p.add_op(OP.QuantizeInt8Rows, [x], [c, s], attrs)
        return build
    add("quantiser BlockSize 128", quant_case([A.u64(K.BlockSize, 128)]))
    add("quantiser Scale 1.5", quant_case([A.f64(K.Scale, 1.5)]))
    add("quantiser Scale 0", quant_case([A.f64(K.Scale, 0.0)]))
    add("quantiser Implementation 8", quant_case([A.u64(K.Implementation, 8)]))
    add("quantiser H256 at width 128", quant_case([A.u64(K.Implementation, 2)], width=128))
    add("quantiser H4096 at width 256", quant_case([A.u64(K.Implementation, 4)]))

    def roles_case(roles, dims=(4, 4)):
        def build(p):
            x = p.add_tensor(BF16, list(dims), roles)
            o = p.add_tensor(BF16, list(dims), OUT)
            p.add_op(OP.SiLU, [x], [o])
        return build
    add("parameter that is neither input nor output", roles_case(int(CONST) | 16))
    add("optimizer state that is a constant", roles_case(int(IN) | int(CONST) | 32))
    add("streamed tensor that is not a constant", roles_case(int(IN) | 8))
    add("unknown role bit", roles_case(int(IN) | 64))
    add("zero dimension", roles_case(int(IN), dims=(4, 0)))
    add("element count overflow", roles_case(int(IN), dims=(2 ** 40, 2 ** 40)))
    return out


CASES = _cases()


@pytest.mark.parametrize("name,data", CASES, ids=[c[0] for c in CASES])
def test_programs_the_reference_verifier_rejects_are_invalid_here(name, data):
    rc, text = check(data)
    assert rc == 1 and text.startswith("DiffIR: "), (rc, text)
    if ob.ref_available():
        ok, why = ref_accepts(data)
        assert not ok, "the reference accepts this program: the case does not test a rule of its verifier"


def test_forms_the_reference_admits_stay_valid():
    """An Output that is also an Input and that no operator writes; attributes of an unexpected kind
    that the operator never reads."""
    def passthrough(p):
        x = p.add_tensor(BF16, [4, 4], int(IN) | int(OUT))
        y = p.add_tensor(BF16, [4, 4], OUT)
        p.add_op(OP.SiLU, [x], [y], [A.f64(K.Axis, 1.0), A.u64(K.Epsilon, 3)])
    data = _simple(passthrough)
    assert check(data) == (0, "")
    if ob.ref_available():
        assert ref_accepts(data)[0]


def _mutate(rng, base: bytes) -> bytes:
    b = bytearray(base[:-32])
    mode = rng.randrange(5)
    words = (len(b) - 8) // 4
    if mode == 0:
        for _ in range(rng.randrange(1, 4)):
            b[rng.randrange(len(b))] = rng.randrange(256)
    elif mode == 1:
        at = 8 + 4 * rng.randrange(words)
        b[at:at + 4] = struct.pack("<I", rng.choice([0, 1, 2, 3, 4, 0xffffffff, 0x7fffffff, 1 << 20, (1 << 20) + 1,
                                                     rng.randrange(80)]))
    elif mode == 2:
        if rng.random() < 0.5:
            b = b[:rng.randrange(8, len(b))]
        else:
            b += bytes(rng.randrange(256) for _ in range(rng.randrange(1, 16)))
    elif mode == 3:
        at = 8 + 4 * rng.randrange(words - 2)
        b[at:at + 8] = struct.pack("<Q", rng.choice([0, 1, 2 ** 63, 2 ** 64 - 1, 2 ** 40, 2 ** 32, rng.randrange(4096)]))
    else:
        i, j = 8 + 4 * rng.randrange(words), 8 + 4 * rng.randrange(words)
        b[i:i + 4], b[j:j + 4] = b[j:j + 4], b[i:i + 4]
    return seal(bytes(b))


@needs_ref
@pytest.mark.parametrize("seed", [1, 2, 3])
def test_mutated_programs_are_judged_like_the_reference_judges_them(seed):
    rng = random.Random(seed)
    seeds = seed_programs()
    counts = {}
    for _ in range(2500):
        data = _mutate(rng, rng.choice(seeds))
        rc, text = check(data)
        ok, why = ref_accepts(data)
        counts[(rc, ok)] = counts.get((rc, ok), 0) + 1
        assert rc in (0, 1, 2), (rc, text)
        if rc == 0:
            assert ok, "accepted here, rejected by the reference: " + why
        if rc == 1:
            assert not ok, "invalid here (%s), accepted by the reference" % text
    assert counts.get((0, True), 0) > 50 and counts.get((1, False), 0) > 1000, counts


def test_container_faults_are_reported_not_crashed_on():
    good = seed_programs()[0]
    assert check(b"") [0] == 1 and check(good[:40])[0] == 1
    assert "SHA-256" in check(good[:-1] + bytes([good[-1] ^ 1]))[1]
    assert "magic" in check(seal(b"XIFIR001" + good[8:-32]))[1]
    assert "version" in check(seal(good[:8] + struct.pack("<I", 2) + good[12:-32]))[1]
    assert check(seal(good[:-32] + b"\0"))[0] == 1          # trailing byte
    assert check(seal(good[:12] + struct.pack("<I", (1 << 20) + 1) + good[16:-32]))[0] == 1   # tensor count
