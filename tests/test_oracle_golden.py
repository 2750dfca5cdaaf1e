"""CPU: the C restatement (oracle/diforacle.c) against the committed vectors that the reference's
own CPU executor produced (tests/golden/hotpath_golden.npz, generator make_golden.py), and, where
the reference build is present, directly against it on fresh seeded inputs. Also the DIFIR001
codec against the reference's decoder/encoder."""
import os

import numpy as np
import pytest

import oracle_bridge as ob
from diffusion_compiler_b200 import diffir as ir

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "hotpath_golden.npz"))


def _eq(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint8).ravel(), np.ascontiguousarray(b).view(np.uint8).ravel())


def test_reference_unit_test_linear_vectors():
    g = GOLDEN
    codes, scales = ob.orc().quantize_int8_rows([g["reftest_linear/x"]], 1, 0.98)
    assert _eq(codes, g["reftest_linear/codes"]) and _eq(scales, g["reftest_linear/row_scales"])
    y = ob.orc().linear_int8_scaled(codes, g["reftest_linear/w"], scales, g["reftest_linear/cs"])
    assert _eq(y, g["reftest_linear/y"])


@pytest.mark.parametrize("impl", [2, 3, 5, 6])
def test_reference_unit_test_h256_vectors(impl):
    clip = 0.9995 if impl in (5, 6) else 1.0
    got = ob.orc().quantize_int8_rows([GOLDEN["reftest_h256/x"]], impl, np.float32(clip), residual=True)
    for name, a in zip(("codes", "scales", "rcodes", "rscales"), got):
        assert _eq(a, GOLDEN["reftest_h256/impl%d_%s" % (impl, name)]), name


@pytest.mark.parametrize("impl", [4, 7])
def test_reference_unit_test_h4096_vectors(impl):
    codes, scales = ob.orc().quantize_int8_rows([GOLDEN["reftest_h4096/x"]], impl)
    assert _eq(codes, GOLDEN["reftest_h4096/impl%d_codes" % impl])
    assert _eq(scales, GOLDEN["reftest_h4096/impl%d_scales" % impl])


@pytest.mark.parametrize("impl", range(1, 8))
def test_seeded_quant_vectors(impl):
    x = GOLDEN["seeded_quant/impl%d_x" % impl]
    K = x.shape[1]
    parts = [np.ascontiguousarray(x[:, :K // 2]), np.ascontiguousarray(x[:, K // 2:])]
    got = ob.orc().quantize_int8_rows(parts, impl, 0.97, residual=True)
    for name, a in zip(("codes", "scales", "rcodes", "rscales"), got):
        assert _eq(a, GOLDEN["seeded_quant/impl%d_%s" % (impl, name)]), name


def test_seeded_linear_vectors():
    g = GOLDEN
    w8, ws = ob.orc().quantize_int8_rows([g["seeded_linear/w_bf16"]], 2)
    assert _eq(w8, g["seeded_linear/w8"]) and _eq(ws, g["seeded_linear/ws"])
    codes, scales = ob.orc().quantize_int8_rows([g["seeded_linear/x"]], 2)
    assert _eq(codes, g["seeded_linear/codes"]) and _eq(scales, g["seeded_linear/row_scales"])
    yb = ob.orc().bias_add(ob.orc().linear_int8_scaled(codes, w8, scales, ws), g["seeded_linear/bias"])
    assert _eq(yb, g["seeded_linear/y_bias"])
    assert _eq(ob.orc().gelu_tanh(yb), g["seeded_linear/y_gelu"])


def test_seeded_attention_vectors():
    g = GOLDEN
    out = ob.orc().attention_exact(g["seeded_attention/q"], g["seeded_attention/k"], g["seeded_attention/v"],
                                   g["seeded_attention/mask"])
    assert _eq(out, g["seeded_attention/out_exact"])


def test_int8_attention_contract_tracks_exact_attention():
    """The INT8 contract (ours) stays within the reference's own bar for its INT8 attention,
    cosine >= 0.9999 against exact attention (reference tests/owned_attention_tests.cpp:122-157)."""
    rng = np.random.default_rng(1)
    B, S, H, KV, D = 1, 192, 2, 1, 128
    one = ob.f32_to_bf16(np.ones(D, np.float32))
    q = ob.orc().rms_norm(ob.f32_to_bf16(rng.standard_normal((B, S, H, D)).astype(np.float32)), one, 1e-6)
    k = ob.orc().rms_norm(ob.f32_to_bf16(rng.standard_normal((B, S, KV, D)).astype(np.float32)), one, 1e-6)
    v = ob.f32_to_bf16(rng.standard_normal((B, S, KV, D)).astype(np.float32))
    q8, qs = ob.orc().quantize_int8_rows([q.reshape(-1, D)], 1)
    k8, ks = ob.orc().quantize_int8_rows([k.reshape(-1, D)], 1)
    a = ob.bf16_to_f32(ob.orc().attention_int8(q8.reshape(B, S, H, D), qs, k8.reshape(B, S, KV, D), ks, v))
    e = ob.bf16_to_f32(ob.orc().attention_exact(q, k, v))
    cos = float(np.dot(a.ravel(), e.ravel()) / (np.linalg.norm(a) * np.linalg.norm(e)))
    assert cos >= 0.9999


def test_thread_count_does_not_change_results():
    rng = np.random.default_rng(3)
    x = ob.f32_to_bf16(rng.standard_normal((33, 768)).astype(np.float32))
    ob.orc().lib.orc_set_threads(1)
    a = ob.orc().quantize_int8_rows([x], 3)
    ob.orc().lib.orc_set_threads(5)
    b = ob.orc().quantize_int8_rows([x], 3)
    ob.orc().lib.orc_set_threads(1)
    assert _eq(a[0], b[0]) and _eq(a[1], b[1])


def test_codec_roundtrip():
    pr = ir.w8a8_linear_program(8, 256, 16, 2, bias=True, gelu=True)["program"]
    data = ir.encode(pr)
    again = ir.decode(data)
    assert ir.encode(again) == data
    with pytest.raises(ValueError):
        ir.decode(data[:-1] + bytes([data[-1] ^ 1]))
    with pytest.raises(ValueError):
        ir.decode(b"XXXXXXXX" + data[8:])


@pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")
def test_codec_against_reference_decoder():
    for pr in (ir.w8a8_linear_program(8, 256, 16, 5, bias=True, gelu=True),
               ir.quantize_program([3, 512], 3, residual=True, dynamic_clip=True),
               ir.attention_program(2, 16, 4, 2, 128, True)):
        ob.ref().encode_check(ir.encode(pr["program"]))


@pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")
@pytest.mark.parametrize("impl", range(1, 8))
def test_restatement_equals_reference_on_fresh_inputs(impl):
    rng = np.random.default_rng(50 + impl)
    K = 4096 if impl in (4, 7) else 768
    x = ob.f32_to_bf16((rng.standard_normal((7, K)) * rng.uniform(0.01, 30)).astype(np.float32))
    pr = ir.quantize_program([7, K], impl, clip=0.9, residual=True)
    res, _ = ob.ref().run(pr["program"], {pr["ids"]["x"][0]: x})
    got = ob.orc().quantize_int8_rows([x], impl, 0.9, residual=True)
    for name, a in zip(("codes", "scales", "rcodes", "rscales"), got):
        assert _eq(a, res[pr["ids"][name]]), name


def test_weight_rows_without_mse_equal_the_pinned_quantiser():
    """orc_quantize_weight_rows without the MSE search is the activation quantiser at clip 1,
    which is pinned against the reference executor; with the search the chosen scale is one of
    the seven candidates and never above the absmax scale."""
    rng = np.random.default_rng(11)
    w = ob.f32_to_bf16((rng.standard_normal((24, 768)) * 0.02).astype(np.float32))
    w[3] = 0  # an all-zero output channel
    for impl in (2, 3, 5, 6):
        codes, scales = ob.orc().quantize_weight_rows(w, impl)
        want_codes, want_scales = ob.orc().quantize_int8_rows([w], impl)
        assert np.array_equal(codes, want_codes) and np.array_equal(scales.view(np.uint32), want_scales.view(np.uint32))
        mcodes, mscales = ob.orc().quantize_weight_rows(w, impl, mse=True)
        assert (mscales <= ob.bf16_to_f32(ob.f32_to_bf16(scales)) * (1 + 2.0 ** -7)).all()
        assert mscales[3] == np.float32(1.0e-30) or mscales[3] == ob.bf16_to_f32(ob.f32_to_bf16(np.float32([1e-30])))[0]
        ratio = mscales[scales > 1e-20] / scales[scales > 1e-20]
        assert ((ratio > 0.75) & (ratio < 1.01)).all()


def test_mse_scale_search_equals_the_reference_packer_fixture():
    """orc_choose_mse_weight_scale against the scales the reference's own packer function chose for the
    same rows (tests/golden/packer_mse_scale.npz, made by tests/golden/make_packer_golden.py from the
    reference tool's source): bit-identical, edge rows included (all zero, one outlier, 1e-20, 1e20)."""
    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "packer_mse_scale.npz"))
    names = sorted({k.split("/")[0] for k in data.files if k.startswith("w")})
    assert names == ["w256", "w4096", "w768"]
    for name in names:
        rows, want = data[name + "/rows"], data[name + "/scale_bits"]
        got = ob.orc().choose_mse_weight_scale(rows).view(np.uint32)
        assert np.array_equal(got, want), name
        assert got[1] == np.float32(1.0e-30).view(np.uint32)  # the all-zero channel


def test_weight_packing_equals_the_reference_packer_fixture():
    """orc_weight_equalization and orc_quantize_weight_rows against whole runs of the reference's own
    packer (rewrite_named_linear_w8a8; the cache tensors are in tests/golden/packer_mse_scale.npz):
    the input-equalisation vector, the scales and the codes, bit for bit, six variant / option mixes."""
    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "packer_mse_scale.npz"))
    keys = sorted({k.split("/")[0] for k in data.files if k.startswith("pack_")})
    assert len(keys) == 6
    for key in keys:
        impl = int(key.split("_")[1][4:])
        equalise, mse = key.split("_")[2] == "eq1", key.split("_")[3] == "mse1"
        w = data[key + "/weight"]
        eq = None
        if equalise:
            eq = ob.orc().weight_equalization(w)
            assert np.array_equal(eq.view(np.uint16).ravel(), data[key + "/input_scale"].ravel()), key
        codes, scales = ob.orc().quantize_weight_rows(w, impl, mse=mse, equalise=eq)
        assert np.array_equal(scales.view(np.uint32), data[key + "/scale_bits"]), key
        assert np.array_equal(codes, data[key + "/codes"]), key


@pytest.mark.skipif(not ob.packer_probe_available(), reason="reference packer probe (oracle/_ref) not present")
def test_mse_scale_search_equals_the_reference_packer_live():
    """The same comparison on fresh seeded rows, against the probe built from the reference tool's
    source, and through the whole weight-row entry: rotate a bf16 weight with the pinned quantiser's
    transform (F32 variant, whose codes expose the rotated row), search the scale with the reference
    function, and find that scale in orc_quantize_weight_rows(mse=True)."""
    rng = np.random.default_rng(23)
    rows = (rng.standard_normal((64, 1024)) * rng.uniform(0.001, 10.0, (64, 1)).astype(np.float32)).astype(np.float32)
    rows[::7, 3] *= 40.0
    got = ob.orc().choose_mse_weight_scale(rows).view(np.uint32)
    want = ob.packer_mse_scales(rows).view(np.uint32)
    assert np.array_equal(got, want)
    # the choice matters: for rows with an outlier the search leaves the absmax scale
    absmax = np.abs(rows).max(axis=1) / np.float32(127.0)
    assert (ob.orc().choose_mse_weight_scale(rows)[::7] < absmax[::7] * 0.99).any()


@pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")
def test_reference_block_amplifies_a_small_attention_difference():
    """Why a whole W8A8 block is not compared at the 2e-3 bar against an executor whose attention
    differs slightly. The reference executor itself, run on the part of the video block behind the
    Attention op at the benchmark widths (hidden 3072, FFN 8192), once from an attention tensor A
    and once from A changed by a few 1e-4 (relative), gives block outputs that differ several
    times more than the inputs did: every QuantizeInt8Rows behind the attention flips the codes that
    sit near a rounding boundary. Reference only; no GPU, no kernel of this repository."""
    import block_oracle
    from diffusion_compiler_b200 import blocks
    rng = np.random.default_rng(17)
    ob.orc().lib.orc_set_threads(8)
    S, hidden, heads, dim, ffn, rotary = 64, 3072, 24, 128, 8192, 96
    quantize = lambda w: ob.orc().quantize_int8_rows([w], 2)
    p, ids, consts, inputs = blocks.synth_video_block(rng, S, hidden, heads, dim, ffn, rotary, quantize)
    _, post, att, _ = block_oracle.split(p)
    attn = (rng.standard_normal((S, heads, dim)) * 0.2).astype(np.float32)
    nudged = attn * (1.0 + 3.0e-4 * rng.standard_normal(attn.shape).astype(np.float32))
    a, b = ob.f32_to_bf16(attn), ob.f32_to_bf16(nudged)
    outs = []
    for tensor in (a, b):
        feed = block_oracle.feed_for(post, {att.outputs[0]: tensor}, consts, inputs)
        out, _ = ob.ref().run(post, feed)
        outs.append(ob.bf16_to_f32(out[ids["out"]]))
    from helpers import rel_l2 as _rel_l2
    d_in = _rel_l2(ob.bf16_to_f32(b), ob.bf16_to_f32(a))
    d_out = _rel_l2(outs[1], outs[0])
    print("attention tensors differ by %.2e, block outputs by %.2e" % (d_in, d_out))
    assert 1e-4 < d_in < 2e-3
    assert d_out > 2.0 * d_in
