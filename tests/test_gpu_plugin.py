"""GPU: the backend plugin entry points (dif_backend_get_v2 / _v1) of libdifb200.so, driven the
way the reference's host drives a plugin, against the committed reference vectors, the CPU oracle
and -- where oracle/_ref is present -- the reference's own plugin loader and CPU executor."""
import os

import numpy as np
import pytest

import oracle_bridge as ob
from diffusion_compiler_b200 import diffir as ir
from helpers import activations, bf16_normal, cosine, rel_l2

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "hotpath_golden.npz"))


def _eq(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint8).ravel(), np.ascontiguousarray(b).view(np.uint8).ravel())


@pytest.fixture(scope="module")
def executor():
    from diffusion_compiler_b200 import plugin
    ex = plugin.PluginExecutor(0)
    yield ex
    ex.close()


def test_reference_unit_test_linear_through_plugin(executor):
    g = GOLDEN
    pr = ir.w8a8_linear_program(2, 16, 16, 1, clip=0.98, bias=False, expose_codes=True)
    ids = pr["ids"]
    prepared = executor.prepare(pr["program"], {ids["weight"]: g["reftest_linear/w"], ids["col_scales"]: g["reftest_linear/cs"]})
    out, tel = prepared.run({ids["x"]: g["reftest_linear/x"]}, warmups=1, iterations=2)
    assert _eq(out[ids["codes"]], g["reftest_linear/codes"])
    assert _eq(out[ids["row_scales"]], g["reftest_linear/row_scales"])
    assert _eq(out[ids["y"]], g["reftest_linear/y"])
    assert tel.mean_milliseconds > 0 and tel.minimum_milliseconds <= tel.maximum_milliseconds
    assert b"difb200" in tel.device_name
    assert prepared.compile_telemetry.resident_bytes > 0


@pytest.mark.parametrize("impl", [2, 3, 5, 6])
def test_reference_unit_test_h256_through_plugin(executor, impl):
    dyn = impl in (5, 6)
    pr = ir.quantize_program([2, 256], impl, residual=True, dynamic_clip=dyn)
    ids = pr["ids"]
    prepared = executor.prepare(pr["program"], {})
    bound = {ids["x"][0]: GOLDEN["reftest_h256/x"]}
    if dyn:
        bound[ids["clip"]] = np.array([0.9995], np.float32)
    out, _ = prepared.run(bound)
    for name in ("codes", "scales", "rcodes", "rscales"):
        assert _eq(out[ids[name]], GOLDEN["reftest_h256/impl%d_%s" % (impl, name)]), name


@pytest.mark.parametrize("impl", [4, 7])
def test_reference_unit_test_h4096_through_plugin(executor, impl):
    pr = ir.quantize_program([1, 4096], impl)
    ids = pr["ids"]
    out, _ = executor.prepare(pr["program"], {}).run({ids["x"][0]: GOLDEN["reftest_h4096/x"]})
    assert _eq(out[ids["codes"]], GOLDEN["reftest_h4096/impl%d_codes" % impl])
    assert _eq(out[ids["scales"]], GOLDEN["reftest_h4096/impl%d_scales" % impl])


@pytest.mark.parametrize("impl", range(1, 8))
def test_seeded_quant_vectors_through_plugin(executor, impl):
    x = GOLDEN["seeded_quant/impl%d_x" % impl]
    K = x.shape[1]
    pr = ir.quantize_program([5, K], impl, clip=0.97, residual=True, part_widths=[K // 2, K // 2])
    ids = pr["ids"]
    out, _ = executor.prepare(pr["program"], {}).run({ids["x"][0]: np.ascontiguousarray(x[:, :K // 2]),
                                                       ids["x"][1]: np.ascontiguousarray(x[:, K // 2:])})
    for name in ("codes", "scales", "rcodes", "rscales"):
        assert _eq(out[ids[name]], GOLDEN["seeded_quant/impl%d_%s" % (impl, name)]), name


def test_seeded_linear_vectors_through_plugin_fused_epilogue(executor):
    g = GOLDEN
    consts = lambda ids: {ids["weight"]: g["seeded_linear/w8"], ids["col_scales"]: g["seeded_linear/ws"],
                          ids["bias"]: g["seeded_linear/bias"]}
    pr = ir.w8a8_linear_program(16, 512, 48, 2, bias=True, gelu=False, expose_codes=True)
    out, _ = executor.prepare(pr["program"], consts(pr["ids"])).run({pr["ids"]["x"]: g["seeded_linear/x"]})
    assert _eq(out[pr["ids"]["codes"]], g["seeded_linear/codes"])
    assert _eq(out[pr["ids"]["y"]], g["seeded_linear/y_bias"])  # bias fused into the GEMM epilogue, same bits
    pr = ir.w8a8_linear_program(16, 512, 48, 2, bias=True, gelu=True)
    out, _ = executor.prepare(pr["program"], consts(pr["ids"])).run({pr["ids"]["x"]: g["seeded_linear/x"]})
    a, b = ob.bf16_to_f32(out[pr["ids"]["y"]]), ob.bf16_to_f32(g["seeded_linear/y_gelu"])
    assert rel_l2(a, b) <= 2e-3 and cosine(a, b) >= 0.9999


def test_attention_with_key_mask_through_plugin(executor):
    g = GOLDEN
    B, S, H, KV, D = 2, 40, 4, 2, 128
    pr = ir.attention_program(B, S, H, KV, D, True)
    ids = pr["ids"]
    out, _ = executor.prepare(pr["program"], {}).run({ids["q"]: g["seeded_attention/q"], ids["k"]: g["seeded_attention/k"],
                                                      ids["v"]: g["seeded_attention/v"],
                                                      ids["mask"]: g["seeded_attention/mask"]})
    got = ob.bf16_to_f32(out[ids["out"]])
    exact = ob.bf16_to_f32(g["seeded_attention/out_exact"])
    assert cosine(got, exact) >= 0.9999  # the reference's own bar for its INT8 attention
    q8, qs = ob.orc().quantize_int8_rows([g["seeded_attention/q"].reshape(-1, D)], 1)
    k8, ks = ob.orc().quantize_int8_rows([g["seeded_attention/k"].reshape(-1, D)], 1)
    want = ob.bf16_to_f32(ob.orc().attention_int8(q8.reshape(B, S, H, D), qs, k8.reshape(B, S, KV, D), ks,
                                                  g["seeded_attention/v"], g["seeded_attention/mask"]))
    assert rel_l2(got, want) <= 2e-3 and cosine(got, want) >= 0.9999


def test_unsupported_and_malformed_programs_fail_closed(executor):
    from diffusion_compiler_b200 import plugin
    p = ir.Program()
    a = p.add_tensor(ir.DType.F32, [1, 4, 8, 8], ir.Role.Input)
    w = p.add_tensor(ir.DType.F32, [4, 4, 3, 3], ir.Role.Constant)
    o = p.add_tensor(ir.DType.F32, [1, 4, 8, 8], ir.Role.Output)
    p.add_op(60, [a, w], [o])  # Conv2d: outside the hot path
    with pytest.raises(plugin.BackendError) as info:
        executor.prepare(p, {w: np.zeros((4, 4, 3, 3), np.float32)})
    assert info.value.status == 2
    pr = ir.attention_program(1, 16, 2, 2, 128, False)
    pr["program"].operations[0].attributes[0] = ir.Attribute.u64(ir.AttrKey.Implementation, 5)
    with pytest.raises(plugin.BackendError) as info:
        executor.prepare(pr["program"], {})
    assert info.value.status == 2  # exact-stream attention is not what this backend lowers
    good = ir.w8a8_linear_program(4, 256, 8, 2)
    prepared = executor.prepare(good["program"], {good["ids"]["weight"]: np.zeros((8, 256), np.int8),
                                                  good["ids"]["col_scales"]: np.ones(8, np.float32),
                                                  good["ids"]["bias"]: np.zeros(8, np.uint16)})
    with pytest.raises(plugin.BackendError) as info:
        prepared.run({good["ids"]["x"]: np.zeros((4, 256), np.uint16)}, iterations=0)
    assert info.value.status == 1


def test_abi_v1_constants_travel_with_execute():
    from diffusion_compiler_b200 import plugin
    g = GOLDEN
    ex = plugin.PluginExecutor(0, abi_version=1)
    pr = ir.w8a8_linear_program(16, 512, 48, 2, bias=True, gelu=False)
    ids = pr["ids"]
    prepared = ex.prepare(pr["program"], {ids["weight"]: g["seeded_linear/w8"], ids["col_scales"]: g["seeded_linear/ws"],
                                          ids["bias"]: g["seeded_linear/bias"]})
    out, _ = prepared.run({ids["x"]: g["seeded_linear/x"]})
    assert _eq(out[ids["y"]], g["seeded_linear/y_bias"])
    prepared.close()
    ex.close()


def _mini_block(M, Hd, N):
    """LayerNormModulate -> W8A8 linear (+bias+GELU) -> W8A8 linear (+bias) -> ResidualGate."""
    p = ir.Program()
    bf = ir.DType.BF16
    x = p.add_tensor(bf, [M, Hd], ir.Role.Input)
    lw = p.add_tensor(bf, [Hd], ir.Role.Constant)
    lb = p.add_tensor(bf, [Hd], ir.Role.Constant)
    sc = p.add_tensor(bf, [1, Hd], ir.Role.Input)
    sh = p.add_tensor(bf, [1, Hd], ir.Role.Input)
    gate = p.add_tensor(bf, [1, Hd], ir.Role.Input)
    xm = p.add_tensor(bf, [M, Hd])
    p.add_op(ir.Opcode.LayerNormModulate, [x, lw, lb, sc, sh], [xm], [ir.Attribute.f64(ir.AttrKey.Epsilon, 1e-6)])

    def w8a8(src, K, Nn, gelu):
        c = p.add_tensor(ir.DType.I8, [M, K])
        r = p.add_tensor(ir.DType.F32, [M])
        w = p.add_tensor(ir.DType.I8, [Nn, K], ir.Role.Constant)
        cs = p.add_tensor(ir.DType.F32, [Nn], ir.Role.Constant)
        b = p.add_tensor(bf, [Nn], ir.Role.Constant)
        y = p.add_tensor(bf, [M, Nn])
        yb = p.add_tensor(bf, [M, Nn])
        p.add_op(ir.Opcode.QuantizeInt8Rows, [src], [c, r],
                 [ir.Attribute.u64(ir.AttrKey.BlockSize, 256), ir.Attribute.u64(ir.AttrKey.Implementation, 2)])
        p.add_op(ir.Opcode.LinearInt8Scaled, [c, w, r, cs], [y])
        p.add_op(ir.Opcode.BiasAdd, [y, b], [yb])
        last = yb
        if gelu:
            yg = p.add_tensor(bf, [M, Nn])
            p.add_op(ir.Opcode.Gelu, [yb], [yg], [ir.Attribute.u64(ir.AttrKey.Approximation, 1)])
            last = yg
        return last, (w, cs, b)

    h, c1 = w8a8(xm, Hd, N, True)
    y, c2 = w8a8(h, N, Hd, False)
    out = p.add_tensor(bf, [M, Hd], ir.Role.Output)
    p.add_op(ir.Opcode.ResidualGate, [x, y, gate], [out])
    return p, dict(x=x, lw=lw, lb=lb, sc=sc, sh=sh, gate=gate, out=out, c1=c1, c2=c2)


@pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")
def test_mini_block_against_reference_executor_and_reference_plugin_host(executor):
    """A modulate -> MLP -> gated-residual slice of a DiT block: (a) our plugin driven by OUR host
    mirror and (b) our plugin driven by the REFERENCE's own dlopen loader (difref_run_plugin) both
    have to agree with the reference CPU executor on the same program and tensors."""
    from diffusion_compiler_b200 import _lib
    rng = np.random.default_rng(9)
    M, Hd, N = 200, 512, 1024
    p, t = _mini_block(M, Hd, N)
    q = lambda a: ob.orc().quantize_int8_rows([a], 2)
    w1, s1 = q(bf16_normal(rng, (N, Hd), 0.02))
    w2, s2 = q(bf16_normal(rng, (Hd, N), 0.02))
    consts = {t["lw"]: ob.f32_to_bf16(np.ones(Hd, np.float32)), t["lb"]: bf16_normal(rng, (Hd,), 0.01),
              t["c1"][0]: w1, t["c1"][1]: s1, t["c1"][2]: bf16_normal(rng, (N,), 0.01),
              t["c2"][0]: w2, t["c2"][1]: s2, t["c2"][2]: bf16_normal(rng, (Hd,), 0.01)}
    inputs = {t["x"]: activations(rng, M, Hd), t["sc"]: bf16_normal(rng, (1, Hd), 0.1),
              t["sh"]: bf16_normal(rng, (1, Hd), 0.1), t["gate"]: bf16_normal(rng, (1, Hd), 1.0)}
    want, _ = ob.ref().run(p, {**consts, **inputs})
    want = ob.bf16_to_f32(want[t["out"]])
    got, _ = executor.prepare(p, consts).run(inputs)
    got = ob.bf16_to_f32(got[t["out"]])
    assert rel_l2(got, want) <= 2e-3 and cosine(got, want) >= 0.9999
    via_ref_host, _ = ob.ref().run(p, {**consts, **inputs}, plugin=_lib.LIB_PATH)
    via_ref_host = ob.bf16_to_f32(via_ref_host[t["out"]])
    assert np.array_equal(via_ref_host, got)
