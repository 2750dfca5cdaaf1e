"""Generates tests/golden/hotpath_golden.npz by running the REFERENCE project's own CPU executor
(oracle/_ref/libdifref.so, built by oracle/Makefile from the reference checkout its REF variable
names) on

  * the inputs of the reference's own unit tests for this path
    (tests/dif_tests.cpp:4259-4312 generic scaled INT8 linear; :4607-4665 H256 ConvRot, four
    variants, four outputs, dynamic clip 0.9995 for the F32 ones; :4667-4710 H4096, two variants);
    the reference pins these only as "CUDA bytes == CPU bytes", so the CPU bytes are the vectors;
  * seeded cases: all seven QuantizeInt8Rows variants with residual outputs and a zero row, a
    W8A8 linear with bias and tanh-GELU, and exact Attention with GQA and a key mask.

Run it where that checkout is present:  python tests/golden/make_golden.py
Every array is stored under "<case>/<name>"; bf16 tensors are uint16 bit patterns.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle_bridge as ob  # noqa: E402
from diffusion_compiler_b200 import diffir as ir  # noqa: E402


def main():
    ref = ob.ref()
    out = {}

    # --- reference unit test: generic scaled INT8 linear (dif_tests.cpp:4259-4312) ---
    x = ob.f32_to_bf16(np.array([(i % 11 - 5) / 2.0 for i in range(32)], np.float32).reshape(2, 16))
    w = np.array([(i % 13) - 6 for i in range(256)], np.int8).reshape(16, 16)
    cs = np.full(16, 0.25, np.float32)
    pr = ir.w8a8_linear_program(2, 16, 16, ir.Int8RowQuantization.Direct, clip=0.98, bias=False, expose_codes=True)
    ids = pr["ids"]
    res, _ = ref.run(pr["program"], {ids["x"]: x, ids["weight"]: w, ids["col_scales"]: cs})
    out.update({"reftest_linear/x": x, "reftest_linear/w": w, "reftest_linear/cs": cs,
                "reftest_linear/codes": res[ids["codes"]], "reftest_linear/row_scales": res[ids["row_scales"]],
                "reftest_linear/y": res[ids["y"]]})

    # --- reference unit test: H256 ConvRot row quantization (dif_tests.cpp:4607-4665) ---
    vals = np.array([((i % 37) - 18) / float((i % 5) + 1) for i in range(512)], np.float32).reshape(2, 256)
    xb = ob.f32_to_bf16(vals)
    out["reftest_h256/x"] = xb
    for impl in (2, 3, 5, 6):
        dyn = impl in (5, 6)
        pr = ir.quantize_program([2, 256], impl, residual=True, dynamic_clip=dyn)
        ids = pr["ids"]
        bound = {ids["x"][0]: xb}
        if dyn:
            bound[ids["clip"]] = np.array([0.9995], np.float32)
        res, _ = ref.run(pr["program"], bound)
        for name in ("codes", "scales", "rcodes", "rscales"):
            out["reftest_h256/impl%d_%s" % (impl, name)] = res[ids[name]]

    # --- reference unit test: H4096 ConvRot (dif_tests.cpp:4667-4710) ---
    vals = np.array([((i % 53) - 26) / float((i % 7) + 1) for i in range(4096)], np.float32).reshape(1, 4096)
    xb = ob.f32_to_bf16(vals)
    out["reftest_h4096/x"] = xb
    for impl in (4, 7):
        pr = ir.quantize_program([1, 4096], impl)
        ids = pr["ids"]
        res, _ = ref.run(pr["program"], {ids["x"][0]: xb})
        out["reftest_h4096/impl%d_codes" % impl] = res[ids["codes"]]
        out["reftest_h4096/impl%d_scales" % impl] = res[ids["scales"]]

    # --- seeded: all variants, residual, zero row, clip 0.97, two concatenated parts ---
    rng = np.random.default_rng(2024)
    for impl in range(1, 8):
        K = 4096 if impl in (4, 7) else 512
        x = ob.f32_to_bf16((rng.standard_normal((5, K)) * 3).astype(np.float32))
        x[3] = 0
        parts = [K // 2, K // 2]
        pr = ir.quantize_program([5, K], impl, clip=0.97, residual=True, part_widths=parts)
        ids = pr["ids"]
        xs = [np.ascontiguousarray(x[:, :K // 2]), np.ascontiguousarray(x[:, K // 2:])]
        res, _ = ref.run(pr["program"], {ids["x"][0]: xs[0], ids["x"][1]: xs[1]})
        out["seeded_quant/impl%d_x" % impl] = x
        for name in ("codes", "scales", "rcodes", "rscales"):
            out["seeded_quant/impl%d_%s" % (impl, name)] = res[ids[name]]

    # --- seeded: W8A8 linear with bias and GELU ---
    M, K, N = 16, 512, 48
    pr = ir.w8a8_linear_program(M, K, N, 2, bias=True, gelu=True, expose_codes=True)
    ids = pr["ids"]
    x = ob.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    wf = ob.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    prw = ir.quantize_program([N, K], 2)
    resw, _ = ref.run(prw["program"], {prw["ids"]["x"][0]: wf})
    w8, ws = resw[prw["ids"]["codes"]], resw[prw["ids"]["scales"]]
    b = ob.f32_to_bf16((rng.standard_normal(N) * 0.01).astype(np.float32))
    res, _ = ref.run(pr["program"], {ids["x"]: x, ids["weight"]: w8, ids["col_scales"]: ws, ids["bias"]: b})
    out.update({"seeded_linear/x": x, "seeded_linear/w_bf16": wf, "seeded_linear/w8": w8, "seeded_linear/ws": ws,
                "seeded_linear/bias": b, "seeded_linear/codes": res[ids["codes"]],
                "seeded_linear/row_scales": res[ids["row_scales"]], "seeded_linear/y_gelu": res[ids["y"]]})
    pr2 = ir.w8a8_linear_program(M, K, N, 2, bias=True, gelu=False)
    i2 = pr2["ids"]
    res2, _ = ref.run(pr2["program"], {i2["x"]: x, i2["weight"]: w8, i2["col_scales"]: ws, i2["bias"]: b})
    out["seeded_linear/y_bias"] = res2[i2["y"]]

    # --- seeded: exact Attention, GQA + key mask ---
    B, S, H, KV, D = 2, 40, 4, 2, 128
    q = ob.f32_to_bf16(rng.standard_normal((B, S, H, D)).astype(np.float32))
    k = ob.f32_to_bf16(rng.standard_normal((B, S, KV, D)).astype(np.float32))
    v = ob.f32_to_bf16(rng.standard_normal((B, S, KV, D)).astype(np.float32))
    mask = np.ones((B, S), np.uint8)
    mask[:, 30:35] = 0
    pr = ir.attention_program(B, S, H, KV, D, True)
    ids = pr["ids"]
    res, _ = ref.run(pr["program"], {ids["q"]: q, ids["k"]: k, ids["v"]: v, ids["mask"]: mask})
    out.update({"seeded_attention/q": q, "seeded_attention/k": k, "seeded_attention/v": v,
                "seeded_attention/mask": mask, "seeded_attention/out_exact": res[ids["out"]]})

    path = os.path.join(HERE, "hotpath_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
