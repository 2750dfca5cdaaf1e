"""GPU: the two DiT blocks at the widths of the benchmark configurations -- hidden 3072, 24 heads
of 128, MLP 12288 (MMDiT double-stream block) and FFN 8192 with rotary 96 (video block) -- on a
few hundred tokens with ragged tails, as DiffIR programs through the plugin against the
reference CPU executor running the SAME program on identical seeded weights and inputs.

Two comparisons per block. (1) Gated at the path's bf16 bar (rel-L2 <= 2e-3, cosine >= 0.9999):
against the reference executor with the one Attention op evaluated by the INT8 contract
(tests/block_oracle.py), which checks every other operator of the block at these widths and the
attention kernel against its contract. (2) Against the reference executor as it is, i.e. with
exact attention: gated at the reference's own bar for an INT8 attention route (cosine >= 0.9999,
reference tests/owned_attention_tests.cpp:122-157) and at rel-L2 <= 1e-2; the measured rel-L2
(about 4e-3 at these widths) is printed. It exceeds 2e-3 by construction: the INT8 codes of Q and K
put the attention output about 5e-3 from the exact one, and every W8A8 linear behind it turns that
into a difference of the size of its own quantisation noise. What these sizes add over the small-width
block tests: ConvRot over 12 (K=3072), 32 (K=8192) and 48 (K=12288) rotation groups inside a
block, 24-head indexing of the fused QKV slices, and the <96, half-split> RoPE with 3-axis
tables. Graph shapes follow the reference's frontends (src/frontend/flux2.cpp:64-445,
tools/difc.cpp:261-345)."""
import numpy as np
import pytest

import oracle_bridge as ob
from block_oracle import reference_with_int8_attention
from diffusion_compiler_b200 import blocks
from helpers import cosine, rel_l2

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")]


def _compare(got, contract, exact, key):
    a, b, e = ob.bf16_to_f32(got), ob.bf16_to_f32(contract), ob.bf16_to_f32(exact)
    assert np.isfinite(a).all()
    r, c = rel_l2(a, b), cosine(a, b)
    r3, c3 = rel_l2(a, e), cosine(a, e)
    print("%s: vs reference with the INT8 attention contract rel-L2 %.3e cosine %.7f; "
          "vs reference with exact attention rel-L2 %.3e cosine %.7f" % (key, r, c, r3, c3))
    assert r <= 2e-3 and c >= 0.9999, (key, r, c)
    assert c3 >= 0.9999 and r3 <= 1e-2, (key, r3, c3)


def test_video_block_at_benchmark_widths_matches_reference_executor():
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(41)
    S, hidden, heads, dim, ffn, rotary = 3 * 5 * 17 + 45, 3072, 24, 128, 8192, 96  # 300 tokens: 2 tiles + a tail
    positions = blocks.video_positions(grid=(3, 5, 17), text_tokens=45)
    quantize = blocks.gpu_weight_quantizer("cuda")  # bit-identical to the CPU packer (checked elsewhere)
    p, ids, consts, inputs = blocks.synth_video_block(rng, S, hidden, heads, dim, ffn, rotary, quantize,
                                                      positions=positions)
    ob.orc().lib.orc_set_threads(8)
    exact, _ = ob.ref().run(p, {**consts, **inputs})
    contract = reference_with_int8_attention(p, {**consts, **inputs})
    ex = plugin.PluginExecutor(0)
    prepared = ex.prepare(p, consts)
    got, _ = prepared.run(inputs)
    prepared.close()
    ex.close()
    _compare(got[ids["out"]], contract[ids["out"]], exact[ids["out"]], "video block 3072/24/8192")


def test_mmdit_block_at_benchmark_widths_matches_reference_executor():
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(43)
    quantize = blocks.gpu_weight_quantizer("cuda")
    # batch 2, 9 x 13 image tokens + 19 text tokens = 136 tokens per batch entry (one tile + a tail)
    p, ids, consts, inputs = blocks.synth_mmdit_block(rng, batch=2, grid=(9, 13), text_tokens=19, hidden=3072,
                                                     heads=24, mlp=12288, quantize=quantize)
    ob.orc().lib.orc_set_threads(8)
    exact, _ = ob.ref().run(p, {**consts, **inputs})
    contract = reference_with_int8_attention(p, {**consts, **inputs})
    ex = plugin.PluginExecutor(0)
    prepared = ex.prepare(p, consts)
    got, _ = prepared.run(inputs)
    prepared.close()
    ex.close()
    for key in ("image_out", "text_out"):
        _compare(got[ids[key]], contract[ids[key]], exact[ids[key]], "MMDiT block 3072/24/12288 " + key)
