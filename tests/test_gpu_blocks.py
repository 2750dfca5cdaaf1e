"""GPU: whole DiT blocks. (1) the video block and the MMDiT double-stream block as DiffIR programs
through the plugin against the reference CPU executor running the SAME program (its Attention is
exact, ours is the INT8 lowering, so the bar is the north star's bf16 tolerance, not bit-exact);
(2) the token-sharded video block, four ranks emulated one after another on one GPU, against the
unsharded block."""
import numpy as np
import pytest

import oracle_bridge as ob
from diffusion_compiler_b200 import blocks
from helpers import cosine, rel_l2

pytestmark = pytest.mark.gpu


def _cpu_quantize(w_bits):
    return ob.orc().quantize_int8_rows([w_bits], 2)


@pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")
def test_video_block_through_plugin_matches_reference_executor():
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(4)
    S, hidden, heads, dim, ffn, rotary = 400, 512, 4, 128, 1024, 96
    p, ids, consts, inputs = blocks.synth_video_block(rng, S, hidden, heads, dim, ffn, rotary, _cpu_quantize)
    want, _ = ob.ref().run(p, {**consts, **inputs})
    ex = plugin.PluginExecutor(0)
    got, tel = ex.prepare(p, consts).run(inputs)
    a, b = ob.bf16_to_f32(got[ids["out"]]), ob.bf16_to_f32(want[ids["out"]])
    assert np.isfinite(a).all()
    assert rel_l2(a, b) <= 2e-3 and cosine(a, b) >= 0.9999, (rel_l2(a, b), cosine(a, b))
    ex.close()


def test_video_block_replayed_from_cuda_graphs_keeps_the_bits():
    """The block's kernels replayed from four CUDA graphs (captured on the first call for fixed
    tensors) give the bits of the kernel-by-kernel run, also after the inputs change in place."""
    import torch
    from diffusion_compiler_b200 import ops
    from diffusion_compiler_b200.sequence_shard import GatherBuffers, ShardPlan, VideoBlock
    rng = np.random.default_rng(8)
    S, hidden, heads, dim, ffn, rotary = 437, 512, 4, 128, 1024, 96
    p, ids, consts, inputs = blocks.synth_video_block(rng, S, hidden, heads, dim, ffn, rotary, _cpu_quantize)
    tensors = {"norm1": consts[ids["norm1"]], "norm2": consts[ids["norm2"]], "q_norm": consts[ids["q_norm"]],
               "k_norm": consts[ids["k_norm"]], "cos": consts[ids["cos"]], "sin": consts[ids["sin"]],
               "linears": {n: (consts[w], consts[cs]) for n, (w, cs, b, N, K) in ids["linears"].items()}}
    block = VideoBlock(tensors, hidden, heads, dim, ffn, rotary, "cuda")
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.bfloat16)
    x = dev(inputs[ids["x"]])
    mods = [dev(inputs[m]) for m in ids["mods"]]
    plan = ShardPlan.make(S, 1)
    gb = GatherBuffers(plan, 0, heads, dim, "cuda")
    for trial in range(2):
        want = block.forward(x, mods, plan, 0, gb=gb).clone()
        got = block.forward(x, mods, plan, 0, gb=gb, graphs=True).clone()
        torch.cuda.synchronize()
        assert torch.equal(want.view(torch.int16), got.view(torch.int16))
        x.mul_(0.5)  # same storage, new values: the second trial replays the graphs of the first
    ops.poll_status()


def test_plugin_rope_fusions_keep_the_bits(monkeypatch):
    """The planner reads last-axis slices in place from QkNormPartialRope and lets that op write
    the attention kernel's INT8 q / k directly (through a Concat along tokens too). Same arithmetic,
    so the block output must not change by a bit against the unfused plan."""
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(6)
    p, ids, consts, inputs = blocks.synth_mmdit_block(rng, batch=2, grid=(8, 8), text_tokens=24, hidden=512, heads=4,
                                                     mlp=1024, quantize=_cpu_quantize)
    results = []
    for fusion in ("1", "0"):
        monkeypatch.setenv("DIFB200_ROPE_FUSION", fusion)
        ex = plugin.PluginExecutor(0)
        got, _ = ex.prepare(p, consts).run(inputs)
        ex.close()
        results.append(got)
    for key in ("image_out", "text_out"):
        assert np.array_equal(results[0][ids[key]], results[1][ids[key]])


def test_plugin_norm_quant_fusion_saves_the_normalised_tensor_and_stays_in_the_bar(monkeypatch):
    """RmsNormModulate -> QuantizeInt8Rows runs as one kernel in the plugin: the normalised tensors
    are not resident any more, and the block output stays well inside the path's bf16 bar against
    the plan with separate kernels (the row statistic is summed in another order, so single codes
    may move by one)."""
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(12)
    S, hidden, heads, dim, ffn, rotary = 400, 512, 4, 128, 1024, 96
    p, ids, consts, inputs = blocks.synth_video_block(rng, S, hidden, heads, dim, ffn, rotary, _cpu_quantize)
    results, resident = [], []
    monkeypatch.setenv("DIFB200_BUFFER_REUSE", "0")  # residency per tensor, so that the saved tensors show
    for fusion in ("1", "0"):
        monkeypatch.setenv("DIFB200_NORM_FUSION", fusion)
        ex = plugin.PluginExecutor(0)
        prepared = ex.prepare(p, consts)
        got, _ = prepared.run(inputs)
        resident.append(int(prepared.compile_telemetry.resident_bytes))
        ex.close()
        results.append(ob.bf16_to_f32(got[ids["out"]]))
    assert resident[1] - resident[0] >= 2 * S * hidden * 2  # two [S, hidden] bf16 tensors fewer
    assert rel_l2(results[0], results[1]) <= 5e-4 and cosine(results[0], results[1]) >= 0.99999


def test_plugin_buffer_reuse_keeps_the_bits_and_saves_memory(monkeypatch):
    """Internal tensors whose lifetimes do not overlap share device memory (the plugin's default):
    the same bits as with one allocation per tensor and fewer resident bytes,
    also when the same executable runs several passes."""
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(16)
    p, ids, consts, inputs = blocks.synth_mmdit_block(rng, batch=2, grid=(8, 8), text_tokens=24, hidden=512, heads=4,
                                                     mlp=1024, quantize=_cpu_quantize)
    results, resident = [], []
    for reuse in ("1", "0"):
        monkeypatch.setenv("DIFB200_BUFFER_REUSE", reuse)
        ex = plugin.PluginExecutor(0)
        prepared = ex.prepare(p, consts)
        got, _ = prepared.run(inputs, warmups=1, iterations=2)
        again, _ = prepared.run(inputs)
        resident.append(int(prepared.compile_telemetry.resident_bytes))
        ex.close()
        for key in ("image_out", "text_out"):
            assert np.array_equal(got[ids[key]], again[ids[key]])
        results.append(got)
    for key in ("image_out", "text_out"):
        assert np.array_equal(results[0][ids[key]], results[1][ids[key]])
    assert resident[0] < resident[1], resident


@pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")
def test_mmdit_double_stream_block_through_plugin_matches_reference_executor():
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(5)
    p, ids, consts, inputs = blocks.synth_mmdit_block(rng, batch=2, grid=(8, 8), text_tokens=24, hidden=512, heads=4,
                                                     mlp=1024, quantize=_cpu_quantize)
    want, _ = ob.ref().run(p, {**consts, **inputs})
    ex = plugin.PluginExecutor(0)
    got, _ = ex.prepare(p, consts).run(inputs)
    for key in ("image_out", "text_out"):
        a, b = ob.bf16_to_f32(got[ids[key]]), ob.bf16_to_f32(want[ids[key]])
        assert np.isfinite(a).all()
        assert rel_l2(a, b) <= 2e-3 and cosine(a, b) >= 0.9999, (key, rel_l2(a, b), cosine(a, b))
    ex.close()


@pytest.mark.parametrize("S,world", [(512, 4), (437, 4)])
def test_token_sharded_video_block_matches_unsharded(S, world):
    """Ranks are emulated sequentially on one GPU: every rank runs its row-local part, the gather
    is done by copying slices between the per-rank buffers, then every rank attends and finishes.
    Without padding (S divisible) the key order and tiling are those of the unsharded run, so the
    outputs are bit-identical; with padding the fp32 accumulation order shifts (tolerance)."""
    import torch
    from diffusion_compiler_b200 import ops
    from diffusion_compiler_b200.sequence_shard import GatherBuffers, ShardPlan, VideoBlock
    rng = np.random.default_rng(6)
    hidden, heads, dim, ffn, rotary = 512, 4, 128, 1024, 96
    p, ids, consts, inputs = blocks.synth_video_block(rng, S, hidden, heads, dim, ffn, rotary, _cpu_quantize)
    tensors = {"norm1": consts[ids["norm1"]], "norm2": consts[ids["norm2"]], "q_norm": consts[ids["q_norm"]],
               "k_norm": consts[ids["k_norm"]], "cos": consts[ids["cos"]], "sin": consts[ids["sin"]],
               "linears": {n: (consts[w], consts[cs]) for n, (w, cs, b, N, K) in ids["linears"].items()}}
    block = VideoBlock(tensors, hidden, heads, dim, ffn, rotary, "cuda")
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.bfloat16)
    x = dev(inputs[ids["x"]])
    mods = [dev(inputs[m]) for m in ids["mods"]]
    full = block.forward(x, mods, ShardPlan.make(S, 1), 0)
    plan = ShardPlan.make(S, world)
    gbs = [GatherBuffers(plan, r, heads, dim, "cuda") for r in range(world)]
    qs = []
    for r in range(world):
        lo, hi = plan.bounds(r)
        qs.append(block.pre_attention(x[lo:hi].contiguous(), [m[lo:hi].contiguous() for m in mods], plan, r, gbs[r]))
    for r in range(world):  # the all-gather: every rank receives every other rank's slice
        for src in range(world):
            for name in ("k8", "ks", "v"):
                getattr(gbs[r], name)[src * plan.slice_len:(src + 1) * plan.slice_len] = \
                    gbs[src].local(getattr(gbs[src], name))
    outs = []
    for r in range(world):
        lo, hi = plan.bounds(r)
        attn = block.attend(qs[r][0], qs[r][1], plan, gbs[r])
        outs.append(block.post_attention(x[lo:hi].contiguous(), attn, [m[lo:hi].contiguous() for m in mods]))
    sharded = torch.cat(outs, dim=0)
    torch.cuda.synchronize()
    ops.poll_status()
    if S % world == 0:
        assert torch.equal(sharded.view(torch.int16), full.view(torch.int16))
    else:
        a, b = sharded.float().cpu().numpy(), full.float().cpu().numpy()
        assert rel_l2(a, b) <= 1e-3 and cosine(a, b) >= 0.99999
