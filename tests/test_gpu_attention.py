"""GPU parity of INT8 attention (difb200_attention_int8 / difb200_attention through the C-ABI)
against the CPU oracle.

Tier 1 (gated, the north star's bf16 bar: rel-L2 <= 2e-3, cosine >= 0.9999): kernel vs
orc_attention_int8, the CPU statement of the kernel's numerical contract on the same INT8 codes.
Tier 3 (gated with the reference's own bar for its INT8 attention, cosine >= 0.9999, reference
tests/owned_attention_tests.cpp:122-157): kernel vs the exact Attention of the reference CPU
executor (restated in orc_attention_exact, bit-identical to it)."""
import numpy as np
import pytest

import oracle_bridge as ob
from helpers import bf16_normal, cosine, from_torch_bf16, rel_l2, to_torch_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from diffusion_compiler_b200 import ops as _ops
    return _ops


def _qkv(rng, B, S, H, KV, D=128):
    """N(0,1) bf16 q/k/v, q and k RMS-normalised per token-head as a DiT block does."""
    one = ob.f32_to_bf16(np.ones(D, np.float32))
    q = ob.orc().rms_norm(bf16_normal(rng, (B, S, H, D)), one, 1e-6)
    k = ob.orc().rms_norm(bf16_normal(rng, (B, S, KV, D)), one, 1e-6)
    v = bf16_normal(rng, (B, S, KV, D))
    return q, k, v


def _check(ops, B, S, H, KV, masked, seed, q_gain=1.0):
    import torch
    rng = np.random.default_rng(seed)
    ob.orc().lib.orc_set_threads(8)
    q, k, v = _qkv(rng, B, S, H, KV)
    if q_gain != 1.0:
        q = ob.f32_to_bf16(ob.bf16_to_f32(q) * np.float32(q_gain))
    valid = None
    if masked:
        valid = np.ones((B, S), np.uint8)
        valid[:, max(0, S - max(1, S // 5)):] = 0  # the last fifth of the keys is padding
        valid[0, 0] = 0
    q8, qs = ob.orc().quantize_int8_rows([q.reshape(-1, 128)], 1)
    k8, ks = ob.orc().quantize_int8_rows([k.reshape(-1, 128)], 1)
    q8, k8 = q8.reshape(B, S, H, 128), k8.reshape(B, S, KV, 128)
    want = ob.orc().attention_int8(q8, qs, k8, ks, v, valid)
    t = lambda a: torch.from_numpy(a).cuda()
    tv = None if valid is None else t(valid)
    got = ops.attention_int8(t(q8), t(qs), t(k8), t(ks), to_torch_bf16(v), tv)
    got2 = ops.attention(to_torch_bf16(q), to_torch_bf16(k), to_torch_bf16(v), tv)
    torch.cuda.synchronize()
    ops.poll_status()
    g, g2, w = (ob.bf16_to_f32(from_torch_bf16(x)) if not isinstance(x, np.ndarray) else ob.bf16_to_f32(x)
                for x in (got, got2, want))
    assert np.isfinite(g).all()
    # quantising q/k on the GPU gives the same codes, hence the same output bits
    assert np.array_equal(from_torch_bf16(got), from_torch_bf16(got2))
    r, c = rel_l2(g, w), cosine(g, w)
    assert r <= 2e-3 and c >= 0.9999, "tier 1: rel-L2 %.3e cosine %.6f" % (r, c)
    if q_gain != 1.0:
        return r, c, None, None
    exact = ob.bf16_to_f32(ob.orc().attention_exact(q, k, v, valid))
    c3, r3 = cosine(g, exact), rel_l2(g, exact)
    assert c3 >= 0.9999, "tier 3: cosine vs exact attention %.6f (rel-L2 %.3e)" % (c3, r3)
    return r, c, r3, c3


@pytest.mark.parametrize("S", [1, 31, 128, 129, 300, 640])
def test_attention_int8_sizes(ops, S):
    _check(ops, 1, S, 2, 2, False, 10 + S)


@pytest.mark.parametrize("B,S,H,KV,masked", [(2, 384, 4, 4, True), (2, 300, 6, 2, True), (1, 520, 8, 1, False),
                                             (2, 257, 3, 3, True)])
def test_attention_int8_gqa_and_mask(ops, B, S, H, KV, masked):
    _check(ops, B, S, H, KV, masked, 77)


@pytest.mark.parametrize("B,S,H,KV,masked", [(1, 300, 2, 2, False), (2, 384, 4, 2, True)])
def test_attention_int8_running_maximum_path(ops, B, S, H, KV, masked):
    """Queries six times larger than a normalised block's: the score bound exceeds the limit of
    the fixed-maximum path, so the kernel keeps a running maximum and rescales its output (tier 1
    only: with logits this peaked the INT8 codes themselves move the exact result)."""
    _check(ops, B, S, H, KV, masked, 91, q_gain=6.0)


def test_attention_all_keys_masked_gives_zero(ops):
    import torch
    rng = np.random.default_rng(5)
    B, S, H, KV = 1, 200, 2, 2
    q, k, v = _qkv(rng, B, S, H, KV)
    valid = torch.zeros(B, S, dtype=torch.uint8, device="cuda")
    out = ops.attention(to_torch_bf16(q), to_torch_bf16(k), to_torch_bf16(v), valid)
    torch.cuda.synchronize()
    assert torch.count_nonzero(out.float()) == 0
    ops.poll_status()


def test_attention_repeatable(ops):
    """Two runs give identical bits (reference gate: repeat-bit-exact, owned_attention_tests.cpp:158-159)."""
    import torch
    rng = np.random.default_rng(6)
    q, k, v = _qkv(rng, 1, 1000, 4, 2)
    a = ops.attention(to_torch_bf16(q), to_torch_bf16(k), to_torch_bf16(v))
    b = ops.attention(to_torch_bf16(q), to_torch_bf16(k), to_torch_bf16(v))
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
