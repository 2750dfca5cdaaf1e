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


@pytest.mark.parametrize("B,Sq,Sk,H,KV,masked,q_gain", [(1, 300, 1100, 4, 2, True, 1.0), (2, 256, 640, 2, 2, False, 1.0),
                                                        (1, 200, 900, 2, 1, True, 6.0)])
def test_attention_chunked_launches_match_the_single_launch(ops, B, Sq, Sk, H, KV, masked, q_gain):
    """The chunked form (keys taken in several launches that carry m, l and the fp32 outputs of
    every query row) against the single launch over all keys: in ring order as the token-sharded
    block consumes slices (own slice first, then the others, one group wrapping around the end of
    the key axis), also with the running-maximum path (q_gain 6). Powers of two scale exactly, so
    only the order of the fp32 sums may differ: rel-L2 <= 1e-4 here, far inside the path's bar."""
    import torch
    rng = np.random.default_rng(300 + Sk)
    q, _, _ = _qkv(rng, B, Sq, H, KV)
    _, k, v = _qkv(rng, B, Sk, H, KV)
    if q_gain != 1.0:
        q = ob.f32_to_bf16(ob.bf16_to_f32(q) * np.float32(q_gain))
    valid = None
    if masked:
        valid = np.ones((B, Sk), np.uint8)
        valid[:, 250:260] = 0          # a padded slice tail in the middle of the key axis
        valid[:, Sk - 37:] = 0
    q8, qs = ob.orc().quantize_int8_rows([q.reshape(-1, 128)], 1)
    k8, ks = ob.orc().quantize_int8_rows([k.reshape(-1, 128)], 1)
    t = lambda a: torch.from_numpy(a).cuda()
    args = (t(q8.reshape(B, Sq, H, 128)), t(qs), t(k8.reshape(B, Sk, KV, 128)), t(ks), to_torch_bf16(v))
    tv = None if valid is None else t(valid)
    whole = ops.attention_int8(*args, tv)
    tiles = (Sk + 127) // 128
    own = 2 if tiles > 3 else 1  # "this rank's slice" starts at tile `own`
    groups = [[(own, 1)], [(own + 1, tiles - own - 1), (0, 1)], [(1, own - 1)]] if own == 2 else \
             [[(own, 1)], [(own + 1, tiles - own - 1), (0, 1)]]
    groups = [[r for r in g if r[1] > 0] for g in groups]
    groups = [g for g in groups if g]
    parts = ops.attention_int8_chunked(*args, groups, tv)
    same_order = ops.attention_int8_chunked(*args, [[(0, 1)], [(1, tiles - 1)]], tv) if tiles > 1 else whole
    torch.cuda.synchronize()
    ops.poll_status()
    a, b, c = (ob.bf16_to_f32(from_torch_bf16(x)) for x in (parts, whole, same_order))
    assert np.isfinite(a).all()
    assert rel_l2(a, b) <= 1e-4 and cosine(a, b) >= 0.999999, (rel_l2(a, b), cosine(a, b))
    # same tile order as the single launch: the carried state continues the very same sums
    assert np.array_equal(from_torch_bf16(same_order), from_torch_bf16(whole)) or rel_l2(c, b) <= 1e-5


@pytest.mark.parametrize("size,grouping", [(2, ()), (4, ()), (8, ()), (8, (1, 2, 5)), (8, (1, 3, 4))])
def test_attention_launch_plans_of_every_rank_match_the_single_launch(ops, size, grouping):
    """The launch plan the token-sharded mode uses (difb200_world_plan: the own slice first, the other
    slices in the groups their ring steps arrive in, ranges that wrap around the end of the key
    axis) for every rank of a world of 2, 4 and 8, on one GPU: each rank's queries against the whole
    gathered key axis in its planned launches must equal the single launch over all keys."""
    import ctypes as C
    import torch
    from diffusion_compiler_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(500 + size)
    H, KV, slice_tokens, local = 2, 2, 256, 200      # slices padded to 2 key tiles, 200 real tokens each
    Sk = size * slice_tokens
    _, k, v = _qkv(rng, 1, Sk, H, KV)
    valid = np.zeros((1, Sk), np.uint8)
    for r in range(size):
        valid[0, r * slice_tokens:r * slice_tokens + local] = 1
    k8, ks = ob.orc().quantize_int8_rows([k.reshape(-1, 128)], 1)
    t = lambda a: torch.from_numpy(a).cuda()
    keys = (t(k8.reshape(1, Sk, KV, 128)), t(ks), to_torch_bf16(v))
    for rank in range(size):
        q, _, _ = _qkv(rng, 1, local, H, KV)
        q8, qs = ob.orc().quantize_int8_rows([q.reshape(-1, 128)], 1)
        cap = 16
        ranges, first, count, n = (C.c_uint32 * (4 * cap))(), (C.c_int32 * cap)(), (C.c_int32 * cap)(), C.c_int32(0)
        sizes = (C.c_int32 * max(1, len(grouping)))(*grouping)
        assert lib.difb200_world_plan(rank, size, slice_tokens // 128, sizes, len(grouping), ranges, first, count, cap,
                                      C.byref(n)) == 0
        groups = [[(ranges[4 * i], ranges[4 * i + 1])] + ([(ranges[4 * i + 2], ranges[4 * i + 3])] if ranges[4 * i + 3] else [])
                  for i in range(n.value)]
        args = (t(q8.reshape(1, local, H, 128)), t(qs)) + keys
        whole = ops.attention_int8(*args, t(valid))
        parts = ops.attention_int8_chunked(*args, groups, t(valid))
        torch.cuda.synchronize()
        a, b = (ob.bf16_to_f32(from_torch_bf16(x)) for x in (parts, whole))
        # Another key order: the fp32 sums of the tensor cores round elsewhere, which moves about one
        # bf16 output in a thousand by one step (rel-L2 near 1e-4). A slice read twice, skipped or taken
        # from the wrong place would show as whole rows off by far more than one step.
        assert np.isfinite(a).all() and rel_l2(a, b) <= 3e-4, (size, rank, rel_l2(a, b))
        assert np.all(np.abs(a - b) <= 2.0 ** -7 * np.abs(b) + 1e-3 * np.abs(b).max()), (size, rank)
        assert np.mean(a != b) <= 0.01, (size, rank, float(np.mean(a != b)))
    ops.poll_status()
