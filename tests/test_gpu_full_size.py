"""Parity at the benchmark's full sizes, where the CPU oracle cannot run everything: rows are
independent in every operator of the path, so a sample of rows checked bit for bit against the
oracle, together with a whole-tensor property that does not need the oracle (the INT32
accumulators of the whole GEMM against an independent integer matrix product, the dequantisation
round trip of the quantiser), covers the full launch."""
import numpy as np
import pytest

import oracle_bridge as ob
from helpers import cosine, from_torch_bf16, rel_l2, to_torch_bf16

pytestmark = pytest.mark.gpu

M_TOKENS = 9216  # benchmark configuration 1: 2 x 4608 tokens


@pytest.fixture(scope="module")
def ops():
    from diffusion_compiler_b200 import ops as _ops
    return _ops


def _sample_rows(rng, rows, count):
    picks = np.concatenate([[0, 127, 128, 255, 256, rows - 1], rng.integers(0, rows, count)])
    return np.unique(picks)


@pytest.mark.parametrize("K", [3072, 12288])
def test_quantizer_full_size_row_sample_and_round_trip(ops, K):
    import torch
    torch.manual_seed(K)
    x = torch.randn(M_TOKENS, K, device="cuda", dtype=torch.float32)
    x[:, ::97] *= 16.0  # outlier channels
    x = x.to(torch.bfloat16)
    codes, scales = ops.quantize_int8_rows([x], 2)
    torch.cuda.synchronize()
    rows = _sample_rows(np.random.default_rng(K), M_TOKENS, 48)
    host = from_torch_bf16(x[torch.from_numpy(rows).cuda()])
    want_codes, want_scales = ob.orc().quantize_int8_rows([host], 2, 1.0)
    assert np.array_equal(codes.cpu().numpy()[rows], want_codes)
    assert np.array_equal(scales.cpu().numpy()[rows].view(np.uint32), want_scales.view(np.uint32))
    # whole tensor: the rotation is orthogonal, so codes * scale has the input's row norms
    deq = (codes.float() * scales[:, None]).pow(2).sum(1).sqrt()
    ref = x.float().pow(2).sum(1).sqrt()
    assert torch.all((deq / ref - 1).abs() < 0.02)
    assert int(codes.abs().max()) <= 127 or int(codes.min()) == -128
    ops.poll_status()


@pytest.mark.parametrize("N,K,gelu", [(9216, 3072, False), (12288, 3072, True), (3072, 12288, False)])
def test_linear_full_size_accumulators_and_row_sample(ops, N, K, gelu):
    """Benchmark projections at M = 9216: every INT32 accumulator against torch's integer matrix
    product (an independent implementation), a row sample of the bf16 outputs against the oracle."""
    import torch
    torch.manual_seed(N + K)
    x8 = torch.randint(-127, 128, (M_TOKENS, K), device="cuda", dtype=torch.int8)
    w8 = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8)
    xs = torch.rand(M_TOKENS, device="cuda") * 0.02 + 1e-3
    ws = torch.rand(N, device="cuda") * 0.002 + 1e-4
    bias = (torch.randn(N, device="cuda") * 0.01).to(torch.bfloat16)
    out, acc = ops.linear_int8_scaled(x8, w8, xs, ws, want_acc=True)
    want_acc = torch._int_mm(x8, w8.t())
    assert torch.equal(acc, want_acc)
    del acc, want_acc
    got = ops.linear_int8_scaled(x8, w8, xs, ws, bias=bias, gelu=gelu)
    torch.cuda.synchronize()
    rows = _sample_rows(np.random.default_rng(N), M_TOKENS, 10)
    ob.orc().lib.orc_set_threads(8)
    idx = torch.from_numpy(rows).cuda()
    want = ob.orc().linear_int8_scaled(x8[idx].cpu().numpy(), w8.cpu().numpy(), xs[idx].cpu().numpy(),
                                       ws.cpu().numpy())
    assert np.array_equal(from_torch_bf16(out[idx]), want)
    want_b = ob.orc().bias_add(want, from_torch_bf16(bias))
    if not gelu:
        assert np.array_equal(from_torch_bf16(got[idx]), want_b)
    else:
        a = ob.bf16_to_f32(from_torch_bf16(got[idx]))
        b = ob.bf16_to_f32(ob.orc().gelu_tanh(want_b))
        assert rel_l2(a, b) <= 2e-3 and cosine(a, b) >= 0.9999  # the path's bf16 bar
    ops.poll_status()


def test_attention_full_sequence_head_sample(ops):
    """Benchmark configuration 2 (B=2, S=4608, H=24, KV=8 with a key mask): two heads of one batch
    entry against the oracle's statement of the kernel's contract on the same INT8 codes."""
    import torch
    torch.manual_seed(2)
    B, S, H, KV, D = 2, 4608, 24, 8, 128
    rms = lambda t: (t.float() / t.float().pow(2).mean(-1, keepdim=True).add(1e-6).sqrt()).to(torch.bfloat16)
    q = rms(torch.randn(B, S, H, D, device="cuda"))
    k = rms(torch.randn(B, S, KV, D, device="cuda"))
    v = torch.randn(B, S, KV, D, device="cuda").to(torch.bfloat16)
    valid = torch.ones(B, S, dtype=torch.uint8, device="cuda")
    valid[:, -300:] = 0
    q8, qs = ops.quantize_int8_rows([q.view(-1, D)], 1)
    k8, ks = ops.quantize_int8_rows([k.view(-1, D)], 1)
    q8, k8 = q8.view(B, S, H, D), k8.view(B, S, KV, D)
    out = ops.attention_int8(q8, qs, k8, ks, v, valid)
    torch.cuda.synchronize()
    ops.poll_status()
    # heads 3 and 4 of batch 1 share kv head 1 (24 / 8 = 3 query heads per kv head)
    heads, kv = [3, 4], 1
    ob.orc().lib.orc_set_threads(8)
    n = lambda t: np.ascontiguousarray(t.cpu().numpy())
    want = ob.orc().attention_int8(n(q8[1:2, :, heads]), n(qs.view(B, S, H)[1:2, :, heads]).reshape(-1),
                                   n(k8[1:2, :, kv:kv + 1]), n(ks.view(B, S, KV)[1:2, :, kv:kv + 1]).reshape(-1),
                                   from_torch_bf16(v[1:2, :, kv:kv + 1].contiguous()), n(valid[1:2]))
    a = ob.bf16_to_f32(from_torch_bf16(out[1:2, :, heads].contiguous()))
    b = ob.bf16_to_f32(want)
    assert np.isfinite(a).all()
    assert rel_l2(a, b) <= 2e-3 and cosine(a, b) >= 0.9999, (rel_l2(a, b), cosine(a, b))


def _attention_row_sample(ops, B, Sq, Sk, H, KV, masked_tail, heads, n_rows, seed):
    """Runs the kernel on the whole problem and checks a sample of query rows of `heads` (which
    must share one kv head) against the three tiers: the kernel's contract on the same codes
    (gated at the path's bf16 bar), the same codes with fp32 softmax weights (reported) and the
    reference's exact Attention (gated at the reference's own cosine bar). Sq < Sk is the
    token-sharded form (attention is not causal, so where the queries sit in the sequence does not
    enter)."""
    import torch
    torch.manual_seed(seed)
    D = 128
    rms = lambda t: (t.float() / t.float().pow(2).mean(-1, keepdim=True).add(1e-6).sqrt()).to(torch.bfloat16)
    q = rms(torch.randn(B, Sq, H, D, device="cuda"))
    k = rms(torch.randn(B, Sk, KV, D, device="cuda"))
    v = torch.randn(B, Sk, KV, D, device="cuda").to(torch.bfloat16)
    valid = None
    if masked_tail:
        valid = torch.ones(B, Sk, dtype=torch.uint8, device="cuda")
        valid[:, -masked_tail:] = 0
    q8, qs = ops.quantize_int8_rows([q.view(-1, D)], 1)
    k8, ks = ops.quantize_int8_rows([k.view(-1, D)], 1)
    q8, k8 = q8.view(B, Sq, H, D), k8.view(B, Sk, KV, D)
    out = ops.attention_int8(q8, qs, k8, ks, v, valid)
    torch.cuda.synchronize()
    ops.poll_status()
    kv = heads[0] // (H // KV)
    assert all(h // (H // KV) == kv for h in heads)
    b = B - 1
    rows = _sample_rows(np.random.default_rng(seed), Sq, n_rows)
    ridx = torch.from_numpy(rows).cuda()
    n = lambda t: np.ascontiguousarray(t.cpu().numpy())
    q8_s = n(q8[b:b + 1][:, ridx][:, :, heads])
    qs_s = n(qs.view(B, Sq, H)[b:b + 1][:, ridx][:, :, heads]).reshape(-1)
    k8_s, ks_s = n(k8[b:b + 1, :, kv:kv + 1]), n(ks.view(B, Sk, KV)[b:b + 1, :, kv:kv + 1]).reshape(-1)
    v_s = from_torch_bf16(v[b:b + 1, :, kv:kv + 1].contiguous())
    valid_s = None if valid is None else n(valid[b:b + 1])
    ob.orc().lib.orc_set_threads(8)
    got = ob.bf16_to_f32(from_torch_bf16(out[b:b + 1][:, ridx][:, :, heads].contiguous()))
    t1 = ob.bf16_to_f32(ob.orc().attention_int8_rows(q8_s, qs_s, k8_s, ks_s, v_s, valid_s))
    t2 = ob.bf16_to_f32(ob.orc().attention_int8_rows(q8_s, qs_s, k8_s, ks_s, v_s, valid_s, fp32_p=True))
    exact = ob.bf16_to_f32(ob.orc().attention_exact_rows(
        from_torch_bf16(q[b:b + 1][:, ridx][:, :, heads].contiguous()),
        from_torch_bf16(k[b:b + 1, :, kv:kv + 1].contiguous()), v_s, valid_s))
    tiers = {"t1_rel_l2": rel_l2(got, t1), "t1_cosine": cosine(got, t1), "t2_rel_l2": rel_l2(got, t2),
             "t3_rel_l2": rel_l2(got, exact), "t3_cosine": cosine(got, exact)}
    print("attention tiers B=%d Sq=%d Sk=%d H=%d KV=%d: %s" % (B, Sq, Sk, H, KV, tiers))
    assert np.isfinite(got).all()
    assert tiers["t1_rel_l2"] <= 2e-3 and tiers["t1_cosine"] >= 0.9999, tiers
    assert tiers["t3_cosine"] >= 0.9999, tiers
    return tiers


def test_attention_dense_benchmark_shape_row_sample(ops):
    """Benchmark configuration 2, dense variant (B=2, S=4608, 24 query and 24 kv heads)."""
    _attention_row_sample(ops, 2, 4608, 4608, 24, 24, 0, heads=[17], n_rows=96, seed=21)


def test_attention_video_sequence_query_shard_row_sample(ops):
    """The video block's attention as one of eight token shards sees it: 4159 local queries
    against the 33272 keys of the whole sequence (Sq < Sk), 24 heads, the last 40 keys masked as
    the padding of an uneven split would be; rows of two heads against the three tiers."""
    for head in (0, 23):
        _attention_row_sample(ops, 1, 4159, 33272, 24, 24, 40, heads=[head], n_rows=40, seed=33 + head)
