"""DiT block graphs built from the hot-path opcodes, and their seeded synthetic tensors.

Two block shapes, both W8A8-rewritten (every Linear is QuantizeInt8Rows(H256ConvRot) +
LinearInt8Scaled, the pattern of reference ``tools/difflux2sample.cpp:2017-2069``) and with
``Attention(Implementation=2)`` so that a backend may bind its INT8 lowering:

* ``mmdit_double_stream_program``: the MMDiT double-stream block in the op sequence of the
  reference's FLUX.2 frontend (``src/frontend/flux2.cpp:64-445``): per stream adaLN
  (LayerNormModulate) -> fused QKV -> slice/reshape -> RMS-norm + interleaved RoPE
  (QkNormPartialRope, Implementation 2) -> concat(text, image) -> joint Attention -> slice ->
  out-proj -> gated residual -> adaLN -> MLP (GELU-tanh) -> gated residual. Dimensions are free
  (benchmark configuration 3: hidden 3072, 24 heads x 128, MLP 12288, 2-axis RoPE theta 10000).
* ``video_block_program``: the single-stream video block the reference emits with
  ``difc make-h3-block-bf16`` (``tools/difc.cpp:261-345``): RmsNormModulate -> q/k/v -> half-split
  partial RoPE -> Attention -> out -> ResidualGate -> RmsNormModulate -> fc1 -> SwiGlu -> fc2 ->
  ResidualGate (benchmark configuration 4: 33272 tokens, hidden 3072, 24 x 128, FFN 8192, rotary 96).

Everything here is host-side graph/tensor construction (numpy); kernels are reached through the
plugin (``plugin.py``) or the device API (``ops.py``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import numpy as np

from .diffir import Attribute, AttrKey, DType, Opcode, Program, Role

H256 = 2


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounding = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    return ((bits + rounding) >> np.uint32(16)).astype(np.uint16)


class _Builder:
    def __init__(self):
        self.p = Program()
        self.linears: Dict[str, Tuple[int, int, int, int, int]] = {}  # name -> (w, cs, bias|0, N, K)

    def bf16(self, dims, role=Role.Internal):
        return self.p.add_tensor(DType.BF16, dims, role)

    def quantize(self, x, lead, K):
        rows = int(np.prod(lead))
        codes = self.p.add_tensor(DType.I8, list(lead) + [K])
        scales = self.p.add_tensor(DType.F32, [rows])
        self.p.add_op(Opcode.QuantizeInt8Rows, [x], [codes, scales],
                      [Attribute.u64(AttrKey.BlockSize, 256), Attribute.u64(AttrKey.Implementation, H256)])
        return codes, scales

    def linear(self, name, quantized, lead, K, N, bias=False, gelu=False, out_role=Role.Internal):
        codes, scales = quantized
        w = self.p.add_tensor(DType.I8, [N, K], Role.Constant)
        cs = self.p.add_tensor(DType.F32, [N], Role.Constant)
        b = self.bf16([N], Role.Constant) if bias else 0
        self.linears[name] = (w, cs, b, N, K)
        last_role = out_role if not bias else Role.Internal
        y = self.bf16(list(lead) + [N], last_role)
        self.p.add_op(Opcode.LinearInt8Scaled, [codes, w, scales, cs], [y])
        if bias:
            yb = self.bf16(list(lead) + [N], Role.Internal if gelu else out_role)
            self.p.add_op(Opcode.BiasAdd, [y, b], [yb])
            y = yb
            if gelu:
                yg = self.bf16(list(lead) + [N], out_role)
                self.p.add_op(Opcode.Gelu, [y], [yg], [Attribute.u64(AttrKey.Approximation, 1)])
                y = yg
        return y


def mmdit_double_stream_program(batch: int, image_tokens: int, text_tokens: int, hidden: int = 3072,
                                heads: int = 24, head_dim: int = 128, mlp: int = 12288, axes_dims=(64, 64),
                                theta: float = 10000.0):
    """Returns (program, ids). ids carries the input/output tensor ids and ``linears``:
    name -> (weight id, column-scale id, bias id, N, K) for the eight quantized linears."""
    assert heads * head_dim == hidden and sum(axes_dims) == head_dim
    b = _Builder()
    p = b.p
    total = text_tokens + image_tokens
    img = b.bf16([batch, image_tokens, hidden], Role.Input)
    txt = b.bf16([batch, text_tokens, hidden], Role.Input)
    pos = p.add_tensor(DType.F32, [batch, total, len(axes_dims)], Role.Input)
    img_mod = b.bf16([batch, 6, hidden], Role.Input)
    txt_mod = b.bf16([batch, 6, hidden], Role.Input)
    ones, zeros = b.bf16([hidden]), b.bf16([hidden])
    p.add_op(Opcode.Fill, [], [ones], [Attribute.f64(AttrKey.Value, 1.0)])
    p.add_op(Opcode.Fill, [], [zeros], [Attribute.f64(AttrKey.Value, 0.0)])
    pairs = head_dim // 2
    pair_axes = p.add_tensor(DType.I32, [pairs], Role.Constant)
    pair_idx = p.add_tensor(DType.I32, [pairs], Role.Constant)
    axis_dims = p.add_tensor(DType.I32, [len(axes_dims)], Role.Constant)
    cosine = p.add_tensor(DType.F32, [batch, total, pairs])
    sine = p.add_tensor(DType.F32, [batch, total, pairs])
    p.add_op(Opcode.RotaryFrequency, [pos, pair_axes, pair_idx, axis_dims], [cosine, sine],
             [Attribute.f64(AttrKey.Theta, theta), Attribute.f64(AttrKey.Ntk, 1.0)])

    def mods(packed):
        rows = []
        for r in range(6):
            t = b.bf16([batch, 1, hidden])
            p.add_op(Opcode.Slice, [packed], [t], [Attribute.u64(AttrKey.Axis, 1), Attribute.u64(AttrKey.Start, r)])
            rows.append(t)
        return rows

    img_mods, txt_mods = mods(img_mod), mods(txt_mod)

    def modulate(x, rows, shift, scale):
        out = b.bf16([batch, rows, hidden])
        p.add_op(Opcode.LayerNormModulate, [x, ones, zeros, scale, shift], [out],
                 [Attribute.f64(AttrKey.Epsilon, 1e-6), Attribute.u64(AttrKey.BlockSize, 128)])
        return out

    qk_scales = {}

    def make_qkv(x, rows, stream):
        packed = b.linear(stream + ".qkv", b.quantize(x, [batch, rows], hidden), [batch, rows], hidden, 3 * hidden,
                          bias=True)
        out = []
        for i, name in enumerate("qkv"):
            flat = b.bf16([batch, rows, hidden])
            p.add_op(Opcode.Slice, [packed], [flat],
                     [Attribute.u64(AttrKey.Axis, 2), Attribute.u64(AttrKey.Start, i * hidden)])
            shaped = b.bf16([batch, rows, heads, head_dim])
            p.add_op(Opcode.Reshape, [flat], [shaped])
            out.append(shaped)
        start = text_tokens if stream == "img" else 0
        attrs = [Attribute.f64(AttrKey.Epsilon, 1e-6), Attribute.u64(AttrKey.Implementation, 2),
                 Attribute.u64(AttrKey.BlockSize, 128), Attribute.u64(AttrKey.RotaryDim, head_dim),
                 Attribute.u64(AttrKey.Start, start), Attribute.u64(AttrKey.RotaryLayout, 1)]
        for i, name in enumerate("qk"):
            w = b.bf16([head_dim], Role.Constant)
            qk_scales[stream + "." + name + "_norm"] = w
            rot = b.bf16([batch, rows, heads, head_dim])
            p.add_op(Opcode.QkNormPartialRope, [out[i], w, cosine, sine], [rot], attrs)
            out[i] = rot
        return out

    img_attn_in = modulate(img, image_tokens, img_mods[0], img_mods[1])
    txt_attn_in = modulate(txt, text_tokens, txt_mods[0], txt_mods[1])
    iq, ik, iv = make_qkv(img_attn_in, image_tokens, "img")
    tq, tk, tv = make_qkv(txt_attn_in, text_tokens, "txt")

    def concat(t, i):
        c = b.bf16([batch, total, heads, head_dim])
        p.add_op(Opcode.Concat, [t, i], [c], [Attribute.u64(AttrKey.Axis, 1)])
        return c

    q, k, v = concat(tq, iq), concat(tk, ik), concat(tv, iv)
    attn = b.bf16([batch, total, heads, head_dim])
    p.add_op(Opcode.Attention, [q, k, v], [attn],
             [Attribute.u64(AttrKey.KvHeads, heads), Attribute.u64(AttrKey.Implementation, 2)])
    attn_flat = b.bf16([batch, total, hidden])
    p.add_op(Opcode.Reshape, [attn], [attn_flat])
    txt_attn = b.bf16([batch, text_tokens, hidden])
    img_attn = b.bf16([batch, image_tokens, hidden])
    p.add_op(Opcode.Slice, [attn_flat], [txt_attn], [Attribute.u64(AttrKey.Axis, 1), Attribute.u64(AttrKey.Start, 0)])
    p.add_op(Opcode.Slice, [attn_flat], [img_attn],
             [Attribute.u64(AttrKey.Axis, 1), Attribute.u64(AttrKey.Start, text_tokens)])

    def branch(residual, attn_rows, rows, m, stream):
        lead = [batch, rows]
        proj = b.linear(stream + ".proj", b.quantize(attn_rows, lead, hidden), lead, hidden, hidden, bias=True)
        r1 = b.bf16(lead + [hidden])
        p.add_op(Opcode.ResidualGate, [residual, proj, m[2]], [r1])
        mlp_in = modulate(r1, rows, m[3], m[4])
        up = b.linear(stream + ".mlp_up", b.quantize(mlp_in, lead, hidden), lead, hidden, mlp, bias=True, gelu=True)
        down = b.linear(stream + ".mlp_down", b.quantize(up, lead, mlp), lead, mlp, hidden, bias=True)
        out = b.bf16(lead + [hidden], Role.Output)
        p.add_op(Opcode.ResidualGate, [r1, down, m[5]], [out])
        return out

    img_out = branch(img, img_attn, image_tokens, img_mods, "img")
    txt_out = branch(txt, txt_attn, text_tokens, txt_mods, "txt")
    ids = {"image": img, "text": txt, "positions": pos, "image_mod": img_mod, "text_mod": txt_mod,
           "pair_axes": pair_axes, "pair_indices": pair_idx, "axis_dims": axis_dims, "image_out": img_out,
           "text_out": txt_out, "linears": b.linears, "qk_scales": qk_scales, "axes_dims": tuple(axes_dims)}
    return p, ids


def video_block_program(S: int, hidden: int = 3072, heads: int = 24, dim: int = 128, ffn: int = 8192,
                        rotary: int = 96):
    """The make-h3-block graph, W8A8-rewritten. Inputs: x and six [S,hidden] modulation tensors
    (scale1, shift1, gate1, scale2, shift2, gate2); constants: norm weights, q/k norm weights,
    cos/sin tables [S,rotary] and the six quantized linears (q, k, v, o, fc1, fc2)."""
    inner = heads * dim
    b = _Builder()
    p = b.p
    x = b.bf16([S, hidden], Role.Input)
    m = [b.bf16([S, hidden], Role.Input) for _ in range(6)]
    w1, w2 = b.bf16([hidden], Role.Constant), b.bf16([hidden], Role.Constant)
    qw, kw = b.bf16([dim], Role.Constant), b.bf16([dim], Role.Constant)
    cosv, sinv = b.bf16([S, rotary], Role.Constant), b.bf16([S, rotary], Role.Constant)
    rms = [Attribute.f64(AttrKey.Epsilon, 1e-5), Attribute.u64(AttrKey.BlockSize, 128)]
    h = b.bf16([S, hidden])
    p.add_op(Opcode.RmsNormModulate, [x, w1, m[0], m[1]], [h], rms)
    hq = b.quantize(h, [S], hidden)
    qkv = []
    for name in ("q", "k", "v"):
        flat = b.linear(name, hq, [S], hidden, inner)
        shaped = b.bf16([S, heads, dim])
        p.add_op(Opcode.Reshape, [flat], [shaped])
        qkv.append(shaped)
    qk_attrs = [Attribute.f64(AttrKey.Epsilon, 1e-5), Attribute.u64(AttrKey.RotaryDim, rotary),
                Attribute.u64(AttrKey.BlockSize, 128)]
    q = b.bf16([S, heads, dim])
    k = b.bf16([S, heads, dim])
    p.add_op(Opcode.QkNormPartialRope, [qkv[0], qw, cosv, sinv], [q], qk_attrs)
    p.add_op(Opcode.QkNormPartialRope, [qkv[1], kw, cosv, sinv], [k], qk_attrs)
    attn = b.bf16([S, heads, dim])
    p.add_op(Opcode.Attention, [q, k, qkv[2]], [attn],
             [Attribute.f64(AttrKey.AttentionScale, 1.0 / np.sqrt(float(dim))),
              Attribute.boolean(AttrKey.Causal, False), Attribute.u64(AttrKey.Implementation, 2)])
    attn_flat = b.bf16([S, inner])
    p.add_op(Opcode.Reshape, [attn], [attn_flat])
    o = b.linear("o", b.quantize(attn_flat, [S], inner), [S], inner, hidden)
    r1 = b.bf16([S, hidden])
    p.add_op(Opcode.ResidualGate, [x, o, m[2]], [r1])
    h2 = b.bf16([S, hidden])
    p.add_op(Opcode.RmsNormModulate, [r1, w2, m[3], m[4]], [h2], rms)
    fc1 = b.linear("fc1", b.quantize(h2, [S], hidden), [S], hidden, 2 * ffn)
    act = b.bf16([S, ffn])
    p.add_op(Opcode.SwiGlu, [fc1], [act])
    fc2 = b.linear("fc2", b.quantize(act, [S], ffn), [S], ffn, hidden)
    out = b.bf16([S, hidden], Role.Output)
    p.add_op(Opcode.ResidualGate, [r1, fc2, m[5]], [out])
    ids = {"x": x, "mods": m, "norm1": w1, "norm2": w2, "q_norm": qw, "k_norm": kw, "cos": cosv, "sin": sinv,
           "out": out, "linears": b.linears}
    return p, ids


# ---------------------------------------------------------------------------------------------
# seeded synthetic tensors
# ---------------------------------------------------------------------------------------------

def video_positions(grid=(21, 30, 52), text_tokens: int = 512) -> np.ndarray:
    """[S,3] (t,h,w) positions: latent grid tokens then text tokens at (index, 0, 0), the
    convention of the reference's H3 conditioning (src/frontend/h3_conditioning.cpp:152-215)."""
    t, h, w = np.meshgrid(np.arange(grid[0]), np.arange(grid[1]), np.arange(grid[2]), indexing="ij")
    lat = np.stack([t.ravel(), h.ravel(), w.ravel()], axis=1).astype(np.float32)
    text = np.zeros((text_tokens, 3), np.float32)
    text[:, 0] = np.arange(text_tokens)
    return np.concatenate([lat, text], axis=0)


def rope_tables_3axis(positions: np.ndarray, rotary: int = 96, theta: float = 10000.0):
    """bf16 cos/sin tables [S, rotary] for half-split partial RoPE over 3 axes: rotary/2 angles
    (16 frequencies per axis), materialised for both halves as the H3 block expects."""
    per_axis = rotary // 2 // positions.shape[1]
    freqs = theta ** (-np.arange(per_axis, dtype=np.float64) / per_axis)
    angles = np.concatenate([positions[:, a:a + 1].astype(np.float64) * freqs[None, :]
                             for a in range(positions.shape[1])], axis=1)
    angles = np.concatenate([angles, angles], axis=1)
    return f32_to_bf16(np.cos(angles).astype(np.float32)), f32_to_bf16(np.sin(angles).astype(np.float32))


def image_positions_2axis(batch: int, text_tokens: int, grid=(64, 64)) -> np.ndarray:
    """F32 [B, text+image, 2]: text tokens at (0,0), image tokens at (row, col)."""
    r, c = np.meshgrid(np.arange(grid[0]), np.arange(grid[1]), indexing="ij")
    img = np.stack([r.ravel(), c.ravel()], axis=1).astype(np.float32)
    pos = np.concatenate([np.zeros((text_tokens, 2), np.float32), img], axis=0)
    return np.ascontiguousarray(np.broadcast_to(pos[None], (batch,) + pos.shape))


def rope_pair_maps(axes_dims) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    pair_axes, pair_idx = [], []
    for a, d in enumerate(axes_dims):
        for i in range(d // 2):
            pair_axes.append(a)
            pair_idx.append(i)
    return (np.array(pair_axes, np.int32), np.array(pair_idx, np.int32), np.array(axes_dims, np.int32))


def random_bf16(rng: np.random.Generator, shape, std: float) -> np.ndarray:
    return f32_to_bf16((rng.standard_normal(shape) * std).astype(np.float32))


def gpu_weight_quantizer(device="cuda"):
    """Weight-side ConvRot on the GPU: QuantizeInt8Rows(H256ConvRot) applied to the rows of a
    bf16 [N,K] weight matrix, which is the reference's offline weight transform with clip 1 and
    no MSE search (reference tools/difflux2sample.cpp:2994-3059)."""
    import torch
    from . import ops

    def quantize(w_bits: np.ndarray):
        w = torch.from_numpy(np.ascontiguousarray(w_bits).view(np.int16)).to(device).view(torch.bfloat16)
        codes, scales = ops.quantize_int8_rows([w], H256)
        return codes.cpu().numpy(), scales.cpu().numpy()

    return quantize


def synth_linears(rng: np.random.Generator, linears, quantize, bias_std: float = 0.01):
    """Seeded N(0,0.02) bf16 weights, ConvRot-quantised by ``quantize``, plus N(0,0.01) biases.
    Returns {tensor id: array} for every constant of the linears."""
    consts = {}
    for name, (w, cs, b, N, K) in linears.items():
        w8, ws = quantize(random_bf16(rng, (N, K), 0.02))
        consts[w], consts[cs] = w8, ws
        if b:
            consts[b] = random_bf16(rng, (N,), bias_std)
    return consts


def synth_video_block(rng: np.random.Generator, S: int, hidden: int, heads: int, dim: int, ffn: int, rotary: int,
                      quantize, positions: np.ndarray = None):
    """(program, ids, constants, inputs) of a video block with seeded synthetic tensors.
    Modulation tensors are broadcast from one conditioning vector through a random linear map,
    as benchmark configuration 4 describes."""
    p, ids = video_block_program(S, hidden, heads, dim, ffn, rotary)
    consts = synth_linears(rng, ids["linears"], quantize)
    one_h = f32_to_bf16(np.ones(hidden, np.float32))
    one_d = f32_to_bf16(np.ones(dim, np.float32))
    consts[ids["norm1"]], consts[ids["norm2"]] = one_h, one_h.copy()
    consts[ids["q_norm"]], consts[ids["k_norm"]] = one_d, one_d.copy()
    if positions is None:
        positions = np.stack([np.arange(S) // 16, (np.arange(S) // 4) % 4, np.arange(S) % 4], axis=1).astype(np.float32)
    consts[ids["cos"]], consts[ids["sin"]] = rope_tables_3axis(positions, rotary)
    cond = rng.standard_normal(hidden).astype(np.float32)
    proj = (rng.standard_normal((6, hidden, 64)) * 0.02).astype(np.float32)
    inputs = {ids["x"]: random_bf16(rng, (S, hidden), 1.0)}
    for i, m in enumerate(ids["mods"]):
        vec = (proj[i] @ cond[:64]).astype(np.float32)
        inputs[m] = f32_to_bf16(np.ascontiguousarray(np.broadcast_to(vec[None, :], (S, hidden))))
    return p, ids, consts, inputs


def synth_mmdit_block(rng: np.random.Generator, batch: int, grid, text_tokens: int, hidden: int, heads: int,
                      mlp: int, quantize):
    """(program, ids, constants, inputs) of an MMDiT double-stream block with seeded tensors."""
    image_tokens = grid[0] * grid[1]
    head_dim = hidden // heads
    p, ids = mmdit_double_stream_program(batch, image_tokens, text_tokens, hidden, heads, head_dim, mlp,
                                         axes_dims=(head_dim // 2, head_dim // 2))
    consts = synth_linears(rng, ids["linears"], quantize)
    for tid in ids["qk_scales"].values():
        consts[tid] = f32_to_bf16(np.ones(head_dim, np.float32))
    pa, pi, ad = rope_pair_maps(ids["axes_dims"])
    consts[ids["pair_axes"]], consts[ids["pair_indices"]], consts[ids["axis_dims"]] = pa, pi, ad
    cond = rng.standard_normal(hidden).astype(np.float32)
    inputs = {ids["image"]: random_bf16(rng, (batch, image_tokens, hidden), 1.0),
              ids["text"]: random_bf16(rng, (batch, text_tokens, hidden), 1.0),
              ids["positions"]: image_positions_2axis(batch, text_tokens, grid)}
    for key in ("image_mod", "text_mod"):
        proj = (rng.standard_normal((6, hidden, 64)) * 0.02).astype(np.float32)
        mod = np.stack([proj[i] @ cond[:64] for i in range(6)], axis=0).astype(np.float32)
        inputs[ids[key]] = f32_to_bf16(np.ascontiguousarray(np.broadcast_to(mod[None], (batch, 6, hidden))))
    return p, ids, consts, inputs
