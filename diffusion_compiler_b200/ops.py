"""Device-resident operators on torch CUDA tensors (torch is only the memory/stream plumbing;
every op below is one call into libdifb200.so).

Names and argument meaning follow the reference opcodes (``QuantizeInt8Rows``,
``LinearInt8Scaled``; reference ``include/dif/ir/ir.hpp:123-139``).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib

EPILOGUE_BIAS = 1
EPILOGUE_GELU_TANH = 2


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _require(t: torch.Tensor, dtype: torch.dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor (there is no CPU path)" % name)
    if t.dtype != dtype:
        raise ValueError("%s must be %s, got %s" % (name, dtype, t.dtype))
    return t.contiguous()


def quantize_int8_rows(parts: Sequence[torch.Tensor], implementation: int = 2, clip: float = 1.0,
                       clip_tensor: Optional[torch.Tensor] = None, residual: bool = False,
                       out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> Tuple[torch.Tensor, ...]:
    """QuantizeInt8Rows: bf16 inputs concatenated on the last axis -> (codes i8, scales f32
    [, residual codes, residual scales]). ``implementation`` is the Int8RowQuantization value.
    ``out`` = (codes, scales) writes into existing contiguous buffers (e.g. a slice of an
    all-gather buffer)."""
    if isinstance(parts, torch.Tensor):
        parts = [parts]
    parts = [_require(p, torch.bfloat16, "input") for p in parts]
    lead = parts[0].shape[:-1]
    rows = 1
    for d in lead:
        rows *= int(d)
    widths = [int(p.shape[-1]) for p in parts]
    for p in parts:
        if p.shape[:-1] != lead:
            raise ValueError("all inputs must share their leading dimensions")
    total = sum(widths)
    dev = parts[0].device
    if out is not None:
        codes, scales = out
        if (codes.dtype != torch.int8 or scales.dtype != torch.float32 or not codes.is_contiguous()
                or not scales.is_contiguous() or codes.numel() != rows * total or scales.numel() != rows):
            raise ValueError("out buffers must be contiguous int8 [rows*width] and float32 [rows]")
    else:
        codes = torch.empty(tuple(lead) + (total,), dtype=torch.int8, device=dev)
        scales = torch.empty((rows,), dtype=torch.float32, device=dev)
    rcodes = torch.empty_like(codes) if residual else None
    rscales = torch.empty_like(scales) if residual else None
    n = len(parts)
    ptrs = (C.c_void_p * n)(*[p.data_ptr() for p in parts])
    ws = (C.c_uint64 * n)(*widths)
    if clip_tensor is not None:
        clip_tensor = _require(clip_tensor, torch.float32, "clip_tensor")
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().difb200_quantize_int8_rows(ptrs, ws, n, rows, int(implementation), float(clip),
                                                         _ptr(clip_tensor), _ptr(codes), _ptr(scales),
                                                         _ptr(rcodes), _ptr(rscales), _stream()))
    return (codes, scales, rcodes, rscales) if residual else (codes, scales)


def rms_norm_modulate_quant(x: torch.Tensor, weight: Optional[torch.Tensor], scale: torch.Tensor,
                            shift: torch.Tensor, epsilon: float = 1e-5, implementation: int = 2, clip: float = 1.0):
    """RmsNormModulate (explicit scale / shift) + QuantizeInt8Rows in one kernel: bf16 [M, K] inputs
    -> (codes i8 [M, K], row scales f32 [M]); the normalised tensor is never written."""
    x = _require(x, torch.bfloat16, "x")
    scale, shift = _require(scale, torch.bfloat16, "scale"), _require(shift, torch.bfloat16, "shift")
    if weight is not None:
        weight = _require(weight, torch.bfloat16, "weight")
    M, K = x.shape
    if scale.shape != x.shape or shift.shape != x.shape:
        raise ValueError("scale and shift must have the shape of x")
    codes = torch.empty((M, K), dtype=torch.int8, device=x.device)
    scales = torch.empty((M,), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().difb200_rms_norm_modulate_quant(_ptr(x), _ptr(weight), _ptr(scale), _ptr(shift), M, K,
                                                           epsilon, implementation, clip, _ptr(codes), _ptr(scales),
                                                           _stream()))
    return codes, scales


def layer_norm_modulate_quant(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, scale: torch.Tensor,
                              shift: torch.Tensor, epsilon: float = 1e-5, implementation: int = 2,
                              clip: float = 1.0):
    """LayerNormModulate + QuantizeInt8Rows in one kernel: x bf16 [M, K], weight / bias bf16 [K],
    scale / shift bf16 [M / r, K] (r rows of x share one modulation row) -> (codes i8 [M, K], row
    scales f32 [M])."""
    x = _require(x, torch.bfloat16, "x")
    weight, bias = _require(weight, torch.bfloat16, "weight"), _require(bias, torch.bfloat16, "bias")
    scale, shift = _require(scale, torch.bfloat16, "scale"), _require(shift, torch.bfloat16, "shift")
    M, K = x.shape
    if scale.shape != shift.shape or scale.shape[-1] != K or M % scale.shape[0] != 0:
        raise ValueError("scale and shift must be [M / r, K]")
    codes = torch.empty((M, K), dtype=torch.int8, device=x.device)
    scales = torch.empty((M,), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().difb200_layer_norm_modulate_quant(_ptr(x), _ptr(weight), _ptr(bias), _ptr(scale), _ptr(shift),
                                                             M, K, M // scale.shape[0], epsilon, implementation, clip,
                                                             _ptr(codes), _ptr(scales), _stream()))
    return codes, scales


def weight_equalization(weight: torch.Tensor) -> torch.Tensor:
    """The offline packer's input-equalisation vector for a bf16 [N, K] weight (reference
    tools/difflux2sample.cpp:2967-2990): sqrt(column absmax / geometric mean of the column
    absmaxes), clamped to [0.5, 2], as bf16 [K]. Weights are divided by it before packing and
    activations multiplied by it at run time."""
    weight = _require(weight, torch.bfloat16, "weight")
    maxima = weight.float().abs().amax(dim=0)
    logs = torch.log(torch.clamp(maxima, min=1.0e-30)).double()
    center = torch.exp(logs.sum() / maxima.numel()).float()
    ratio = torch.sqrt(maxima / torch.clamp(center, min=1.0e-30))
    return torch.clamp(ratio, 0.5, 2.0).to(torch.bfloat16)


def quantize_weight_rows(weight: torch.Tensor, implementation: int = 2, mse_scale: bool = False,
                         input_scale: Optional[torch.Tensor] = None):
    """Weight-side packing of a bf16 [N, K] matrix: I8 codes [N, K] and per-output-channel scales
    [N] (reference tools/difflux2sample.cpp:2994-3059); ``mse_scale`` picks each row's scale by the
    offline packer's MSE search (:1225-1259); ``input_scale`` is the bf16 [K] equalisation vector
    the weights are divided by first."""
    weight = _require(weight, torch.bfloat16, "weight")
    if weight.dim() != 2:
        raise ValueError("weight must be a bf16 [N, K] matrix")
    N, K = weight.shape
    if input_scale is not None:
        input_scale = _require(input_scale, torch.bfloat16, "input_scale")
        if input_scale.numel() != K:
            raise ValueError("input_scale must have K entries")
    codes = torch.empty((N, K), dtype=torch.int8, device=weight.device)
    scales = torch.empty((N,), dtype=torch.float32, device=weight.device)
    _lib.check(_lib.lib().difb200_quantize_weight_rows(_ptr(weight), _ptr(input_scale), N, K, implementation,
                                                        1 if mse_scale else 0, _ptr(codes), _ptr(scales), _stream()))
    return codes, scales


def linear_int8_scaled(x8: torch.Tensor, w8: torch.Tensor, row_scales: torch.Tensor,
                       col_scales: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False,
                       want_acc: bool = False, out: Optional[torch.Tensor] = None):
    """LinearInt8Scaled (+ fused BiasAdd / tanh-Gelu): x8 [..,K] i8, w8 [N,K] i8 -> bf16 [..,N]."""
    x8 = _require(x8, torch.int8, "x8")
    w8 = _require(w8, torch.int8, "w8")
    row_scales = _require(row_scales, torch.float32, "row_scales")
    col_scales = _require(col_scales, torch.float32, "col_scales")
    K = int(x8.shape[-1])
    M = x8.numel() // K
    N = int(w8.shape[0])
    if w8.shape[1] != K or row_scales.numel() != M or col_scales.numel() != N:
        raise ValueError("shapes must flatten as [M,K] x [N,K] with row [M] and column [N] scales")
    flags = 0
    if bias is not None:
        bias = _require(bias, torch.bfloat16, "bias")
        flags |= EPILOGUE_BIAS
    if gelu:
        flags |= EPILOGUE_GELU_TANH
    if out is None:
        out = torch.empty(tuple(x8.shape[:-1]) + (N,), dtype=torch.bfloat16, device=x8.device)
    acc = torch.empty((M, N), dtype=torch.int32, device=x8.device) if want_acc else None
    with torch.cuda.device(x8.device):
        _lib.check(_lib.lib().difb200_linear_int8_scaled(_ptr(x8), _ptr(w8), _ptr(row_scales), _ptr(col_scales),
                                                         _ptr(bias), flags, M, N, K, _ptr(out), _ptr(acc),
                                                         _stream()))
    return (out, acc) if want_acc else out


def w8a8_linear(x: torch.Tensor, w8: torch.Tensor, col_scales: torch.Tensor,
                bias: Optional[torch.Tensor] = None, gelu: bool = False, implementation: int = 2,
                clip: float = 1.0, out: Optional[torch.Tensor] = None,
                scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """The W8A8 int8-convrot linear in one call: quantize x [..,K] bf16, multiply with w8 [N,K].
    ``scratch`` = (codes int8 [M,K], row scales f32 [M]) may be passed to reuse buffers."""
    x = _require(x, torch.bfloat16, "x")
    w8 = _require(w8, torch.int8, "w8")
    col_scales = _require(col_scales, torch.float32, "col_scales")
    K = int(x.shape[-1])
    M = x.numel() // K
    N = int(w8.shape[0])
    flags = 0
    if bias is not None:
        bias = _require(bias, torch.bfloat16, "bias")
        flags |= EPILOGUE_BIAS
    if gelu:
        flags |= EPILOGUE_GELU_TANH
    if scratch is None:
        scratch = (torch.empty((M, K), dtype=torch.int8, device=x.device),
                   torch.empty((M,), dtype=torch.float32, device=x.device))
    codes, scales = scratch
    if codes.numel() < M * K or scales.numel() < M:
        raise ValueError("scratch buffers are too small")
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().difb200_w8a8_linear(_ptr(x), _ptr(w8), _ptr(col_scales), _ptr(bias), flags,
                                                  int(implementation), float(clip), M, N, K, _ptr(codes),
                                                  _ptr(scales), _ptr(out), _stream()))
    return out


def attention_int8(q8: torch.Tensor, qs: torch.Tensor, k8: torch.Tensor, ks: torch.Tensor, v: torch.Tensor,
                   key_valid: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                   out: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """INT8 attention on quantised Q/K ([B,Sq,H,128] / [B,Sk,KV,128] int8 + per token-head f32
    scales) and bf16 V [B,Sk,KV,128]; key_valid is an optional [B,Sk] uint8/bool key mask.
    Sq < Sk is the token-sharded form (local queries, all-gathered keys/values)."""
    q8 = _require(q8, torch.int8, "q8")
    k8 = _require(k8, torch.int8, "k8")
    qs = _require(qs, torch.float32, "qs")
    ks = _require(ks, torch.float32, "ks")
    v = _require(v, torch.bfloat16, "v")
    B, Sq, H, D = (int(d) for d in q8.shape)
    Sk, KV = int(k8.shape[1]), int(k8.shape[2])
    if tuple(v.shape) != (B, Sk, KV, D) or qs.numel() != B * Sq * H or ks.numel() != B * Sk * KV:
        raise ValueError("q8/qs, k8/ks and v shapes do not agree")
    if key_valid is not None:
        key_valid = key_valid.to(torch.uint8).contiguous()
        if key_valid.numel() != B * Sk:
            raise ValueError("key_valid must be [B,Sk]")
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    if out is None:
        out = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q8.device)
    L = _lib.lib()
    nbytes = int(L.difb200_attention_int8_scratch_bytes(B, Sk, KV))
    if scratch is None or scratch.numel() < nbytes:
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q8.device)
    with torch.cuda.device(q8.device):
        _lib.check(L.difb200_attention_int8(_ptr(q8), _ptr(qs), _ptr(k8), _ptr(ks), _ptr(v), _ptr(key_valid),
                                            B, Sq, Sk, H, KV, D, float(scale), _ptr(scratch), scratch.numel(),
                                            _ptr(out), _stream()))
    return out


def attention_int8_chunked(q8: torch.Tensor, qs: torch.Tensor, k8: torch.Tensor, ks: torch.Tensor, v: torch.Tensor,
                           tile_groups: Sequence[Sequence[Tuple[int, int]]], key_valid: Optional[torch.Tensor] = None,
                           scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """attention_int8 as a sequence of launches, one per entry of ``tile_groups``; an entry is one or
    two (first tile, tile count) ranges of 128-key tiles. The unnormalised state of every query row
    is carried from launch to launch; the last launch writes the bf16 result. The groups must
    cover every key tile exactly once (the token-sharded block launches one group per set of
    key / value slices that have arrived)."""
    q8 = _require(q8, torch.int8, "q8")
    k8 = _require(k8, torch.int8, "k8")
    qs, ks = _require(qs, torch.float32, "qs"), _require(ks, torch.float32, "ks")
    v = _require(v, torch.bfloat16, "v")
    B, Sq, H, D = (int(d) for d in q8.shape)
    Sk, KV = int(k8.shape[1]), int(k8.shape[2])
    if key_valid is not None:
        key_valid = key_valid.to(torch.uint8).contiguous()
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    if out is None:
        out = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q8.device)
    L = _lib.lib()
    scratch = torch.empty(int(L.difb200_attention_int8_scratch_bytes(B, Sk, KV)), dtype=torch.uint8, device=q8.device)
    state = torch.empty(int(L.difb200_attention_int8_state_bytes(B, Sq, H)), dtype=torch.uint8, device=q8.device)
    groups = [list(g) for g in tile_groups]
    with torch.cuda.device(q8.device):
        for i, group in enumerate(groups):
            if not 1 <= len(group) <= 2:
                raise ValueError("a launch covers one or two tile ranges")
            flat = [int(x) for r in group for x in r] + [0, 0] * (2 - len(group))
            ranges = (C.c_uint32 * 4)(*flat)
            _lib.check(L.difb200_attention_int8_chunk(_ptr(q8), _ptr(qs), _ptr(k8), _ptr(ks), _ptr(v), _ptr(key_valid),
                                                      B, Sq, Sk, H, KV, D, float(scale), _ptr(scratch), scratch.numel(),
                                                      _ptr(out), ranges, 1 if i > 0 else 0,
                                                      1 if i + 1 < len(groups) else 0, _ptr(state), _stream()))
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, key_valid: Optional[torch.Tensor] = None,
              scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
              scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """DiffIR Attention on bf16 q [B,S,H,128], k/v [B,S,KV,128] through the INT8 lowering."""
    q = _require(q, torch.bfloat16, "q")
    k = _require(k, torch.bfloat16, "k")
    v = _require(v, torch.bfloat16, "v")
    B, S, H, D = (int(d) for d in q.shape)
    KV = int(k.shape[2])
    if key_valid is not None:
        key_valid = key_valid.to(torch.uint8).contiguous()
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    if out is None:
        out = torch.empty((B, S, H, D), dtype=torch.bfloat16, device=q.device)
    L = _lib.lib()
    nbytes = int(L.difb200_attention_scratch_bytes(B, S, H, KV))
    if scratch is None:
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(L.difb200_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(key_valid), B, S, H, KV, D, float(scale),
                                       _ptr(scratch), scratch.numel(), _ptr(out), _stream()))
    return out


def poll_status() -> None:
    """Raises if a kernel recorded that one of its bounded device-side waits ran out."""
    _lib.check(_lib.lib().difb200_poll_status())
