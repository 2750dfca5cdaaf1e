"""Token partition of the video DiT block and a device-API harness of its sharded form.

The reference has no multi-GPU layer (one device per Executor, reference
``include/dif/runtime/executor.hpp:683``); the sequence-partitioned form of the block that
``blocks.video_block_program`` describes lives in the native library: with ``DIFB200_WORLD_SIZE``
set, every rank's plugin context runs the block program on its token slice and exchanges the INT8
key codes, their per-token-head scales and the bf16 values with the other ranks (pushes into
peer-mapped buffers or NCCL: ``csrc/world.cu``, ``csrc/plugin.cu``). Rank r owns a contiguous slice of the tokens; weights,
norm weights and RoPE tables are replicated; everything except attention is row-local; queries
stay local and each rank attends from its own queries to all keys; nothing is reduced afterwards.

This module holds the partition arithmetic (``ShardPlan``) that the benchmark and the tests share
with that mode, and ``VideoBlock``: the same block issued kernel by kernel through the device API
on one GPU, with the gather buffers laid out as a rank of a larger world would see them. Tests
use it to emulate the ranks of a world one after another on a single GPU (slices copied between
per-rank buffers in place of the exchange) and to check the CUDA-graph replay of the block.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

H256 = 2
DIRECT = 1


@dataclass
class ShardPlan:
    """Contiguous token slices of equal padded length."""
    tokens: int
    world: int
    slice_len: int  # padded length of every slice

    @staticmethod
    def make(tokens: int, world: int) -> "ShardPlan":
        if tokens <= 0 or world <= 0:
            raise ValueError("tokens and world must be positive")
        return ShardPlan(tokens, world, (tokens + world - 1) // world)

    def bounds(self, rank: int) -> Tuple[int, int]:
        lo = min(rank * self.slice_len, self.tokens)
        return lo, min(lo + self.slice_len, self.tokens)

    def local_tokens(self, rank: int) -> int:
        lo, hi = self.bounds(rank)
        return hi - lo

    @property
    def padded_tokens(self) -> int:
        return self.slice_len * self.world

    def key_valid(self, device="cpu") -> Optional[torch.Tensor]:
        """[1, padded_tokens] uint8 mask of real keys in gathered order, or None if no padding."""
        if self.padded_tokens == self.tokens:
            return None
        valid = torch.zeros(self.padded_tokens, dtype=torch.uint8)
        for r in range(self.world):
            valid[r * self.slice_len: r * self.slice_len + self.local_tokens(r)] = 1
        return valid.reshape(1, -1).to(device)


class GatherBuffers:
    """Full-sequence K codes / K scales / V buffers whose local slice the producers write."""

    def __init__(self, plan: ShardPlan, rank: int, kv_heads: int, dim: int, device):
        self.plan, self.rank = plan, rank
        P = plan.padded_tokens
        self.k8 = torch.zeros((P, kv_heads, dim), dtype=torch.int8, device=device)
        self.ks = torch.zeros((P, kv_heads), dtype=torch.float32, device=device)
        self.v = torch.zeros((P, kv_heads, dim), dtype=torch.bfloat16, device=device)

    def local(self, t: torch.Tensor) -> torch.Tensor:
        lo = self.rank * self.plan.slice_len
        return t[lo: lo + self.plan.slice_len]


class VideoBlock:
    """Device-resident weights of one video block and its (optionally token-sharded) forward.

    ``tensors`` maps the constant names of ``blocks.video_block_program`` to numpy arrays:
    norm1, norm2, q_norm, k_norm, cos, sin (bf16 bit patterns) and, per linear, (w8, col_scales).
    """

    def __init__(self, tensors: Dict[str, object], hidden: int, heads: int, dim: int, ffn: int, rotary: int,
                 device):
        from . import ops
        self.ops = ops
        self.hidden, self.heads, self.dim, self.ffn, self.rotary = hidden, heads, dim, ffn, rotary
        self.device = device

        def bf(a):
            return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(device).view(torch.bfloat16)

        self.norm1, self.norm2 = bf(tensors["norm1"]), bf(tensors["norm2"])
        self.q_norm, self.k_norm = bf(tensors["q_norm"]), bf(tensors["k_norm"])
        self.cos, self.sin = bf(tensors["cos"]), bf(tensors["sin"])
        self.lin = {name: (torch.from_numpy(w).to(device), torch.from_numpy(s).to(device))
                    for name, (w, s) in tensors["linears"].items()}
        self._scratch = None
        self._graphs = {}
        self._valid = {}

    def _glue(self, name, *args):
        from . import _lib
        _lib.check(getattr(_lib.lib(), name)(*args))

    def pre_attention(self, x: torch.Tensor, mods: List[torch.Tensor], plan: ShardPlan, rank: int,
                      gb: GatherBuffers, on_v_ready=None, on_k_ready=None):
        """Row-local part up to the exchange: norm+modulate, q/k/v projections, q/k norm + RoPE,
        per-token-head quantisation. K codes/scales and V land in this rank's slice of ``gb``.
        The order is V, then K, then Q, and ``on_v_ready`` / ``on_k_ready`` are called as soon as
        the respective slice is enqueued, so that their all-gathers can run under the remaining
        work. Returns the local query codes and scales."""
        import ctypes as C
        ops = self.ops
        S_loc = x.shape[0]
        lo, _ = plan.bounds(rank)
        H, D, hid = self.heads, self.dim, self.hidden
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: C.c_void_p(t.data_ptr())
        new = lambda *shape: torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        # norm + modulate + ConvRot quantisation in one kernel: the normalised tensor is never written
        codes, scales = ops.rms_norm_modulate_quant(x, self.norm1, mods[0], mods[1], 1e-5, H256)
        v_local = gb.local(gb.v)[:S_loc]
        ops.linear_int8_scaled(codes, *self._w("v", scales), out=v_local.view(S_loc, H * D))  # into the gather buffer
        if on_v_ready is not None:
            on_v_ready()

        def norm_rope_quant(name, w, codes, scales):
            """q/k projection, then QkNormPartialRope + per-token-head quantisation in one kernel:
            codes and scales are written where the caller wants them."""
            y = ops.linear_int8_scaled(codes_in, *self._w(name, scales_in))
            self._glue("difb200_qk_norm_rope_quant", p(y), p(w), p(self.cos), p(self.sin), None, p(codes), p(scales),
                       2, S_loc, H, self.rotary, self.rotary, S_loc, self.cos.shape[0], lo, 1e-5, 0, stream)

        codes_in, scales_in = codes, scales
        # K codes and scales are produced directly inside this rank's slice of the gather buffers
        norm_rope_quant("k", self.k_norm, gb.local(gb.k8)[:S_loc], gb.local(gb.ks)[:S_loc])
        if on_k_ready is not None:
            on_k_ready()
        q8 = torch.empty((S_loc, H, D), dtype=torch.int8, device=self.device)
        qs = torch.empty((S_loc * H,), dtype=torch.float32, device=self.device)
        norm_rope_quant("q", self.q_norm, q8, qs)
        return q8.view(1, S_loc, H, D), qs

    def attend(self, q8: torch.Tensor, qs: torch.Tensor, plan: ShardPlan, gb: GatherBuffers) -> torch.Tensor:
        """Local queries against the gathered keys/values of the whole sequence."""
        H, D, P = self.heads, self.dim, plan.padded_tokens
        key = (plan.tokens, plan.world)
        if key not in self._valid:  # built once (a host-to-device copy has no place in a graph capture)
            self._valid[key] = plan.key_valid(self.device)
        return self.ops.attention_int8(q8, qs, gb.k8.view(1, P, H, D), gb.ks, gb.v.view(1, P, H, D),
                                       self._valid[key], scale=1.0 / float(np.sqrt(D)))

    def post_attention(self, x: torch.Tensor, attn: torch.Tensor, mods: List[torch.Tensor]) -> torch.Tensor:
        """Row-local part after attention: out-proj, gated residual, norm+modulate, SwiGLU MLP."""
        import ctypes as C
        ops = self.ops
        S_loc = x.shape[0]
        H, D, hid = self.heads, self.dim, self.hidden
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: C.c_void_p(t.data_ptr())
        new = lambda *shape: torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        o = ops.w8a8_linear(attn.view(S_loc, H * D), *self.lin["o"])
        r1 = new(S_loc, hid)
        self._glue("difb200_residual_gate", p(x), p(o), p(mods[2]), p(r1), 2, S_loc, hid, S_loc, stream)
        codes2, scales2 = ops.rms_norm_modulate_quant(r1, self.norm2, mods[3], mods[4], 1e-5, H256)
        fc1 = ops.linear_int8_scaled(codes2, *self._w("fc1", scales2))
        act = new(S_loc, self.ffn)
        self._glue("difb200_swiglu", p(fc1), p(act), 2, S_loc, self.ffn, 2 * self.ffn, 0, 0, stream)
        fc2 = ops.w8a8_linear(act, *self.lin["fc2"])
        out = new(S_loc, hid)
        self._glue("difb200_residual_gate", p(r1), p(fc2), p(mods[5]), p(out), 2, S_loc, hid, S_loc, stream)
        return out

    def forward(self, x: torch.Tensor, mods: List[torch.Tensor], plan: ShardPlan, rank: int,
                gb: Optional[GatherBuffers] = None, events: Optional[dict] = None,
                graphs: bool = False) -> torch.Tensor:
        """The block on one GPU (``plan.world`` == 1, or the local part of an emulated rank whose
        gather buffers the caller has filled). x and the six modulation tensors are [S_local,
        hidden]. With ``graphs`` the kernels of the block are replayed from four CUDA graphs (V
        part, K part, Q part, attention + rest), captured on the first call for these very tensors."""
        def mark(name):
            if events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.setdefault(name, []).append(ev)

        if gb is None:
            gb = GatherBuffers(plan, rank, self.heads, self.dim, self.device)
        if graphs:
            return self._forward_graphed(x, mods, plan, rank, gb, mark)
        mark("start")
        q8, qs = self.pre_attention(x, mods, plan, rank, gb)
        mark("pre_attention")
        attn = self.attend(q8, qs, plan, gb)
        mark("attention")
        out = self.post_attention(x, attn, mods)
        mark("end")
        return out

    def _forward_graphed(self, x, mods, plan, rank, gb, mark):
        key = (x.data_ptr(), tuple(m.data_ptr() for m in mods), gb.k8.data_ptr(), plan.tokens, plan.world, rank)
        state = self._graphs.get(key)
        if state is None:
            state = self._capture(x, mods, plan, rank, gb)
            self._graphs[key] = state
        mark("start")
        state["v"].replay()
        state["k"].replay()
        state["q"].replay()
        mark("pre_attention")
        state["rest"].replay()
        mark("end")
        return state["out"]

    def _capture(self, x, mods, plan, rank, gb):
        """Records the four kernel sequences of this block for these very tensors.
        pre_attention reports the end of its V and K parts through callbacks: a capture ends and
        the next begins inside them. The returned output tensor is overwritten by every replay."""
        self.forward(x, mods, plan, rank, gb=gb)  # lazy allocations and one-time set-up, outside a capture
        torch.cuda.synchronize()
        pool = torch.cuda.graph_pool_handle()
        graph = {name: torch.cuda.CUDAGraph() for name in ("v", "k", "q", "rest")}
        current = {"name": "v"}

        def switch(to):
            graph[current["name"]].capture_end()
            current["name"] = to
            graph[to].capture_begin(pool=pool)

        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            graph["v"].capture_begin(pool=pool)
            q8, qs = self.pre_attention(x, mods, plan, rank, gb, on_v_ready=lambda: switch("k"),
                                        on_k_ready=lambda: switch("q"))
            switch("rest")
            attn = self.attend(q8, qs, plan, gb)
            out = self.post_attention(x, attn, mods)
            graph["rest"].capture_end()
        torch.cuda.current_stream().wait_stream(stream)
        state = dict(graph)
        state["out"] = out
        return state

    def _w(self, name, scales):
        w8, cs = self.lin[name]
        return w8, scales, cs
