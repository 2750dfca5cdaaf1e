"""DiffIR program model and the DIFIR001 wire format (host side).

This mirrors the part of the reference's IR that the quantized DiT hot path needs:
``Program{TensorDesc[], Operation[]}``, the dtype / role / opcode / attribute-key codes
(reference ``include/dif/ir/ir.hpp:16-293``) and the binary encoding that crosses the
backend plugin boundary (reference ``src/ir/codec.cpp:370-476``):

    "DIFIR001", u32 version=1, u32 #tensors, u32 #ops,
    tensors {u32 id, u32 dtype, u32 roles, u32 rank, u64 dims[rank]},
    ops {u32 id, u32 opcode, u32 #in, u32 #out, u32 #attr, u32 in[], u32 out[],
         attr {u32 key, u32 kind, u64 bits}[]},
    SHA-256 of everything before it; all little-endian.

The native plugin has its own decoder; this module is what tests, the benchmark and users
of the Python layer build programs with.
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Dict, List, Sequence

MAGIC = b"DIFIR001"
VERSION = 1
MAX_RANK = 8


class DType(IntEnum):
    F32 = 1
    BF16 = 2
    F16 = 3
    I8 = 4
    I32 = 5
    Bool = 6
    FP8E4M3 = 7
    FP8E8M0 = 8


DTYPE_SIZE = {DType.F32: 4, DType.BF16: 2, DType.F16: 2, DType.I8: 1, DType.I32: 4,
              DType.Bool: 1, DType.FP8E4M3: 1, DType.FP8E8M0: 1}


class Role(IntEnum):
    Internal = 0
    Input = 1
    Output = 2
    Constant = 4
    Streamed = 8
    Parameter = 16
    OptimizerState = 32


class Opcode(IntEnum):
    Add = 1
    Multiply = 2
    RmsNormModulate = 3
    SwiGlu = 4
    ResidualGate = 5
    Linear = 6
    QkNormPartialRope = 7
    Attention = 8
    BiasAdd = 10
    SiLU = 16
    RmsNorm = 17
    Fill = 18
    Cast = 21
    RotaryPosition = 24
    AffineLastDim = 29
    LayerNorm = 30
    Gelu = 49
    Sigmoid = 50
    Reshape = 51
    BroadcastTo = 52
    Slice = 53
    RotaryFrequency = 54
    RotaryApply = 55
    BooleanMaskToBias = 56
    Concat = 59
    QuantizeInt8Rows = 67
    LinearInt8Scaled = 68
    LayerNormModulate = 75


class AttrKey(IntEnum):
    Epsilon = 1
    BlockSize = 2
    Heads = 3
    HeadDim = 4
    RotaryDim = 5
    AttentionScale = 6
    Causal = 7
    Implementation = 9
    GateFirst = 13
    Value = 15
    Scale = 18
    KvHeads = 39
    Approximation = 40
    Axis = 41
    Start = 42
    Theta = 43
    Ntk = 44
    WeightOffset = 45
    RotaryLayout = 46
    LinearBiasMode = 55
    ReductionTileSize = 56
    ModulationLayout = 57
    WorkspaceLimitBytes = 58
    MaskQueries = 73


class AttrKind(IntEnum):
    U64 = 1
    I64 = 2
    F64 = 3
    Bool = 4


class Int8RowQuantization(IntEnum):
    """Row transform / rounding contract of QuantizeInt8Rows (ir.hpp:285-293)."""
    Direct = 1
    H256ConvRot = 2
    H256SignedConvRot = 3
    H4096SignedConvRot = 4
    H256F32ConvRot = 5
    H256F32SignedConvRot = 6
    H4096F32SignedConvRot = 7


class GeluApproximation(IntEnum):
    Tanh = 1
    ExactErf = 2


@dataclass
class Attribute:
    key: int
    kind: int
    bits: int

    @staticmethod
    def u64(key: int, value: int) -> "Attribute":
        return Attribute(int(key), AttrKind.U64, int(value) & 0xFFFFFFFFFFFFFFFF)

    @staticmethod
    def i64(key: int, value: int) -> "Attribute":
        return Attribute(int(key), AttrKind.I64, struct.unpack("<Q", struct.pack("<q", int(value)))[0])

    @staticmethod
    def f64(key: int, value: float) -> "Attribute":
        return Attribute(int(key), AttrKind.F64, struct.unpack("<Q", struct.pack("<d", float(value)))[0])

    @staticmethod
    def boolean(key: int, value: bool) -> "Attribute":
        return Attribute(int(key), AttrKind.Bool, 1 if value else 0)


@dataclass
class TensorDesc:
    id: int
    dtype: int
    roles: int
    dims: List[int]

    def element_count(self) -> int:
        n = 1
        for d in self.dims:
            n *= int(d)
        return n

    def byte_count(self) -> int:
        return self.element_count() * DTYPE_SIZE[DType(self.dtype)]

    def has_role(self, role: int) -> bool:
        return (self.roles & int(role)) != 0


@dataclass
class Operation:
    id: int
    opcode: int
    inputs: List[int]
    outputs: List[int]
    attributes: List[Attribute] = field(default_factory=list)


@dataclass
class Program:
    tensors: List[TensorDesc] = field(default_factory=list)
    operations: List[Operation] = field(default_factory=list)
    version: int = VERSION

    def tensor(self, tensor_id: int) -> TensorDesc:
        for t in self.tensors:
            if t.id == tensor_id:
                return t
        raise KeyError(tensor_id)

    # small builder helpers -------------------------------------------------
    def add_tensor(self, dtype: int, dims: Sequence[int], roles: int = Role.Internal) -> int:
        tid = len(self.tensors) + 1
        self.tensors.append(TensorDesc(tid, int(dtype), int(roles), [int(d) for d in dims]))
        return tid

    def add_op(self, opcode: int, inputs: Sequence[int], outputs: Sequence[int],
               attributes: Sequence[Attribute] = ()) -> int:
        oid = len(self.operations) + 1
        self.operations.append(Operation(oid, int(opcode), list(inputs), list(outputs), list(attributes)))
        return oid

    def with_role(self, role: int) -> List[TensorDesc]:
        """Tensors carrying ``role``, in program order (the order views cross the ABI in)."""
        return [t for t in self.tensors if t.has_role(role)]


def encode(program: Program) -> bytes:
    """Serialise to DIFIR001 bytes (codec.cpp:370-405)."""
    out = bytearray(MAGIC)
    out += struct.pack("<III", program.version, len(program.tensors), len(program.operations))
    for t in program.tensors:
        out += struct.pack("<IIII", t.id, int(t.dtype), t.roles, len(t.dims))
        for d in t.dims:
            out += struct.pack("<Q", d)
    for op in program.operations:
        out += struct.pack("<IIIII", op.id, int(op.opcode), len(op.inputs), len(op.outputs),
                           len(op.attributes))
        for i in op.inputs:
            out += struct.pack("<I", i)
        for o in op.outputs:
            out += struct.pack("<I", o)
        for a in op.attributes:
            out += struct.pack("<IIQ", int(a.key), int(a.kind), a.bits)
    out += hashlib.sha256(bytes(out)).digest()
    return bytes(out)


def decode(data: bytes) -> Program:
    """Parse DIFIR001 bytes; raises ValueError on the conditions codec.cpp:407-476 rejects."""
    if len(data) < len(MAGIC) + 12 + 32:
        raise ValueError("DiffIR file is too small")
    payload, digest = data[:-32], data[-32:]
    if hashlib.sha256(payload).digest() != digest:
        raise ValueError("DiffIR SHA-256 mismatch")
    if payload[:8] != MAGIC:
        raise ValueError("invalid DiffIR magic")
    pos = 8

    def take(fmt: str):
        nonlocal pos
        size = struct.calcsize(fmt)
        if pos + size > len(payload):
            raise ValueError("truncated DiffIR payload")
        values = struct.unpack_from(fmt, payload, pos)
        pos += size
        return values

    version, n_tensors, n_ops = take("<III")
    if version != VERSION:
        raise ValueError("unsupported DiffIR version")
    if n_tensors > (1 << 20) or n_ops > (1 << 20):
        raise ValueError("DiffIR count is too large")
    program = Program(version=version)
    for _ in range(n_tensors):
        tid, dtype, roles, rank = take("<IIII")
        if rank == 0 or rank > MAX_RANK:
            raise ValueError("invalid DiffIR tensor rank")
        dims = [take("<Q")[0] for _ in range(rank)]
        program.tensors.append(TensorDesc(tid, dtype, roles, dims))
    for _ in range(n_ops):
        oid, opcode, n_in, n_out, n_attr = take("<IIIII")
        if max(n_in, n_out, n_attr) > (1 << 20):
            raise ValueError("DiffIR count is too large")
        inputs = [take("<I")[0] for _ in range(n_in)]
        outputs = [take("<I")[0] for _ in range(n_out)]
        attrs = [Attribute(*take("<IIQ")) for _ in range(n_attr)]
        program.operations.append(Operation(oid, opcode, inputs, outputs, attrs))
    if pos != len(payload):
        raise ValueError("trailing bytes in DiffIR payload")
    return program


# ---------------------------------------------------------------------------
# Program builders for the hot path
# ---------------------------------------------------------------------------

def w8a8_linear_program(M: int, K: int, N: int, implementation: int = Int8RowQuantization.H256ConvRot,
                        clip: float = 1.0, bias: bool = True, gelu: bool = False,
                        expose_codes: bool = False) -> Dict[str, object]:
    """``QuantizeInt8Rows -> LinearInt8Scaled [-> BiasAdd [-> Gelu(tanh)]]`` on a bf16 [M,K] input.

    This is the op sequence the reference's W8A8 rewrite puts in place of a ``Linear``
    (``tools/difflux2sample.cpp:2017-2069``). Returns the program and the tensor ids by name.
    With ``expose_codes`` the INT8 codes and row scales are program outputs too.
    """
    p = Program()
    x = p.add_tensor(DType.BF16, [M, K], Role.Input)
    code_role = Role.Output if expose_codes else Role.Internal
    codes = p.add_tensor(DType.I8, [M, K], code_role)
    row = p.add_tensor(DType.F32, [M], code_role)
    w = p.add_tensor(DType.I8, [N, K], Role.Constant)
    col = p.add_tensor(DType.F32, [N], Role.Constant)
    ids = {"x": x, "codes": codes, "row_scales": row, "weight": w, "col_scales": col}
    last_is_output = not bias and not gelu
    y = p.add_tensor(DType.BF16, [M, N], Role.Output if last_is_output else Role.Internal)
    p.add_op(Opcode.QuantizeInt8Rows, [x], [codes, row],
             [Attribute.u64(AttrKey.BlockSize, 256), Attribute.f64(AttrKey.Scale, clip),
              Attribute.u64(AttrKey.Implementation, int(implementation))])
    p.add_op(Opcode.LinearInt8Scaled, [codes, w, row, col], [y])
    ids["y"] = y
    if bias:
        b = p.add_tensor(DType.BF16, [N], Role.Constant)
        yb = p.add_tensor(DType.BF16, [M, N], Role.Internal if gelu else Role.Output)
        p.add_op(Opcode.BiasAdd, [y, b], [yb])
        ids["bias"] = b
        ids["y"] = yb
    if gelu:
        yg = p.add_tensor(DType.BF16, [M, N], Role.Output)
        p.add_op(Opcode.Gelu, [ids["y"]], [yg],
                 [Attribute.u64(AttrKey.Approximation, int(GeluApproximation.Tanh))])
        ids["y"] = yg
    return {"program": p, "ids": ids}


def quantize_program(rows_shape: Sequence[int], implementation: int, clip: float = 1.0,
                     residual: bool = False, dynamic_clip: bool = False,
                     part_widths: Sequence[int] = ()) -> Dict[str, object]:
    """A single QuantizeInt8Rows op (verify.cpp:949-1027): 1..n bf16 inputs concatenated on the
    last axis, optional trailing F32[1] clip input, 2 or 4 outputs."""
    p = Program()
    lead = list(rows_shape[:-1])
    widths = list(part_widths) if part_widths else [rows_shape[-1]]
    xs = [p.add_tensor(DType.BF16, lead + [w], Role.Input) for w in widths]
    total = sum(widths)
    rows = 1
    for d in lead:
        rows *= d
    codes = p.add_tensor(DType.I8, lead + [total], Role.Output)
    scales = p.add_tensor(DType.F32, [rows], Role.Output)
    outs = [codes, scales]
    ids = {"x": xs, "codes": codes, "scales": scales}
    if residual:
        rc = p.add_tensor(DType.I8, lead + [total], Role.Output)
        rs = p.add_tensor(DType.F32, [rows], Role.Output)
        outs += [rc, rs]
        ids.update({"rcodes": rc, "rscales": rs})
    ins = list(xs)
    attrs = [Attribute.u64(AttrKey.BlockSize, 256),
             Attribute.u64(AttrKey.Implementation, int(implementation))]
    if dynamic_clip:
        c = p.add_tensor(DType.F32, [1], Role.Input)
        ins.append(c)
        ids["clip"] = c
    else:
        attrs.append(Attribute.f64(AttrKey.Scale, clip))
    p.add_op(Opcode.QuantizeInt8Rows, ins, outs, attrs)
    return {"program": p, "ids": ids}


def attention_program(B: int, S: int, H: int, KV: int, D: int, masked: bool,
                      scale: float | None = None) -> Dict[str, object]:
    """``[BooleanMaskToBias(MaskQueries=false) ->] Attention(Implementation=2, KvHeads)`` on bf16
    [B,S,H,D] queries and [B,S,KV,D] keys/values (verify.cpp:1250-1324, 228-243)."""
    p = Program()
    q = p.add_tensor(DType.BF16, [B, S, H, D], Role.Input)
    k = p.add_tensor(DType.BF16, [B, S, KV, D], Role.Input)
    v = p.add_tensor(DType.BF16, [B, S, KV, D], Role.Input)
    ids = {"q": q, "k": k, "v": v}
    ins = [q, k, v]
    if masked:
        m = p.add_tensor(DType.Bool, [B, S], Role.Input)
        bias = p.add_tensor(DType.BF16, [B, 1, S, S], Role.Internal)
        p.add_op(Opcode.BooleanMaskToBias, [m], [bias], [Attribute.boolean(AttrKey.MaskQueries, False)])
        ins.append(bias)
        ids["mask"] = m
    out = p.add_tensor(DType.BF16, [B, S, H, D], Role.Output)
    attrs = [Attribute.u64(AttrKey.Implementation, 2), Attribute.u64(AttrKey.KvHeads, KV)]
    if scale is not None:
        attrs.append(Attribute.f64(AttrKey.AttentionScale, scale))
    p.add_op(Opcode.Attention, ins, [out], attrs)
    ids["out"] = out
    return {"program": p, "ids": ids}
