"""ctypes access to the two CPU checkers under oracle/ (test infrastructure).

``orc``  : oracle/_build/liboracle.so, the plain-C restatement (always available after
           ``__graft_entry__.build()`` or ``make -C oracle oracle``).
``ref``  : oracle/_ref/libdifref.so, the reference project's own CPU executor compiled from
           its sources (present only where it was built; tests that need it skip otherwise).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Dict, List, Optional, Sequence

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORC_PATH = os.path.join(ORACLE_DIR, "_build", "liboracle.so")
REF_PATH = os.path.join(ORACLE_DIR, "_ref", "libdifref.so")

_p8 = C.POINTER(C.c_int8)
_pu8 = C.POINTER(C.c_uint8)
_pu16 = C.POINTER(C.c_uint16)
_pf = C.POINTER(C.c_float)
_pi32 = C.POINTER(C.c_int32)
_pu64 = C.POINTER(C.c_uint64)


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns, round-to-nearest-even on the raw bits."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounding = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    return ((bits + rounding) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def _ptr(a: Optional[np.ndarray], typ):
    if a is None:
        return C.cast(None, typ)
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(typ)


def build_oracle() -> None:
    subprocess.run(["make", "-s", "-C", ORACLE_DIR, "oracle"], check=True)


class _Orc:
    def __init__(self) -> None:
        if not os.path.exists(ORC_PATH):
            build_oracle()
        self.lib = C.CDLL(ORC_PATH)
        L = self.lib
        L.orc_quantize_int8_rows.restype = C.c_int
        L.orc_quantize_int8_rows.argtypes = [C.POINTER(_pu16), _pu64, C.c_uint64, C.c_uint64, C.c_int,
                                             C.c_float, _p8, _pf, _p8, _pf]
        L.orc_linear_int8_scaled.restype = None
        L.orc_linear_int8_scaled.argtypes = [_p8, _p8, _pf, _pf, C.c_uint64, C.c_uint64, C.c_uint64,
                                             _pi32, _pu16]
        L.orc_bias_add.restype = None
        L.orc_bias_add.argtypes = [_pu16, _pu16, C.c_uint64, C.c_uint64, _pu16]
        L.orc_gelu_tanh.restype = None
        L.orc_gelu_tanh.argtypes = [_pu16, C.c_uint64, _pu16]
        L.orc_rms_norm.restype = None
        L.orc_rms_norm.argtypes = [_pu16, _pu16, C.c_uint64, C.c_uint64, C.c_float, C.c_float, _pu16]
        L.orc_rotary_apply.restype = None
        L.orc_rotary_apply.argtypes = [_pu16, _pf, _pf] + [C.c_uint64] * 5 + [_pu16]
        for name in ("orc_attention_exact",):
            getattr(L, name).restype = None
        L.orc_attention_exact.argtypes = [_pu16, _pu16, _pu16, _pu8] + [C.c_uint64] * 5 + [C.c_float, _pu16]
        L.orc_attention_int8.restype = None
        L.orc_attention_int8.argtypes = [_p8, _pf, _p8, _pf, _pu16, _pu8] + [C.c_uint64] * 5 + \
                                        [C.c_float, _pi32, _pu16]
        L.orc_attention_int8_rows.restype = None
        L.orc_attention_int8_rows.argtypes = [_p8, _pf, _p8, _pf, _pu16, _pu8] + [C.c_uint64] * 6 + \
                                             [C.c_float, C.c_int, _pu16]
        L.orc_attention_exact_rows.restype = None
        L.orc_attention_exact_rows.argtypes = [_pu16, _pu16, _pu16, _pu8] + [C.c_uint64] * 6 + [C.c_float, _pu16]

    def quantize_int8_rows(self, parts: Sequence[np.ndarray], implementation: int, clip: float = 1.0,
                           residual: bool = False):
        parts = [np.ascontiguousarray(p, dtype=np.uint16) for p in parts]
        rows = int(np.prod(parts[0].shape[:-1]))
        widths = np.array([p.shape[-1] for p in parts], dtype=np.uint64)
        total = int(widths.sum())
        codes = np.empty((rows, total), np.int8)
        scales = np.empty(rows, np.float32)
        rcodes = np.empty((rows, total), np.int8) if residual else None
        rscales = np.empty(rows, np.float32) if residual else None
        arr = (_pu16 * len(parts))(*[_ptr(p, _pu16) for p in parts])
        rc = self.lib.orc_quantize_int8_rows(arr, _ptr(widths, _pu64), len(parts), rows, int(implementation),
                                             float(clip), _ptr(codes, _p8), _ptr(scales, _pf),
                                             _ptr(rcodes, _p8), _ptr(rscales, _pf))
        if rc != 0:
            raise ValueError("illegal width for this ConvRot variant")
        return (codes, scales, rcodes, rscales) if residual else (codes, scales)

    def quantize_weight_rows(self, weight: np.ndarray, implementation: int, mse: bool = False,
                             equalise: Optional[np.ndarray] = None):
        weight = np.ascontiguousarray(weight, dtype=np.uint16)
        rows, columns = weight.shape
        codes = np.empty((rows, columns), np.int8)
        scales = np.empty(rows, np.float32)
        if equalise is not None:
            equalise = np.ascontiguousarray(equalise, dtype=np.uint16)
        self.lib.orc_quantize_weight_rows.restype = C.c_int
        self.lib.orc_quantize_weight_rows.argtypes = [_pu16, _pu16, C.c_uint64, C.c_uint64, C.c_int, C.c_int, _p8, _pf]
        rc = self.lib.orc_quantize_weight_rows(_ptr(weight, _pu16), _ptr(equalise, _pu16), rows, columns,
                                               int(implementation), 1 if mse else 0, _ptr(codes, _p8),
                                               _ptr(scales, _pf))
        if rc != 0:
            raise ValueError("illegal width or variant for weight packing")
        return codes, scales

    def choose_mse_weight_scale(self, rows_f32: np.ndarray) -> np.ndarray:
        """The packer's MSE row-scale search alone, on fp32 rows [rows, columns]."""
        rows_f32 = np.ascontiguousarray(rows_f32, dtype=np.float32)
        rows, columns = rows_f32.shape
        scales = np.empty(rows, np.float32)
        self.lib.orc_choose_mse_weight_scale.restype = None
        self.lib.orc_choose_mse_weight_scale.argtypes = [_pf, C.c_uint64, C.c_uint64, _pf]
        self.lib.orc_choose_mse_weight_scale(_ptr(rows_f32, _pf), rows, columns, _ptr(scales, _pf))
        return scales

    def weight_equalization(self, weight: np.ndarray) -> np.ndarray:
        weight = np.ascontiguousarray(weight, dtype=np.uint16)
        rows, columns = weight.shape
        out = np.empty(columns, np.uint16)
        self.lib.orc_weight_equalization.restype = None
        self.lib.orc_weight_equalization.argtypes = [_pu16, C.c_uint64, C.c_uint64, _pu16]
        self.lib.orc_weight_equalization(_ptr(weight, _pu16), rows, columns, _ptr(out, _pu16))
        return out

    def linear_int8_scaled(self, x8, w8, row, col, want_acc=False):
        x8 = np.ascontiguousarray(x8, np.int8)
        w8 = np.ascontiguousarray(w8, np.int8)
        row = np.ascontiguousarray(row, np.float32)
        col = np.ascontiguousarray(col, np.float32)
        M, K = x8.shape
        N = w8.shape[0]
        out = np.empty((M, N), np.uint16)
        acc = np.empty((M, N), np.int32) if want_acc else None
        self.lib.orc_linear_int8_scaled(_ptr(x8, _p8), _ptr(w8, _p8), _ptr(row, _pf), _ptr(col, _pf), M, N, K,
                                        _ptr(acc, _pi32), _ptr(out, _pu16))
        return (out, acc) if want_acc else out

    def bias_add(self, y, bias):
        y = np.ascontiguousarray(y, np.uint16)
        bias = np.ascontiguousarray(bias, np.uint16)
        out = np.empty_like(y)
        self.lib.orc_bias_add(_ptr(y, _pu16), _ptr(bias, _pu16), y.size, bias.size, _ptr(out, _pu16))
        return out

    def gelu_tanh(self, y):
        y = np.ascontiguousarray(y, np.uint16)
        out = np.empty_like(y)
        self.lib.orc_gelu_tanh(_ptr(y, _pu16), y.size, _ptr(out, _pu16))
        return out

    def rms_norm(self, x, weight, eps=1e-6, weight_offset=0.0):
        x = np.ascontiguousarray(x, np.uint16)
        weight = np.ascontiguousarray(weight, np.uint16)
        cols = x.shape[-1]
        out = np.empty_like(x)
        self.lib.orc_rms_norm(_ptr(x, _pu16), _ptr(weight, _pu16), x.size // cols, cols, eps, weight_offset,
                              _ptr(out, _pu16))
        return out

    def rotary_apply(self, x, cosine, sine):
        x = np.ascontiguousarray(x, np.uint16)
        cosine = np.ascontiguousarray(cosine, np.float32)
        sine = np.ascontiguousarray(sine, np.float32)
        B, S, H, D = x.shape
        out = np.empty_like(x)
        self.lib.orc_rotary_apply(_ptr(x, _pu16), _ptr(cosine, _pf), _ptr(sine, _pf), B, S, H, D,
                                  cosine.shape[-1], _ptr(out, _pu16))
        return out

    def attention_exact(self, q, k, v, key_valid=None, scale=None):
        q = np.ascontiguousarray(q, np.uint16)
        k = np.ascontiguousarray(k, np.uint16)
        v = np.ascontiguousarray(v, np.uint16)
        B, S, H, D = q.shape
        KV = k.shape[2]
        scale = float(1.0 / np.sqrt(float(D))) if scale is None else scale
        kvp = None if key_valid is None else np.ascontiguousarray(key_valid, np.uint8)
        out = np.empty_like(q)
        self.lib.orc_attention_exact(_ptr(q, _pu16), _ptr(k, _pu16), _ptr(v, _pu16), _ptr(kvp, _pu8),
                                     B, S, H, KV, D, scale, _ptr(out, _pu16))
        return out

    def attention_int8(self, q8, qs, k8, ks, v, key_valid=None, scale=None, want_acc=False):
        q8 = np.ascontiguousarray(q8, np.int8)
        k8 = np.ascontiguousarray(k8, np.int8)
        qs = np.ascontiguousarray(qs, np.float32)
        ks = np.ascontiguousarray(ks, np.float32)
        v = np.ascontiguousarray(v, np.uint16)
        B, S, H, D = q8.shape
        KV = k8.shape[2]
        scale = float(1.0 / np.sqrt(float(D))) if scale is None else scale
        kvp = None if key_valid is None else np.ascontiguousarray(key_valid, np.uint8)
        out = np.empty((B, S, H, D), np.uint16)
        acc = np.empty((S, S), np.int32) if want_acc else None
        self.lib.orc_attention_int8(_ptr(q8, _p8), _ptr(qs, _pf), _ptr(k8, _p8), _ptr(ks, _pf), _ptr(v, _pu16),
                                    _ptr(kvp, _pu8), B, S, H, KV, D, scale, _ptr(acc, _pi32), _ptr(out, _pu16))
        return (out, acc) if want_acc else out


    def attention_int8_rows(self, q8, qs, k8, ks, v, key_valid=None, scale=None, fp32_p=False):
        """INT8 attention of a query sample [B,Sq,H,D] against all keys [B,S,KV,D]; fp32_p keeps
        the softmax weights unrounded (the reported middle tier)."""
        q8 = np.ascontiguousarray(q8, np.int8)
        k8 = np.ascontiguousarray(k8, np.int8)
        qs = np.ascontiguousarray(qs, np.float32)
        ks = np.ascontiguousarray(ks, np.float32)
        v = np.ascontiguousarray(v, np.uint16)
        B, Sq, H, D = q8.shape
        S, KV = k8.shape[1], k8.shape[2]
        scale = float(1.0 / np.sqrt(float(D))) if scale is None else scale
        kvp = None if key_valid is None else np.ascontiguousarray(key_valid, np.uint8)
        out = np.empty((B, Sq, H, D), np.uint16)
        self.lib.orc_attention_int8_rows(_ptr(q8, _p8), _ptr(qs, _pf), _ptr(k8, _p8), _ptr(ks, _pf), _ptr(v, _pu16),
                                         _ptr(kvp, _pu8), B, Sq, S, H, KV, D, scale, 1 if fp32_p else 0,
                                         _ptr(out, _pu16))
        return out

    def attention_exact_rows(self, q, k, v, key_valid=None, scale=None):
        """Exact Attention of a query sample [B,Sq,H,D] against all keys [B,S,KV,D]."""
        q = np.ascontiguousarray(q, np.uint16)
        k = np.ascontiguousarray(k, np.uint16)
        v = np.ascontiguousarray(v, np.uint16)
        B, Sq, H, D = q.shape
        S, KV = k.shape[1], k.shape[2]
        scale = float(1.0 / np.sqrt(float(D))) if scale is None else scale
        kvp = None if key_valid is None else np.ascontiguousarray(key_valid, np.uint8)
        out = np.empty_like(q)
        self.lib.orc_attention_exact_rows(_ptr(q, _pu16), _ptr(k, _pu16), _ptr(v, _pu16), _ptr(kvp, _pu8),
                                          B, Sq, S, H, KV, D, scale, _ptr(out, _pu16))
        return out


class _View(C.Structure):
    _fields_ = [("tensor_id", C.c_uint32), ("data", C.c_void_p), ("byte_count", C.c_uint64)]


class _Ref:
    """The reference project's CPU executor / plugin host behind oracle/ref_driver.cpp."""

    def __init__(self) -> None:
        self.lib = C.CDLL(REF_PATH)
        common = [C.c_char_p, C.c_size_t, C.POINTER(_View), C.c_size_t, C.POINTER(_View), C.c_size_t,
                  C.c_uint32, C.c_uint32, C.POINTER(C.c_double), C.c_char_p, C.c_size_t]
        self.lib.difref_run.restype = C.c_int
        self.lib.difref_run.argtypes = common
        self.lib.difref_run_plugin.restype = C.c_int
        self.lib.difref_run_plugin.argtypes = [C.c_char_p, C.c_int] + common
        self.lib.difref_encode_check.restype = C.c_int
        self.lib.difref_encode_check.argtypes = [C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]

    @staticmethod
    def _np_dtype(dtype: int):
        return {1: np.float32, 2: np.uint16, 3: np.uint16, 4: np.int8, 5: np.int32, 6: np.uint8}[int(dtype)]

    def run(self, program, bound: Dict[int, np.ndarray], outputs: Optional[List[int]] = None,
            plugin: Optional[str] = None, device: int = 0, warmups: int = 0, iterations: int = 1):
        from diffusion_compiler_b200 import diffir
        data = diffir.encode(program)
        if outputs is None:
            outputs = [t.id for t in program.with_role(diffir.Role.Output)]
        keep = []
        bviews = (_View * max(1, len(bound)))()
        for i, (tid, arr) in enumerate(bound.items()):
            arr = np.ascontiguousarray(arr)
            keep.append(arr)
            bviews[i] = _View(tid, arr.ctypes.data, arr.nbytes)
        outs = {}
        oviews = (_View * max(1, len(outputs)))()
        for i, tid in enumerate(outputs):
            desc = program.tensor(tid)
            arr = np.zeros(desc.dims, self._np_dtype(desc.dtype))
            outs[tid] = arr
            oviews[i] = _View(tid, arr.ctypes.data, arr.nbytes)
        err = C.create_string_buffer(1024)
        ms = C.c_double(0.0)
        if plugin is None:
            rc = self.lib.difref_run(data, len(data), bviews, len(bound), oviews, len(outputs), warmups,
                                     iterations, C.byref(ms), err, 1024)
        else:
            rc = self.lib.difref_run_plugin(plugin.encode(), device, data, len(data), bviews, len(bound),
                                            oviews, len(outputs), warmups, iterations, C.byref(ms), err, 1024)
        if rc != 0:
            raise RuntimeError("reference: " + err.value.decode(errors="replace"))
        return outs, ms.value

    def encode_check(self, data: bytes) -> None:
        err = C.create_string_buffer(1024)
        rc = self.lib.difref_encode_check(data, len(data), err, 1024)
        if rc != 0:
            raise RuntimeError("reference codec: " + err.value.decode(errors="replace"))


_orc = None
_ref = None


def orc() -> _Orc:
    global _orc
    if _orc is None:
        _orc = _Orc()
    return _orc


PACKER_PROBE = os.path.join(ORACLE_DIR, "_ref", "difpacker_scale")


def packer_probe_available() -> bool:
    return os.path.exists(PACKER_PROBE)


def packer_mse_scales(rows_f32: np.ndarray) -> np.ndarray:
    """choose_mse_int8_weight_scale of the reference's own packer (oracle/_ref/difpacker_scale, which
    includes the reference tool's source) on fp32 rows [rows, columns]."""
    import subprocess
    import tempfile
    rows_f32 = np.ascontiguousarray(rows_f32, dtype=np.float32)
    with tempfile.NamedTemporaryFile(suffix=".f32") as f:
        rows_f32.tofile(f.name)
        out = subprocess.run([PACKER_PROBE, f.name, str(rows_f32.shape[0]), str(rows_f32.shape[1])],
                             check=True, capture_output=True, text=True).stdout.split()
    return np.array([int(h, 16) for h in out], np.uint32).view(np.float32)


def packer_pack(weight_bf16: np.ndarray, implementation: int, equalise: bool, mse: bool, directory: str) -> str:
    """The reference packer (rewrite_named_linear_w8a8 of tools/difflux2sample.cpp, through
    oracle/_ref/difpacker_scale) on one bf16 weight matrix; returns the path of the cache file it wrote."""
    import subprocess
    weight_bf16 = np.ascontiguousarray(weight_bf16, dtype=np.uint16)
    source = os.path.join(directory, "weight.bf16")
    cache = os.path.join(directory, "cache")
    os.makedirs(cache, exist_ok=True)
    weight_bf16.tofile(source)
    out = subprocess.run([PACKER_PROBE, "pack", source, str(weight_bf16.shape[0]), str(weight_bf16.shape[1]),
                          str(int(implementation)), "1" if equalise else "0", "1" if mse else "0", cache],
                         check=True, capture_output=True, text=True).stdout.split()
    files = [f for f in out if f.endswith(".safetensors")]
    assert len(files) == 1, out
    return files[0]


def ref_available() -> bool:
    return os.path.exists(REF_PATH)


def ref() -> _Ref:
    global _ref
    if _ref is None:
        _ref = _Ref()
    return _ref
