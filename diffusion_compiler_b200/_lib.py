"""ctypes binding of libdifb200.so. There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdifb200.so")

_lib = None


class Difb200Error(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__("difb200 status %d: %s" % (status, text))
        self.status = status


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libdifb200.so is not built (%s). Run `python -m diffusion_compiler_b200.build`; "
                "there is no CPU or PyTorch fallback." % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        vp, u64, u32, i32, f32 = C.c_void_p, C.c_uint64, C.c_uint32, C.c_int32, C.c_float
        L.difb200_last_error.restype = C.c_char_p
        L.difb200_version.restype = C.c_int
        L.difb200_poll_status.restype = C.c_int
        L.difb200_launch_count.restype = u64
        L.difb200_set_wait_limit_ns.restype = None
        L.difb200_set_wait_limit_ns.argtypes = [u64]
        L.difb200_test_withhold_gemm_load.restype = None
        L.difb200_test_withhold_gemm_load.argtypes = [u32]
        L.difb200_selftest_host.restype = C.c_int
        L.difb200_quantize_int8_rows.restype = C.c_int
        L.difb200_quantize_int8_rows.argtypes = [C.POINTER(vp), C.POINTER(u64), u32, u64, i32, f32, vp,
                                                 vp, vp, vp, vp, vp]
        L.difb200_rms_norm_modulate_quant.restype = C.c_int
        L.difb200_rms_norm_modulate_quant.argtypes = [vp, vp, vp, vp, u64, u64, f32, i32, f32, vp, vp, vp]
        L.difb200_layer_norm_modulate_quant.restype = C.c_int
        L.difb200_layer_norm_modulate_quant.argtypes = [vp, vp, vp, vp, vp, u64, u64, u64, f32, i32, f32, vp, vp, vp]
        L.difb200_quantize_weight_rows.restype = C.c_int
        L.difb200_quantize_weight_rows.argtypes = [vp, vp, u64, u64, i32, i32, vp, vp, vp]
        L.difb200_linear_int8_scaled.restype = C.c_int
        L.difb200_linear_int8_scaled.argtypes = [vp, vp, vp, vp, vp, u32, u64, u64, u64, vp, vp, vp]
        L.difb200_w8a8_linear.restype = C.c_int
        L.difb200_w8a8_linear.argtypes = [vp, vp, vp, vp, u32, i32, f32, u64, u64, u64, vp, vp, vp, vp]
        L.difb200_w8a8_linear_static.restype = C.c_int
        L.difb200_w8a8_linear_static.argtypes = [vp, vp, vp, vp, u32, i32, f32, u64, u64, u64, vp, i32, vp]
        L.difb200_attention_int8_scratch_bytes.restype = u64
        L.difb200_attention_int8_scratch_bytes.argtypes = [u64, u64, u64]
        L.difb200_attention_int8.restype = C.c_int
        L.difb200_attention_int8.argtypes = [vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, u64, u64, f32, vp, u64, vp, vp]
        L.difb200_attention_int8_state_bytes.restype = u64
        L.difb200_attention_int8_state_bytes.argtypes = [u64, u64, u64]
        L.difb200_attention_int8_chunk.restype = C.c_int
        L.difb200_attention_int8_chunk.argtypes = [vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, u64, u64, f32, vp, u64,
                                                   vp, C.POINTER(u32), i32, i32, vp, vp]
        pu8, pu64, pi32, pu32 = C.POINTER(C.c_uint8), C.POINTER(u64), C.POINTER(i32), C.POINTER(u32)
        for name, args in (
                ("difb200_world_unique_id", [pu8]),
                ("difb200_world_rendezvous", [C.c_char_p, i32, i32, pu8, u32]),
                ("difb200_world_create", [pu8, i32, i32, C.POINTER(vp)]),
                ("difb200_world_destroy", [vp]),
                ("difb200_world_exchange", [vp, i32, C.POINTER(vp), pu64, i32, vp]),
                ("difb200_world_bind", [vp, u64, vp, C.POINTER(vp), C.POINTER(vp), pi32]),
                ("difb200_world_unbind", [vp, vp]),
                ("difb200_world_push", [vp, vp, i32, pu64, pu64, i32, vp]),
                ("difb200_world_selftest_flags", [u64, i32]),
                ("difb200_sharded_attention", [vp, vp, vp, vp, vp, vp, vp, vp, u64, u64, u64, u64, f32, vp, u64, vp,
                                               vp, vp]),
                ("difb200_world_plan", [i32, i32, u32, pi32, i32, pu32, pi32, pi32, i32, pi32]),
                ("difb200_world_selftest_fake", [i32, i32, u32])):
            getattr(L, name).restype = C.c_int
            getattr(L, name).argtypes = args
        pcs = C.POINTER(C.c_char_p)
        for name, args in (
                ("difb200_cache_open", [C.c_char_p, C.POINTER(vp)]),
                ("difb200_cache_close", [vp]),
                ("difb200_cache_tensor", [vp, C.c_char_p, C.POINTER(u32), C.POINTER(u32), C.POINTER(u64),
                                          C.POINTER(vp), C.POINTER(u64)]),
                ("difb200_cache_write", [C.c_char_p, u32, pcs, C.POINTER(u32), C.POINTER(u32), C.POINTER(u64),
                                         C.POINTER(vp)]),
                ("difb200_program_fingerprint", [C.c_char_p, u64, C.POINTER(C.c_uint8)]),
                ("difb200_cvr1_check", [C.POINTER(u32), C.c_char_p, u64, u32]),
                ("difb200_build_convrot_cache", [C.c_char_p, C.c_char_p, u64, u32, C.POINTER(u32), C.POINTER(vp),
                                                 C.POINTER(u64), C.POINTER(u64), C.POINTER(C.c_uint8), vp])):
            getattr(L, name).restype = C.c_int
            getattr(L, name).argtypes = args
        L.difb200_cvr1_identity.restype = None
        L.difb200_cvr1_identity.argtypes = [u32, C.POINTER(C.c_uint8), C.POINTER(C.c_uint8), C.POINTER(u32)]
        L.difb200_measure_i8_mma_peak.restype = C.c_int
        L.difb200_measure_i8_mma_peak.argtypes = [i32, u32, C.POINTER(C.c_double), C.POINTER(C.c_double), vp]
        L.difb200_executable_profile.restype = C.c_int
        L.difb200_executable_profile.argtypes = [vp, C.POINTER(u32), C.POINTER(C.c_double), C.POINTER(u64), u32,
                                                 C.POINTER(u32)]
        L.difb200_program_check.restype = C.c_int
        L.difb200_program_check.argtypes = [C.c_char_p, u64]
        L.difb200_executable_exchange.restype = C.c_int
        L.difb200_executable_exchange.argtypes = [vp]
        L.difb200_attention_scratch_bytes.restype = u64
        L.difb200_attention_scratch_bytes.argtypes = [u64, u64, u64, u64]
        L.difb200_attention.restype = C.c_int
        L.difb200_attention.argtypes = [vp, vp, vp, vp, u64, u64, u64, u64, u64, f32, vp, u64, vp, vp]
        for name, args in (
                ("difb200_rms_norm_modulate", [vp, vp, vp, vp, vp, u32, u64, u64, f32, vp]),
                ("difb200_layer_norm_modulate", [vp, vp, vp, vp, vp, vp, u32, u64, u64, u64, f32, vp]),
                ("difb200_qk_norm_rope", [vp, vp, vp, vp, vp, u32, u32, u64, u64, u64, u64, u64, u64, u64, u64, f32,
                                          i32, vp]),
                ("difb200_qk_norm_rope_quant", [vp, vp, vp, vp, vp, vp, vp, u32, u64, u64, u64, u64, u64, u64, u64,
                                                f32, i32, vp]),
                ("difb200_residual_gate", [vp, vp, vp, vp, u32, u64, u64, u64, vp]),
                ("difb200_swiglu", [vp, vp, u32, u64, u64, u64, u64, i32, vp])):
            getattr(L, name).restype = C.c_int
            getattr(L, name).argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise Difb200Error(status, lib().difb200_last_error().decode(errors="replace"))
