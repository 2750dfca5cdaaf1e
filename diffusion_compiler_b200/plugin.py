"""Host-side mirror of the reference's plugin executor, over the C-ABI of libdifb200.so.

The reference drives a backend plugin through ``Executor.prepare(program, bindings)`` and
``PreparedExecution.run(inputs, options)`` (reference ``include/dif/runtime/executor.hpp:662-680``,
``src/backend/plugin.cpp:119-296``). This module does the same calls -- ``dif_backend_get_v2``,
``create``, ``compile`` with the Constant-role tensors in program order, ``execute`` with the
Input-role tensors and zero-filled host outputs -- from Python with numpy host buffers, so the
parity tests read like the reference's own.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, Optional

import numpy as np

from . import _lib, diffir


class BackendError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__("backend plugin status %d: %s" % (status, text))
        self.status = status


class _Error(C.Structure):
    _fields_ = [("data", C.c_char_p), ("capacity", C.c_size_t)]


class _View(C.Structure):
    _fields_ = [("tensor_id", C.c_uint32), ("dtype", C.c_uint32), ("rank", C.c_uint32),
                ("dims", C.POINTER(C.c_uint64)), ("host_data", C.c_void_p), ("byte_count", C.c_uint64)]


class _RunOptions(C.Structure):
    _fields_ = [("warmups", C.c_uint32), ("iterations", C.c_uint32), ("minimum_free_bytes", C.c_uint64)]


class Telemetry(C.Structure):
    _fields_ = [("mean_milliseconds", C.c_double), ("minimum_milliseconds", C.c_double),
                ("maximum_milliseconds", C.c_double), ("free_bytes_before", C.c_uint64),
                ("free_bytes_after", C.c_uint64), ("device_name", C.c_char * 256)]


class _CompileOptions(C.Structure):
    _fields_ = [("minimum_free_bytes", C.c_uint64), ("flags", C.c_uint64)]


class CompileTelemetry(C.Structure):
    _fields_ = [("preparation_milliseconds", C.c_double), ("resident_bytes", C.c_uint64),
                ("free_bytes_before", C.c_uint64), ("free_bytes_after", C.c_uint64),
                ("device_name", C.c_char * 256)]


_CREATE = C.CFUNCTYPE(C.c_int, C.c_int32, C.POINTER(C.c_void_p), C.POINTER(_Error))
_DESTROY = C.CFUNCTYPE(None, C.c_void_p)
_COMPILE_V2 = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(_View), C.c_size_t,
                          C.POINTER(_CompileOptions), C.POINTER(C.c_void_p), C.POINTER(CompileTelemetry),
                          C.POINTER(_Error))
_COMPILE_V1 = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_void_p), C.POINTER(_Error))
_EXECUTE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(_View), C.c_size_t, C.POINTER(_View), C.c_size_t,
                       C.POINTER(_RunOptions), C.POINTER(Telemetry), C.POINTER(_Error))


class ApiV2(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("backend_name", C.c_char_p),
                ("capabilities", C.c_uint64), ("create", _CREATE), ("destroy", _DESTROY), ("compile", _COMPILE_V2),
                ("destroy_executable", _DESTROY), ("execute", _EXECUTE)]


class ApiV1(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("backend_name", C.c_char_p),
                ("capabilities", C.c_uint64), ("create", _CREATE), ("destroy", _DESTROY), ("compile", _COMPILE_V1),
                ("destroy_executable", _DESTROY), ("execute", _EXECUTE)]


_NP = {1: np.float32, 2: np.uint16, 3: np.uint16, 4: np.int8, 5: np.int32, 6: np.uint8}


def api_v2() -> ApiV2:
    L = _lib.lib()
    L.dif_backend_get_v2.restype = C.POINTER(ApiV2)
    return L.dif_backend_get_v2().contents


def api_v1() -> ApiV1:
    L = _lib.lib()
    L.dif_backend_get_v1.restype = C.POINTER(ApiV1)
    return L.dif_backend_get_v1().contents


def _views(program: diffir.Program, tensors, arrays: Dict[int, np.ndarray], keep: list):
    views = (_View * max(1, len(tensors)))()
    for i, t in enumerate(tensors):
        arr = np.ascontiguousarray(arrays[t.id])
        if arr.nbytes != t.byte_count():
            raise ValueError("tensor %d: %d bytes bound, program says %d" % (t.id, arr.nbytes, t.byte_count()))
        dims = (C.c_uint64 * len(t.dims))(*t.dims)
        keep += [arr, dims]
        views[i] = _View(t.id, int(t.dtype), len(t.dims), dims, arr.ctypes.data, arr.nbytes)
    return views


class PreparedExecution:
    """A compiled, device-resident program (reference ``PluginPreparedExecution``)."""

    def __init__(self, executor: "PluginExecutor", program: diffir.Program, handle, telemetry, v2: bool,
                 constants: Dict[int, np.ndarray]):
        self._executor, self.program, self._handle, self.compile_telemetry = executor, program, handle, telemetry
        self._v2, self._constants = v2, constants
        executor._prepared.add(self)

    def run(self, inputs: Dict[int, np.ndarray], warmups: int = 0, iterations: int = 1,
            minimum_free_bytes: int = 0, outputs: Optional[Dict[int, np.ndarray]] = None):
        api = self._executor.api
        p = self.program
        keep: list = []
        in_tensors = p.with_role(diffir.Role.Input)
        bound = dict(inputs)
        if not self._v2:  # v1: constants travel with every execute call
            in_tensors = in_tensors + p.with_role(diffir.Role.Constant)
            bound.update(self._constants)
        in_views = _views(p, in_tensors, bound, keep)
        out_tensors = p.with_role(diffir.Role.Output)
        if outputs is None:
            outputs = {t.id: np.zeros(t.dims, _NP[int(t.dtype)]) for t in out_tensors}
        out_views = _views(p, out_tensors, outputs, keep)
        # _views made contiguous copies only if needed; write-back targets must be the originals
        for i, t in enumerate(out_tensors):
            out_views[i].host_data = outputs[t.id].ctypes.data
        options = _RunOptions(warmups, iterations, minimum_free_bytes)
        telemetry = Telemetry()
        buf = C.create_string_buffer(1024)
        err = _Error(C.cast(buf, C.c_char_p), 1024)
        rc = api.execute(self._handle, in_views, len(in_tensors), out_views, len(out_tensors), C.byref(options),
                         C.byref(telemetry), C.byref(err))
        if rc != 0:
            raise BackendError(rc, buf.value.decode(errors="replace"))
        return outputs, telemetry

    def profile(self) -> Dict[int, tuple]:
        """{opcode: (milliseconds, steps)} summed over the timed passes since the last call; filled only
        when DIFB200_PROFILE=1 was in the environment at prepare() (difb200_executable_profile)."""
        from . import _lib
        cap = 64
        opcodes, ms, steps, n = (C.c_uint32 * cap)(), (C.c_double * cap)(), (C.c_uint64 * cap)(), C.c_uint32(0)
        _lib.check(_lib.lib().difb200_executable_profile(self._handle, opcodes, ms, steps, cap, C.byref(n)))
        return {int(opcodes[i]): (float(ms[i]), int(steps[i])) for i in range(n.value)}

    def exchange(self) -> str:
        """How a token-sharded executable moves its slices: "none" (one rank), "nccl" or "direct"
        (difb200_executable_exchange)."""
        from . import _lib
        return ("none", "nccl", "direct")[int(_lib.lib().difb200_executable_exchange(self._handle))]

    def close(self):
        if self._handle:
            self._executor.api.destroy_executable(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PluginExecutor:
    """``make_plugin_executor(library, device)`` of the reference, for libdifb200.so."""

    def __init__(self, device: int = 0, abi_version: int = 2):
        self.api = api_v2() if abi_version == 2 else api_v1()
        self._v2 = abi_version == 2
        ctx = C.c_void_p()
        buf = C.create_string_buffer(1024)
        err = _Error(C.cast(buf, C.c_char_p), 1024)
        rc = self.api.create(device, C.byref(ctx), C.byref(err))
        if rc != 0:
            raise BackendError(rc, buf.value.decode(errors="replace"))
        self._ctx = ctx
        # executables must be destroyed before their context (reference src/backend/plugin.cpp:96-99,
        # 186-191), so the executor closes what it prepared before it destroys the context
        self._prepared = weakref.WeakSet()

    def prepare(self, program: diffir.Program, constants: Dict[int, np.ndarray],
                minimum_free_bytes: int = 0) -> PreparedExecution:
        data = diffir.encode(program)
        exe = C.c_void_p()
        buf = C.create_string_buffer(1024)
        err = _Error(C.cast(buf, C.c_char_p), 1024)
        telemetry = CompileTelemetry()
        if self._v2:
            keep: list = []
            tensors = program.with_role(diffir.Role.Constant)
            views = _views(program, tensors, constants, keep)
            options = _CompileOptions(minimum_free_bytes, 1)
            rc = self.api.compile(self._ctx, data, len(data), views, len(tensors), C.byref(options), C.byref(exe),
                                  C.byref(telemetry), C.byref(err))
        else:
            rc = self.api.compile(self._ctx, data, len(data), C.byref(exe), C.byref(err))
        if rc != 0:
            raise BackendError(rc, buf.value.decode(errors="replace"))
        return PreparedExecution(self, program, exe, telemetry, self._v2, dict(constants))

    def close(self):
        if self._ctx:
            for prepared in list(self._prepared):
                prepared.close()
            self.api.destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
