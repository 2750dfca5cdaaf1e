"""ConvRot INT8 weight caches through the native library (``csrc/convrot_cache.cu``): the
SafeTensors files the reference keeps quantised Linear weights in -- per-projection ``weight`` /
``scale`` pairs (reference ``tools/difflux2sample.cpp:3079-3091``) and the generic cache with its
``__meta__.convrot_int8`` identity record (reference ``src/runtime/cuda_executor.cpp:4266-4364``,
``tools/difh3convrot.cpp:51,208-231``). This module only marshals numpy arrays to the C entry points."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from . import _lib, diffir

_NP = {1: np.float32, 2: np.uint16, 3: np.uint16, 4: np.int8, 5: np.int32, 6: np.uint8, 7: np.uint8, 8: np.uint8}
CVR1_MAGIC = 0x31525643
IDENTITY = "__meta__.convrot_int8"


def write(path: str, tensors: Dict[str, Tuple[int, np.ndarray]]) -> None:
    """Writes {name: (DiffIR dtype code, array)} in the given order."""
    names = list(tensors)
    n = len(names)
    arrays = [np.ascontiguousarray(tensors[k][1]) for k in names]
    c_names = (C.c_char_p * n)(*[k.encode() for k in names])
    dtypes = (C.c_uint32 * n)(*[int(tensors[k][0]) for k in names])
    ranks = (C.c_uint32 * n)(*[a.ndim for a in arrays])
    dims = (C.c_uint64 * (8 * n))()
    for i, a in enumerate(arrays):
        for j, d in enumerate(a.shape):
            dims[8 * i + j] = d
    data = (C.c_void_p * n)(*[a.ctypes.data for a in arrays])
    _lib.check(_lib.lib().difb200_cache_write(path.encode(), n, c_names, dtypes, ranks, dims, data))


class Cache:
    """A cache file opened for reading; tensors come back as numpy copies."""

    def __init__(self, path: str):
        self._h = C.c_void_p()
        _lib.check(_lib.lib().difb200_cache_open(path.encode(), C.byref(self._h)))

    def tensor(self, name: str) -> Tuple[int, np.ndarray]:
        dtype, rank, nbytes = C.c_uint32(), C.c_uint32(), C.c_uint64()
        dims = (C.c_uint64 * 8)()
        data = C.c_void_p()
        _lib.check(_lib.lib().difb200_cache_tensor(self._h, name.encode(), C.byref(dtype), C.byref(rank), dims,
                                                   C.byref(data), C.byref(nbytes)))
        raw = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nbytes.value,)).copy()
        shape = tuple(int(dims[i]) for i in range(rank.value))
        return dtype.value, raw.view(_NP.get(dtype.value, np.uint8)).reshape(shape if dtype.value else (-1,))

    def identity(self) -> np.ndarray:
        return self.tensor(IDENTITY)[1].view(np.uint32)

    def close(self):
        if self._h:
            _lib.lib().difb200_cache_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def fingerprint(program: diffir.Program) -> bytes:
    data = diffir.encode(program)
    out = (C.c_uint8 * 32)()
    _lib.check(_lib.lib().difb200_program_fingerprint(data, len(data), out))
    return bytes(out)


def cvr1_identity(projections: int, program_digest: bytes, index_digest: Optional[bytes] = None) -> np.ndarray:
    out = (C.c_uint32 * 20)()
    pd = (C.c_uint8 * 32)(*program_digest)
    idg = (C.c_uint8 * 32)(*index_digest) if index_digest else None
    _lib.lib().difb200_cvr1_identity(projections, pd, idg, out)
    return np.array(out[:], np.uint32)


def cvr1_check(identity: np.ndarray, program: Optional[diffir.Program], projections: int) -> None:
    ident = (C.c_uint32 * 20)(*[int(x) for x in np.asarray(identity, np.uint32)])
    data = diffir.encode(program) if program is not None else None
    _lib.check(_lib.lib().difb200_cvr1_check(ident, data, len(data) if data else 0, projections))


def build(path: str, program: diffir.Program, weights: Dict[int, np.ndarray], index_digest: Optional[bytes] = None):
    """Quantises the bf16 [N, K] weight matrices {weight tensor id: bit patterns} on the current GPU and
    writes the generic cache of ``program``."""
    import torch
    ids = list(weights)
    n = len(ids)
    arrays = [np.ascontiguousarray(weights[i], np.uint16) for i in ids]
    data = diffir.encode(program)
    idg = (C.c_uint8 * 32)(*index_digest) if index_digest else None
    _lib.check(_lib.lib().difb200_build_convrot_cache(
        path.encode(), data, len(data), n, (C.c_uint32 * n)(*ids), (C.c_void_p * n)(*[a.ctypes.data for a in arrays]),
        (C.c_uint64 * n)(*[a.shape[0] for a in arrays]), (C.c_uint64 * n)(*[a.shape[1] for a in arrays]), idg,
        C.c_void_p(torch.cuda.current_stream().cuda_stream)))
