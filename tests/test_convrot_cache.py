"""ConvRot INT8 weight caches: the files this library writes must be readable by the reference's
own SafeTensors reader, files written by the reference's own writer must load here, and the
generic cache's identity record must follow the reference's rules (magic "CVR1", version, group
256, projection count, program fingerprint: reference src/runtime/cuda_executor.cpp:4266-4364,
tools/difh3convrot.cpp:208-231; container src/weights/safetensors.cpp; per-projection pairs
tools/difflux2sample.cpp:3079-3091). The reference side runs through oracle/_ref. CPU tests; the
GPU test builds a cache with the weight-side quantiser and binds it as plugin constants."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_bridge as ob
from diffusion_compiler_b200 import convrot_cache, diffir

needs_ref = pytest.mark.skipif(not ob.ref_available(), reason="reference build (oracle/_ref) not present")


def _ref():
    lib = C.CDLL(ob.REF_PATH)
    return lib


def _ref_read(path, name, capacity=1 << 24):
    lib = _ref()
    dtype, rank, nbytes = C.c_uint32(), C.c_uint32(), C.c_uint64()
    dims = (C.c_uint64 * 8)()
    buf = (C.c_uint8 * capacity)()
    err = C.create_string_buffer(1024)
    rc = lib.difref_read_safetensor(path.encode(), name.encode(), C.byref(dtype), C.byref(rank), dims, buf,
                                    C.c_uint64(capacity), C.byref(nbytes), err, C.c_size_t(1024))
    if rc != 0:
        raise RuntimeError(err.value.decode())
    return dtype.value, tuple(dims[i] for i in range(rank.value)), bytes(buf[:nbytes.value])


def _ref_write(path, tensors):
    lib = _ref()
    names = list(tensors)
    n = len(names)
    arrays = [np.ascontiguousarray(tensors[k][1]) for k in names]
    dims = (C.c_uint64 * (8 * n))()
    for i, a in enumerate(arrays):
        for j, d in enumerate(a.shape):
            dims[8 * i + j] = d
    err = C.create_string_buffer(1024)
    rc = lib.difref_write_safetensors(path.encode(), C.c_size_t(n), (C.c_char_p * n)(*[k.encode() for k in names]),
                                      (C.c_uint32 * n)(*[tensors[k][0] for k in names]),
                                      (C.c_uint32 * n)(*[a.ndim for a in arrays]), dims,
                                      (C.c_void_p * n)(*[a.ctypes.data for a in arrays]),
                                      (C.c_uint64 * n)(*[a.nbytes for a in arrays]), err, C.c_size_t(1024))
    if rc != 0:
        raise RuntimeError(err.value.decode())


def _pair(rng, N=24, K=512):
    w = ob.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    codes, scales = ob.orc().quantize_weight_rows(w, 2)
    return w, codes, scales


@needs_ref
def test_pair_cache_written_here_is_read_by_the_reference(tmp_path):
    rng = np.random.default_rng(0)
    _, codes, scales = _pair(rng)
    eq = ob.f32_to_bf16(np.linspace(0.5, 2.0, codes.shape[1]).astype(np.float32))
    path = str(tmp_path / "block0.safetensors")
    convrot_cache.write(path, {"weight": (4, codes), "scale": (1, scales), "input_scale": (2, eq)})
    assert not os.path.exists(path + ".building")
    for name, (dtype, arr) in {"weight": (4, codes), "scale": (1, scales), "input_scale": (2, eq)}.items():
        got_dtype, dims, data = _ref_read(path, name)
        assert got_dtype == dtype and dims == arr.shape and data == arr.tobytes()


@needs_ref
def test_pair_cache_written_by_the_reference_loads_here(tmp_path):
    rng = np.random.default_rng(1)
    _, codes, scales = _pair(rng, 40, 256)
    path = str(tmp_path / "ref.safetensors")
    _ref_write(path, {"weight": (4, codes), "scale": (1, scales)})
    # byte for byte the file this library's writer produces for the same tensors
    ours = str(tmp_path / "ours.safetensors")
    convrot_cache.write(ours, {"weight": (4, codes), "scale": (1, scales)})
    assert open(path, "rb").read() == open(ours, "rb").read()
    with convrot_cache.Cache(path) as cache:
        dtype, w = cache.tensor("weight")
        assert dtype == 4 and np.array_equal(w, codes)
        dtype, s = cache.tensor("scale")
        assert dtype == 1 and np.array_equal(s.view(np.uint32), scales.view(np.uint32))
        with pytest.raises(Exception):
            cache.tensor("input_scale")


def test_unfinished_and_malformed_files_are_refused(tmp_path):
    path = str(tmp_path / "c.safetensors")
    open(path + ".building", "wb").write(b"partial")
    with pytest.raises(Exception) as info:
        convrot_cache.write(path, {"weight": (4, np.zeros((2, 256), np.int8))})
    assert "incomplete cache" in str(info.value) and not os.path.exists(path)
    for blob in (b"", b"\x08\x00\x00\x00\x00\x00\x00\x00{}      ", b"\xff" * 16,
                 b"\x40\x00\x00\x00\x00\x00\x00\x00" + b'{"w":{"dtype":"I8","shape":[4],"data_offsets":[0,9]}}'.ljust(64)):
        bad = str(tmp_path / "bad.safetensors")
        open(bad, "wb").write(blob)
        with pytest.raises(Exception):
            convrot_cache.Cache(bad)


def _two_linear_program():
    p = diffir.Program()
    x = p.add_tensor(diffir.DType.BF16, [8, 512], diffir.Role.Input)
    w1 = p.add_tensor(diffir.DType.BF16, [256, 512], diffir.Role.Constant)
    y = p.add_tensor(diffir.DType.BF16, [8, 256])
    w2 = p.add_tensor(diffir.DType.BF16, [512, 256], diffir.Role.Constant)
    z = p.add_tensor(diffir.DType.BF16, [8, 512], diffir.Role.Output)
    p.add_op(diffir.Opcode.Linear, [x, w1], [y])
    p.add_op(diffir.Opcode.Linear, [y, w2], [z])
    return p, (w1, w2)


@needs_ref
def test_program_fingerprint_and_identity_record_follow_the_reference():
    p, _ = _two_linear_program()
    data = diffir.encode(p)
    want = (C.c_uint8 * 32)()
    err = C.create_string_buffer(1024)
    assert _ref().difref_fingerprint(data, C.c_size_t(len(data)), want, err, C.c_size_t(1024)) == 0, err.value
    digest = convrot_cache.fingerprint(p)
    assert digest == bytes(want)
    index = bytes(range(32))
    ident = convrot_cache.cvr1_identity(2, digest, index)
    assert ident.shape == (20,) and ident[0] == convrot_cache.CVR1_MAGIC and tuple(ident[1:4]) == (1, 256, 2)
    assert ident[4:12].tobytes() == digest and ident[12:20].tobytes() == index  # little-endian words
    convrot_cache.cvr1_check(ident, p, 2)
    with pytest.raises(Exception) as info:
        convrot_cache.cvr1_check(ident, p, 3)
    assert "projection count" in str(info.value)
    other, _ = _two_linear_program()
    other.tensors[0].dims[0] = 9
    other.tensors[2].dims[0] = 9
    other.tensors[4].dims[0] = 9
    with pytest.raises(Exception) as info:
        convrot_cache.cvr1_check(ident, other, 2)
    assert "fingerprint mismatch" in str(info.value)
    bad = ident.copy()
    bad[2] = 128
    with pytest.raises(Exception) as info:
        convrot_cache.cvr1_check(bad, p, 2)
    assert "unsupported format metadata" in str(info.value)


@pytest.mark.gpu
@needs_ref
def test_cache_built_on_the_gpu_matches_the_cpu_packer_and_binds_as_plugin_constants(tmp_path):
    """difb200_build_convrot_cache on a two-Linear program: the reference's reader sees the identity
    record and the tensors under the names its loader asks for, the codes and scales equal the CPU
    packer's bit for bit, and bound as the constants of the W8A8 rewrite of the program they give
    the reference executor's result."""
    from diffusion_compiler_b200 import plugin
    rng = np.random.default_rng(3)
    p, (w1, w2) = _two_linear_program()
    weights = {w1: ob.f32_to_bf16((rng.standard_normal((256, 512)) * 0.02).astype(np.float32)),
               w2: ob.f32_to_bf16((rng.standard_normal((512, 256)) * 0.02).astype(np.float32))}
    path = str(tmp_path / "generic.safetensors")
    convrot_cache.build(path, p, weights, index_digest=bytes(32))
    dtype, dims, data = _ref_read(path, convrot_cache.IDENTITY)
    assert dtype == 5 and dims == (20,)
    ident = np.frombuffer(data, np.uint32)
    convrot_cache.cvr1_check(ident, p, 2)
    packed = {}
    with convrot_cache.Cache(path) as cache:
        for wid, bits in weights.items():
            want_codes, want_scales = ob.orc().quantize_weight_rows(bits, 2)
            _, codes = cache.tensor("linear.%d.weight" % wid)
            _, scales = cache.tensor("linear.%d.scale" % wid)
            assert np.array_equal(codes, want_codes)
            assert np.array_equal(scales.view(np.uint32), want_scales.view(np.uint32))
            assert _ref_read(path, "linear.%d.weight" % wid)[2] == want_codes.tobytes()
            packed[wid] = (codes, scales)
    # the W8A8 rewrite of the program with the cache's tensors as constants, on both executors
    q = diffir.Program()
    x = q.add_tensor(diffir.DType.BF16, [8, 512], diffir.Role.Input)
    consts, cur, K = {}, x, 512
    for i, wid in enumerate((w1, w2)):
        N = packed[wid][0].shape[0]
        codes = q.add_tensor(diffir.DType.I8, [8, K])
        row = q.add_tensor(diffir.DType.F32, [8])
        w = q.add_tensor(diffir.DType.I8, [N, K], diffir.Role.Constant)
        cs = q.add_tensor(diffir.DType.F32, [N], diffir.Role.Constant)
        y = q.add_tensor(diffir.DType.BF16, [8, N], diffir.Role.Output if i == 1 else diffir.Role.Internal)
        q.add_op(diffir.Opcode.QuantizeInt8Rows, [cur], [codes, row],
                 [diffir.Attribute.u64(diffir.AttrKey.BlockSize, 256), diffir.Attribute.u64(diffir.AttrKey.Implementation, 2)])
        q.add_op(diffir.Opcode.LinearInt8Scaled, [codes, w, row, cs], [y])
        consts[w], consts[cs] = packed[wid]
        cur, K = y, N
    inputs = {x: ob.f32_to_bf16(rng.standard_normal((8, 512)).astype(np.float32))}
    want, _ = ob.ref().run(q, {**consts, **inputs})
    ex = plugin.PluginExecutor(0)
    prepared = ex.prepare(q, consts)
    got, _ = prepared.run(inputs)
    prepared.close()
    ex.close()
    assert np.array_equal(got[cur], want[cur])


needs_packer = pytest.mark.skipif(not ob.packer_probe_available(),
                                  reason="reference packer probe (oracle/_ref/difpacker_scale) not present")


@needs_packer
@pytest.mark.parametrize("impl,N,K", [(1, 40, 384), (2, 40, 768), (3, 40, 768), (5, 24, 512), (6, 24, 512),
                                      (4, 8, 4096), (7, 8, 4096)])
@pytest.mark.parametrize("equalise,mse", [(False, False), (True, False), (False, True), (True, True)])
def test_reference_packer_output_equals_the_restatement_and_loads_here(tmp_path, impl, N, K, equalise, mse):
    """The reference's OWN offline W8A8 packer (rewrite_named_linear_w8a8 of tools/difflux2sample.cpp,
    run on a one-Linear program through oracle/_ref/difpacker_scale) writes its cache file for a seeded
    bf16 weight; this library's reader loads that file, and the restatements the GPU weight quantiser
    is tested against -- orc_weight_equalization, orc_quantize_weight_rows with and without the MSE
    scale search -- reproduce its three tensors bit for bit, for every QuantizeInt8Rows variant."""
    rng = np.random.default_rng(1000 * impl + 2 * int(equalise) + int(mse))
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    w[:, rng.integers(0, K, 6)] *= 12.0   # a few loud input channels: what equalisation is for
    w[2] = 0.0                            # an all-zero output channel
    w[3, 7] = 1.5                         # one outlier in a row: what the MSE search is for
    w = ob.f32_to_bf16(w)
    path = ob.packer_pack(w, impl, equalise, mse, str(tmp_path))
    assert ("weight-equalized" in path) == equalise and ("mse-weight-scale" in path) == mse
    with convrot_cache.Cache(path) as cache:
        dt_w, codes = cache.tensor("weight")
        dt_s, scales = cache.tensor("scale")
        assert dt_w == int(diffir.DType.I8) and dt_s == int(diffir.DType.F32)
        assert codes.shape == (N, K) and scales.shape == (N,)
        eq = None
        if equalise:
            dt_e, eq = cache.tensor("input_scale")
            assert dt_e == int(diffir.DType.BF16) and eq.shape == (K,)
    if equalise:
        want_eq = ob.orc().weight_equalization(w)
        assert np.array_equal(eq.view(np.uint16).ravel(), want_eq.view(np.uint16).ravel())
    if impl == 1:
        return  # Direct weights are not a ConvRot variant of orc_quantize_weight_rows; the file loaded, the vector matched
    want_codes, want_scales = ob.orc().quantize_weight_rows(w, impl, mse=mse, equalise=eq if equalise else None)
    assert np.array_equal(scales.view(np.uint32), want_scales.view(np.uint32))
    assert np.array_equal(codes.view(np.int8), want_codes)


def test_mutated_cache_files_are_refused_or_read_never_crashed_on(tmp_path):
    """Seeded mutations of a valid file (header bytes flipped, truncation, a wrong length word, junk
    inserted into the JSON, tokens replaced, 2000 levels of nesting): the reader either opens the file
    and serves or refuses each tensor, or refuses the file with an error -- it never faults."""
    import random
    import struct
    from diffusion_compiler_b200 import _lib
    rng = random.Random(5)
    good = str(tmp_path / "good.safetensors")
    convrot_cache.write(good, {"weight": (int(diffir.DType.I8), np.arange(64, dtype=np.int8).reshape(4, 16)),
                               "scale": (int(diffir.DType.F32), np.ones(4, np.float32))})
    raw = open(good, "rb").read()
    opened = refused = 0
    for _ in range(600):
        b = bytearray(raw)
        mode = rng.randrange(6)
        if mode == 0:
            for _ in range(rng.randrange(1, 6)):
                b[rng.randrange(0, min(len(b), 208))] = rng.randrange(256)
        elif mode == 1:
            b = b[:rng.randrange(0, len(b))]
        elif mode == 2:
            b[0:8] = struct.pack("<Q", rng.choice([0, 1, 7, 2 ** 63, 2 ** 64 - 1, len(b), 2 * len(b), rng.randrange(2 ** 40)]))
        elif mode == 3:
            at = rng.randrange(8, min(len(b), 200))
            b[at:at] = bytes(rng.randrange(256) for _ in range(rng.randrange(1, 40)))
        elif mode == 4:
            body = bytes(b[8:])
            token = rng.choice([b'"data_offsets"', b'"shape"', b'"dtype"', b"[", b"]", b"{", b"}", b":", b",", b'"I8"'])
            b = b[:8] + body.replace(token, rng.choice([b"", b'"x"', b"[[", b"-1", b"1e999", b"9" * 30, b"null", b'"\\']), 1)
        else:
            b = bytearray(struct.pack("<Q", 4000) + b"[" * 2000 + b"]" * 2000)
        path = str(tmp_path / "mutated.safetensors")
        with open(path, "wb") as f:
            f.write(bytes(b))
        try:
            with convrot_cache.Cache(path) as cache:
                for name in ("weight", "scale", "absent"):
                    try:
                        cache.tensor(name)
                    except (_lib.Difb200Error, KeyError, ValueError):
                        pass
            opened += 1
        except (_lib.Difb200Error, ValueError):
            refused += 1
    assert opened + refused == 600 and refused > 300
