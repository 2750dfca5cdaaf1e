"""CPU checks of the C-ABI: the library loads and exports every symbol that include/difb200/*.h
declares, the plugin API tables are well-formed, the restated ABI header has the reference's
layout, and without a CUDA device the product fails loudly instead of falling back."""
import ctypes as C
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")


def _reference_root():
    """The reference checkout the oracle recipe builds from (its REF variable)."""
    res = subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "print-ref"],
                         capture_output=True, text=True)
    return res.stdout.strip()


REF_ABI = os.path.join(_reference_root(), "include", "dif", "backend", "abi.h")


@pytest.fixture(scope="module")
def lib():
    from diffusion_compiler_b200 import _lib, build
    build.build()
    return _lib.lib()


def _declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(INCLUDE, "difb200")):
        text = open(os.path.join(INCLUDE, "difb200", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"#define[^\n]*", "", text)
        for m in re.finditer(r"(?:DIFB200_EXPORT|DIF_BACKEND_EXPORT)\s+[^;(]*?\b(\w+)\s*\(", text):
            names.add(m.group(1))
    return names


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert {"dif_backend_get_v2", "dif_backend_get_v1", "difb200_quantize_int8_rows",
            "difb200_linear_int8_scaled", "difb200_attention_int8"} <= names
    for name in names:
        assert hasattr(lib, name), "libdifb200.so does not export %s" % name


def test_api_tables(lib):
    from diffusion_compiler_b200 import plugin
    for api, version, typ in ((plugin.api_v2(), 2, plugin.ApiV2), (plugin.api_v1(), 1, plugin.ApiV1)):
        assert api.abi_version == version
        assert api.struct_size == C.sizeof(typ)
        assert api.backend_name == b"difb200"
        assert api.capabilities & 0b1010 == 0b1010  # BF16 | I8
        for field in ("create", "destroy", "compile", "destroy_executable", "execute"):
            assert C.cast(getattr(api, field), C.c_void_p).value


def test_per_device_bookkeeping_selftest(lib):
    """One-time kernel set-up (shared-memory opt-in, resident CTA pairs) is keyed by device
    ordinal, a failed set-up is retried, and the wait-limit state round-trips: the library's
    host-only self-check, which touches no GPU."""
    assert lib.difb200_selftest_host() == 0, lib.difb200_last_error().decode()


def test_create_without_gpu_fails_loudly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from diffusion_compiler_b200 import plugin
    with pytest.raises(plugin.BackendError) as info:
        plugin.PluginExecutor(0)
    assert info.value.status == 2 and "no CPU path" in str(info.value)


def test_ops_reject_cpu_tensors(lib):
    import torch
    from diffusion_compiler_b200 import ops
    with pytest.raises(ValueError):
        ops.quantize_int8_rows([torch.zeros(4, 256, dtype=torch.bfloat16)], 2)


@pytest.mark.skipif(not os.path.exists(REF_ABI), reason="reference header not present on this machine")
def test_abi_layout_matches_reference(tmp_path):
    """Compile a checker that includes both headers under renamed identifiers and compares
    sizeof / offsetof of every structure and the values of every enumerator."""
    structs = {
        "dif_backend_error": ["data", "capacity"],
        "dif_backend_tensor_view": ["tensor_id", "dtype", "rank", "dims", "host_data", "byte_count"],
        "dif_backend_run_options": ["warmups", "iterations", "minimum_free_bytes"],
        "dif_backend_telemetry": ["mean_milliseconds", "minimum_milliseconds", "maximum_milliseconds",
                                  "free_bytes_before", "free_bytes_after", "device_name"],
        "dif_backend_api_v1": ["struct_size", "abi_version", "backend_name", "capabilities", "create", "destroy",
                               "compile", "destroy_executable", "execute"],
        "dif_backend_compile_options_v2": ["minimum_free_bytes", "flags"],
        "dif_backend_compile_telemetry_v2": ["preparation_milliseconds", "resident_bytes", "free_bytes_before",
                                             "free_bytes_after", "device_name"],
        "dif_backend_api_v2": ["struct_size", "abi_version", "backend_name", "capabilities", "create", "destroy",
                               "compile", "destroy_executable", "execute"],
    }
    enums = ["DIF_BACKEND_OK", "DIF_BACKEND_INVALID_ARGUMENT", "DIF_BACKEND_UNSUPPORTED", "DIF_BACKEND_OUT_OF_MEMORY",
             "DIF_BACKEND_COMPILE_ERROR", "DIF_BACKEND_EXECUTION_ERROR", "DIF_BACKEND_INTERNAL_ERROR",
             "DIF_BACKEND_CAP_F32", "DIF_BACKEND_CAP_BF16", "DIF_BACKEND_CAP_F16", "DIF_BACKEND_CAP_I8",
             "DIF_BACKEND_CAP_TRAINING", "DIF_BACKEND_CAP_ASYNC", "DIF_BACKEND_COMPILE_COPY_CONSTANTS"]

    def side(header, tag):
        text = open(header).read()
        # give every dif_backend identifier a per-side suffix so both headers can coexist
        return re.sub(r"\b(dif_backend_\w+|DIF_BACKEND_\w+)\b", lambda m: m.group(1) + tag, text)

    src = ["#include <stddef.h>", "#include <stdint.h>", side(REF_ABI, "_ref"),
           side(os.path.join(INCLUDE, "difb200", "abi.h"), "_own")]
    for s, fields in structs.items():
        src.append("_Static_assert(sizeof(%s_ref) == sizeof(%s_own), \"%s size\");" % (s, s, s))
        for f in fields:
            src.append("_Static_assert(offsetof(%s_ref, %s) == offsetof(%s_own, %s), \"%s.%s\");" % (s, f, s, f, s, f))
    for e in enums:
        src.append("_Static_assert((long long)%s_ref == (long long)%s_own, \"%s\");" % (e, e, e))
    src.append("int main(void) { return 0; }")
    path = tmp_path / "abi_check.c"
    path.write_text("\n".join(src))
    res = subprocess.run(["gcc", "-std=c11", "-fsyntax-only", str(path)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
