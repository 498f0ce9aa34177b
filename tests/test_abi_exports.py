"""The C ABI: every function declared in include/*.h is exported by the built libraries, and the ctypes
signature table names exactly those functions.  No compute calls (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    src = open(os.path.join(ROOT, "include", header)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(esp_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def built():
    from loongserve_b200 import build
    build.build_all(force=False)
    from loongserve_b200 import _lib
    return _lib


def test_attention_header_symbols_exported(built):
    names = _declared("esp_attention.h")
    assert len(names) >= 17
    lib = C.CDLL(built.ATTN_LIB)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in esp_attention.h but not exported"
    table = set(built.ATTN_SIGNATURES) | set(built.ATTN_STRING_FUNCS) | {"esp_pool_can_use"}
    assert table == set(names) - {"esp_pool"}


def test_rnccl_header_symbols_exported(built):
    names = [n for n in _declared("esp_rnccl.h") if n != "esp_rnccl_comm"]
    import torch  # noqa: F401  (loads the NCCL copy the library binds to)
    lib = C.CDLL(built.RNCCL_LIB)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in esp_rnccl.h but not exported"
    assert set(built.RNCCL_SIGNATURES) | {"esp_rnccl_stream", "esp_rnccl_last_error"} == set(names)


def test_argument_counts_match_header(built):
    src = open(os.path.join(ROOT, "include", "esp_attention.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    for name, args in built.ATTN_SIGNATURES.items():
        mt = re.search(r"\b" + name + r"\s*\((.*?)\)\s*;", src, flags=re.S)
        assert mt, name
        params = [p for p in mt.group(1).split(",") if p.strip() and p.strip() != "void"]
        assert len(params) == len(args), f"{name}: header has {len(params)} parameters, ctypes table {len(args)}"


def test_error_strings_and_argument_checks(built):
    lib = built.attn()
    assert lib.esp_strerror(0) == b"ok"
    assert b"unsupported" in lib.esp_strerror(-5)
    # argument validation happens on the host before any CUDA call
    assert lib.esp_kv_scatter(None, 0, 0, None, 0, 0, None, 0, 5, 1, 8, 2, 0, None) == -1
    assert lib.esp_decode_merge(None, None, None, None, None, 1, 1, 128, 1, 1, 2, None) == -1
    assert lib.esp_kv_scatter(None, 0, 0, None, 0, 0, None, 0, 0, 1, 8, 2, 0, None) == 0     # empty input is a no-op


def test_ops_refuse_cpu_tensors(built):
    import torch
    from loongserve_b200 import kv_ops
    with pytest.raises(RuntimeError, match="CUDA"):
        kv_ops.destindex_copy_kv(torch.zeros(2, 2, 8), torch.zeros(2, dtype=torch.int32), torch.zeros(4, 2, 8))


def test_abi_version_matches_header_and_python_table(built):
    src = open(os.path.join(ROOT, "include", "esp_attention.h")).read()
    header_version = int(re.search(r"#define\s+ESP_ABI_VERSION\s+(\d+)", src).group(1))
    lib = C.CDLL(built.ATTN_LIB)
    lib.esp_abi_version.restype = C.c_int
    assert lib.esp_abi_version() == header_version == built.ESP_ABI_VERSION


def test_build_entry_point_runs():
    import __graft_entry__ as g
    g.build()


def test_headers_compile_as_plain_c_and_link(tmp_path, built):
    """The boundary is a C ABI: both headers must be usable from a C99 translation unit, and a C program linked against
    the library must resolve and call a symbol (no device work: the version query)."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("gcc not available")
    src = tmp_path / "abi.c"
    src.write_text('#include "esp_attention.h"\n#include "esp_rnccl.h"\n'
                   'int main(void) { return esp_abi_version() == ESP_ABI_VERSION ? 0 : 1; }\n')
    exe = tmp_path / "abi"
    libdir = os.path.dirname(built.ATTN_LIB)
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-l:libesp_attention.so", f"-Wl,-rpath,{libdir}"], check=True)
    env = dict(os.environ)
    import torch
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    env["LD_LIBRARY_PATH"] = os.pathsep.join([torch_lib, "/usr/local/cuda/lib64", env.get("LD_LIBRARY_PATH", "")])
    assert subprocess.run([str(exe)], env=env).returncode == 0
