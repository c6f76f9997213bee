"""The C-ABI shared library loads without a GPU and exports every symbol the header declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


@pytest.fixture(scope="module")
def lib():
    from chitudiffusion_b200 import _lib, build

    build.build()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "chitu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(chitu_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert "chitu_b200_attn_fwd" in names and len(names) >= 7
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/chitu_b200.h but not exported"


def test_binding_lists_the_same_symbols(lib):
    from chitudiffusion_b200 import _lib

    assert sorted(_lib.EXPORTS) == _declared_functions()


def test_version_caps_and_argument_errors_need_no_gpu(lib):
    assert lib.chitu_b200_version() >= 100
    assert lib.chitu_b200_caps() & 1
    # argument validation happens before any CUDA call
    rc = lib.chitu_b200_attn_fwd(None, None, None, None, None, 1, 1, 1, 1, 128, None, None, None, 1.0, 0, None, None)
    assert rc == -1
    assert b"null" in lib.chitu_b200_last_error()
    st = (ctypes.c_int64 * 4)(128, 128, 128, 1)
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    rc = lib.chitu_b200_attn_fwd(p, p, p, p, None, 1, 1, 1, 1, 64, st, st, st, 1.0, 0, None, None)
    assert rc == -2 and b"head_dim" in lib.chitu_b200_last_error()


def test_backend_construction_and_cpu_tensors_fail_loudly():
    import torch

    from chitudiffusion_b200 import B200AttnBackend

    backend = B200AttnBackend("b200")
    assert backend.impl == "b200"
    with pytest.raises(RuntimeError):
        B200AttnBackend("flash_attn")
    q = torch.zeros(1, 4, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        backend(q, q, q)


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C11 (no torch types, no C++ in the signatures)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "use_header.c"
    src.write_text('#include "chitu_b200.h"\nint probe(void) { return (int)chitu_b200_version(); }\n')
    include = os.path.join(os.path.dirname(__file__), "..", "include")
    proc = subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-I", include, "-c", str(src), "-o",
                           str(tmp_path / "use_header.o")], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
