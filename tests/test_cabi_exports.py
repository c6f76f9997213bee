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


def test_exchange_entries_validate_their_descriptors_without_a_gpu(lib):
    from chitudiffusion_b200 import _lib

    st = (ctypes.c_int64 * 4)(128, 128, 128, 1)
    buf = ctypes.create_string_buffer(256)
    p = ctypes.addressof(buf)
    dests = _lib.ptr_array([p, p])
    # push mode without its descriptors
    rc = lib.chitu_b200_attn_fwd_exchange_push(p, p, p, dests, 2, 128, 128, 128, 0, 1, 256, 256, 1, 128, st, st, st,
                                               1.0, 0, 1, None, 0, 128, None, None, None, None)
    assert rc == -1 and b"descriptor" in lib.chitu_b200_last_error()
    # the flag exchange without a sync block
    rc = lib.chitu_b200_attn_fwd_exchange(p, p, p, dests, 2, 128, 128, 128, 0, 1, 256, 256, 1, 128, st, st, st, 1.0,
                                          0, 1, None, 0, 128, 0, None, 0, 0, 0, None, None, None)
    assert rc == -1 and b"sync" in lib.chitu_b200_last_error()
    # a sync descriptor whose rank is outside the group
    blocks = (ctypes.c_void_p * 2)(p, p)
    bad = _lib.PeerSyncDesc(ctypes.cast(blocks, ctypes.POINTER(ctypes.c_void_p)), 5, 2)
    assert lib.chitu_b200_peer_wait_outputs(ctypes.byref(bad), None, None) == -1
    # the timer stamp wants an 8-byte aligned slot; the merge setting can be read back
    assert lib.chitu_b200_stamp(None, None) == -1
    assert lib.chitu_b200_stamp(p + 4, None) == -1
    old = lib.chitu_b200_set_cluster_merge(-1)
    assert old in (0, 1) and lib.chitu_b200_set_cluster_merge(old) == old
    # split workspace: header of counters plus whole 128-row tiles of fp32 rows and log-sum-exps
    assert lib.chitu_b200_attn_splitkv_workspace_bytes(1, 300, 3, 128, 1) == 0
    assert lib.chitu_b200_attn_splitkv_workspace_bytes(1, 300, 3, 128, 2) == 65536 + 2 * (3 * 2 * 256) * 129 * 4


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
