"""The C-ABI library loads without a GPU and exports every symbol the header
declares; entry points that need no device behave.  No compute calls here."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from tensorpencil_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_functions():
    src = open(os.path.join(ROOT, "include", "tpb200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tpb_[a-z0-9_]+)\s*\(", src)))


def test_header_and_binding_agree(lib):
    from tensorpencil_b200 import _lib
    names = declared_functions()
    assert len(names) >= 20
    assert sorted(_lib.SIGNATURES) == names
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in tpb200.h but not exported"


def test_version_and_strings(lib):
    assert lib.tpb_version() >= 100
    assert lib.tpb_status_string(0) == b"ok"
    assert b"timed out" in lib.tpb_status_string(-4)
    assert lib.tpb_convrot_w4_expanded_bytes(12288, 3072) == 12288 * 3072


def test_create_without_device_reports_no_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.tpb_create(C.byref(h), 0)
    assert rc == -6 and not h.value  # TPB_ERR_NO_DEVICE; no fallback object is handed out


def test_null_handle_is_rejected(lib):
    assert lib.tpb_destroy(None) == -1
    assert lib.tpb_convrot_prep(None, None, None, 0, 1, 256, 8, None, None, None) == -1
    assert lib.tpb_stream_prefetch(None, 0) == -1


def test_backend_refuses_to_run_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from tensorpencil_b200.backend import Backend
    with pytest.raises(RuntimeError, match="no CPU path"):
        Backend(0)


def test_product_never_imports_the_oracle():
    """The oracle is test infrastructure: nothing in the package may import it."""
    pkg = os.path.join(ROOT, "tensorpencil_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cuh", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), (dirpath, f)
