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


def test_elementwise_wrappers_refuse_outputs_they_would_overrun():
    """The stand-alone elementwise ops write f32.  A bf16 tensor passed as the in-place operand
    would be overrun on the device, so the mirror refuses it before anything is launched (the
    checks need no device: they run on CPU tensors here, on an object without a handle)."""
    import torch
    from tensorpencil_b200.backend import Backend
    be = Backend.__new__(Backend)              # no device, no library: the checks come first
    a16 = torch.zeros(8, 256, dtype=torch.bfloat16)
    b16 = torch.zeros(8, 256, dtype=torch.bfloat16)
    a32 = torch.zeros(8, 256, dtype=torch.float32)
    mod = torch.zeros(3 * 256)
    for call in (lambda: be.siluMul(a16, b16, 8 * 256), lambda: be.sigmoidMul(a16, b16, 8 * 256),
                 lambda: be.rmsMod(a32, a16, mod, 8, 256, 0, 256, 1e-5),
                 lambda: be.gatedAdd(a16, b16, mod, 8 * 256, 256, 0)):
        with pytest.raises(TypeError, match="float32"):
            call()
    with pytest.raises(ValueError, match="hold"):
        be.siluMul(a32[:4], a32, 8 * 256)          # output shorter than the element count
    with pytest.raises(ValueError, match="contiguous"):
        be.sigmoidMul(a32.t(), a32.t(), 8 * 256)
    with pytest.raises(TypeError, match="same dtype"):
        be.siluMul(a32, b16, 8 * 256)


def test_product_never_imports_the_oracle():
    """The oracle is test infrastructure: nothing in the package may import it."""
    pkg = os.path.join(ROOT, "tensorpencil_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cuh", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), (dirpath, f)


def test_piece_size_of_the_shared_link_streamer_matches_the_python_slot_size(lib):
    """tpb_stream_piece_bytes is plain arithmetic (no device): g equal pieces, rounded up to 256 bytes, cover
    the image; offload.slot_size is g of them."""
    import random
    from tensorpencil_b200.offload import slot_size
    rnd = random.Random(7)
    for _ in range(200):
        nbytes, g = rnd.randrange(1, 200_000_000), rnd.choice([1, 2, 3, 4, 8])
        piece = int(lib.tpb_stream_piece_bytes(nbytes, g))
        assert piece % 256 == 0 and piece * g >= nbytes and (piece - 256) * g < nbytes
        if g > 1:
            assert slot_size(nbytes, g) == piece * g
    assert slot_size(12345, 1) == 12345
    assert int(lib.tpb_stream_piece_bytes(1000, 0)) == 0
