"""CPU-only checks of the C-ABI boundary: the library builds, loads, exports every symbol that
include/tangq.h declares, and refuses to run without a GPU instead of falling back."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    hdr = open(os.path.join(ROOT, "include", "tangq.h")).read()
    return re.findall(r"TQ_API [\w\* ]+?(tq_\w+)\(", hdr)


@pytest.fixture(scope="module")
def lib():
    from tang_b200 import _build, load

    _build.build_library()
    return load()


def test_header_symbols_exported(lib):
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in tangq.h but not exported by libtangq.so"


def test_prototypes_cover_header(lib):
    from tang_b200._lib import PROTOTYPES

    assert set(PROTOTYPES) == set(_declared())


def test_no_oracle_in_product():
    """The product package must not reach into oracle/ (the oracle is only a checker)."""
    pkg = os.path.join(ROOT, "tang_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f


def test_no_gpu_fails_loudly(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import tang_b200

    with pytest.raises(tang_b200.TangqError):
        tang_b200.QuantComputeDevice(0)
    ctx = ctypes.c_void_p()
    assert lib.tq_ctx_create(0, None, ctypes.byref(ctx)) != 0 and not ctx.value
    assert lib.tq_last_error(None) is not None
