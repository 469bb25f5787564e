"""The C-ABI library loads on a machine without a GPU and exports every symbol include/qmk_b200.h declares
(no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "qmk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qmk_[a-z_0-9]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from qimeng_megakernel_b200 import _build, _lib
    _build.build()
    return _lib.load()


def test_header_and_binding_agree(lib):
    from qimeng_megakernel_b200 import _lib
    declared = declared_symbols()
    bound = sorted(name for name, _, _ in _lib.SYMBOLS)
    assert declared == bound, f"header declares {set(declared) ^ set(bound)} differently from the ctypes table"


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/qmk_b200.h but not exported"


def test_abi_version_and_strerror(lib):
    from qimeng_megakernel_b200 import _lib
    assert lib.qmk_abi_version() == _lib.ABI_VERSION
    assert lib.qmk_strerror(0) == b"ok"
    assert b"bounded device-side wait" in lib.qmk_strerror(_lib.ERR_DEVICE_TIMEOUT)
    assert lib.qmk_strerror(-12345) == b"unknown error"


def test_null_arguments_are_rejected_without_a_gpu(lib):
    h = ctypes.c_void_p()
    assert lib.qmk_create(None, None, 0, ctypes.byref(h)) == -1
    assert lib.qmk_decode_step(None, 0, None) == -1
    assert lib.qmk_step_bytes(None, 0) == 0
    lib.qmk_destroy(None)        # must be a no-op


def test_missing_library_raises_import_error(tmp_path):
    from qimeng_megakernel_b200 import mk_kernel
    with pytest.raises(ImportError):
        mk_kernel.get_mk(tmp_path)


def test_unsupported_descriptor_is_rejected(lib):
    """Validation that happens before any CUDA call: a descriptor that matches no compiled shape."""
    from qimeng_megakernel_b200 import _lib
    desc = _lib.ModelDesc(_lib.ABI_VERSION, _lib.ARCH_LLAMA, 2, 1000, 8192, 32, 8, 64, 4096, 128, 1e-5, 0.125, 0.0, 0, 0, 0)
    w = _lib.WeightPtrs(**{n: 256 for n, _ in _lib.WeightPtrs._fields_})
    h = ctypes.c_void_p()
    # neither kernel takes a hidden size that is not a multiple of 64, a head_dim of 32, or 3 query heads per kv head
    assert lib.qmk_create(ctypes.byref(desc), ctypes.byref(w), 0, ctypes.byref(h)) == -2
    desc.hidden_size = 2048
    desc.head_dim = 32
    assert lib.qmk_create(ctypes.byref(desc), ctypes.byref(w), 0, ctypes.byref(h)) == -2
    desc.head_dim = 64
    desc.num_attention_heads = 24
    assert lib.qmk_create(ctypes.byref(desc), ctypes.byref(w), 0, ctypes.byref(h)) == -2
    desc.num_attention_heads = 32
    desc.arch = 7
    assert lib.qmk_create(ctypes.byref(desc), ctypes.byref(w), 0, ctypes.byref(h)) == -2
    desc.arch = _lib.ARCH_LLAMA
    desc.abi_version = 99
    assert lib.qmk_create(ctypes.byref(desc), ctypes.byref(w), 0, ctypes.byref(h)) == -1
    desc.abi_version = _lib.ABI_VERSION
    w.qkv = 257                                     # misaligned
    assert lib.qmk_create(ctypes.byref(desc), ctypes.byref(w), 0, ctypes.byref(h)) == -1
