"""The shared library loads without a GPU and exports every symbol include/straydog_gpu_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "straydog_gpu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sdx?_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from straydog_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), name


def test_binding_covers_the_header():
    from straydog_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    _lib.load()


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        return
    from straydog_b200.backend import Backend, StraydogError
    try:
        Backend(0, 1 << 30)
    except StraydogError as error:
        assert str(error)
    else:
        raise AssertionError("sd_create succeeded without a GPU")
