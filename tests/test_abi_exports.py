"""CPU-side checks of the drop-in boundary: the library builds, loads and exports every
symbol the public header declares; argument validation answers without touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cuda_lib():
    from vla_cpp_b200 import build

    build.build()
    from vla_cpp_b200 import api

    return api.lib()


def declared_symbols():
    names = []
    for hdr in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        names += re.findall(r"VLAB200_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)
    return names


def declared_model_api_symbols():
    """The seven functions of include/vla.h (ABI v1)."""
    text = open(os.path.join(ROOT, "include", "vla.h")).read()
    return re.findall(r"VLA_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)


def test_header_and_binding_list_agree(cuda_lib):
    from vla_cpp_b200 import api

    assert sorted(declared_symbols()) == sorted(api.EXPORTS)


def test_every_declared_symbol_is_exported(cuda_lib):
    for name in declared_symbols():
        assert hasattr(cuda_lib, name), name


def test_model_level_abi_is_exported(cuda_lib):
    names = declared_model_api_symbols()
    assert sorted(names) == sorted(["vla_abi_version", "vla_model_load", "vla_model_free", "vla_model_config",
                                    "vla_predict", "vla_free_actions", "vla_last_stats"])
    for name in names:
        assert hasattr(cuda_lib, name), name
    assert cuda_lib.vla_abi_version() == 1


def test_abi_version(cuda_lib):
    assert cuda_lib.vlab200_abi_version() == 1


def test_argument_checks_need_no_gpu(cuda_lib):
    null = C.c_void_p(0)
    one = C.c_void_p(16)
    assert cuda_lib.vlab200_act_quant(null, null, null, 4, 128, null) == -1
    assert cuda_lib.vlab200_act_quant(one, one, one, 4, 100, null) == -4  # K % 8
    assert cuda_lib.vlab200_ternary_linear(null, null, null, null, null, null, 1, 1, 16, 128, 0, null) == -1
    # N % 16 and K % 128 are hard requirements of the ladder pack
    assert cuda_lib.vlab200_ternary_linear(one, one, one, null, one, one, 1, 1, 24, 128, 0, null) == -4
    assert cuda_lib.vlab200_ternary_linear(one, one, one, null, one, one, 1, 1, 16, 100, 0, null) == -4
    assert cuda_lib.vlab200_ternary_linear(one, one, one, null, one, one, 1, 0, 16, 128, 0, null) == 0  # M = 0
