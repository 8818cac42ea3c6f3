"""include/vla.h (ABI v1): the header is plain C, its struct layout equals the reference header's, and the
NULL-handle / status-code contract holds with no model and with a metadata-only checkpoint.  Host only.

The golden layout (tests/golden/vla_h_layout.txt) is the output of tests/c/vla_h_layout.c compiled against the
REFERENCE's include/vla.h by tests/golden/make_golden.py; here the same program is compiled against this
repository's header and the two outputs must be identical."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")
LIBDIR = os.path.join(ROOT, "vla_cpp_b200")


def _cc(tmp_path, src, out, link=False):
    cmd = ["gcc", "-std=c99", "-Wall", "-Werror", "-I", INC, os.path.join(ROOT, "tests", "c", src), "-o", str(tmp_path / out)]
    if link:
        cmd += ["-L", LIBDIR, "-lvla_b200", "-Wl,-rpath," + LIBDIR]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return str(tmp_path / out)


def test_struct_layout_equals_the_reference_header(tmp_path):
    exe = _cc(tmp_path, "vla_h_layout.c", "layout")
    got = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    want = open(os.path.join(ROOT, "tests", "golden", "vla_h_layout.txt")).read()
    assert got == want


def test_null_handles_and_status_codes_without_a_model(tmp_path):
    import vla_cpp_b200

    vla_cpp_b200.lib()
    exe = _cc(tmp_path, "c_api_no_model.c", "capi", link=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and "c api: ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("arch", ["pi0", "smolvla"])
def test_load_resolves_the_config_from_checkpoint_metadata(tmp_path, arch):
    """vla_model_load needs no GPU: it parses the GGUF metadata with the reference's required keys
    (src/models/pi0.cpp:258-293, src/models/smolvla.cpp:590-632) and vla_model_config reports the resolved values."""
    gguf = pytest.importorskip("gguf")
    import numpy as np
    import vla_cpp_b200

    vla_cpp_b200.lib()
    path = tmp_path / "m.gguf"
    w = gguf.GGUFWriter(str(path), arch)
    p = arch + "."
    vals = dict(hidden=2048, intermediate=16384, n_q_heads=8, n_kv_heads=1, head_dim=256, n_layers=18, expert_h=1024,
                expert_inter=4096, chunk_size=50, num_steps=10, max_state_dim=32, max_action_dim=32, real_state_dim=8,
                real_action_dim=7, tokenizer_max_length=48)
    for k, v in vals.items():
        w.add_uint32(p + k, v)
    w.add_float64(p + "min_period", 4e-3)
    w.add_float64(p + "max_period", 4.0)
    if arch == "smolvla":
        w.add_uint32("smolvla.self_attn_every_n_layers", 2)
        w.add_uint32("smolvla.n_img_tokens", 64)
        w.add_uint32("smolvla.vocab_size", 49280)
    w.add_tensor("dummy", np.zeros(4, np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    exe = _cc(tmp_path, "c_api_no_model.c", "capi", link=True)
    r = subprocess.run([exe, str(path)], capture_output=True, text=True)
    assert r.returncode == 0 and "c api: ok" in r.stdout, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("config ")][0]
    assert "hidden=2048 expert_h=1024 n_layers=18 n_suffix=50 n_lang=48" in line
    assert "q_full=2048 kv_full=256 steps=10" in line and "min=0.004 max=4 denorm=1" in line
    if arch == "pi0":
        assert "n_img=256" in line and "every=0" in line and "rms_eps=1e-06" in line
    else:
        assert "n_img=64" in line and "every=2" in line and "rms_eps=1e-05" in line

    # the C++ face (include/vla_model.hpp, the shape of the reference's src/model.h) on the same file
    cpp = str(tmp_path / "cppapi")
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", INC, os.path.join(ROOT, "tests", "c", "cpp_api.cpp"), "-o", cpp,
                    "-L", LIBDIR, "-lvla_b200", "-Wl,-rpath," + LIBDIR], check=True, capture_output=True, text=True)
    r = subprocess.run([cpp, str(path)], capture_output=True, text=True)
    assert r.returncode == 0 and "cpp api: ok" in r.stdout and "expert_h=1024 n_suffix=50 steps=10" in r.stdout, r.stdout + r.stderr

    # a checkpoint that lacks a required key does not load
    bad = tmp_path / "bad.gguf"
    w = gguf.GGUFWriter(str(bad), arch)
    w.add_uint32(p + "hidden", 2048)
    w.add_tensor("dummy", np.zeros(4, np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    import ctypes as C

    L = vla_cpp_b200.lib()
    L.vla_model_load.restype = C.c_void_p
    L.vla_model_load.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
    assert L.vla_model_load(None, str(bad).encode(), None) is None
    assert b"missing" in L.vlab200_last_error()
