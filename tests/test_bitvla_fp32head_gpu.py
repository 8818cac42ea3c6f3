"""BitVLA's float32 proprioception projector and action head (bitvla_fp32head_* of this library) against the reference's
own CUDA implementation (oracle/_ref/libbitvla_fp32head_ref.so: src/kernels/bitvla/bitvla_fp32head_cuda.cu compiled
unmodified, cuBLAS SGEMM) and against a float64 numpy restatement.

Bar: rel-L2 <= 1e-5 against both -- float32 arithmetic on either side, only the order of the sums differs."""
import ctypes as C
import os

import numpy as np
import pytest

from tests.gpu_util import ROOT, rel_l2, require_cuda

pytestmark = pytest.mark.gpu

NAMES = ["pp_fc1_w", "pp_fc1_b", "pp_fc2_w", "pp_fc2_b", "ah_ln1_w", "ah_ln1_b", "ah_fc1_w", "ah_fc1_b", "ah_b0_lnw", "ah_b0_lnb",
         "ah_b0_w", "ah_b0_b", "ah_b1_lnw", "ah_b1_lnb", "ah_b1_w", "ah_b1_b", "ah_ln2_w", "ah_ln2_b", "ah_fc2_w", "ah_fc2_b"]


def bind(lib):
    fp = C.POINTER(C.c_float)
    lib.bitvla_fp32head_cuda_init.restype = C.c_void_p
    lib.bitvla_fp32head_cuda_init.argtypes = [C.c_int] * 4 + [C.c_float] + [fp] * 20
    lib.bitvla_fp32head_proprio_forward.restype = C.c_int
    lib.bitvla_fp32head_proprio_forward.argtypes = [C.c_void_p, fp, fp, C.c_void_p]
    lib.bitvla_fp32head_action_forward.restype = C.c_int
    lib.bitvla_fp32head_action_forward.argtypes = [C.c_void_p, fp, fp, C.c_void_p]
    lib.bitvla_fp32head_cuda_free.restype = None
    lib.bitvla_fp32head_cuda_free.argtypes = [C.c_void_p]
    return lib


def reference_head_lib():
    p = os.path.join(ROOT, "oracle", "_ref", "libbitvla_fp32head_ref.so")
    return bind(C.CDLL(p)) if os.path.exists(p) else None


def make_head(rng, proprio_dim, hidden, action_dim):
    D = action_dim * hidden
    shapes = dict(pp_fc1_w=(hidden, proprio_dim), pp_fc1_b=(hidden,), pp_fc2_w=(hidden, hidden), pp_fc2_b=(hidden,),
                  ah_ln1_w=(D,), ah_ln1_b=(D,), ah_fc1_w=(hidden, D), ah_fc1_b=(hidden,), ah_b0_lnw=(hidden,), ah_b0_lnb=(hidden,),
                  ah_b0_w=(hidden, hidden), ah_b0_b=(hidden,), ah_b1_lnw=(hidden,), ah_b1_lnb=(hidden,), ah_b1_w=(hidden, hidden),
                  ah_b1_b=(hidden,), ah_ln2_w=(hidden,), ah_ln2_b=(hidden,), ah_fc2_w=(action_dim, hidden), ah_fc2_b=(action_dim,))
    w = {}
    for k, shp in shapes.items():
        if k.endswith(("lnw", "ln1_w", "ln2_w")):
            w[k] = rng.uniform(0.8, 1.2, shp).astype(np.float32)
        elif len(shp) == 2:
            w[k] = (rng.standard_normal(shp) * shp[1] ** -0.5).astype(np.float32)
        else:
            w[k] = (rng.standard_normal(shp) * 0.1).astype(np.float32)
    return w


def drive(lib, w, cfg, state, ah_in):
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    ctx = lib.bitvla_fp32head_cuda_init(cfg["proprio_dim"], cfg["hidden"], cfg["chunk"], cfg["action_dim"], cfg["ah_ln_eps"],
                                        *[fp(w[n]) for n in NAMES])
    assert ctx, "bitvla_fp32head_cuda_init returned NULL"
    try:
        pp = np.zeros(cfg["hidden"], np.float32)
        act = np.zeros((cfg["chunk"], cfg["action_dim"]), np.float32)
        assert lib.bitvla_fp32head_proprio_forward(ctx, fp(state), fp(pp), None) == 0
        assert lib.bitvla_fp32head_action_forward(ctx, fp(ah_in), fp(act), None) == 0
        return pp, act
    finally:
        lib.bitvla_fp32head_cuda_free(ctx)


# BitVLA's own sizes (proprio 8, hidden 2560, chunk 8, 7 action dims: fc1 is 2560 x 17920) and odd small ones
# (K not a multiple of 4, fewer columns than a CTA serves, more rows than one pass)
@pytest.mark.parametrize("cfg", [dict(proprio_dim=8, hidden=2560, chunk=8, action_dim=7, ah_ln_eps=1e-5),
                                 dict(proprio_dim=5, hidden=70, chunk=3, action_dim=3, ah_ln_eps=1e-5),
                                 dict(proprio_dim=9, hidden=129, chunk=11, action_dim=2, ah_ln_eps=1e-6)])
def test_head_against_reference_cuda_and_float64(oracle, cfg):
    require_cuda()
    from vla_cpp_b200 import api

    rng = np.random.default_rng(cfg["hidden"])
    w = make_head(rng, cfg["proprio_dim"], cfg["hidden"], cfg["action_dim"])
    state = rng.standard_normal(cfg["proprio_dim"]).astype(np.float32)
    ah_in = rng.standard_normal((cfg["chunk"], cfg["action_dim"] * cfg["hidden"])).astype(np.float32)
    pp, act = drive(bind(api.lib()), w, cfg, state, ah_in)
    assert api.device_status() == 0
    want = oracle.bitvla_fp32head(w, cfg, state=state, ah_in=ah_in)
    e_pp, e_act = rel_l2(pp, want["proprio"]), rel_l2(act, want["action"])
    msg = f"fp32 head hidden={cfg['hidden']}: vs float64 proprio {e_pp:.2e}, action {e_act:.2e}"
    assert e_pp <= 1e-5 and e_act <= 1e-5, msg
    ref = reference_head_lib()
    if ref is not None:
        rpp, ract = drive(ref, w, cfg, state, ah_in)
        r_pp, r_act = rel_l2(pp, rpp), rel_l2(act, ract)
        msg += f"; vs reference CUDA proprio {r_pp:.2e}, action {r_act:.2e}; reference vs float64 {rel_l2(ract, want['action']):.2e}"
        assert r_pp <= 1e-5 and r_act <= 1e-5, msg
    print(msg)


def test_head_rejects_bad_arguments():
    require_cuda()
    from vla_cpp_b200 import api

    L = bind(api.lib())
    assert not L.bitvla_fp32head_cuda_init(0, 16, 2, 2, 1e-5, *([None] * 20))
    assert not L.bitvla_fp32head_cuda_init(4, 16, 2, 2, 1e-5, *([None] * 20))  # null weights
    assert L.bitvla_fp32head_proprio_forward(None, None, None, None) == -1
