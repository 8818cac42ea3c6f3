"""The whole Euler loop of one observation as one persistent kernel (csrc/chunk_loop.cu) against the launch-per-operator
path of the same engine and against the oracle (src/models/pi0.cpp:570-588, src/models/smolvla.cpp:1393-1418)."""
import os

import numpy as np
import pytest

from tests.gpu_util import require_cuda

pytestmark = pytest.mark.gpu


def _engine(torch, vb, policy, seed=3):
    import bench

    return bench.build_pi0_engine(torch, vb, torch.device("cuda", 0), 1, seed, policy)


def _with_loop(flag, fn):
    old = os.environ.get("VLAB200_CHUNK_LOOP")
    os.environ["VLAB200_CHUNK_LOOP"] = flag
    try:
        return fn()
    finally:
        if old is None:
            del os.environ["VLAB200_CHUNK_LOOP"]
        else:
            os.environ["VLAB200_CHUNK_LOOP"] = old


@pytest.mark.parametrize("policy", ["pi0", "smolvla", "pi05"])
def test_loop_kernel_matches_operator_path(policy):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    eng, x0, state = _engine(torch, vb, policy)
    ref = _with_loop("0", lambda: eng.denoise(x0, state))
    out = _with_loop("1", lambda: eng.denoise(x0, state))
    again = _with_loop("1", lambda: eng.denoise(x0, state))
    torch.cuda.synchronize()
    assert vb.device_status() == 0
    assert torch.isfinite(out).all()
    rel = ((out - ref).norm() / ref.norm()).item()
    assert rel <= 1e-2, rel  # both paths round activations to bf16 at different points
    assert torch.equal(out, again)  # every sum has a fixed order


def test_loop_kernel_hidden_key_range_and_prefix_length():
    """SmolVLA-shaped: a pad range hides prefix keys; then the prefix in use shrinks (the phase table is rebuilt)."""
    torch = require_cuda()
    import vla_cpp_b200 as vb

    eng, x0, state = _engine(torch, vb, "smolvla", seed=7)
    pad = torch.tensor([[140, 170]], dtype=torch.int32, device="cuda")
    ref = _with_loop("0", lambda: eng.denoise(x0, state, pad_ranges=pad))
    out = _with_loop("1", lambda: eng.denoise(x0, state, pad_ranges=pad))
    plain = _with_loop("1", lambda: eng.denoise(x0, state))
    torch.cuda.synchronize()
    assert ((out - ref).norm() / ref.norm()).item() <= 1e-2
    assert ((out - plain).norm() / plain.norm()).item() > 1e-4  # the hidden keys matter
    eng.set_prefix_len(eng.prefix_len - 33)
    ref2 = _with_loop("0", lambda: eng.denoise(x0, state))
    out2 = _with_loop("1", lambda: eng.denoise(x0, state))
    torch.cuda.synchronize()
    assert vb.device_status() == 0
    assert ((out2 - ref2).norm() / ref2.norm()).item() <= 1e-2
    assert ((out2 - plain).norm() / plain.norm()).item() > 1e-4


@pytest.mark.parametrize("policy", ["pi0", "smolvla"])
def test_loop_kernel_full_depth_against_oracle(oracle, policy):
    """The benchmark configurations at full depth (18 x 10 and 16 x 10 layer-steps), one observation, forced through the
    loop kernel: final action chunk rel-L2 <= 1e-2 against the float32 oracle, as for the operator path."""
    from tests.test_engine_gpu import PI0_FULL, SMOLVLA_FULL, run_case

    if policy == "pi0":
        w, d = _with_loop("1", lambda: run_case(oracle, 71, n_obs=1, P=816, check_obs=[0], sigma=0.02, **PI0_FULL))
    else:
        w, d = _with_loop("1", lambda: run_case(oracle, 72, n_obs=1, P=177, pos_base=170, pad=(160, 176), check_obs=[0], sigma=0.02,
                                               **SMOLVLA_FULL))
    print(f"loop kernel {policy} full depth: rel_l2={w:.3e} displacement rel_l2={d:.3e}")
    assert w < 1e-2 and d < 3e-2, (w, d)


def test_loop_kernel_other_shapes_against_oracle(oracle):
    """head_dim 128 (its own kernel instantiation), and a small SmolVLA-shaped expert with cross-attention layers, a hidden key
    range and rebased suffix positions; one observation each, so both take the loop kernel."""
    from tests.test_engine_gpu import run_case

    w, d = _with_loop("1", lambda: run_case(oracle, 73, n_obs=1, P=40, model=0, L=2, H=128, n_q=2, n_kv=1, hd=128, inter=256,
                                           chunk=10, A=32, sd=32, T=2))
    assert w < 1e-2 and d < 3e-2, (w, d)
    w, d = _with_loop("1", lambda: run_case(oracle, 74, n_obs=1, P=30, pos_base=27, pad=(20, 29), model=1, L=4, H=192, n_q=6, n_kv=2,
                                           hd=64, inter=384, chunk=10, A=32, sd=32, T=2, self_every=2))
    assert w < 1e-2 and d < 3e-2, (w, d)
