"""The allocation-free entry point (vlab200_denoise_attn_loop_static) against the regular one.

Some callers cannot allocate device memory at all -- a plugin whose host application owns the
allocator and passes in only inputs and outputs, or a control loop in which cudaMalloc (a
device-wide synchronising call) is forbidden.  For them the library carries the query scratch
buffer inside its own image.  The file name keeps this test last in collection order."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _setup(torch, vb, n_obs, seed, H=720, n_q=15, n_kv=5, S=51, P=177):
    hd, L, T = 64, 2, 2
    g = torch.Generator(device="cuda").manual_seed(seed)
    st = vb.KvStore(L, n_obs, n_kv, hd, P, S)
    for l in range(L):
        st.write_prefix(l, torch.randn((n_obs, P, n_kv, hd), device="cuda", generator=g),
                        torch.randn((n_obs, P, n_kv, hd), device="cuda", generator=g))
    w = (torch.randn((L, (n_q + 2 * n_kv) * hd, H), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    ln = 1 + 0.1 * torch.randn((L, H), device="cuda", generator=g)
    op = vb.DenoiseAttn(st, H, n_q, S, ln, w, 1e-5, vb.MASK_CAUSAL)
    xs = [torch.randn((T, L, n_obs * S, H), device="cuda", generator=g).to(torch.bfloat16) for _ in range(2)]
    return op, xs


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vla_cpp_b200 as vb

    op, xs = _setup(torch, vb, n_obs=5, seed=11)
    for x in xs:  # two calls in a row share the built-in array
        ref = op.run(x).clone()
        op.out.zero_()
        got = op.run_static(x).clone()
        assert vb.device_status() == 0
        # same kernels, same inputs: the outputs are identical bit for bit
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
        assert got.float().abs().max().item() > 0
    # the property the entry point exists for: a call takes no device memory, neither from the driver
    # nor from torch's caching allocator (the first call above already looked up the array's address)
    torch.cuda.synchronize()
    free0, alloc0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    op.run_static(xs[0])
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free0 and torch.cuda.memory_allocated() == alloc0


def test_static_scratch_limit_is_exactly_16_mib():
    """128 observations x 16 heads x 64 tokens x 64 x 2 bytes fill the built-in array to the last byte and must
    pass; one observation more must be refused."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vla_cpp_b200 as vb

    shape = dict(H=256, n_q=16, n_kv=4, S=64, P=64)
    op, xs = _setup(torch, vb, n_obs=128, seed=13, **shape)
    ref = op.run(xs[0]).clone()
    op.out.zero_()
    got = op.run_static(xs[0])
    assert vb.device_status() == 0
    assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
    op, xs = _setup(torch, vb, n_obs=129, seed=14, **shape)
    with pytest.raises(vb.VlaB200Error) as e:
        op.run_static(xs[0])
    assert e.value.code == -4


def test_static_scratch_entry_point_rejects_oversized_requests():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vla_cpp_b200 as vb

    # 200 observations need 200 * 15 * 51 * 64 * 2 = 19.6 MB of queries: over the 16 MiB built in
    op, xs = _setup(torch, vb, n_obs=200, seed=12)
    with pytest.raises(vb.VlaB200Error) as e:
        op.run_static(xs[0])
    assert e.value.code == -4 and "16777216" in str(e.value)
    op.run(xs[0])  # the regular entry point takes the same request
    assert vb.device_status() == 0
