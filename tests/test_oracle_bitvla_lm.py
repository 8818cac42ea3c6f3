"""CPU checks of the oracle's BitVLA language-model block (the composite restatement of
src/kernels/bitvla/bitvla_lm_cuda.cu:395-525 used as the checker of the GPU stack test)."""
import numpy as np

from tests.test_bitvla_lm_gpu import SMALL, make_layer


def _case(oracle, seq=48, n_layers=2):
    rng = np.random.default_rng(5)
    layers = [make_layer(oracle, rng, SMALL) for _ in range(n_layers)]
    out_norm = oracle.bf16_round(rng.uniform(0.8, 1.2, SMALL["hidden"]).astype(np.float32))
    x = oracle.bf16_round(rng.standard_normal((seq, SMALL["hidden"])).astype(np.float32))
    return x, layers, out_norm


def test_stack_is_finite_bf16_and_deterministic(oracle):
    x, layers, out_norm = _case(oracle)
    a = oracle.bitvla_lm_forward(x, layers, out_norm, SMALL)
    b = oracle.bitvla_lm_forward(x, layers, out_norm, SMALL)
    assert a.shape == x.shape and np.isfinite(a).all()
    assert np.array_equal(a, b)
    assert np.array_equal(a, oracle.bf16_round(a))  # every output is a bf16 value


def test_sequences_do_not_interact_and_rows_do(oracle):
    """Bidirectional attention: changing the LAST token changes the FIRST token's output; a second
    sequence is an independent call."""
    x, layers, out_norm = _case(oracle, seq=16, n_layers=1)
    a = oracle.bitvla_lm_forward(x, layers, out_norm, SMALL)
    x2 = x.copy()
    x2[-1] = -x2[-1]
    b = oracle.bitvla_lm_forward(x2, layers, out_norm, SMALL)
    assert not np.array_equal(a[0], b[0])


def test_rounding_sensitivity_sets_the_gpu_bar(oracle, monkeypatch):
    """Rounding the attention probabilities to bf16 before instead of after the division by the row
    sum is mathematically the same softmax; the stack output moves by percents because four int8
    re-quantisations and the squared gate amplify it.  The GPU stack test allows 5e-2 for that reason."""
    x, layers, out_norm = _case(oracle, seq=96)
    ref = oracle.bitvla_lm_forward(x, layers, out_norm, SMALL)
    real_round = oracle.bf16_round
    calls = {"n": 0}

    def jitter(v):  # perturb every rounded tensor's input by far less than a bf16 ulp
        calls["n"] += 1
        return real_round(np.asarray(v, np.float32) * np.float32(1.0 + 2.0 ** -12))

    monkeypatch.setattr(oracle, "bf16_round", jitter)
    moved = oracle.bitvla_lm_forward(x, layers, out_norm, SMALL)
    assert calls["n"] > 0
    err = float(np.linalg.norm(moved - ref) / np.linalg.norm(ref))
    assert 1e-4 < err < 5e-2, err
