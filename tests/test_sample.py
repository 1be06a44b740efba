"""The CPU sampler (crates/ksearch_gemma/src/sample.rs:9-81) against the reference's own known-answer tests
(sample.rs:91-117) and a NumPy restatement of its arithmetic.  Host code: runs without a GPU."""
import numpy as np
import pytest

from ksearch_b200.sample import sample_softcap_min_p


def _pack(oracle, v):
    """f32 -> f16 bits with the reference's own converter (ksearch_gguf::f32_to_f16, as its tests pack logits)."""
    return oracle.f32_to_f16_ref(np.asarray(v, np.float32))


def test_reference_known_answers(oracle):
    # greedy_picks_argmax_after_softcap
    assert sample_softcap_min_p(_pack(oracle, [1.0, 9.0, 3.0]), 30.0, 0.0, 0.05, 1) == 1
    # min_p_keeps_only_the_peak_when_peaked
    peaked = _pack(oracle, [0.0, 20.0, 0.0])
    assert {sample_softcap_min_p(peaked, 30.0, 1.0, 0.05, s) for s in range(1, 64)} == {1}
    # temperature_samples_near_ties_after_softcap
    ties = _pack(oracle, [8.0, 8.05, 0.0])
    counts = np.bincount([sample_softcap_min_p(ties, 30.0, 1.0, 0.05, s) for s in range(1, 256)], minlength=3)
    assert counts[0] > 0 and counts[1] > 0 and counts[2] == 0


def _np_sample(x, cap, temperature, min_p, seed):
    x = np.asarray(x, np.float32)
    y = (np.float32(cap) * np.tanh(x / np.float32(cap))).astype(np.float32) if cap > 0 else x
    best = int(np.argmax(y))                      # first of equal values
    if temperature < 1e-6:
        return best
    p = np.exp(((y - y[best]) / np.float32(temperature)).astype(np.float32)).astype(np.float32)
    p = p * np.float32(1.0 / max(float(p.sum(dtype=np.float32)), 1e-30))
    p[p < p.max() * max(min_p, 0.0)] = 0
    filtered = float(p.sum(dtype=np.float32))
    if filtered <= 1e-9:
        return best
    state = ((seed | 1) + 0x9E3779B9) & 0xFFFFFFFF
    z = state
    z = ((z ^ (z >> 16)) * 0x7feb352d) & 0xFFFFFFFF
    z = ((z ^ (z >> 15)) * 0x846ca68b) & 0xFFFFFFFF
    z ^= z >> 16
    r = np.float32(np.float32(z) / np.float32(4294967296.0)) * np.float32(filtered)
    cdf = np.cumsum(p, dtype=np.float32)
    hit = np.flatnonzero(r < cdf)
    return int(hit[0]) if hit.size else len(x) - 1


@pytest.mark.parametrize("temperature,min_p,cap", [(0.0, 0.05, 30.0), (0.7, 0.05, 30.0), (1.0, 0.0, 30.0), (1.3, 0.2, 0.0)])
def test_against_numpy_restatement(temperature, min_p, cap):
    rng = np.random.default_rng(5)
    agree = total = 0
    for trial in range(40):
        x = (rng.standard_normal(257) * 4).astype(np.float32)
        for seed in (1, 2, 77, 4096, 0xFFFFFFFF):
            got = sample_softcap_min_p(x, cap, temperature, min_p, seed)
            want = _np_sample(x, cap, temperature, min_p, seed)
            total += 1
            agree += got == want
            assert 0 <= got < 257
    # libm and NumPy may round exp / tanh differently in the last place: a draw that lands on a cdf edge can differ
    assert agree >= total - 2
    assert sample_softcap_min_p(x, cap, temperature, min_p, 9) == sample_softcap_min_p(x, cap, temperature, min_p, 9)


def test_f16_and_f32_inputs_agree_and_ties_go_to_the_first(oracle):
    x = np.array([3.0, 7.5, 7.5, -2.0], np.float32)           # exact in f16
    assert sample_softcap_min_p(x, 30.0, 0.0, 0.05, 1) == 1     # the first of the equal maxima
    bits = _pack(oracle, x)
    for seed in range(1, 40):
        assert sample_softcap_min_p(bits, 30.0, 0.9, 0.05, seed) == sample_softcap_min_p(x, 30.0, 0.9, 0.05, seed)
    assert sample_softcap_min_p(np.array([0.5], np.float32), 30.0, 1.0, 0.05, 3) == 0
