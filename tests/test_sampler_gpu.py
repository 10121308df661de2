"""The device sampler (sample_topk_kernel through quintrit_b200_sample_logits) against the numpy restatement of the reference's sampler
(quintrit-runtime/src/sampler.rs:59-143): same token and same generator state, draw after draw, on vocabulary-sized logits with ties at the
cut, infinities and both signs of zero."""
import numpy as np
import pytest

import quintrit_b200 as q
from oracle import sampler

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,top_k,top_p,temperature", [(131072, 40, 0.9, 0.8), (131072, 1024, 1.0, 1.3), (128256, 2, 0.5, 0.7), (5000, 7, 0.95, 2.0), (1025, 1024, 0.99, 1.0), (300, 40, 0.9, 0.8)])
def test_draws_equal_the_reference_sampler(n, top_k, top_p, temperature):
    rng = np.random.default_rng(n + top_k)
    ref = sampler.Sampler(temperature, top_k, top_p, seed=1234)
    state = ref.state
    for draw in range(6):
        logits = (rng.standard_normal(n) * 4.0).astype(np.float32)
        if draw == 1:  # coarse values: many exact ties, also across the k-th largest (the lower ids win)
            logits = np.round(logits * 2.0) / 2.0
        if draw == 2:
            logits[rng.integers(0, n, 20)] = -np.inf
            logits[rng.integers(0, n, 3)] = -0.0
        if draw == 3:  # a peaked distribution: the nucleus is one or two candidates
            logits[int(rng.integers(0, n))] = 60.0
        if draw == 4:  # all equal: the first top_k ids are the candidates
            logits[:] = 1.5
        want = ref.sample(logits)
        got, state = q.sample_logits(logits, temperature, top_k, top_p, state)
        assert got == want and state == ref.state, (draw, got, want)


def test_arguments():
    lg = np.zeros(100, np.float32)
    for args in [(0.0, 10, 0.9, 1), (1.0, 0, 0.9, 1), (1.0, 100, 0.9, 1), (1.0, 2000, 0.9, 1), (1.0, 10, 0.0, 1), (1.0, 10, 1.5, 1), (1.0, 10, 0.9, 0)]:
        with pytest.raises(q.QuintritError) as e:
            q.sample_logits(lg, *args)
        assert e.value.code == 2
