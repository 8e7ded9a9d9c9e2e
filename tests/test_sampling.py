"""The host sampler against the plain sampler written from the reference (tests/plain_qwen2.py)."""
import numpy as np

import plain_qwen2 as plain


def test_host_sampler_equals_plain_sampler():
    from hfcpu_b200.sampling import Rng, SamplingParams, sample_host
    rs = np.random.RandomState(0)
    for trial in range(200):
        V = int(rs.choice([17, 512, 1000]))
        l = (rs.randn(V) * rs.choice([0.5, 2, 5])).astype(np.float32)
        if trial % 5 == 0:
            l[rs.randint(V, size=6)] = l[0]
        p = SamplingParams(temp=float(rs.choice([0, 0.7, 1.0, 2.0])), top_k=int(rs.choice([0, 1, 5, 40, 2000])),
                           top_p=float(rs.choice([1.0, 0.95, 0.5])), min_p=float(rs.choice([0, 0.05, 0.3])))
        r1, r2 = Rng(trial), plain.Rng(trial)
        for _ in range(3):
            assert sample_host(l, p, r1) == plain.sample(l, p.temp, p.top_k, p.top_p, p.min_p, r2)


def test_rng_sequence():
    """xorshift64* with the reference's seeding (src/sample.c:9-23): values in [0, 1), seeds differ, seed 0 works.
    (The draws themselves are pinned on the reference's own in tests/test_golden.py.)"""
    from hfcpu_b200.sampling import Rng
    a, b = Rng(0), Rng(1)
    xs, ys = [float(a.uniform()) for _ in range(1000)], [float(b.uniform()) for _ in range(1000)]
    assert all(0 <= x < 1 for x in xs) and xs != ys and 0.4 < sum(xs) / 1000 < 0.6
    assert Rng(0).state == 0x1234567


def test_logprobs():
    from hfcpu_b200.sampling import logprob, top_logprobs
    l = np.array([1.0, 3.0, 2.0, 3.0], dtype=np.float32)
    ref = l - np.log(np.exp(l.astype(np.float64)).sum())
    assert abs(logprob(l, 2) - ref[2]) < 1e-6
    top = top_logprobs(l, 3)
    assert [i for i, _ in top] == [1, 3, 2] and abs(top[0][1] - ref[1]) < 1e-6
