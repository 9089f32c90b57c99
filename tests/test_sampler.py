"""The token sampler of the library (host code, no GPU) against its definition in the reference
(design-tests/nn/gpu/src/diary.rs:686-744): greedy at temperature <= 0, else softmax(logits / temperature) in f32, the
top-k kept with ties in index order, one SplitMix64 draw over their mass."""
import ctypes as C

import numpy as np
import pytest

from ava_b200 import build, engine


@pytest.fixture(scope="module", autouse=True)
def _lib():
    build.build()


def test_splitmix64_reference_vector():
    # design-tests/nn/data/src/rng.rs: `reference_vector_seed_zero`
    r = engine.Rng(0)
    assert [r.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def restated_pick(logits, temperature, top_k, rng):
    """The sampler written out again in numpy, on the library's exp (the only transcendental in it)."""
    L = engine.lib()
    L.ava_host_expf.restype, L.ava_host_expf.argtypes = C.c_float, [C.c_float]
    x = np.asarray(logits, np.float32)
    if temperature <= 0:
        return int(np.argmax(x))
    z = (x * np.float32(1.0 / float(np.float32(temperature))) + np.float32(0)).astype(np.float32)
    mx = z.max()
    e = np.array([L.ava_host_expf(float(v)) for v in (z - mx).astype(np.float32)], np.float32)
    s = np.float32(0)
    for v in e:
        s = np.float32(s + v)
    p = (e / s).astype(np.float32)
    order = sorted(range(len(p)), key=lambda j: (-p[j], j))[:max(1, min(top_k, len(p)))]
    total = float(sum(float(p[j]) for j in order))
    r = (rng.next_u64() >> 11) / float(1 << 53) * total
    out = order[-1]
    for j in order:
        r -= float(p[j])
        if r <= 0:
            out = j
            break
    return out


@pytest.mark.parametrize("temperature,top_k", [(1.0, 40), (0.7, 5), (1.5, 1), (1.0, 10_000), (0.05, 3)])
def test_draws_follow_the_definition(temperature, top_k):
    rng = np.random.default_rng(int(temperature * 100) + top_k)
    a, b = engine.Rng(17), engine.Rng(17)
    for trial in range(25):
        lg = (rng.normal(size=300) * 3).astype(np.float32)
        if trial % 5 == 0:
            lg[10:14] = lg.max() + 1.0          # ties among the most likely: index order decides
        assert engine.pick(lg, temperature, top_k, a) == restated_pick(lg, temperature, top_k, b), trial
    assert a.state.value == b.state.value      # one generator step per draw


def test_greedy_takes_the_lowest_index_and_no_draw():
    lg = np.array([0.5, 2.0, -1.0, 2.0, 2.0], np.float32)
    r = engine.Rng(5)
    assert engine.pick(lg, 0.0, 40, r) == 1 and engine.pick(lg, -1.0, 40, None) == 1
    assert r.state.value == 5
    tok, lp, slp = engine.pick(lg, 0.0, 40, None, traced=True)
    want = 2.0 - np.log(np.exp(lg.astype(np.float64)).sum())
    assert tok == 1 and slp == 0.0 and lp == pytest.approx(want, abs=1e-6)


def test_traced_log_probabilities():
    rng = np.random.default_rng(1)
    lg = (rng.normal(size=500) * 2).astype(np.float32)
    tok, lp, slp = engine.pick(lg, 0.8, 7, engine.Rng(3), traced=True)
    x = lg.astype(np.float64)
    assert lp == pytest.approx(x[tok] - np.log(np.exp(x - x.max()).sum()) - x.max(), abs=1e-5)
    p = np.exp(x / 0.8 - (x / 0.8).max())
    p /= p.sum()
    top = np.sort(p)[::-1][:7]
    assert p[tok] >= top[-1] * (1 - 1e-6)
    assert slp == pytest.approx(np.log(p[tok] / top.sum()), abs=1e-4)
    # the draws spread as the kept mass says (a coarse check over many draws of one distribution)
    r = engine.Rng(99)
    counts = np.zeros(500)
    for _ in range(4000):
        counts[engine.pick(lg, 0.8, 7, r)] += 1
    kept = np.argsort(-p)[:7]
    assert counts.sum() == counts[kept].sum()
    assert np.abs(counts[kept] / 4000 - p[kept] / p[kept].sum()).max() < 0.03
