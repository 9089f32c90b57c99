"""The oracle's chunk-parallel forms of the fast-weight memory against its own token loops, on the cases the
reference's tests use (design-tests/nn/gpu/src/arch/tests.rs:700-753 `chunked_memory_matches_the_token_loop`:
per-head and per-channel gates, momentum 0 / 0.5 / 0.7, lengths 16, 24, 32, 40, 128, from zero and from a carried
state, log alpha shifted by -6 so that products of rates underflow, bound 1e-4 of max(1, max|ref|);
design-tests/nn/gpu/tests/smoke.rs:373-391: the chunk-64 WY form of the plain delta rule against stepping with
repeated keys over 128 tokens, bound 1e-3).  CPU only."""
import numpy as np
import pytest


def unit(x):
    return (x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)).astype(np.float32)


def log_sigmoid(x):
    return (-(np.maximum(-x, 0) + np.log1p(np.exp(-np.abs(x))))).astype(np.float32)


def rel(a, b):
    return float(np.abs(a - b).max() / max(1.0, float(np.abs(b).max())))


CASES = [(False, 0.0, 32, 2.0), (True, 0.0, 32, 2.0), (False, 0.5, 40, 2.0), (True, 0.5, 24, 2.0), (True, 0.0, 32, -6.0), (True, 0.7, 16, -6.0),
         (False, 0.0, 128, 1.0)]


@pytest.mark.parametrize("n", range(len(CASES)))
@pytest.mark.parametrize("carried", [False, True])
def test_chunked_memory_matches_the_token_loop(orc, n, carried):
    chan, m, t, shift = CASES[n]
    hs = 8
    g = hs if chan else 1
    for head in range(4):                       # the reference's 2 rows x 2 heads
        rng = np.random.default_rng(100 * n + head)
        q, k = unit(rng.normal(size=(t, hs))), unit(rng.normal(size=(t, hs)))
        e = unit(rng.normal(size=(t, hs))) if chan else k.copy()
        v = rng.normal(size=(t, hs)).astype(np.float32)
        la = log_sigmoid(3.0 * rng.normal(size=(t, g)) + shift)
        bw = (2.0 / (1.0 + np.exp(-rng.normal(size=(t, g))))).astype(np.float32)
        f0 = (0.3 * rng.normal(size=(hs, hs))).astype(np.float32) if carried else None
        s0 = (0.3 * rng.normal(size=(hs, hs))).astype(np.float32) if carried and m > 0 else None
        y1, f1, s1 = orc.delta_rec(q, k, e, v, la, bw, m, f0, s0)
        y2, f2, s2 = orc.delta_chunk(q, k, e, v, la, bw, m, f0, s0)
        assert np.isfinite(y2).all()
        assert rel(y2, y1) < 1e-4, (head, rel(y2, y1))
        assert rel(f2, f1) < 1e-4, (head, rel(f2, f1))
        assert (s1 is None) == (s2 is None)
        if s1 is not None:
            assert rel(s2, s1) < 1e-4


def test_token_loop_is_the_fused_steps_head(orc):
    """The oracle's `delta_rec` (the reference's tensor-op loop, src/arch.rs:1091-1136) and its `head_rows` (the fused
    step's loop, src/model/fstep/arch.rs:256-337) are the same rule: they agree to rounding token after token."""
    rng = np.random.default_rng(3)
    t, hs = 12, 16
    q, k, e = unit(rng.normal(size=(t, hs))), unit(rng.normal(size=(t, hs))), unit(rng.normal(size=(t, hs)))
    v = rng.normal(size=(t, hs)).astype(np.float32)
    la = log_sigmoid(3.0 * rng.normal(size=(t, hs)) + 2.0)
    bw = (2.0 / (1.0 + np.exp(-rng.normal(size=(t, hs))))).astype(np.float32)
    y1, f1, _ = orc.delta_rec(q, k, e, v, la, bw)
    f = np.zeros((hs, hs), np.float32)
    for i in range(t):
        ex = np.exp(la[i]).astype(np.float32)
        y, f, _ = orc.head_rows(e[i], v[i], k[i] * bw[i], e[i] * (bw[i] * ex), q[i] * ex, ex, float((q[i] * (k[i] * bw[i])).sum()),
                                float((q[i] * (e[i] * (bw[i] * ex))).sum()), f)
        assert rel(y, y1[i]) < 1e-5, i
    assert rel(f, f1) < 1e-5


def test_wy_form_of_the_plain_rule_against_stepping_with_repeated_keys(orc):
    """`delta_rule_from` (chunk 64, (I + A)^-1 by block doubling) against the plain rule stepped token by token over 128
    tokens whose second half repeats one token: the case a Neumann series blows up on (tests/smoke.rs:373-391)."""
    rng = np.random.default_rng(7)
    t, hs = 128, 32
    q, k = unit(rng.normal(size=(t, hs))), unit(rng.normal(size=(t, hs)))
    v = rng.normal(size=(t, hs)).astype(np.float32)
    k[64:], q[64:], v[64:] = k[64], q[64], v[64]
    la = log_sigmoid(rng.normal(size=t) + 3.0)
    beta = (1.0 / (1.0 + np.exp(-rng.normal(size=t)))).astype(np.float32)
    y, f = orc.delta_rule_from(q, k, v, la, beta)
    fs = np.zeros((hs, hs), np.float32)
    for i in range(t):
        fs, ys = orc.delta_plain(fs, k[i], v[i], q[i], float(np.exp(la[i])), float(beta[i]))
        assert np.abs(ys - y[i]).max() < 1e-3, i
    assert np.abs(fs - f).max() < 1e-3
    # and from a carried state, in two windows
    y_a, f_a = orc.delta_rule_from(q[:64], k[:64], v[:64], la[:64], beta[:64])
    y_b, f_b = orc.delta_rule_from(q[64:], k[64:], v[64:], la[64:], beta[64:], f_a)
    assert np.abs(np.concatenate([y_a, y_b]) - y).max() < 1e-4 and np.abs(f_b - f).max() < 1e-4


def test_inverse_by_block_doubling(orc):
    rng = np.random.default_rng(1)
    for c in (1, 2, 4, 16, 64):
        a = np.tril(rng.normal(size=(c, c)), -1).astype(np.float32)
        t = orc.inv_unit_lower(a)
        assert np.abs(t @ (np.eye(c, dtype=np.float32) + a) - np.eye(c)).max() < 5e-3 * max(1.0, float(np.abs(t).max()))
