"""The chunk-parallel (tensor-core) form of the fast-weight memory on the GPU: its batched limb product against float64,
and the whole chunked pass against the oracle's token loop at the reference's own bound for its chunked form
(design-tests/nn/gpu/src/arch/tests.rs:700-753: 1e-4 of max(1, max|ref|))."""
import numpy as np
import pytest

from ava_b200 import build, engine

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib():
    build.build()
    engine.lib()


@pytest.mark.parametrize("batch,m,n,k", [(1, 128, 128, 64), (3, 128, 768, 768), (2, 768, 768, 128), (5, 128, 128, 768), (2, 256, 64, 192)])
def test_batched_limb_product_is_an_f32_product(batch, m, n, k):
    """Three bf16 limbs per operand and the six leading limb products: every operand is carried to 2^-24, so the result
    agrees with the float64 product to the rounding of the f32 additions (1e-5 of the sum of magnitudes allowed; measured up to 5e-6 at K = 768: the tensor core truncates where an ordered f32 sum rounds)."""
    rng = np.random.default_rng(m + n + k)
    a = (rng.normal(size=(batch, m, k)) * np.exp(rng.normal(size=(batch, m, k)))).astype(np.float32)
    b = (rng.normal(size=(batch, n, k)) * np.exp(rng.normal(size=(batch, n, k)))).astype(np.float32)
    got = engine.op_tc_bgemm(a, b)
    want = np.einsum("bmk,bnk->bmn", a.astype(np.float64), b.astype(np.float64))
    mag = np.einsum("bmk,bnk->bmn", np.abs(a).astype(np.float64), np.abs(b).astype(np.float64))
    assert float((np.abs(got - want) / mag).max()) < 1e-5
    # the decaying update: c = colscale * c + a . b^T, and the limbs written for the new c sum to it exactly
    c0 = rng.normal(size=(batch, m, n)).astype(np.float32)
    g = rng.uniform(0.2, 1.0, (batch, n)).astype(np.float32)
    c1, limb_sum = engine.op_tc_bgemm(a, b, colscale=g, c_in=c0)
    want1 = g[:, None, :].astype(np.float64) * c0 + want
    assert float((np.abs(c1 - want1) / (mag + np.abs(c0))).max()) < 1e-5
    assert np.array_equal(limb_sum.view(np.uint32), c1.view(np.uint32))


def _chunk_case(rng, t, hb, hs, rate_bias):
    unit = lambda x: (x / np.linalg.norm(x, axis=-1, keepdims=True)).astype(np.float32)
    q, k, e = (unit(rng.normal(size=(t, hb, hs))) for _ in range(3))
    v = rng.normal(size=(t, hb, hs)).astype(np.float32)
    la = (-np.log1p(np.exp(-(rng.normal(size=(t, hb, hs)) + rate_bias)))).astype(np.float32)  # log sigmoid
    b = (1.0 / (1.0 + np.exp(-rng.normal(size=(t, hb, hs))))).astype(np.float32)
    f0 = (0.1 * rng.normal(size=(hb, hs, hs))).astype(np.float32)
    return q, k, e, v, la, b, f0


@pytest.mark.parametrize("t,hb,hs,rate_bias", [(64, 1, 128, 3.0), (128, 3, 128, 2.0), (256, 2, 256, 4.0), (128, 2, 768, 3.0)])
def test_chunked_memory_agrees_with_the_token_loop(t, hb, hs, rate_bias):
    """y and the state after t tokens from the chunk-parallel kernels (64-token chunks, state carried from chunk to
    chunk and from a non-zero start) against the oracle's token loop, at the reference's bound for its own chunked
    form: 1e-4 of max(1, max|ref|)."""
    from oracle import oracle

    rng = np.random.default_rng(t + hb + hs)
    q, k, e, v, la, b, f0 = _chunk_case(rng, t, hb, hs, rate_bias)
    w = (k * b).astype(np.float32)
    ah = (e * (b * np.exp(la))).astype(np.float32)
    y, f1, oor = engine.op_mem_chunk(q, e, w, ah, v, la, f0)
    assert not oor
    for h in range(hb):
        yr, fr, _ = oracle.delta_rec(q[:, h], k[:, h], e[:, h], v[:, h], la[:, h], b[:, h], f0=f0[h])
        assert float(np.abs(y[:, h] - yr).max()) <= 1e-4 * max(1.0, float(np.abs(yr).max())), h
        assert float(np.abs(f1[h] - fr).max()) <= 1e-4 * max(1.0, float(np.abs(fr).max())), h


def test_chunked_memory_refuses_rates_outside_its_range():
    """Rates that forget by more than e^-60 inside one chunk cannot be written as products of per-token scalings in
    f32; the pass says so and touches nothing."""
    rng = np.random.default_rng(5)
    q, k, e, v, la, b, f0 = _chunk_case(rng, 64, 1, 128, -3.0)  # log rates near -3 per token: -190 over the chunk
    y, f1, oor = engine.op_mem_chunk(q, e, k * b, e * (b * np.exp(la)), v, la, f0)
    assert oor
    assert np.array_equal(f1, f0) and not y.any()


def _bf16_round(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


@pytest.mark.parametrize("rows,t,n0,start,heads", [(1, 64, 0, 0, 1), (2, 200, 37, 3, 2), (1, 256, 300, 0, 3), (3, 130, 1000, 11, 1)])
def test_engram_chunk_read_is_the_causal_softmax(rows, t, n0, start, heads):
    """The causal read of a whole chunk (tensor cores, two passes, keys in tiles of 64) against float64: token i sees
    the n0 keys held before the chunk and the chunk's keys 0 .. i, all as the store keeps them (bf16).  Chunk lengths
    that do and do not fill a tile of 128 queries, stores that start inside the ring, never-written slots full of NaN."""
    rng = np.random.default_rng(rows + t + n0 + heads)
    d = 64 * heads
    qkv = rng.normal(size=(t, rows, 3 * d)).astype(np.float32)
    qkv[:, :, :d] *= 3.0   # sharp scores: a few keys carry most of a row's weight
    kp = rng.normal(size=(rows, heads, n0, 64)).astype(np.float32)
    vp = rng.normal(size=(rows, heads, n0, 64)).astype(np.float32)
    got = engine.op_engram_chunk(qkv, kp, vp, start=start)
    worst = 0.0
    for r in range(rows):
        for h in range(heads):
            q = qkv[:, r, h * 64:(h + 1) * 64].astype(np.float64)
            k = np.concatenate([_bf16_round(kp[r, h]), _bf16_round(qkv[:, r, d + h * 64:d + (h + 1) * 64])]).astype(np.float64)
            v = np.concatenate([_bf16_round(vp[r, h]), _bf16_round(qkv[:, r, 2 * d + h * 64:2 * d + (h + 1) * 64])]).astype(np.float64)
            s = q @ k.T / 8.0
            vis = np.arange(n0 + t)[None, :] <= (n0 + np.arange(t))[:, None]
            s = np.where(vis, s, -np.inf)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            want = (p / p.sum(axis=1, keepdims=True)) @ v
            worst = max(worst, float(np.abs(got[:, r, h * 64:(h + 1) * 64] - want).max()) / max(1.0, float(np.abs(want).max())))
    print("engram chunk read against float64:", worst)
    assert worst <= 2e-5
