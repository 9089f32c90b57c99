"""Each CUDA kernel against the CPU oracle on the same seeded inputs, through the C ABI (teacher-forced: the kernel gets
exactly the inputs the oracle's function gets).  Integer and ordered-sum work must agree bit for bit; where exp / ln /
x^-1/2 enter, the oracle is run on the engine's own host arithmetic, which makes those bit-exact too."""
import numpy as np
import pytest

from ava_b200 import build, config, engine

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.fixture(scope="module", autouse=True)
def _lib():
    build.build()
    engine.lib()


@pytest.fixture()
def orc_same_math(orc):
    orc.set_math(*engine.host_math())
    yield orc
    orc.reset_math()


def test_device_math_equals_host_math():
    L = engine.lib()
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.uniform(-104, 89, 200000), rng.normal(0, 1, 100000), [0.0, -0.0, np.inf, -np.inf, np.nan, 88.72, -103.9]]).astype(np.float32)
    got = engine.op_math(0, x)
    want = np.array([L.ava_host_expf(float(v)) for v in x[:5000]], np.float32)
    assert np.array_equal(bits(got[:5000]), bits(want))
    tail = np.array([L.ava_host_expf(float(v)) for v in x[-7:]], np.float32)
    assert np.array_equal(bits(got[-7:]), bits(tail))
    y = np.abs(np.concatenate([rng.lognormal(0, 20, 100000), rng.uniform(0.4, 2.6, 100000), [0.0, 1.0, np.inf, 1e-40]])).astype(np.float32)
    got = engine.op_math(1, y)
    idx = np.r_[0:3000, 100000:103000, y.size - 4:y.size]
    want = np.array([L.ava_host_logf(float(v)) for v in y[idx]], np.float32)
    assert np.array_equal(bits(got[idx]), bits(want))
    got = engine.op_math(2, y[:100000] + np.float32(1e-30))
    want = np.array([L.ava_host_rsqrtf(float(v)) for v in (y[:3000] + np.float32(1e-30))], np.float32)
    assert np.array_equal(bits(got[:3000]), bits(want))


@pytest.mark.parametrize("m,din,dout", [(1, 128, 64), (5, 768, 768), (1, 768, 3072), (8, 3072, 784), (3, 192, 48), (70, 768, 3840), (256, 3072, 768), (33, 128, 320), (256, 768, 4112)])
def test_q8_matmul_bits(orc, m, din, dout):
    rng = np.random.default_rng(m * 7 + dout)
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = (rng.uniform(0.5, 1.5, dout) / 127).astype(np.float32)
    x = rng.normal(size=(m, din)).astype(np.float32)
    if m > 2:
        x[1] = 0.0
        x[2] = rng.integers(-2, 3, din)   # spikes: the sum is an exact integer
        x[0, ::5] = -0.0
    orc.set_threads(8)
    try:
        want = orc.q8_matmul(x, q, sc)
    finally:
        orc.set_threads(1)
    got = engine.op_q8_matmul(x, q, sc)
    assert np.array_equal(bits(got), bits(want))
    if m > 2:
        exact = (x[2].astype(np.int64) @ q.astype(np.int64)).astype(np.float32) * sc
        assert np.array_equal(bits(got[2]), bits(exact))


@pytest.mark.parametrize("m,din,dout", [(1, 64, 64), (5, 128, 132), (70, 768, 3840), (256, 3072, 768), (130, 768, 16384), (300, 2048, 196)])
def test_tensor_core_product_agrees_to_rounding(orc, m, din, dout):
    """The tcgen05 form of the product: exact products, the tensor core's summation order.  Against the reference's
    ordered sum it may differ by the rounding of the additions only: at most 4e-6 of the sum of the terms' magnitudes
    (measured: 1.3e-6 to 2.3e-6), and spike rows (small integers) come out exact."""
    rng = np.random.default_rng(m + dout)
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = (rng.uniform(0.5, 1.5, dout) / 127).astype(np.float32)
    x = (rng.normal(size=(m, din)) * np.exp(rng.normal(size=(m, din)))).astype(np.float32)
    if m > 2:
        x[1] = 0.0
        x[2] = rng.integers(-2, 3, din)
    orc.set_threads(8)
    try:
        want = orc.q8_matmul(x, q, sc)
    finally:
        orc.set_threads(1)
    got = engine.op_q8_tc_matmul(x, q, sc)
    mag = (np.abs(x).astype(np.float64) @ np.abs(q).astype(np.float64)) * sc + 1e-30
    assert float(np.max(np.abs(got.astype(np.float64) - want) / mag)) <= 4e-6
    if m > 2:
        assert not got[1].any()
        assert np.array_equal(bits(got[2]), bits(want[2]))   # integer sums below 2^24: exact in any order
    with pytest.raises(engine.NotApplicable):
        engine.op_q8_tc_matmul(x[:, :48], q[:48], sc)


@pytest.mark.parametrize("density", [0.0, 0.02, 0.25, 0.6, 1.0])
@pytest.mark.parametrize("din,dout", [(768, 768), (3072, 768), (128, 320)])
@pytest.mark.parametrize("m", [9, 3])
def test_event_sum_bits(orc, density, din, dout, m):
    """The event-sum kernel (non-zero inputs only, in order) gives the dense sum's bits at any density; nine rows take
    the kernel for batches, three the one for a few sequences."""
    rng = np.random.default_rng(int(density * 100) + din)
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = (rng.uniform(0.5, 1.5, dout) / 127).astype(np.float32)
    x = np.zeros((m, din), np.float32)
    on = rng.random((m, din)) < density
    x[on] = rng.normal(size=on.sum())
    x[0][on[0]] = rng.integers(-2, 3, on[0].sum())   # spikes
    x[1, ::7] = -0.0
    want = orc.q8_matmul(x, q, sc)
    got = engine.op_q8_matmul(x, q, sc, event=True)
    assert np.array_equal(bits(got), bits(want))
    assert np.array_equal(bits(engine.op_q8_matmul(x, q, sc)), bits(want))


@pytest.mark.parametrize("m,din,dout,density", [(8, 64, 128, 0.5), (77, 3072, 768, 0.25), (256, 768, 768, 0.05), (19, 192, 784, 0.3), (130, 2048, 208, 0.6), (5, 128, 64, 0.2)])
def test_event_sum_bits_many_rows(orc, m, din, dout, density):
    """The event sum of a batch of rows: the dense sum's bits for every row, for row counts and widths that do and do not
    fill a block's columns, with rows of all zeros, -0 (skipped) and a NaN (kept: src/int8.rs:261-269)."""
    rng = np.random.default_rng(m + din + dout)
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = (rng.uniform(0.5, 1.5, dout) / 127).astype(np.float32)
    x = np.zeros((m, din), np.float32)
    on = rng.random((m, din)) < density
    x[on] = rng.normal(size=on.sum())
    x[0][on[0]] = rng.integers(-2, 3, on[0].sum())
    x[1, ::7] = -0.0
    x[2] = 0.0
    x[m - 1, din // 2] = np.nan
    orc.set_threads(8)
    try:
        want = orc.q8_matmul(x, q, sc)
    finally:
        orc.set_threads(1)
    got = engine.op_q8_matmul(x, q, sc, event=True)
    assert np.array_equal(bits(got[:m - 1]), bits(want[:m - 1]))
    assert np.isnan(got[m - 1]).all() and np.isnan(want[m - 1]).all()
    assert not np.isnan(got[:m - 1]).any()


@pytest.mark.parametrize("m,din,dout", [(128, 64, 64), (256, 768, 768), (1024, 768, 128), (128, 3072, 68)])
def test_spike_rows_on_the_tensor_cores_are_the_event_sums_bits(orc, m, din, dout):
    """Rows of spikes (integers in -2..2) times int8 weights with one bf16 limb each side on tcgen05: every partial sum is
    an integer below 2^24, so the accumulator is exact in any order; times the scale and added to what is there, the
    result is the bits of the ordered sum followed by the same multiply and add."""
    rng = np.random.default_rng(m + din + dout)
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = (rng.uniform(0.5, 1.5, dout) / 127).astype(np.float32)
    x = (rng.integers(-2, 3, (m, din)) * (rng.random((m, din)) < 0.3)).astype(np.float32)
    x[0] = 2.0   # the largest sums a row can make
    x[1] = -2.0
    y0 = rng.normal(size=(m, dout)).astype(np.float32)
    got = engine.op_q8_spike_tc_matmul(x, q, sc, y0)
    orc.set_threads(8)
    try:
        prod = orc.q8_matmul(x, q, sc)
    finally:
        orc.set_threads(1)
    want = (y0 + prod).astype(np.float32)   # one rounding, as the residual add has
    assert np.array_equal(bits(got), bits(want))


def test_event_sum_more_rows_than_a_grid_dimension(orc):
    """70000 token-rows (a long prompt chunk of many sequences): more than one grid dimension holds (65535), so the
    rows go on in a second one; first, middle and last rows against the oracle, all rows against the dense kernel."""
    rng = np.random.default_rng(70000)
    m, din, dout = 70000, 64, 64
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = (rng.uniform(0.5, 1.5, dout) / 127).astype(np.float32)
    x = (rng.integers(-2, 3, (m, din)) * (rng.random((m, din)) < 0.3)).astype(np.float32)
    got = engine.op_q8_matmul(x, q, sc, event=True)
    dense = engine.op_q8_matmul(x, q, sc, event=False)
    assert np.array_equal(bits(got), bits(dense))
    pick = np.r_[0:4, 32766:32770, 65534:65538, m - 3:m]
    assert np.array_equal(bits(got[pick]), bits(orc.q8_matmul(x[pick], q, sc)))


@pytest.mark.parametrize("m,n", [(1, 64), (7, 768), (300, 2048)])
def test_rmsnorm_bits(orc_same_math, m, n):
    rng = np.random.default_rng(n)
    x = (rng.normal(size=(m, n)) * rng.uniform(0.01, 30, (m, 1))).astype(np.float32)
    g = rng.uniform(0.5, 1.5, n).astype(np.float32)
    want = np.stack([orc_same_math.rmsnorm(x[r], g) for r in range(m)])
    assert np.array_equal(bits(engine.op_rmsnorm(x, g)), bits(want))


@pytest.mark.parametrize("spikes", [0, 1, 2])
@pytest.mark.parametrize("alif", [False, True])
def test_lif_exact(orc, spikes, alif):
    rng = np.random.default_rng(spikes * 2 + alif)
    m, d = 9, 768
    cur = rng.normal(0, 1.2, (m, d)).astype(np.float32)
    beta = rng.uniform(0.8, 0.99, d).astype(np.float32)
    th = rng.uniform(0.8, 1.2, d).astype(np.float32)
    v0 = rng.normal(0, 1, (m, d)).astype(np.float32)
    s0 = rng.integers(-2, 3, (m, d)).astype(np.float32) if spikes == 2 else rng.integers(0, 2, (m, d)).astype(np.float32)
    kw = {}
    if alif:
        kw = dict(rho=rng.uniform(0.9, 0.99, d).astype(np.float32), gain=rng.uniform(0.5, 1.5, d).astype(np.float32))
        a0 = rng.uniform(0, 1, (m, d)).astype(np.float32)
    # some membranes exactly on a threshold
    cur[0, :8] = 0.0
    v0[0, :8] = 0.0
    s1, v1, a1 = engine.op_lif(cur, beta, v0, s0, theta=th, a0=a0 if alif else None, spikes=spikes, **kw)
    for r in range(m):
        ws, wv, wa = orc.lif(cur[r], beta, v0[r], s0[r], theta=th, a0=a0[r] if alif else None, spikes=spikes, **kw)
        assert np.array_equal(s1[r], ws)
        assert np.array_equal(bits(v1[r]), bits(wv))
        if alif:
            assert np.array_equal(bits(a1[r]), bits(wa))


def test_lif_hand_vectors():
    """The reference's hand-worked spikes (arch/tests.rs:431-445) through the kernel."""
    cur = [2.5, -1.2, 0.3, -3.0, 1.0, 0.99]
    for spikes, want in ((1, [1, -1, 1, -1, 1, 0]), (2, [2, -2, 2, -2, 2, -1]), (0, [1, 0, 0, 0, 1, 0])):
        v = np.zeros((1, 1), np.float32)
        s = np.zeros((1, 1), np.float32)
        got = []
        for i in cur:
            s, v, _ = engine.op_lif(np.array([[i]], np.float32), np.zeros(1, np.float32), v, s, spikes=spikes)
            got.append(float(s[0, 0]))
        assert got == [float(w) for w in want]


@pytest.mark.parametrize("n,k", [(256, 64), (3072, 768), (8192, 2048), (1000, 999), (64, 64)])
@pytest.mark.parametrize("relu2", [0, 1])
def test_kwta_exact(orc, n, k, relu2):
    rng = np.random.default_rng(n + k)
    m = 6
    u = rng.normal(size=(m, n)).astype(np.float32)
    u[1, : n // 2] = u[1, 0]            # a big tie
    u[2] = -np.abs(u[2])                # all negative
    u[3, ::3] = 0.0
    u[3, 1::3] = -0.0
    u[4] = np.round(u[4] * 4) / 4       # many ties at the threshold
    got = engine.op_kwta(u, k, relu2)
    for r in range(m):
        want = orc.kwta(u[r], k, relu2)
        assert np.array_equal(got[r] != 0, want != 0), r
        assert np.array_equal(got[r], want), r


@pytest.mark.parametrize("hs,m", [(32, 5), (64, 12), (128, 3), (256, 2), (768, 3)])
def test_mem_heads_bits(orc, hs, m):
    rng = np.random.default_rng(hs)
    unit = lambda x: (x / np.sqrt((x * x).sum(-1, keepdims=True))).astype(np.float32)
    e = unit(rng.normal(size=(m, hs)))
    k = unit(rng.normal(size=(m, hs)))
    q = unit(rng.normal(size=(m, hs)))
    v = rng.normal(size=(m, hs)).astype(np.float32)
    ex = rng.uniform(0.9, 1.0, (m, hs)).astype(np.float32)
    be = rng.uniform(0.05, 1.5, (m, hs)).astype(np.float32)
    w, ah, qg = k * be, e * (be * ex), q * ex
    qw = rng.normal(size=m).astype(np.float32)
    qa = rng.normal(size=m).astype(np.float32)
    f = rng.normal(0, 0.3, (m, hs, hs)).astype(np.float32)
    f[0] = 0.0
    y, f1 = engine.op_mem_heads(e, v, w, ah, qg, ex, qw, qa, f)
    for i in range(m):
        wy, wf, _ = orc.head_rows(e[i], v[i], w[i], ah[i], qg[i], ex[i], float(qw[i]), float(qa[i]), f[i])
        assert np.array_equal(bits(y[i]), bits(wy)), i
        assert np.array_equal(bits(f1[i]), bits(wf)), i
    # twice over the same state: the second call reads what the first wrote
    y2, f2 = engine.op_mem_heads(e, v, w, ah, qg, ex, qw, qa, f1)
    wy, wf, _ = orc.head_rows(e[1], v[1], w[1], ah[1], qg[1], ex[1], float(qw[1]), float(qa[1]), f1[1])
    assert np.array_equal(bits(f2[1]), bits(wf)) and np.array_equal(bits(y2[1]), bits(wy))


@pytest.mark.parametrize("hs,m", [(768, 40), (64, 700), (128, 200), (256, 77)])
def test_mem_heads_bits_when_a_block_walks_several_items(orc, hs, m):
    """The state pass keeps as many blocks as the GPU holds at once and each walks several (row, slice) items, the
    next item's rows streaming in while the current one is updated: with more items than blocks every buffer, barrier
    phase and hand-over between items is exercised.  Same bits as `head_rows` (src/model/fstep/arch.rs:256-337)."""
    rng = np.random.default_rng(hs + m)
    unit = lambda x: (x / np.sqrt((x * x).sum(-1, keepdims=True))).astype(np.float32)
    e, k, q = (unit(rng.normal(size=(m, hs))) for _ in range(3))
    v = rng.normal(size=(m, hs)).astype(np.float32)
    ex = rng.uniform(0.9, 1.0, (m, hs)).astype(np.float32)
    be = rng.uniform(0.05, 1.5, (m, hs)).astype(np.float32)
    w, ah, qg = k * be, e * (be * ex), q * ex
    qw, qa = rng.normal(size=m).astype(np.float32), rng.normal(size=m).astype(np.float32)
    f = rng.normal(0, 0.3, (m, hs, hs)).astype(np.float32)
    y, f1 = engine.op_mem_heads(e, v, w, ah, qg, ex, qw, qa, f)
    y2, f2 = engine.op_mem_heads(e, v, w, ah, qg, ex, qw, qa, f1)
    for i in list(range(0, m, max(1, m // 16))) + [m - 1]:
        wy, wf, _ = orc.head_rows(e[i], v[i], w[i], ah[i], qg[i], ex[i], float(qw[i]), float(qa[i]), f[i])
        assert np.array_equal(bits(y[i]), bits(wy)), i
        assert np.array_equal(bits(f1[i]), bits(wf)), i
        wy2, wf2, _ = orc.head_rows(e[i], v[i], w[i], ah[i], qg[i], ex[i], float(qw[i]), float(qa[i]), wf)
        assert np.array_equal(bits(y2[i]), bits(wy2)) and np.array_equal(bits(f2[i]), bits(wf2)), i


@pytest.mark.parametrize("hs,m,chunk", [(768, 20, 3), (768, 400, 0), (768, 3, 5), (64, 8, 0), (256, 50, 1)])
def test_mem_heads_bounded_wait_runs_out_and_the_state_stays(hs, m, chunk):
    """Every wait on a copy barrier inside the state pass is bounded.  Nothing is made to fault or hang here: all the
    copies complete, only one barrier per block is told to expect 16 bytes more than will arrive, with a limit of a few
    thousand polls.  The kernel must give up, raise its status bit (a step then returns AVA_ERR_CUDA) and leave every
    bit of the state as it was: a block that gave up neither updates nor stores."""
    import ctypes as C
    changed = C.c_int32(-1)
    rc = engine.lib().ava_debug_mem_heads_wait_runs_out(0, m, hs, chunk, 4000, C.byref(changed))
    assert rc == engine.ERR_CUDA
    assert changed.value == 0
    # and the device is fine afterwards: the same kernel, undisturbed, gives the usual bits
    x = np.full((1, hs), 0.01, np.float32)
    engine.op_mem_heads(x, x, x, x, x, np.ones((1, hs), np.float32), np.ones(1, np.float32), np.ones(1, np.float32), np.zeros((1, hs, hs), np.float32))


@pytest.mark.parametrize("n", [1, 2, 3, 70, 1500])
@pytest.mark.parametrize("bf16", [False, True])
def test_attend_bits(orc_same_math, n, bf16):
    orc = orc_same_math
    rng = np.random.default_rng(n)
    m, hs = 12, 64
    q = rng.normal(size=(m, hs)).astype(np.float32)
    kc = rng.normal(size=(m, n, hs)).astype(np.float32)
    vc = rng.normal(size=(m, n, hs)).astype(np.float32)
    got = engine.op_attend(q, kc, vc, bf16)
    if bf16:
        rb = np.vectorize(orc.bf16_round, otypes=[np.float32])
        kc, vc = rb(kc), rb(vc)
    scale = np.float32(1.0 / np.sqrt(float(hs)))
    for hh in range(m):
        want = orc.attend(q[hh], kc[hh], vc[hh], scale)
        assert np.array_equal(bits(got[hh]), bits(want)), hh
