"""The CPU oracle against the reference's own hand-worked vectors and the identities its tests assert.

Sources (paths inside the reference project):
  design-tests/nn/gpu/src/arch/tests.rs:431-445    signed integer spikes by hand
  design-tests/nn/grad/tests/lif.rs:7-10,46-50     LIF three-step trace
  design-tests/nn/gpu/src/arch/tests.rs:317-364    momentum recurrence by hand (F1 = U1, F2 = a2 F1 + M U1 + U2)
  design-tests/nn/parts/src/quant.rs:111-125       quantiser error bound
  design-tests/nn/gpu/src/int8/tests.rs:60-119     SIMD == scalar, event == dense, threads, row alone == row in batch
  design-tests/nn/gpu/src/int8/tests.rs:394-457    event-list semantics, concat identity
  design-tests/nn/gpu/tests/smoke.rs:156           kWTA keeps u >= kth
"""
import numpy as np
import pytest

from ava_b200 import config, synth


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---------------------------------------------------------------------------------------------- spikes by hand
def run_lif(orc, cur, beta, spikes, theta=1.0):
    v = np.zeros(1, np.float32)
    s = np.zeros(1, np.float32)
    out_s, out_v = [], []
    for i in cur:
        s, v, _ = orc.lif(np.array([i], np.float32), np.array([beta], np.float32), v, s,
                          theta=np.array([theta], np.float32), spikes=spikes, slope=4.0)
        out_s.append(float(s[0]))
        out_v.append(float(v[0]))
    return out_s, out_v


def test_integer_spikes_by_hand(orc):
    cur = [2.5, -1.2, 0.3, -3.0, 1.0, 0.99]
    assert run_lif(orc, cur, 0.0, config.SPIKES_TERNARY)[0] == [1.0, -1.0, 1.0, -1.0, 1.0, 0.0]
    assert run_lif(orc, cur, 0.0, config.SPIKES_INT2)[0] == [2.0, -2.0, 2.0, -2.0, 2.0, -1.0]
    assert run_lif(orc, cur, 0.0, config.SPIKES_BINARY)[0] == [1.0, 0.0, 0.0, 0.0, 1.0, 0.0]


def test_lif_three_step_trace(orc):
    s, v = run_lif(orc, [0.8, 0.9, 0.3], 0.5, config.SPIKES_BINARY)
    assert s == [0.0, 1.0, 0.0]
    np.testing.assert_allclose(v, [0.8, 1.3, -0.05], atol=1e-6)


def test_spikes_are_integers_and_silent_at_rest(orc):
    rng = np.random.default_rng(0)
    d = 4096
    cur = rng.normal(0, 1.5, d).astype(np.float32)
    beta = rng.uniform(0.8, 0.99, d).astype(np.float32)
    v0 = rng.normal(0, 1, d).astype(np.float32)
    s0 = rng.integers(-2, 3, d).astype(np.float32)
    a0 = rng.uniform(0, 1, d).astype(np.float32)
    rho = np.full(d, 0.95, np.float32)
    gain = np.ones(d, np.float32)
    th = rng.uniform(0.8, 1.2, d).astype(np.float32)
    s, v, a = orc.lif(cur, beta, v0, s0, theta=th, rho=rho, gain=gain, a0=a0, spikes=2)
    assert set(np.unique(s)).issubset({-2.0, -1.0, 0.0, 1.0, 2.0})
    # the reference's rule: s = sign(v) min(floor(|v| / theta_t), 2)
    th_t = th + a * gain
    want = np.sign(v) * np.minimum(np.floor(np.abs(v) / th_t), 2)
    near = np.abs(np.abs(v) / th_t - np.round(np.abs(v) / th_t)) < 1e-5
    assert np.array_equal(s[~near], want[~near].astype(np.float32))
    z = np.zeros(8, np.float32)
    s, v, _ = orc.lif(z, np.full(8, 0.9, np.float32), z, z, spikes=2)
    assert not s.any() and not v.any()


# ---------------------------------------------------------------------------------------------- fast weights
def delta_rec64(q, k, e, v, alpha, b, m, f0, s0):
    """The recurrence of the reference's token loop (arch.rs:1091-1136) in float64, per-channel gates."""
    upd = np.outer(b * k, v) - alpha[:, None] * np.outer(b * e, e @ f0)
    s1 = m * s0 + upd
    f1 = alpha[:, None] * f0 + s1
    return q @ f1, f1, s1


def head_inputs(rng, hs):
    unit = lambda x: x / np.sqrt((x * x).sum() + 1e-6)
    q, k, e = (unit(rng.normal(size=hs)) for _ in range(3))
    v = rng.normal(size=hs)
    alpha = 1 / (1 + np.exp(-(rng.normal(size=hs) + 2)))
    b = 2 / (1 + np.exp(-rng.normal(size=hs)))
    return q, k, e, v, alpha, b


def oracle_head(orc, q, k, e, v, alpha, b, m, f0, s0):
    f32 = lambda x: np.asarray(x, np.float32)
    q, k, e, v, alpha, b = map(f32, (q, k, e, v, alpha, b))
    w = k * b
    ah = e * (b * alpha)
    qg = q * alpha
    qw = np.float32(0)
    qa = np.float32(0)
    for c in range(len(q)):
        qw = np.float32(qw + q[c] * w[c])
        qa = np.float32(qa + q[c] * ah[c])
    kw = {}
    if m > 0:
        kw = dict(mom=m, qs=q * np.float32(m), p2=e * np.float32(0), s0=f32(s0))
    return orc.head_rows(e, v, w, ah, qg, alpha, float(qw), float(qa), f32(f0), **kw)


@pytest.mark.parametrize("m", [0.0, 0.5, 0.7])
def test_head_rows_is_the_token_recurrence(orc, m):
    rng = np.random.default_rng(3)
    hs = 24
    f = np.zeros((hs, hs))
    s = np.zeros((hs, hs))
    f32, s32 = f.astype(np.float32), s.astype(np.float32)
    for _ in range(12):
        q, k, e, v, alpha, b = head_inputs(rng, hs)
        y, f, s = delta_rec64(q, k, e, v, alpha, b, m, f, s)
        y32, f32, s32n = oracle_head(orc, q, k, e, v, alpha, b, m, f32, s32)
        if m > 0:
            s32 = s32n
        np.testing.assert_allclose(y32, y, atol=2e-5)
        np.testing.assert_allclose(f32, f, atol=2e-5)
        if m > 0:
            np.testing.assert_allclose(s32, s, atol=2e-5)


def test_momentum_first_two_steps_by_hand(orc):
    """F1 = U1 and F2 = alpha2 F1 + M U1 + U2 with U_i = b k v^T - alpha b e (e^T F_prev)."""
    rng = np.random.default_rng(5)
    hs, m = 8, 0.7
    z = np.zeros((hs, hs), np.float32)
    i1, i2 = head_inputs(rng, hs), head_inputs(rng, hs)

    def U(inp, fprev):
        q, k, e, v, alpha, b = inp
        return np.outer(b * k, v) - alpha[:, None] * np.outer(b * e, e @ fprev)

    _, f1, s1 = oracle_head(orc, *i1, m, z, z)
    u1 = U(i1, np.zeros((hs, hs)))
    np.testing.assert_allclose(f1, u1, atol=1e-6)
    _, f2, _ = oracle_head(orc, *i2, m, f1, s1)
    want = i2[4][:, None] * u1 + m * u1 + U(i2, u1)
    np.testing.assert_allclose(f2, want, atol=1e-5)


def test_error_correcting_write_then_read(orc):
    """The benchmark corner (alpha = 1, b = eta, erase key = key, no momentum) is W += eta (v - W k) k^T with
    W = F^T, read after the write; and it agrees with the plain delta rule of the older block."""
    rng = np.random.default_rng(7)
    hs, eta = 16, np.float32(0.1)
    F = rng.normal(size=(hs, hs)).astype(np.float32)
    unit = lambda x: (x / np.sqrt((x * x).sum() + 1e-6)).astype(np.float32)
    k, q = unit(rng.normal(size=hs)), unit(rng.normal(size=hs))
    v = rng.normal(size=hs).astype(np.float32)
    one = np.ones(hs, np.float32)
    y, f1, _ = oracle_head(orc, q, k, k, v, one, one * eta, 0.0, F, None)
    W = F.T.astype(np.float64)
    W1 = W + eta * np.outer(v - W @ k, k)
    np.testing.assert_allclose(f1, W1.T, atol=1e-5)
    np.testing.assert_allclose(y, W1 @ q, atol=1e-5)
    f1p, yp = orc.delta_plain(F, k, v, q, 1.0, float(eta))
    np.testing.assert_allclose(f1p, f1, atol=1e-5)
    np.testing.assert_allclose(yp, y, atol=1e-5)


# ---------------------------------------------------------------------------------------------- quantiser + int8
def test_quantiser_bound_and_rounding(orc):
    rng = np.random.default_rng(1)
    w = rng.normal(0, 0.02, (96, 200)).astype(np.float32)
    w[:, 7] = 0.0
    q, sc = orc.quantize_int8(w)
    assert q.dtype == np.int8 and q.nbytes * 4 == w.nbytes
    assert sc[7] == 1.0 and not q[:, 7].any()
    np.testing.assert_array_equal(sc[np.arange(200) != 7], (np.abs(w).max(0) / np.float32(127.0))[np.arange(200) != 7])
    assert np.all(np.abs(w - q.astype(np.float32) * sc) <= sc / 2 + 1e-9)
    assert np.abs(q).max() == 127
    # half away from zero: 2.5 scale -> 3, -2.5 scale -> -3
    w2 = np.array([[127.0, 127.0], [2.5, -2.5]], np.float32)
    q2, sc2 = orc.quantize_int8(w2)
    assert sc2.tolist() == [1.0, 1.0] and q2[1].tolist() == [3, -3]


def chain_f32(x, q, sc):
    """y[c] = (fma chain over j ascending of x[j] * q[j][c] from +0) * scale[c], in exact arithmetic per step."""
    din, dout = q.shape
    acc = np.zeros(dout, np.float32)
    for j in range(din):
        # a product of an f32 and a small integer is exact in float64, so float64 add then one rounding = fma
        acc = (x[j].astype(np.float64) * q[j].astype(np.float64) + acc.astype(np.float64)).astype(np.float32)
    return acc * sc


@pytest.mark.parametrize("dout", [64, 200, 4112 // 16])
def test_q8_matmul_is_the_ordered_fma_chain(orc, dout):
    rng = np.random.default_rng(2)
    din = 96
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = rng.uniform(0.5, 1.5, dout).astype(np.float32) / 127
    x = rng.normal(size=(3, din)).astype(np.float32)
    y = orc.q8_matmul(x, q, sc)
    for r in range(3):
        assert np.array_equal(bits(y[r]), bits(chain_f32(x[r], q, sc)))
    # against the dequantised float64 product
    np.testing.assert_allclose(y, x.astype(np.float64) @ (q.astype(np.float64) * sc), rtol=0, atol=1e-4)


def test_simd_equals_scalar_and_threads_do_not_matter(orc):
    rng = np.random.default_rng(4)
    din, dout, m = 256, 4112, 13
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = rng.uniform(0.5, 1.5, dout).astype(np.float32) / 127
    x = rng.normal(size=(m, din)).astype(np.float32)
    x[3] = 0.0
    x[5, ::3] = -0.0
    ref = None
    try:
        for simd in (True, False):
            for th in (1, 2, 4, 8):
                orc.set_simd(simd)
                orc.set_threads(th)
                y = orc.q8_matmul(x, q, sc)
                if ref is None:
                    ref = y
                assert np.array_equal(bits(y), bits(ref)), (simd, th)
        # a row alone gives the bits it has inside the batch
        for r in (0, 3, 5, 12):
            assert np.array_equal(bits(orc.q8_matmul(x[r:r + 1], q, sc)[0]), bits(ref[r]))
    finally:
        orc.set_simd(True)
        orc.set_threads(1)


@pytest.mark.parametrize("density", [0.01, 0.08, 0.3, 0.6])
@pytest.mark.parametrize("graded", [False, True])
def test_event_sum_equals_dense_sum(orc, density, graded):
    rng = np.random.default_rng(6)
    din, dout, m = 384, 384, 5
    q = rng.integers(-127, 128, (din, dout)).astype(np.int8)
    sc = rng.uniform(0.5, 1.5, dout).astype(np.float32) / 127
    x = np.zeros((m, din), np.float32)
    on = rng.random((m, din)) < density
    x[on] = rng.integers(-2, 3, on.sum()) if graded else 1.0
    try:
        orc.set_event_max(0.5)
        y_ev = orc.q8_matmul(x, q, sc)
        n_ev = orc.last_event_rows()
        orc.set_event_max(-1.0)
        y_dense = orc.q8_matmul(x, q, sc)
        assert orc.last_event_rows() == 0
    finally:
        orc.set_event_max(0.5)
    assert n_ev == int(((x != 0).sum(1) <= 0.5 * din).sum())
    assert np.array_equal(bits(y_ev), bits(y_dense))
    # integer rows: the sum is an exact integer, so an int32 accumulation converted once gives the same bits
    y_int = (x.astype(np.int64) @ q.astype(np.int64)).astype(np.float32) * sc
    assert np.array_equal(bits(y_ev), bits(y_int))


def test_event_rule_counts_minus_zero_as_zero_and_nan_as_set(orc):
    din, dout = 64, 64
    q = np.ones((din, dout), np.int8)
    sc = np.ones(dout, np.float32)
    x = np.zeros((1, din), np.float32)
    x[0, :40] = -0.0
    x[0, 40] = 1e-40  # a denormal is not zero
    x[0, 41] = 3.0
    y = orc.q8_matmul(x, q, sc)
    assert orc.last_event_rows() == 1
    assert np.all(y == np.float32(3.0) + np.float32(1e-40))
    x[0, 42] = np.nan
    assert np.isnan(orc.q8_matmul(x, q, sc)).all()


def test_concat_gives_each_parts_own_bits(orc):
    rng = np.random.default_rng(8)
    din = 128
    parts = [(rng.integers(-127, 128, (din, n)).astype(np.int8), rng.uniform(0.5, 1.5, n).astype(np.float32)) for n in (64, 128, 192)]
    x = rng.normal(size=(2, din)).astype(np.float32)
    merged = orc.q8_matmul(x, np.concatenate([p[0] for p in parts], 1), np.concatenate([p[1] for p in parts]))
    c = 0
    for q, sc in parts:
        assert np.array_equal(bits(merged[:, c:c + q.shape[1]]), bits(orc.q8_matmul(x, q, sc)))
        c += q.shape[1]


# ---------------------------------------------------------------------------------------------- kWTA, norms, attention
def test_kwta_keeps_every_unit_at_or_above_the_kth(orc):
    rng = np.random.default_rng(9)
    u = rng.normal(size=1024).astype(np.float32)
    u[10:20] = u[5]  # ties
    for k in (1, 128, 256, 1023, 1024, 2000):
        a = orc.kwta(u, k, False)
        if k >= u.size:
            assert np.array_equal(a, np.maximum(u, 0))
            continue
        kth = np.sort(u)[::-1][k - 1]
        assert orc.kth_largest(u, k) == kth
        keep = u >= kth
        assert keep.sum() >= k
        assert np.array_equal(a != 0, keep & (u > 0))
        assert np.array_equal(a[keep & (u > 0)], u[keep & (u > 0)])
        a2 = orc.kwta(u, k, True)
        assert np.array_equal(a2, a * a)


def test_rmsnorm_and_friends(orc):
    rng = np.random.default_rng(10)
    x = rng.normal(size=384).astype(np.float32)
    g = rng.uniform(0.5, 1.5, 384).astype(np.float32)
    y = orc.rmsnorm(x, g)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-5) * g
    np.testing.assert_allclose(y, want, rtol=2e-6)
    h = orc.l2_heads(x, 64)
    np.testing.assert_allclose((h.reshape(6, 64).astype(np.float64) ** 2).sum(1), 1.0, rtol=1e-5)
    n = orc.head_norm(x, 64)
    np.testing.assert_allclose((n.reshape(6, 64).astype(np.float64) ** 2).mean(1), 1.0, rtol=1e-4)
    assert abs(orc.lib().orc_sigmoid(0.0) - 0.5) < 1e-7
    np.testing.assert_allclose(orc.lib().orc_log_sigmoid(-3.0), -np.log1p(np.exp(3.0)), rtol=1e-6)
    # gemv: the 1-, 2- and many-input forms
    for k in (1, 2, 3, 40):
        xv = rng.normal(size=k).astype(np.float32)
        w = rng.normal(size=(k, 7)).astype(np.float32)
        np.testing.assert_allclose(orc.gemv(xv, w), xv.astype(np.float64) @ w, atol=1e-5)


def test_attend_is_softmax_attention(orc):
    rng = np.random.default_rng(11)
    for n in (1, 2, 9, 70):
        hs = 32
        q = rng.normal(size=hs).astype(np.float32)
        kc = rng.normal(size=(n, hs)).astype(np.float32)
        vc = rng.normal(size=(n, hs)).astype(np.float32)
        sc = 1 / np.sqrt(hs)
        s = kc.astype(np.float64) @ q * sc
        p = np.exp(s - s.max())
        p /= p.sum()
        np.testing.assert_allclose(orc.attend(q, kc, vc, np.float32(sc)), p @ vc, atol=2e-6)


def test_bf16_round(orc):
    assert orc.bf16_round(1.0) == 1.0
    assert orc.bf16_round(1.0 + 2 ** -8) == 1.0            # tie to even
    assert orc.bf16_round(1.0 + 3 * 2 ** -8) == 1.0 + 2 ** -6
    assert orc.bf16_round(-0.30078125) == -0.30078125   # already a bf16 value


# ---------------------------------------------------------------------------------------------- model level identities
@pytest.fixture(scope="module")
def tiny_model(orc):
    cfg = config.tiny(mem_momentum=0.5)
    return cfg, orc.OracleModel(cfg, synth.model(cfg, 0, "awake"))


def test_rows_are_independent_and_stream_equals_batch(orc, tiny_model):
    cfg, m = tiny_model
    ids = synth.token_ids(cfg["vocab"], 3, 24)
    st = m.state(3)
    all_logits = st.forward(ids)
    for r in range(3):
        s1 = m.state(1)
        for t in range(24):
            lg = s1.step(ids[r:r + 1, t])
            assert np.array_equal(bits(lg[0]), bits(all_logits[r, t])), (r, t)
        for name in ("lif.0.v", "lif.2.s", "lif.1.a", "mem.1.f", "mem.2.s", "eng.k", "eng.v"):
            assert np.array_equal(bits(s1.get(0, name)), bits(st.get(r, name))), name
        assert s1.seen(0) == 24


def test_threads_do_not_change_a_step(orc, tiny_model):
    cfg, m = tiny_model
    ids = synth.token_ids(cfg["vocab"], 4, 6)
    outs = []
    try:
        for th in (1, 3, 8):
            orc.set_threads(th)
            outs.append(m.state(4).forward(ids, last_only=True))
    finally:
        orc.set_threads(1)
    assert all(np.array_equal(bits(o), bits(outs[0])) for o in outs)


def test_select_forks_a_state(orc, tiny_model):
    cfg, m = tiny_model
    ids = synth.token_ids(cfg["vocab"], 1, 10)
    st = m.state(1)
    st.forward(ids)
    two = st.select([0, 0])
    a = two.step(np.array([5, 9], np.uint32))
    b = st.select([0]).step(np.array([9], np.uint32))
    assert np.array_equal(bits(a[1]), bits(b[0]))
    assert not np.array_equal(a[0], a[1])


def test_engram_cap_drops_the_oldest(orc):
    cfg = config.tiny(eng_cap=6)
    m = orc.OracleModel(cfg, synth.model(cfg, 0, "awake"))
    free = orc.OracleModel(config.tiny(), synth.model(cfg, 0, "awake"))
    ids = synth.token_ids(cfg["vocab"], 1, 9)
    s_cap, s_free = m.state(1), free.state(1)
    l_cap, l_free = s_cap.forward(ids), s_free.forward(ids)
    enh, hs = cfg["d"] // cfg["eng_head_size"], cfg["eng_head_size"]
    assert s_cap.get(0, "eng.k").size == enh * 6 * hs and s_free.get(0, "eng.k").size == enh * 9 * hs
    assert np.array_equal(bits(l_cap[0, :6]), bits(l_free[0, :6]))
    assert not np.array_equal(l_cap[0, 8], l_free[0, 8])


def test_benchmark_recipe_is_the_stated_corner(orc):
    """alpha = 1, write strength 0.1, erase key = key; spikes stay a few per cent of the channels."""
    cfg = config.make(512, 128, 2, head_size=128, eng_block=1, eng_head_size=64, eng_store_bf16=1)
    m = orc.OracleModel(cfg, synth.model(cfg, 0, "bench"))
    st = m.state(1)
    ids = synth.token_ids(cfg["vocab"], 1, 30)
    orc.trace_enable(True)
    try:
        for t in range(30):
            st.step(ids[:, t])
        assert np.all(orc.trace("ex", 1) == 1.0)
        np.testing.assert_allclose(orc.trace("w", 1), orc.trace("k", 1) * 0.1, rtol=1e-6)
        assert np.array_equal(orc.trace("ek", 1), orc.trace("k", 1))
        k = st.get(0, "eng.k")
        assert np.array_equal(k, np.array([orc.bf16_round(v) for v in k], np.float32))
    finally:
        orc.trace_enable(False)


def _stp_efficacies(orc, U, F, D, spikes, mix=0.0):
    lg = lambda p: np.float32(np.log(p / (1 - p)))
    u, x, effs, outs = np.zeros(1, np.float32), np.ones(1, np.float32), [], []
    for sv in spikes:
        o, u, x, e = orc.stp(np.array([sv], np.float32), [lg(U)], [lg(F)], [lg(D)], [mix], u, x)
        effs.append(float(e[0]))
        outs.append(float(o[0]))
    return effs, outs


def test_stp_depresses_facilitates_and_starts_as_no_change(orc):
    """design-tests/nn/parts/src/stp.rs `depresses_facilitates_and_starts_as_no_change`: with mix 0 the spikes pass
    unchanged; a depressing synapse (U 0.8, no facilitation memory, slow recovery) weakens each spike of a train, the
    first at efficacy 1; a facilitating one (U 0.1, long facilitation, fast recovery) strengthens them past 2 by the
    fifth; with mix 1 the output is the efficacy-weighted spike."""
    rng = np.random.default_rng(4)
    s = (rng.normal(size=9) >= 0.3).astype(np.float32)
    _, outs = _stp_efficacies(orc, 0.2, float(np.exp(-1 / 20)), float(np.exp(-1 / 5)), s, mix=0.0)
    assert np.allclose(outs, s, atol=1e-7)
    e, _ = _stp_efficacies(orc, 0.8, 1e-4, 0.99, [1.0] * 5)
    assert abs(e[0] - 1.0) < 1e-4 and all(b < a for a, b in zip(e, e[1:]))
    e, _ = _stp_efficacies(orc, 0.1, 0.95, 1e-4, [1.0] * 5)
    assert abs(e[0] - 1.0) < 1e-4 and all(b > a for a, b in zip(e, e[1:])) and e[4] > 2.0
    e, outs = _stp_efficacies(orc, 0.1, 0.95, 1e-4, s, mix=1.0)
    assert np.allclose(outs, s * np.array(e, np.float32), atol=1e-6)


def test_stp_signed_multilevel_spikes_stay_bounded(orc):
    """stp.rs `signed_multilevel_spikes_keep_the_rule_bounded`: int2 spikes (-2..2), also a sustained run of -2, keep
    every efficacy finite and at most 1 / U."""
    rng = np.random.default_rng(8)
    rnd = np.clip(np.round(rng.normal(size=600) * 1.5), -2, 2).astype(np.float32)
    for spikes in (rnd, np.full(300, -2.0, np.float32)):
        e, _ = _stp_efficacies(orc, 0.05, 0.99, 0.5, spikes)
        assert np.isfinite(e).all() and np.abs(e).max() <= 1.0 / 0.05 + 1e-3


def test_new_parts_start_as_no_change(orc):
    """The reference initialises the synapse's mix and the dendrites' B to zero and the nucleus's read-out
    and bias too, so that a model with the parts starts as the model without them (nn/parts/src/stp.rs:61, src/v51.rs:399,
    src/v50.rs:20-22), and the relay's gate matrices and biases (src/v51b.rs:282-283): the whole step must then give the
    same bits."""
    from ava_b200 import config, synth
    base = config.tiny(head_size=64)
    full = config.tiny(head_size=64, stp=1, dendrite=1, neuromod=3, thalamus=1, dopamine=1, mood=4, cb_units=512, letters=1, rhythm=1)
    w0 = synth.model(base, 3, "awake")
    w1 = synth.model(full, 3, "awake")
    for k in w1:
        if k.endswith("parts.stp.mix") or k.endswith("v51.dend_b") or k.endswith("v51.da_w") or k.endswith("v51.da_c") or k.endswith("v51.mood_g") \
                or k in ("nm.wn", "nm.bn", "th.gate", "th.bias", "cbh.wo", "v51.letters.wo") or k.endswith("v51.rh_w") or k.endswith("v51.rh_r"):  # nucleus and relay then send 2 sigmoid(0) = 1
            w1[k] = np.zeros_like(w1[k])
    m0, m1 = orc.OracleModel(base, w0), orc.OracleModel(full, w1)
    s0, s1 = m0.state(2), m1.state(2)
    ids = synth.token_ids(base["vocab"], 2, 12)
    for t in range(12):
        a, b = s0.step(ids[:, t]), s1.step(ids[:, t])
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), t
    assert (s1.get(0, "parts.1.stp_x") != 1.0).any()          # the synapse's state moved all the same


def test_relay_gates_follow_their_formula(orc):
    """--thalamus (src/v51b.rs:312-321): block i's gates are 2 sigmoid(tanh(acc / sqrt(i + 1)) G_i + c_i), acc the sum of the
    reads rmsnorm(x_j) R_j of the blocks' input and of the outputs of the blocks before i.  Checked in f64 on the
    oracle's own traces of the stream, and that the gates move the logits."""
    from ava_b200 import config, synth
    cfg = config.tiny(head_size=64, thalamus=1)
    w = synth.model(cfg, 11, "awake")
    m = orc.OracleModel(cfg, w)
    s = m.state(1)
    ids = synth.token_ids(cfg["vocab"], 1, 4)
    orc.trace_enable(True)
    try:
        for t in range(4):
            with_gates = s.step(ids[:, t]).copy()
        d, L = cfg["d"], cfg["n_blocks"]
        xs = [orc.trace("x_in", -1)[:d]] + [orc.trace("x_out", i)[:d] for i in range(L - 1)]
        acc = np.zeros(16)
        for i in range(L):
            x = xs[i].astype(np.float64)
            acc = acc + (x / np.sqrt((x * x).mean() + 1e-5)) @ w["th.read"][i].astype(np.float64)
            z = np.tanh(acc / np.sqrt(i + 1.0)) @ w["th.gate"][i].astype(np.float64) + w["th.bias"][i]
            want = 2.0 / (1.0 + np.exp(-z))
            got = orc.trace("th_g", i)[:2]
            assert np.allclose(got, want, rtol=0, atol=2e-5), (i, got, want)
            assert (np.abs(got - 1.0) > 1e-3).all()
    finally:
        orc.trace_enable(False)
    plain = dict(cfg, thalamus=0)
    s0 = orc.OracleModel(plain, {k: v for k, v in w.items() if not k.startswith("th.")}).state(1)
    for t in range(4):
        without = s0.step(ids[:, t])
    assert np.abs(with_gates - without).max() > 1e-3


def test_surprise_mood_and_dopamine_follow_their_formulas(orc):
    """--dopamine / --mood (src/model/fstep/arch_f3.rs:106-186): the surprise at token t is the cross entropy of the
    head's logits for block 0's normed output at t - 1 (0 at the first token), z = s / ln V, the mood
    m = (z win + bin) sigmoid(-lam) + m sigmoid(lam).  Checked in f64 on the carried tensors token by token."""
    from ava_b200 import config, synth
    cfg = config.tiny(head_size=64, dopamine=1, mood=4)
    w = synth.model(cfg, 5, "awake")
    m = orc.OracleModel(cfg, w)
    s = m.state(1)
    ids = synth.token_ids(cfg["vocab"], 1, 6)
    q, sc = orc.quantize_int8(np.ascontiguousarray(w["tok_emb"].T))
    head = q.astype(np.float64) * sc.astype(np.float64)
    lam, win, b = (w["v51.mood." + k].astype(np.float64) for k in ("lam", "win", "bin"))
    mood = np.zeros(4)
    sig = lambda x: 1.0 / (1.0 + np.exp(-x))
    for t in range(6):
        prev, valid = s.get(0, "v51.prev").astype(np.float64), float(s.get(0, "v51.pvalid")[0])
        assert valid == (0.0 if t == 0 else 1.0)
        s.step(ids[:, t])
        lg = prev @ head
        ce = (np.log(np.exp(lg - lg.max()).sum()) + lg.max() - lg[ids[0, t]]) * valid
        assert abs(float(s.get(0, "v51.last_s")[0]) - ce) < 1e-4, t
        mood = (ce / np.log(cfg["vocab"]) * win + b) * sig(-lam) + mood * sig(lam)
        assert np.allclose(s.get(0, "v51.mood"), mood, rtol=0, atol=1e-5), t
    assert float(s.get(0, "v51.last_s")[0]) > 1.0   # an untrained model is surprised
    # both parts move the logits
    plain = dict(cfg, dopamine=0, mood=0)
    s0 = orc.OracleModel(plain, {k: v for k, v in w.items() if "v51." not in k}).state(1)
    s1 = m.state(1)
    for t in range(3):
        a, b2 = s0.step(ids[:, t]), s1.step(ids[:, t])
    assert np.abs(a - b2).max() > 1e-3


def test_cerebellum_wiring_and_correction(orc):
    """--cerebellum-head: the wiring's properties the reference's own test asks for (src/v51b/tests.rs:94-102: four
    distinct inputs per unit, weights +-1/2), the generator's first draw by hand, and the correction against a numpy
    restatement of src/model/fstep/arch_f3.rs:207-283 (top G/32 units, rectified, unit length, read out)."""
    from ava_b200 import config, synth
    idx, w = orc.cb_wiring(256, 1024)
    assert idx.shape == (1024, 4) and all(len(set(r)) == 4 for r in idx.tolist()) and idx.max() < 256
    assert set(np.unique(w).tolist()) == {-0.5, 0.5}
    s = 0x51B0CE7E | 1                      # xorshift64 (13, 7, 17), by hand
    s ^= (s << 13) & (2**64 - 1); s ^= s >> 7; s ^= (s << 17) & (2**64 - 1)
    assert idx[0, 0] == s % 256
    cfg = config.tiny(head_size=64, cb_units=512)
    wts = synth.model(cfg, 9, "awake")
    st = orc.OracleModel(cfg, wts).state(1)
    ids = synth.token_ids(cfg["vocab"], 1, 3)
    d, g = cfg["d"], 512
    ix, sg = orc.cb_wiring(2 * d, g)
    orc.trace_enable(True)
    try:
        for t in range(3):
            st.step(ids[:, t])
            xf, got = orc.trace("x_final", -1)[:d].astype(np.float64), orc.trace("x_cb", -1)[:d]
            e = wts["tok_emb"][ids[0, t]].astype(np.float64)
            u = np.concatenate([xf, e / np.sqrt((e * e).mean() + 1e-5)])
            h = (u[ix] * sg).sum(1)
            kth = np.sort(h)[-g // 32]
            a = np.maximum(np.where(h >= kth, h, 0.0), 0.0)
            code = a / (np.sqrt((a * a).sum()) + 1e-6)
            assert (code != 0).sum() <= g // 32
            want = xf + code @ wts["cbh.wo"].astype(np.float64)
            assert np.allclose(got, want, rtol=0, atol=2e-5), t
            assert np.abs(got - xf).max() > 1e-3
    finally:
        orc.trace_enable(False)


def test_letters_follow_their_formula(orc):
    """--letters (src/v51.rs:455-469,492-501): a token's input is its embedding plus l Wo with
    l = sum over its first 16 bytes of tanh(byte[b] + end[min(len - 1 - j, 15)] + pos[j]) / sqrt(min(len, 16));
    a token without bytes adds nothing.  Checked in f64 against the oracle's trace of the input."""
    from ava_b200 import config, synth
    cfg = config.tiny(head_size=64, letters=1)
    w = synth.model(cfg, 2, "awake")
    data, off = w["token_bytes"]
    st = orc.OracleModel(cfg, w).state(1)
    E, P, Q, Wo = (w["v51.letters." + k].astype(np.float64) for k in ("byte", "pos", "end", "wo"))
    orc.trace_enable(True)
    try:
        for tok in (0, 3, 7, int(np.argmax(np.diff(off)))):   # token 3 has no bytes; the last is a longest one
            st.step(np.array([tok], np.uint32))
            b = data[off[tok]:off[tok + 1]]
            used = min(len(b), 16)
            l = np.zeros(64)
            for j in range(used):
                l += np.tanh(E[b[j]] + Q[min(len(b) - 1 - j, 15)] + P[j])
            want = w["tok_emb"][tok].astype(np.float64) + (l / np.sqrt(used) if used else l) @ Wo
            got = orc.trace("x_let", -1)[: cfg["d"]]
            assert np.allclose(got, want, rtol=0, atol=1e-5), tok
            assert (np.abs(got - w["tok_emb"][tok]).max() > 1e-4) == (used > 0)
    finally:
        orc.trace_enable(False)


def test_rhythm_clocks_follow_their_formula(orc):
    """--rhythm (src/model/fstep/arch_f4.rs:47-92): each clock's time is (1 - reset) * (1 + time) with reset =
    sigmoid(head_norm(x) wr + br), its phase time * exp(lw), the features cos and sin of the phases.  In f64 on the
    carried times; with the reference's start (reset bias -10) the times count the tokens."""
    from ava_b200 import config, synth
    cfg = config.tiny(head_size=64, rhythm=1)
    w = synth.model(cfg, 4, "awake")
    st = orc.OracleModel(cfg, w).state(1)
    ids = synth.token_ids(cfg["vocab"], 1, 8)
    times = np.zeros(2)
    orc.trace_enable(True)
    try:
        for t in range(8):
            st.step(ids[:, t])
            x = w["tok_emb"][ids[0, t]].astype(np.float64)
            pre = (x / np.sqrt((x * x).mean() + 1e-5)) @ w["v51.rhythm.wr"].astype(np.float64) + w["v51.rhythm.br"]
            times = (1.0 + times) / (1.0 + np.exp(pre))            # 1 - sigmoid(pre) = sigmoid(-pre)
            assert np.allclose(st.get(0, "v51.rh"), times, rtol=2e-5, atol=0), t
            ph = times * np.exp(w["v51.rhythm.lw"].astype(np.float64))
            want = np.array([np.cos(ph[0]), np.sin(ph[0]), np.cos(ph[1]), np.sin(ph[1])])
            assert np.allclose(orc.trace("rh_f", -1)[:4], want, rtol=0, atol=1e-4), t
    finally:
        orc.trace_enable(False)
    quiet = dict(w)
    quiet["v51.rhythm.wr"] = np.zeros_like(w["v51.rhythm.wr"])
    quiet["v51.rhythm.br"] = np.full(2, -10.0, np.float32)
    s2 = orc.OracleModel(cfg, quiet).state(1)
    for t in range(8):
        s2.step(ids[:, t])
    assert np.allclose(s2.get(0, "v51.rh"), [8.0, 8.0], atol=2e-3)


def test_shared_sine_and_cosine_are_correctly_rounded():
    """The library's sine and cosine (double arithmetic, one rounding to float) against numpy's double results rounded to
    float, over the range the phases take."""
    from ava_b200 import engine
    L = engine.lib()
    rng = np.random.default_rng(0)
    for scale in (1.0, 100.0, 1e4, 1e6):
        for x in (rng.uniform(-scale, scale, 2000).astype(np.float32)):
            assert L.ava_host_sinf(float(x)) == float(np.float32(np.sin(np.float64(x))))
            assert L.ava_host_cosf(float(x)) == float(np.float32(np.cos(np.float64(x))))
    assert L.ava_host_sinf(0.0) == 0.0 and L.ava_host_cosf(0.0) == 1.0 and np.isnan(L.ava_host_sinf(float("inf")))
