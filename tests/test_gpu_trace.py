"""`Model::step_trace` (design-tests/nn/gpu/src/model/fstep/arch.rs:420-476) through the library: the traced step gives the
plain step's logits and state bit for bit (the reference's own check, src/model/fstep/trace_tests.rs), its copies are
the oracle's intermediates bit for bit, and its sizes follow their formulas."""
import numpy as np
import pytest

from ava_b200 import build, config, engine, synth

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("kw", [dict(head_size=64), dict(head_size=32, stp=1, dendrite=1, neuromod=3, rhythm=1, mem_momentum=0.5),
                                dict(head_size=128, eng_block=-1, spikes=0, alif=0, theta=0, lif_scale=0, value_residual=0, relu2=0, dense=0, out_gate=0,
                                     fast_mem=0)])
def test_traced_token(orc, kw):
    build.build()
    orc.set_math(*engine.host_math())
    try:
        cfg = config.tiny(**kw)
        w = synth.model(cfg, 6, "awake")
        gm, om = engine.Model(cfg, w), orc.OracleModel(cfg, w)
        plain, traced, os_ = gm.state(1, 64), gm.state(1, 64), om.state(1)
        ids = synth.token_ids(cfg["vocab"], 1, 10, seed0=4)
        d, L, hs = cfg["d"], cfg["n_blocks"], cfg["head_size"]
        nh = d // hs
        orc.trace_enable(True)
        for t in range(10):
            f_before = [os_.get(0, f"mem.{i}.f").astype(np.float64) for i in range(L)] if cfg["fast_mem"] else None
            want_logits = gm.step(plain, ids[:, t])[0]
            logits, rec = gm.step_trace(traced, int(ids[0, t]))
            os_.step(ids[:, t])
            assert np.array_equal(bits(logits), bits(want_logits)), t
            x_in = orc.trace("x_in", -1)[:d].astype(np.float64)
            assert abs(float(rec[("input_rms", -1)][0]) - np.sqrt((x_in * x_in).mean())) < 1e-6
            for i in range(L):
                assert np.array_equal(bits(rec[("spikes", i)]), bits(orc.trace("stp_out" if cfg["stp"] else "spikes", i)[:d])), (t, i)
                hidden = orc.trace("a_dend" if cfg["dendrite"] and cfg["fast_mem"] else "a", i)
                # equal as numbers: a unit the k-WTA drops is max(u * 0, 0), whose sign of zero the reference leaves to the platform
                assert np.array_equal(rec[("hidden", i)], hidden) and not np.isnan(hidden).any(), (t, i)
                u = orc.trace("u", i)
                kth = np.sort(u)[-cfg["kwta_k"]]
                assert np.array_equal(rec[("winners", i)], (u >= kth).astype(np.float32)), (t, i)
                assert rec[("winners", i)].sum() >= cfg["kwta_k"]
                if cfg["fast_mem"]:
                    ex, be, yraw = (orc.trace(n, i)[:d].astype(np.float64) for n in ("ex", "be", "y_raw"))
                    f1 = os_.get(0, f"mem.{i}.f").astype(np.float64).reshape(nh, hs, hs)
                    f0 = f_before[i].reshape(nh, hs, hs)
                    wr = np.sqrt(((f1 - f0 * ex.reshape(nh, hs, 1)) ** 2).sum((1, 2)))
                    assert np.allclose(rec[("mem_write", i)], wr, rtol=2e-5, atol=1e-7), (t, i)
                    assert np.allclose(rec[("mem_read", i)], np.sqrt((yraw.reshape(nh, hs) ** 2).sum(1)), rtol=2e-6, atol=1e-9)
                    assert np.allclose(rec[("mem_keep", i)], ex.reshape(nh, hs).mean(1), rtol=2e-6)
                    assert np.allclose(rec[("mem_gate", i)], be.reshape(nh, hs).mean(1), rtol=2e-6)
                else:
                    assert ("mem_write", i) not in rec
                if i == cfg["eng_block"]:
                    ehs = cfg["eng_head_size"]
                    enh, n = d // ehs, t + 1
                    attn = rec[("engram_attn", i)].reshape(enh, n).astype(np.float64)
                    kk = os_.get(0, "eng.k").astype(np.float64).reshape(enh, n, ehs)
                    q = orc.trace("eng_qkv", i)[:d].astype(np.float64).reshape(enh, ehs)
                    sc = np.einsum("hnc,hc->hn", kk, q) / np.sqrt(ehs)
                    p = np.exp(sc - sc.max(1, keepdims=True))
                    assert np.allclose(attn, p / p.sum(1, keepdims=True), rtol=0, atol=2e-6), t
                    assert np.array_equal(bits(rec[("engram_read", i)]), bits(orc.trace("eng_r", i)[:d])), t
        # the traced state went the plain state's way
        for name in [f"lif.{i}.v" for i in range(L)] + ([f"mem.{L - 1}.f"] if cfg["fast_mem"] else []) + (["eng.k"] if cfg["eng_block"] >= 0 else []):
            assert np.array_equal(bits(traced.get(0, name)), bits(plain.get(0, name))), name
    finally:
        orc.trace_enable(False)
        orc.reset_math()


def test_trace_wants_one_row_and_an_uncapped_store():
    build.build()
    cfg = config.tiny(head_size=64)
    m = engine.Model(cfg, synth.model(cfg, 1, "awake"))
    with pytest.raises(engine.EngineError):
        m.step_trace(m.state(2, 16), 1)
    capped = config.tiny(head_size=64, eng_cap=4)
    m2 = engine.Model(capped, synth.model(capped, 1, "awake"))
    with pytest.raises(engine.NotApplicable):
        m2.step_trace(m2.state(1, 16), 1)
