"""`State::save` / `State::load` (design-tests/nn/gpu/src/state.rs:1114-1329) through the library: the file carries the
reference's tensor names and shapes, a loaded state continues bit for bit, and a file of another model is refused
(the reference's own tests: src/state/tests.rs, save -> load -> same logits)."""
import numpy as np
import pytest

from ava_b200 import build, config, engine, synth

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.fixture(scope="module", autouse=True)
def _lib():
    build.build()
    engine.lib()


@pytest.mark.parametrize("name,kw", [("ava04_small", dict()), ("momentum_bf16", dict(mem_momentum=0.5, head_size=64, eng_store_bf16=1)),
                                     ("capped", dict(eng_cap=6)), ("stp", dict(stp=1)), ("kind_s", None),
                                     ("nine_parts", dict(stp=1, neuromod=3, dendrite=1, dopamine=1, mood=4, thalamus=1, cb_units=512, letters=1,
                                                         rhythm=1, head_size=64, mem_momentum=0.5))])
def test_saved_state_continues_bit_for_bit(tmp_path, name, kw):
    cfg = config.kind_s(320, 128, 3) if kw is None else config.tiny(**kw)
    m = engine.Model(cfg, synth.model(cfg, 1, "awake"))
    rows, d, L = 3, cfg["d"], cfg["n_blocks"]
    # rows of different lengths: one state per length, joined
    lens = [9, 4, 9]
    ids = synth.token_ids(cfg["vocab"], rows, 30, seed0=3)
    parts = []
    for r, n in enumerate(lens):
        st = m.state(1, 64)
        m.forward_with_state(ids[r:r + 1, :n], st, last_only=True)
        parts.append(st)
    st = engine.State.cat(parts)
    path = str(tmp_path / "conv.safetensors")
    st.save(path)

    ck = engine.Checkpoint(path)
    names = set(ck.names())
    assert {"meta.seen", "meta.model", "meta.blocks", "meta.cap", "meta.hist", "meta.hist_len", "lif.0.v", f"lif.{L - 1}.s"} <= names
    assert ck.get("meta.seen").tolist() == lens and ck.get("meta.blocks").tolist() == [L]
    assert ck.get("meta.cap").tolist() == [cfg["eng_cap"], 0]
    fp = ck.get("meta.model")
    assert (int(fp[0]) << 32 | int(fp[1])) == m.fingerprint
    assert ck.get("lif.1.v").shape == (rows, d) and ck.get("meta.hist").shape == (rows, 17)
    if cfg["stp"]:
        assert ck.get("parts.0.stp_u").shape == (rows, d) and (ck.get("parts.1.stp_x") != 1.0).any()
    if cfg["mood"]:   # the reference's names and shapes for what the surprise, the mood and the clocks carry (src/v51.rs:1012)
        assert ck.get("v51.prev").shape == (rows, d) and ck.get("v51.pvalid").tolist() == [1.0] * rows and ck.get("v51.last_s").shape == (rows,)
        assert ck.get("v51.mood").shape == (rows, cfg["mood"]) and ck.get("v51.rh").shape == (rows, 2) and (ck.get("v51.rh") > 0).all()
    if cfg["fast_mem"]:
        hs = cfg["head_size"]
        assert ck.get("mem.0.f").shape == (rows * d // hs, hs, hs)
        assert ("mem.0.s" in names) == (cfg["mem_momentum"] > 0)
    if cfg["eng_block"] >= 0:
        ehs = cfg["eng_head_size"]
        held = [min(n, cfg["eng_cap"]) if cfg["eng_cap"] else n for n in lens]
        S = max(held)
        k = ck.get("eng.k")
        assert k.shape == (rows, d // ehs, S, ehs) and ck.get("eng.valid").tolist() == held
        pad = ck.get("eng.pad")
        assert pad.shape == (rows, S) and (pad[1, :S - held[1]] == np.float32(-1e9)).all() and not pad[0].any() and not pad[1, S - held[1]:].any()
        assert not k[1, :, :S - held[1]].any()                           # shorter rows are padded on the left
        assert np.array_equal(bits(k[1, :, S - held[1]:].reshape(d // ehs, held[1], ehs)), bits(st.get(1, "eng.k").reshape(d // ehs, held[1], ehs)))
    else:
        assert "eng.k" not in names

    back = m.load_state(path, 64)
    assert [back.seen(r) for r in range(rows)] == lens
    for t in range(9, 16):
        a = m.step(st, ids[:, t])
        b = m.step(back, ids[:, t])
        assert np.array_equal(bits(a), bits(b)), t

    # another model (other weights) refuses the file; so does a model with another cap
    other = engine.Model(cfg, synth.model(cfg, 2, "awake"))
    assert other.fingerprint != m.fingerprint
    with pytest.raises(engine.EngineError):
        other.load_state(path, 64)
    with pytest.raises(engine.EngineError):
        m.load_state(str(tmp_path / "absent.safetensors"), 64)


def test_fresh_state_has_no_store_in_the_file(tmp_path):
    cfg = config.tiny()
    m = engine.Model(cfg, synth.model(cfg, 1, "awake"))
    st = m.state(2, 16)
    path = str(tmp_path / "fresh.safetensors")
    st.save(path)
    assert "eng.k" not in engine.Checkpoint(path).names()
    back = m.load_state(path, 16)
    tok = np.array([3, 4], np.uint32)
    assert np.array_equal(bits(m.step(st, tok)), bits(m.step(back, tok)))


def test_conversation_store(tmp_path):
    cfg = config.kind_s(320, 128, 2)
    m = engine.Model(cfg, synth.model(cfg, 1, "awake"))
    other = engine.Model(cfg, synth.model(cfg, 2, "awake"))
    store = engine.ConvStore(str(tmp_path / "conversations"))
    assert store.path("anna-2") == str(tmp_path / "conversations" / "state-anna-2.safetensors")
    odd = store.path("who is there?")
    assert odd.endswith(".safetensors") and "state-h" in odd and len(odd.split("state-h")[1]) == 16 + len(".safetensors")
    assert store.load("anna-2", m) == ("fresh", None)
    st = m.state(1, 32)
    m.step(st, np.array([7], np.uint32))
    store.save("anna-2", st)
    store.save("who is there?", st)
    kind, back = store.load("anna-2", m, 32)
    assert kind == "resumed" and back.seen(0) == 1
    tok = np.array([9], np.uint32)
    assert np.array_equal(bits(m.step(st, tok)), bits(m.step(back, tok)))
    assert store.load("anna-2", other) == ("stale", None)
    assert store.load("who is there?", m, 32)[0] == "resumed"
