"""Checkpoints through the library's loader into the engine, against the oracle fed the same f32 tensors
(design-tests/nn/gpu/src/ckpt.rs:51-76 `load_auto`, src/model.rs:949-991 `set_int8`): the quantiser runs on both sides,
so every logit and the whole state must again be the same bits.

One test takes a released checkpoint of the reference when the environment names one (AVA_M_CKPT: the file
release/ava-m/model.safetensors of the reference project, kind S); it is skipped otherwise."""
import os

import numpy as np
import pytest

from ava_b200 import build, ckpt, config, engine, synth

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


def run_both(orc, gm, om, cfg, rows, T, names):
    ids = synth.token_ids(cfg["vocab"], rows, T, seed0=5)
    gs, os_ = gm.state(rows, T + 4), om.state(rows)
    for t in range(T):
        lg, lo = gm.step(gs, ids[:, t]), os_.step(ids[:, t])
        assert np.array_equal(bits(lg), bits(lo)), (t, float(np.abs(lg - lo).max()))
    for r in range(rows):
        for name in names:
            assert np.array_equal(bits(gs.get(r, name)), bits(os_.get(r, name))), (r, name)
    return gs


NINE_PARTS = dict(stp=1, neuromod=3, dendrite=1, dopamine=1, mood=4, thalamus=1, cb_units=512, letters=1, rhythm=1)


@pytest.mark.parametrize("kind", ["S", "D", "D with the nine Ava-0.4 parts"])
def test_synthetic_checkpoint_runs_to_the_oracles_bits(orc_same_math, tmp_path, kind):
    orc = orc_same_math
    parts = kind.startswith("D with")
    kind = kind[0]
    cfg = config.kind_s(320, 128, 3) if kind == "S" else config.tiny(mem_momentum=0.5, head_size=64, **(NINE_PARTS if parts else {}))
    weights = synth.model(cfg, 2, "awake")
    path = ckpt.save(str(tmp_path), cfg, weights)
    flags = ckpt.flags_of(cfg)
    if parts:   # the model file has the parts' tensors under the reference's names; the spellings come from the tokenizer
        assert all(w in flags for w in ("--stp", "--neuromod 3", "--dendrite", "--letters", "--dopamine", "--mood", "--rhythm", "--thalamus",
                                        "--cerebellum-head 512"))
    gm = engine.Model.from_checkpoint(path, kind, flags, token_bytes=weights.get("token_bytes"))
    for k in NINE_PARTS:
        assert gm.cfg[k] == cfg[k], k
    for k in ("d", "n_blocks", "hidden", "kwta_k", "head_size", "eng_block", "spikes", "alif", "theta", "fast_mem"):
        assert gm.cfg[k] == cfg[k], k
    ck = engine.Checkpoint(path)
    ow = {n: ck.get(n) for n in ck.names()}
    if parts:
        ow["token_bytes"] = weights["token_bytes"]
    om = orc.OracleModel(gm.cfg, ow)
    names = [f"lif.{i}.{k}" for i in range(cfg["n_blocks"]) for k in ("v", "s")]
    if kind == "D":
        names += ["mem.0.f", "mem.2.s", "eng.k"]
    if parts:
        names += ["parts.1.stp_x", "v51.prev", "v51.last_s", "v51.mood", "v51.rh"]
    gs = run_both(orc, gm, om, gm.cfg, rows=3, T=40, names=names)
    assert (gs.get(0, "lif.1.s") != 0).any()


def test_released_kind_s_checkpoint(orc_same_math):
    path = os.environ.get("AVA_M_CKPT", "")
    if not os.path.isfile(path):
        pytest.skip("AVA_M_CKPT does not name the reference's release/ava-m/model.safetensors")
    orc = orc_same_math
    gm = engine.Model.from_checkpoint(path, "S")
    assert (gm.cfg["d"], gm.cfg["n_blocks"], gm.cfg["vocab"], gm.cfg["hidden"], gm.cfg["kwta_k"]) == (384, 8, 4096, 1536, 192)
    ck = engine.Checkpoint(path)
    om = orc.OracleModel(gm.cfg, {n: ck.get(n) for n in ck.names()})
    orc.set_threads(8)
    try:
        gs = run_both(orc, gm, om, gm.cfg, rows=4, T=96, names=[f"lif.{i}.{k}" for i in range(8) for k in ("v", "s")])
    finally:
        orc.set_threads(1)
    share = float(np.mean([(gs.get(r, f"lif.{i}.s") != 0).mean() for r in range(4) for i in range(8)]))
    print("released kind-S checkpoint: spike share after 96 uniform tokens", share)
    assert 0.01 < share < 0.5
    # chunked prompt reading gives the stepped bits on real weights too
    ids = synth.token_ids(gm.cfg["vocab"], 4, 96, seed0=5)
    st = gm.state(4, 100)
    lg = gm.forward_with_state(ids, st, last_only=True)
    assert np.array_equal(bits(st.get(2, "lif.7.v")), bits(gs.get(2, "lif.7.v")))
    assert lg.shape == (4, gm.cfg["vocab"])
