"""The checkpoint loader (host side of the library: no GPU): safetensors header and data, configuration detection as
design-tests/nn/gpu/src/ckpt.rs:21-47 does it, the arch.txt flag words of design-tests/nn/gpu/src/arch.rs:273-420."""
import os
import struct

import numpy as np
import pytest

from ava_b200 import build, ckpt, config, engine, synth

AVA04_FLAGS = ("--head-size 64 --timescales fixed --gates channel --value-residual --kwta 1/4 --mlp-act relu2 --mem-momentum 0.5 "
               "--resid-fix --residual dense --lif-init logspaced --lif-scale --spikes int2 --alif --lif-reset-grad --homeostasis 0.1")


@pytest.fixture(scope="module", autouse=True)
def _lib():
    build.build()


def test_round_trip_of_a_synthetic_checkpoint(tmp_path):
    cfg = config.tiny(mem_momentum=0.5, head_size=64)
    w = synth.model(cfg, 3, "awake")
    path = ckpt.save(str(tmp_path), cfg, w)
    ck = engine.Checkpoint(path)
    want = ckpt.dequantised(w)
    assert sorted(ck.names()) == sorted(want)
    for i in range(len(ck)):
        name, dt, shape = ck.info(i)
        assert dt == "F32" and shape == want[name].shape
        assert np.array_equal(ck.get(name).view(np.uint32), want[name].view(np.uint32)), name
    flags = open(os.path.join(tmp_path, "arch.txt")).read().strip()
    got = ck.config("D", flags)
    for k in config.FIELDS_I32 + config.FIELDS_F32:
        if k not in ("eng_store_bf16", "eng_cap", "slope"):          # not in a file: the caller's choice
            assert got[k] == pytest.approx(cfg[k]), k
    ck.close()


def test_kind_s_is_detected_from_names():
    cfg = config.kind_s(320, 128, 3)
    w = synth.model(cfg, 0, "awake")
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        ck = engine.Checkpoint(ckpt.save(d, cfg, w))
        got = ck.config("S")
        assert got == {**cfg, "slope": got["slope"]}
        with pytest.raises(engine.NotApplicable):
            ck.config("S", "--alif")                 # block options are for model D
        with pytest.raises(engine.NotApplicable):
            ck.config("D")                           # per-head gates: not covered
        with pytest.raises(engine.NotApplicable):
            ck.config("A")


def test_arch_flag_words():
    base = config.make(4112, 384, 8, head_size=32, spikes=0, alif=0, theta=0, lif_scale=0, value_residual=0, relu2=0, dense=0, out_gate=1)
    got = engine.arch_flags(AVA04_FLAGS, base)
    assert (got["head_size"], got["value_residual"], got["kwta_k"], got["relu2"], got["dense"], got["lif_scale"], got["spikes"], got["alif"],
            got["theta"]) == (64, 1, 384, 1, 1, 1, 2, 1, 1)
    assert got["mem_momentum"] == 0.5
    # the released Ava 0.4 adds nine parts the engine does not have: the first of them is named
    assert engine.arch_flags(AVA04_FLAGS + " --stp", base)["stp"] == 1
    got = engine.arch_flags(AVA04_FLAGS + " --stp --dendrite", base)
    assert (got["stp"], got["dendrite"]) == (1, 1)
    got = engine.arch_flags(AVA04_FLAGS + " --stp --neuromod 3 --dendrite", base)
    assert (got["stp"], got["neuromod"], got["dendrite"]) == (1, 3, 1)
    got = engine.arch_flags(AVA04_FLAGS + " --stp --neuromod 3 --dendrite --thalamus --dopamine --mood", base)
    assert (got["neuromod"], got["thalamus"], got["dopamine"], got["mood"]) == (3, 1, 1, 4)
    assert engine.arch_flags(AVA04_FLAGS + " --mood-units 2", base)["mood"] == 2
    assert engine.arch_flags(AVA04_FLAGS + " --cerebellum-head 12288", base)["cb_units"] == 12288
    with pytest.raises(engine.EngineError, match="multiple of 32"):
        engine.arch_flags(AVA04_FLAGS + " --cerebellum-head 100", base)
    assert engine.arch_flags(AVA04_FLAGS + " --letters", base)["letters"] == 1
    # the released Ava 0.4 line (release/ava-0.4/arch.txt) is covered whole; a part the engine lacks is still named
    got = engine.arch_flags(AVA04_FLAGS + " --stp --neuromod 3 --dendrite --letters --dopamine --mood --rhythm --thalamus --cerebellum-head 12288", base)
    assert all(got[k] for k in ("stp", "neuromod", "dendrite", "letters", "dopamine", "mood", "rhythm", "thalamus", "cb_units"))
    with pytest.raises(engine.NotApplicable, match="--columns"):
        engine.arch_flags(AVA04_FLAGS + " --stp --columns 4", base)
    with pytest.raises(engine.NotApplicable, match="gates"):
        engine.arch_flags("--head-size 64", base)
    with pytest.raises(engine.NotApplicable, match="sigmoid"):
        engine.arch_flags("--gates channel --gate sigmoid", base)
    with pytest.raises(engine.EngineError, match="not a block flag"):
        engine.arch_flags("--gates channel banana", base)
    with pytest.raises(engine.EngineError, match="1/n"):
        engine.arch_flags("--gates channel --kwta 0.3", base)
    assert engine.arch_flags("--gates channel --kwta 0.125", base)["kwta_k"] == base["hidden"] // 8


def test_f16_and_bf16_tensors_widen_exactly(tmp_path):
    a = np.array([0.0, -0.0, 1.0, -2.5, 6.1e-5, 5.96e-8, 65504.0, np.inf], np.float16)
    b = np.array([1.0, -3.140625, 1e-30, 3.3895314e38], np.float32)
    b16 = (b.view(np.uint32) >> 16).astype(np.uint16)
    path = str(tmp_path / "x.safetensors")
    raw_a, raw_b = a.tobytes(), b16.tobytes()
    header = ('{"h":{"dtype":"F16","shape":[%d],"data_offsets":[0,%d]},"__metadata__":{"format":"pt","note":"a \\"quoted\\" word"},'
              '"b":{"dtype":"BF16","shape":[2,2],"data_offsets":[%d,%d]}}' % (a.size, len(raw_a), len(raw_a), len(raw_a) + len(raw_b))).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + raw_a + raw_b)
    ck = engine.Checkpoint(path)
    assert np.array_equal(ck.get("h").view(np.uint32), a.astype(np.float32).view(np.uint32))
    assert np.array_equal(ck.get("b").view(np.uint32).ravel(), (b16.astype(np.uint32) << 16))
    assert ck.info(1)[2] == (2, 2) or ck.info(0)[2] == (2, 2)


@pytest.mark.parametrize("damage", ["short", "header_len", "offsets", "dtype", "json", "twice", "shape_wraps", "begin_after_end"])
def test_damaged_files_are_refused(tmp_path, damage):
    path = str(tmp_path / "bad.safetensors")
    good = '{"t":{"dtype":"F32","shape":[2],"data_offsets":[0,8]}}'
    data = b"\0" * 8
    if damage == "short":
        blob = b"\1\2\3"
    elif damage == "header_len":
        blob = struct.pack("<Q", 10_000) + good.encode() + data
    elif damage == "offsets":
        blob = struct.pack("<Q", len(good)) + good.replace("[0,8]", "[0,12]").encode() + data
    elif damage == "dtype":
        h = good.replace("F32", "I64")
        blob = struct.pack("<Q", len(h)) + h.encode() + data
    elif damage == "json":
        h = good[:-3]
        blob = struct.pack("<Q", len(h)) + h.encode() + data
    elif damage == "shape_wraps":
        # 2^31 x 2^31 x 4 elements of 4 bytes: the byte count wraps to 0 in 64 bits, so a naive product matches [0,0]
        h = good.replace("[2]", "[2147483648,2147483648,4]").replace("[0,8]", "[0,0]")
        blob = struct.pack("<Q", len(h)) + h.encode() + data
    elif damage == "begin_after_end":
        h = good.replace("[0,8]", "[8,0]")
        blob = struct.pack("<Q", len(h)) + h.encode() + data
    else:
        h = '{"t":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"t":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
        blob = struct.pack("<Q", len(h)) + h.encode() + data
    open(path, "wb").write(blob)
    with pytest.raises((engine.EngineError, engine.NotApplicable)):
        engine.Checkpoint(path)
    with pytest.raises(engine.EngineError):
        engine.Checkpoint(str(tmp_path / "absent.safetensors"))


# the reference project, when it is mounted beside this repository (or where AVA_REFERENCE_DIR says)
REF_AVA_M = os.path.join(os.environ.get("AVA_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "..", "reference")),
                         "release", "ava-m")


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF_AVA_M, "model.safetensors")), reason="the reference's released Ava-M is not on this machine")
def test_released_ava_m_scores_text_like_its_model_card(orc):
    """The released kind-S checkpoint through the loader, the quantiser and the oracle's step: English text must score
    near the card's validation loss (3.98 nats per token on its own held-out text; ln 4096 = 8.32 for a model that
    knows nothing).  This pins loader + kind-S step + quantiser on real trained weights as far as can be done without
    the reference's binary."""
    ck = engine.Checkpoint(os.path.join(REF_AVA_M, "model.safetensors"))
    cfg = ck.config("S")
    assert (cfg["d"], cfg["n_blocks"], cfg["vocab"], cfg["hidden"], cfg["kwta_k"]) == (384, 8, 4096, 1536, 192)
    # byte-level BPE of the release ("ava-bpe v1": 256 bytes, EOS, PAD, then one merge per line), greedy by merge rank
    lines = open(os.path.join(REF_AVA_M, "bpe.txt")).read().split("\n")
    rank = {tuple(map(int, l.split())): i for i, l in enumerate(x for x in lines[1:] if x.strip())}

    def encode(text):
        out = []
        for word in __import__("re").findall(r" ?[^ ]+| +", text):
            t = list(word.encode())
            while len(t) > 1:
                best = min(((rank.get((t[i], t[i + 1]), 1 << 30), i) for i in range(len(t) - 1)))
                if best[0] == 1 << 30:
                    break
                t[best[1]:best[1] + 2] = [258 + best[0]]
            out += t
        return out

    ids = encode("The weather was fine in the morning, so the children went out to play in the garden behind the house. "
                 "After a while their mother called them in for lunch, and they sat down at the table and talked about what they had seen.")
    om = orc.OracleModel(cfg, {n: ck.get(n) for n in ck.names()})
    st = om.state(1)
    nll = []
    for a, b in zip(ids[:-1], ids[1:]):
        lg = st.step(np.array([a], np.uint32))[0].astype(np.float64)
        lp = lg - lg.max()
        nll.append(-(lp[b] - np.log(np.exp(lp).sum())))
    assert np.mean(nll) < 5.0, np.mean(nll)      # measured 4.24
