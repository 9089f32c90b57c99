"""The engram store of one long sequence split by position over several ranks (benchmark configuration 4), checked on
ONE GPU: two ranks are two engines in this process on the same device, and the two collectives (broadcast of q,k,v,
all-gather of the partial softmax statistics) are plain copies between their buffers.  The kernels of the two ranks run
one after another, never waiting on each other.  The real NCCL run on 2+ GPUs is tests/multi_gpu_split_kv.py."""
import numpy as np
import pytest

from ava_b200 import build, config, engine, longctx, shard, synth

pytestmark = pytest.mark.gpu


def test_kv_owner_rule():
    assert [shard.kv_owner(p, 4, 3) for p in range(14)] == [0, 0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2, 2, 2]


NINE_PARTS = dict(stp=1, neuromod=3, dendrite=1, dopamine=1, mood=4, thalamus=1, cb_units=512, letters=1, rhythm=1)


@pytest.mark.parametrize("world,parts", [(1, False), (2, False), (3, False), (2, True)])
def test_split_store_decode_matches_the_oracle(orc, world, parts):
    import torch
    build.build()
    orc.set_math(*engine.host_math())
    try:
        cfg = config.tiny(eng_head_size=64, eng_store_bf16=1, **(NINE_PARTS if parts else {}))
        carried = [f"lif.{i}.{k}" for i in range(cfg["n_blocks"]) for k in "vsa"] + [f"mem.{i}.f" for i in range(cfg["n_blocks"])]
        if parts:   # the step is cut in two at the engram: what the parts carry must survive the cut as well
            carried += [f"parts.{i}.{k}" for i in range(cfg["n_blocks"]) for k in ("stp_u", "stp_x")]
            carried += ["v51.prev", "v51.pvalid", "v51.last_s", "v51.mood", "v51.rh"]
        w = synth.model(cfg, 0, "awake")
        om = orc.OracleModel(cfg, w)
        prompt_len, decode = 37, 12
        ids = synth.token_ids(cfg["vocab"], 1, prompt_len + decode, seed0=3)
        # the prompt is read on rank 0 with the whole store; then the store is dealt out by position
        ranks = [longctx.SplitKV(engine.Model(cfg, w), 1, 64, r, world, dist=None, seg_len=8) for r in range(world)]
        full = ranks[0].m.state(1, 64)
        ranks[0].m.forward_with_state(ids[:, :prompt_len], full, last_only=True)
        os_ = om.state(1)
        os_.forward(ids[:, :prompt_len], last_only=True)
        heads, hs = cfg["d"] // cfg["eng_head_size"], cfg["eng_head_size"]
        k_full = full.get(0, "eng.k").reshape(heads, prompt_len, hs)
        v_full = full.get(0, "eng.v").reshape(heads, prompt_len, hs)
        block = -(-prompt_len // world)
        for sk in ranks:
            sk.take_prompt_store(k_full, v_full, prompt_len, block)
        # rank 0 continues from the prompt's membranes and fast weights
        for name in carried:
            ranks[0].state.put(0, name, full.get(0, name))
        dev = torch.device("cuda", 0)
        logits = torch.empty(1, cfg["vocab"], dtype=torch.float32, device=dev)
        for t in range(decode):
            tok = torch.tensor([int(ids[0, prompt_len + t])], dtype=torch.int32, device=dev)
            torch.cuda.synchronize()
            ranks[0].begin(tok.data_ptr())
            ranks[0].m.sync()
            for sk in ranks[1:]:
                sk.qkv.copy_(ranks[0].qkv)               # the broadcast
            torch.cuda.synchronize()
            for sk in ranks:
                sk.partial_read()
                sk.m.sync()
            ranks[0].gathered.copy_(torch.stack([sk.partial for sk in ranks]))   # the all-gather
            torch.cuda.synchronize()
            ranks[0].end(logits.data_ptr(), None)
            ranks[0].m.sync()
            want = os_.step(ids[:, prompt_len + t])
            got = logits.cpu().numpy()
            np.testing.assert_allclose(got, want, rtol=0, atol=1e-4 * max(1.0, float(np.abs(want).max())), err_msg=f"token {t}")
            # keep both on one trajectory: rounding differences may flip a spike later on
            for name in carried:
                ranks[0].state.put(0, name, os_.get(0, name))
        # every position is on exactly one rank, the decoded ones on the last
        counts = [sk.state.get(0, "eng.k").size // cfg["d"] for sk in ranks]
        assert sum(counts) == prompt_len + decode
        assert counts[-1] >= decode
    finally:
        orc.reset_math()


def test_split_step_as_one_call_with_its_own_communicator():
    """ava_split_step on one rank: NCCL loaded by the library (dlopen), a communicator of one rank made through the C
    ABI, the token stepped as one call; the logits are the bits of the three-call form on a twin state (with one rank
    the all-gather is a copy either way), and the communicator's broadcast and all-gather ran on the engine's stream.  Each token is
    waited for with ava_split_wait (the bounded wait that asks NCCL for its asynchronous error)."""
    import ctypes as C
    import torch
    build.build()
    ver = C.c_int32(0)
    if engine.lib().ava_nccl_version(C.byref(ver)) != 0:
        pytest.skip("no NCCL library to load")
    cfg = config.tiny(eng_head_size=64, eng_store_bf16=1)
    w = synth.model(cfg, 0, "awake")
    ids = synth.token_ids(cfg["vocab"], 1, 24, seed0=5)
    dev = torch.device("cuda", 0)
    outs = []
    for one_call in (False, True):
        sk = longctx.SplitKV(engine.Model(cfg, w), 1, 64, 0, 1, dist=None, seg_len=8)
        engine.lib().ava_state_set_kv_shard(sk.state.h, 0, 1, 64, 0)
        if one_call:
            sk.make_comm()
        logits = torch.empty(1, cfg["vocab"], dtype=torch.float32, device=dev)
        got = []
        for t in range(24):
            tok = torch.tensor([int(ids[0, t])], dtype=torch.int32, device=dev)
            torch.cuda.synchronize()
            if one_call:
                sk.step_c(tok.data_ptr(), logits.data_ptr(), None)
            else:
                sk.begin(tok.data_ptr())
                sk.partial_read()
                sk.m.sync()
                sk.gathered.copy_(sk.partial.unsqueeze(0))
                torch.cuda.synchronize()
                sk.end(logits.data_ptr(), None)
            if one_call:
                sk.wait(20000)  # the bounded wait: stream drained, no asynchronous NCCL error, communicator kept
                assert sk.comm is not None
            sk.m.sync()
            got.append(logits.cpu().numpy().copy())
        if one_call:
            sk.close_comm()
        outs.append(np.stack(got))
    assert ver.value >= 20000
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
