"""The batched generation loop of the library (`ava_generate`) against the same thing done by hand with the step calls,
as design-tests/nn/gpu/src/state.rs:1388-1458 defines it: prompts of different lengths, groups smaller than the
batch, rows leaving at EOS or at the caller's stop rule, greedy on the device and sampled through a callback.  Rows are
independent and every step is bit-exact, so the tokens must be identical, not just close."""
import numpy as np
import pytest

from ava_b200 import build, config, engine, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib():
    build.build()
    engine.lib()


@pytest.fixture(scope="module")
def model():
    cfg = config.tiny()
    return engine.Model(cfg, synth.model(cfg, 4, "awake"))


def by_hand(model, prompt, max_new, eos, choose, stop=None):
    """One prompt alone: read it, then step token by token."""
    st = model.state(1, len(prompt) + max_new + 2)
    lg = model.forward_with_state(np.asarray([prompt], np.uint32), st, last_only=True)[0]
    out = []
    for step in range(max_new):
        tok = choose(lg)
        if tok == eos:
            break
        out.append(tok)
        if stop is not None and stop(out):
            break
        if step + 1 == max_new:
            break
        lg = model.step(st, np.array([tok], np.uint32))[0]
    return out


def prompts_of(cfg, lens):
    ids = synth.token_ids(cfg["vocab"], len(lens), max(lens), seed0=21)
    return [ids[r, :n].tolist() for r, n in enumerate(lens)]


def test_greedy_equals_one_prompt_at_a_time(model):
    lens = [5, 9, 5, 1, 12, 9, 5]
    prompts = prompts_of(model.cfg, lens)
    free = [by_hand(model, p, 14, 1 << 30, lambda lg: int(np.argmax(lg))) for p in prompts]
    got = model.generate(prompts, 14, batch_rows=4, eos=1 << 30)
    assert got == free
    assert all(len(g) == 14 for g in got)
    # an EOS that some rows meet early: those rows leave, the others go on unchanged
    eos = free[2][3]
    want = [by_hand(model, p, 14, eos, lambda lg: int(np.argmax(lg))) for p in prompts]
    assert model.generate(prompts, 14, batch_rows=3, eos=eos) == want
    assert len(want[2]) == 3 and any(len(w) == 14 for w in want)
    # a stop rule per prompt
    stop = lambda r, toks: len(toks) >= 2 + r
    want = [by_hand(model, p, 14, 1 << 30, lambda lg: int(np.argmax(lg)), stop=lambda t, r=r: stop(r, t)) for r, p in enumerate(prompts)]
    assert model.generate(prompts, 14, batch_rows=16, eos=1 << 30, stop_fn=stop) == want
    assert [len(w) for w in want] == [2, 3, 4, 5, 6, 7, 8]


def test_sampled_through_the_callback(model):
    prompts = prompts_of(model.cfg, [6, 6, 3])
    # one generator per prompt, so the draws do not depend on how rows are grouped
    def run(batch_rows):
        rngs = [engine.Rng(100 + r) for r in range(len(prompts))]
        return model.generate(prompts, 10, batch_rows=batch_rows, eos=1 << 30, pick_fn=lambda r, lg: engine.pick(lg, 0.9, 20, rngs[r]))
    a, b = run(8), run(2)
    assert a == b
    want = []
    for r, p in enumerate(prompts):
        rng = engine.Rng(100 + r)
        want.append(by_hand(model, p, 10, 1 << 30, lambda lg: engine.pick(lg, 0.9, 20, rng)))
    assert a == want
    assert a != model.generate(prompts, 10, eos=1 << 30)      # and it is not the greedy continuation


def test_arguments(model):
    with pytest.raises(engine.EngineError):
        model.generate([[1, 2], []], 4)
    assert model.generate([[1, 2, 3]], 0) == [[]]
    def boom(r, lg):
        raise KeyError("from the callback")
    with pytest.raises(KeyError):
        model.generate([[1, 2, 3]], 4, pick_fn=boom)
