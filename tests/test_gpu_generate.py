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


@pytest.mark.parametrize("temperature,top_k,vocab", [(1.0, 40, 16384), (0.7, 5, 4096), (1.3, 1, 500), (1.0, 1024, 2000), (0.9, 100000, 700), (0.02, 40, 16384)])
def test_device_sampler_draws_what_the_host_sampler_draws(temperature, top_k, vocab):
    """The sampler kernel against ava_pick on the same logits and the same uniform numbers: the same tokens, ties at the
    top and at the cut included."""
    rng = np.random.default_rng(top_k + vocab)
    rows = 24
    lg = (rng.normal(size=(rows, vocab)) * 3).astype(np.float32)
    lg[1, 10:14] = lg[1].max() + 1.0                       # ties among the most likely
    lg[2] = np.round(lg[2])                                # many ties everywhere (and at the top_k cut)
    lg[3] = 0.0                                            # all equal: index order decides
    lg[4, 7] = 80.0                                        # one token takes all the mass
    gen = engine.Rng(77)
    states, u = [], []
    for r in range(rows):
        states.append(gen.state.value)
        u.append((gen.next_u64() >> 11) / float(1 << 53))
    got = engine.op_sample(lg, temperature, top_k, u)
    for r in range(rows):
        want = engine.pick(lg[r], temperature, top_k, engine.Rng(states[r]))
        assert got[r] == want, (r, int(got[r]), want)


def test_generate_sampled_equals_the_callback_form(model):
    prompts = prompts_of(model.cfg, [6, 6, 3, 9, 6])
    for batch_rows in (8, 2):
        rng = engine.Rng(5)
        want = model.generate(prompts, 12, batch_rows=batch_rows, eos=1 << 30, pick_fn=lambda r, lg: engine.pick(lg, 0.8, 16, rng))
        rng2 = engine.Rng(5)
        got = model.generate_sampled(prompts, 12, 0.8, 16, rng2, batch_rows=batch_rows, eos=1 << 30)
        assert got == want
        assert rng2.state.value == rng.state.value       # the same number of draws
    # an EOS that rows meet on the way, and a stop rule
    eos = want[0][4]
    rng, rng2 = engine.Rng(9), engine.Rng(9)
    stop = lambda r, toks: len(toks) >= 3 + r
    want = model.generate(prompts, 12, eos=eos, pick_fn=lambda r, lg: engine.pick(lg, 0.8, 16, rng), stop_fn=stop)
    assert model.generate_sampled(prompts, 12, 0.8, 16, rng2, eos=eos, stop_fn=stop) == want
    # temperature 0 is the greedy loop
    assert model.generate_sampled(prompts, 6, 0.0, 16, engine.Rng(1), eos=1 << 30) == model.generate(prompts, 6, eos=1 << 30)


def test_a_top_k_the_device_sampler_does_not_cover_is_drawn_on_the_host():
    """`diary::pick` works for any top_k (src/diary.rs:686-718); the device sampler holds at most 1024 kept tokens.  The
    generation loop decides once per call: beyond that it steps with logits out and draws with the host sampler from the
    same generator, so the tokens equal the callback form; the single step refuses before the state moves."""
    cfg = config.tiny(vocab=2048)
    m = engine.Model(cfg, synth.model(cfg, 4, "awake"))
    prompts = prompts_of(cfg, [6, 3, 6])
    rng, rng2 = engine.Rng(11), engine.Rng(11)
    want = m.generate(prompts, 9, batch_rows=8, eos=1 << 30, pick_fn=lambda r, lg: engine.pick(lg, 0.9, 1500, rng))
    got = m.generate_sampled(prompts, 9, 0.9, 1500, rng2, batch_rows=8, eos=1 << 30)
    assert got == want and all(len(g) == 9 for g in got)
    assert rng2.state.value == rng.state.value
    st = m.state(2, 16)
    m.step(st, np.array([1, 2], np.uint32))
    before = (st.seen(0), st.get(0, "lif.0.v").copy(), st.get(1, "mem.1.f").copy())
    with pytest.raises(engine.NotApplicable):
        m.step_sample(st, np.array([3, 4], np.uint32), 0.9, 1500, np.array([0.25, 0.5]))
    assert st.seen(0) == before[0]
    assert np.array_equal(st.get(0, "lif.0.v"), before[1]) and np.array_equal(st.get(1, "mem.1.f"), before[2])
