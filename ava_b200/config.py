"""Model configurations of the block step.

The fields mirror the reference's `Config` (design-tests/nn/gpu/src/model.rs:158-177) and the block options of
`Arch` (design-tests/nn/gpu/src/arch.rs:149-197) that the per-token step reads; the dict has exactly the fields of
`ava_config` in include/ava_engine.h, in the same order.
"""
from __future__ import annotations

FIELDS_I32 = ("vocab", "d", "n_blocks", "hidden", "kwta_k", "head_size", "eng_block", "eng_head_size",
              "eng_store_bf16", "eng_cap", "gate_rank", "spikes", "alif", "theta", "lif_scale", "value_residual",
              "relu2", "dense", "out_gate", "fast_mem", "dendrite", "neuromod", "stp", "thalamus", "dopamine", "mood", "cb_units", "letters", "rhythm")
FIELDS_F32 = ("mem_momentum", "slope")

SPIKES_BINARY, SPIKES_TERNARY, SPIKES_INT2 = 0, 1, 2


def make(vocab, d, n_blocks, *, hidden=None, kwta_k=None, head_size=64, eng_block=-1, eng_head_size=32,
         eng_store_bf16=0, eng_cap=0, gate_rank=32, spikes=SPIKES_INT2, alif=1, theta=1, lif_scale=1,
         value_residual=1, relu2=1, dense=1, out_gate=1, fast_mem=1, dendrite=0, neuromod=0, stp=0, thalamus=0, dopamine=0, mood=0, cb_units=0, letters=0, rhythm=0, mem_momentum=0.0, slope=4.0) -> dict:
    hidden = 4 * d if hidden is None else hidden
    kwta_k = hidden // 4 if kwta_k is None else kwta_k
    cfg = dict(vocab=vocab, d=d, n_blocks=n_blocks, hidden=hidden, kwta_k=kwta_k, head_size=head_size,
               eng_block=eng_block, eng_head_size=eng_head_size, eng_store_bf16=eng_store_bf16, eng_cap=eng_cap,
               gate_rank=gate_rank, spikes=spikes, alif=alif, theta=theta, lif_scale=lif_scale,
               value_residual=value_residual, relu2=relu2, dense=dense, out_gate=out_gate, fast_mem=fast_mem, dendrite=dendrite, neuromod=neuromod, stp=stp, thalamus=thalamus, dopamine=dopamine, mood=mood, cb_units=cb_units, letters=letters, rhythm=rhythm,
               mem_momentum=float(mem_momentum), slope=float(slope))
    assert d % head_size == 0
    assert eng_block < n_blocks
    if eng_block >= 0:
        assert d % eng_head_size == 0
    return cfg


def ava04_shaped(scaled: bool = False) -> dict:
    """The benchmark model: 12 blocks, d 768, wide 3072, kWTA 768, vocab 16384, ONE 768x768 fast-synapse matrix per
    block (one memory head of size d), one attention read of 12 heads x 64 in block 6 with a bf16 store.
    `scaled`: 24 blocks, d 2048, wide 8192, vocab 32768, engram in block 12."""
    if scaled:
        return make(32768, 2048, 24, head_size=2048, eng_block=12, eng_head_size=64, eng_store_bf16=1)
    return make(16384, 768, 12, head_size=768, eng_block=6, eng_head_size=64, eng_store_bf16=1)


def kind_s(vocab, d, n_blocks, **kw) -> dict:
    """The reference's model kind S (design-tests/nn/gpu/src/model.rs:105-118): blocks of a spiking memory with binary
    spikes and a fixed threshold, and the sparse MLP with relu; no fast-weight memory, no engram.  The k-WTA keeps an
    eighth of the wide layer (KWTA_DIV, model.rs:41).  The released Ava-M is one (d 384, 8 blocks, vocabulary 4096)."""
    base = dict(head_size=d, kwta_k=4 * d // 8, eng_block=-1, spikes=SPIKES_BINARY, alif=0, theta=0, lif_scale=0, value_residual=0, relu2=0,
                dense=0, out_gate=0, fast_mem=0)
    base.update(kw)
    return make(vocab, d, n_blocks, **base)


def tiny(**kw) -> dict:
    """A small model with every option on, for tests (d 128, 3 blocks as the reference's golden recipe)."""
    base = dict(vocab=320, d=128, n_blocks=3, head_size=32, eng_block=1, eng_head_size=32)
    base.update(kw)
    return make(base.pop("vocab"), base.pop("d"), base.pop("n_blocks"), **base)
