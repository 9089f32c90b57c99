"""Seeded synthetic weights and token ids for the block step.

The reference's benchmark inputs (validation shards, question files) and the released Ava 0.4 weights are not
available, so the measurements and the parity tests run on synthetic models of the same shapes.  The generator is
SplitMix64 with the constants of the reference's one random number generator
(design-tests/nn/data/src/rng.rs:11-31); uniforms are (next >> 11) / 2^53 as in
design-tests/nn/gpu/src/bin/int8_bench.rs:141-150.  Every tensor draws from its own stream, seeded
mix64(seed ^ fnv1a64(name)), so a tensor's values do not depend on which other tensors exist.

Two recipes:
  * "bench": int8 weights q ~ U{-127..127}, per-output scales ~ U(0.5, 1.5)/127 (times one documented gain per
    matrix so that a unit-RMS input gives a unit-RMS output), leak ~ U(0.8, 0.99), threshold 1, adaptation rate
    0.05 (rho 0.95, gain 1), gate projections zero with alpha = 1 and write strength 0.1, erase key = key, fast
    synapse zero-init, tied embedding ~ N(0, 0.02^2).
  * "awake": the same matrices, but every small parameter that the reference initialises to zero gets seeded noise
    so that every term of the step is exercised (the reference's tests do the same,
    design-tests/nn/gpu/src/state/tests.rs:14-34).
"""
from __future__ import annotations

import math

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_MASK = (1 << 64) - 1


def _finalize(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def splitmix64(seed: int, n: int) -> np.ndarray:
    """The first n outputs of SplitMix64(seed) as uint64."""
    with np.errstate(over="ignore"):
        k = np.arange(1, n + 1, dtype=np.uint64)
        return _finalize(np.uint64(seed & _MASK) + k * _GAMMA)


def mix64(x: int) -> int:
    return int(splitmix64(x, 1)[0])


def fnv1a64(s: str) -> int:
    h = 0xCBF29CE484222325
    for b in s.encode():
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return h


def uniform(seed: int, n: int) -> np.ndarray:
    """n uniforms in [0, 1) as float64."""
    return (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) / float(1 << 53)


def normal(seed: int, n: int) -> np.ndarray:
    """n standard normals (Box-Muller on pairs of uniforms of one stream)."""
    m = (n + 1) // 2
    u = uniform(seed, 2 * m)
    u1, u2 = np.maximum(u[0::2], 2.0 ** -53), u[1::2]
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2 * np.pi * u2), r * np.sin(2 * np.pi * u2)])
    return z[:n]


class _Gen:
    def __init__(self, seed: int):
        self.seed = seed

    def s(self, name: str) -> int:
        return mix64(self.seed ^ fnv1a64(name))

    def u(self, name, shape, lo=0.0, hi=1.0):
        n = int(np.prod(shape))
        return (lo + (hi - lo) * uniform(self.s(name), n)).astype(np.float32).reshape(shape)

    def n(self, name, shape, std):
        n = int(np.prod(shape))
        return (std * normal(self.s(name), n)).astype(np.float32).reshape(shape)

    def q8(self, name, din, dout, gain):
        """int8 weights uniform over -127..127 and scales U(0.5, 1.5)/127 * gain, one per output."""
        q = (np.floor(uniform(self.s(name + ".q"), din * dout) * 255.0) - 127.0).astype(np.int8).reshape(din, dout)
        sc = ((0.5 + uniform(self.s(name + ".scale"), dout)) / 127.0 * gain).astype(np.float32)
        return q, sc


def logit(p: float) -> float:
    return math.log(p / (1.0 - p))


# std of U{-127..127} * (mean scale 1/127): a unit-RMS input through an unscaled matrix gives RMS 0.5774*sqrt(din)
_W_STD = math.sqrt((255.0 ** 2 - 1) / 12.0) / 127.0


def model(cfg: dict, seed: int = 0, recipe: str = "bench", unit_gain: bool = True) -> dict:
    """name -> f32 array, or (int8 [din, dout], f32 scale [dout]) for the int8 matrices.  The output head is not in
    the dict: it is the quantised transpose of tok_emb, built by whoever loads the weights."""
    assert recipe in ("bench", "awake")
    g = _Gen(seed)
    d, H, V, L = cfg["d"], cfg["hidden"], cfg["vocab"], cfg["n_blocks"]
    nh, r = d // cfg["head_size"], cfg["gate_rank"]
    awake = recipe == "awake"
    w = {}

    def gain(din, extra=1.0):
        return extra / (_W_STD * math.sqrt(din)) if unit_gain else extra

    w["tok_emb"] = g.n("tok_emb", (V, d), 0.02)
    w["final.norm"] = 1.0 + g.n("final.norm", (d,), 0.05) if awake else np.ones(d, np.float32)
    if cfg.get("neuromod"):
        k = cfg["neuromod"]
        w["nm.norm"] = (1.0 + g.n("nm.norm", (d,), 0.05)).astype(np.float32) if awake else np.ones(d, np.float32)
        w["nm.wn"] = g.n("nm.wn", (d, k), 0.05) if awake else np.zeros((d, k), np.float32)
        w["nm.bn"] = g.n("nm.bn", (k,), 0.3) if awake else np.zeros(k, np.float32)
    if cfg.get("rhythm"):
        # the reference's start: periods of 16 and 3.2 tokens, a reset bias of -10 (never); the awake recipe resets now and then
        w["v51.rhythm.lw"] = np.log(2.0 * np.pi / np.array([16.0, 3.2])).astype(np.float32)
        w["v51.rhythm.wr"] = g.n("v51.rhythm.wr", (d, 2), 2.0 / math.sqrt(d)) if awake else np.zeros((d, 2), np.float32)
        w["v51.rhythm.br"] = np.array([-2.0, -1.0], np.float32) if awake else np.full(2, -10.0, np.float32)
    if cfg.get("mood"):
        k = cfg["mood"]
        w["v51.mood.lam"] = g.n("v51.mood.lam", (k,), 1.0) + 2.0
        w["v51.mood.win"] = (1.0 + g.n("v51.mood.win", (k,), 0.3)).astype(np.float32)
        w["v51.mood.bin"] = g.n("v51.mood.bin", (k,), 0.1) if awake else np.zeros(k, np.float32)
    if cfg.get("letters"):
        # spellings of 0 to 20 bytes (longer than the 16 places the part reads, and one empty), seeded
        rng = np.random.default_rng(seed * 7919 + 17)
        lens = rng.integers(1, 21, size=V)
        lens[min(3, V - 1)] = 0
        off = np.zeros(V + 1, np.int64)
        off[1:] = np.cumsum(lens)
        w["token_bytes"] = (rng.integers(0, 256, size=int(off[-1]), dtype=np.uint8), off)
        s3 = 1.0 / math.sqrt(3.0)
        w["v51.letters.byte"] = g.n("v51.letters.byte", (256, 64), s3)
        w["v51.letters.pos"] = g.n("v51.letters.pos", (16, 64), s3)
        w["v51.letters.end"] = g.n("v51.letters.end", (16, 64), s3)
        w["v51.letters.wo"] = g.n("v51.letters.wo", (64, d), 0.02) if awake else np.zeros((64, d), np.float32)
    if cfg.get("cb_units"):
        w["cbh.wo"] = g.n("cbh.wo", (cfg["cb_units"], d), 0.05) if awake else np.zeros((cfg["cb_units"], d), np.float32)
    if cfg.get("thalamus"):
        # the reference starts the reads as seeded noise / sqrt(d) and the gates at zero (every gate exactly 1)
        w["th.read"] = g.n("th.read", (L, d, 16), 1.0 / math.sqrt(d))
        w["th.gate"] = g.n("th.gate", (L, 16, 2), 0.5) if awake else np.zeros((L, 16, 2), np.float32)
        w["th.bias"] = g.n("th.bias", (L, 2), 0.3) if awake else np.zeros((L, 2), np.float32)
    for i in range(L):
        p = f"b{i}."
        ones = lambda nm: (1.0 + g.n(p + nm, (d,), 0.05)).astype(np.float32) if awake else np.ones(d, np.float32)
        # the spiking memory: leak ~ U(0.8, 0.99) per channel, stored as its logit (the reference keeps the parameter)
        beta = g.u(p + "mem.beta", (d,), 0.8, 0.99).astype(np.float64)
        w[p + "mem.norm"] = ones("mem.norm")
        w[p + "mem.beta"] = np.log(beta / (1.0 - beta)).astype(np.float32)
        # the input current is scaled by (1 - beta) in the step; the extra gain keeps the spike share in the
        # reference's measured range (a few per cent)
        w[p + "mem.win"] = g.q8(p + "mem.win", d, d, gain(d, 2.5))
        w[p + "mem.wout"] = g.q8(p + "mem.wout", d, d, gain(d, 0.5))
        if cfg["theta"]:
            w[p + "mem.theta"] = g.u(p + "mem.theta", (d,), 0.8, 1.2) if awake else np.ones(d, np.float32)
        if cfg["alif"]:
            rho = 0.95
            jitter = g.n(p + "mem.arho", (d,), 0.2) if awake else np.zeros(d, np.float32)
            w[p + "mem.arho"] = (logit(rho) + jitter).astype(np.float32)
            w[p + "mem.again"] = g.u(p + "mem.again", (d,), 0.5, 1.5) if awake else np.ones(d, np.float32)
        if cfg["stp"]:
            # the synapse of the spikes: U around 0.2, facilitation and recovery of a few tokens, a real mix
            for nm, lo, hi in (("u_param", 0.1, 0.5), ("f_param", 0.5, 0.98), ("d_param", 0.5, 0.95)):
                pv = g.u(p + "parts.stp." + nm, (d,), lo, hi).astype(np.float64)
                w[p + "parts.stp." + nm] = np.log(pv / (1.0 - pv)).astype(np.float32)
            w[p + "parts.stp.mix"] = g.u(p + "parts.stp.mix", (d,), 0.0, 1.0) if awake else np.full(d, 0.5, np.float32)
        # the fast-weight memory (kinds D and A; kind S has none)
        if cfg["fast_mem"]:
            w[p + "hebb.norm"] = ones("hebb.norm")
            for nm in ("wq", "wk", "wv", "wo"):
                w[p + "hebb." + nm] = g.q8(p + "hebb." + nm, d, d, gain(d, 0.5 if nm == "wo" else 1.0))
            if cfg["out_gate"]:
                w[p + "hebb.wg"] = g.q8(p + "hebb.wg", d, d, gain(d))
            if awake:
                w[p + "hebb.we"] = g.q8(p + "hebb.we", d, d, gain(d, 0.3))
                w[p + "hebb.wa"] = g.n(p + "hebb.wa", (d, nh), 0.02)
                w[p + "hebb.wb"] = g.n(p + "hebb.wb", (d, nh), 0.02)
                w[p + "hebb.ba"] = g.n(p + "hebb.ba", (nh,), 0.1)
                w[p + "hebb.bb"] = g.n(p + "hebb.bb", (nh,), 0.1)
                w[p + "hebb.wa1"] = g.n(p + "hebb.wa1", (d, r), 0.02)
                w[p + "hebb.wa2"] = g.n(p + "hebb.wa2", (r, d), 0.1)
                w[p + "hebb.wb1"] = g.n(p + "hebb.wb1", (d, r), 0.02)
                w[p + "hebb.wb2"] = g.n(p + "hebb.wb2", (r, d), 0.1)
                # per-channel keep offsets: logit of a decay in (0.9, 0.999)
                ga = g.u(p + "hebb.off", (d,), 0.9, 0.999).astype(np.float64)
                w[p + "hebb.off"] = np.log(ga / (1 - ga)).astype(np.float32)
            else:
                # alpha = 1 (log_sigmoid of a large offset is -0), write strength 2 sigmoid(bb) = 0.1, erase key = key
                w[p + "hebb.we"] = (np.zeros((d, d), np.int8), g.q8(p + "hebb.we", d, d, gain(d))[1])
                w[p + "hebb.wa"] = np.zeros((d, nh), np.float32)
                w[p + "hebb.wb"] = np.zeros((d, nh), np.float32)
                w[p + "hebb.ba"] = np.zeros(nh, np.float32)
                w[p + "hebb.bb"] = np.full(nh, logit(0.05), np.float32)
                w[p + "hebb.wa1"] = np.zeros((d, r), np.float32)
                w[p + "hebb.wa2"] = np.zeros((r, d), np.float32)
                w[p + "hebb.wb1"] = np.zeros((d, r), np.float32)
                w[p + "hebb.wb2"] = np.zeros((r, d), np.float32)
                w[p + "hebb.off"] = np.full(d, 40.0, np.float32)
            if cfg["value_residual"] and i > 0:
                w[p + "hebb.vres"] = g.n(p + "hebb.vres", (2,), 0.1) if awake else np.zeros(2, np.float32)
        if i == cfg["eng_block"]:
            w[p + "eng.norm"] = ones("eng.norm")
            for nm in ("wq", "wk", "wv", "wo"):
                w[p + "eng." + nm] = g.q8(p + "eng." + nm, d, d, gain(d, 0.5 if nm == "wo" else 1.0))
        if cfg.get("dendrite") and cfg["fast_mem"]:
            w[p + "v51.dend_a"] = g.n(p + "v51.dend_a", (d, 32), 1.0 / math.sqrt(d))
            w[p + "v51.dend_b"] = g.n(p + "v51.dend_b", (32, H), 0.3) if awake else np.zeros((32, H), np.float32)
        if cfg.get("rhythm") and cfg["fast_mem"]:
            w[p + "v51.rh_w"] = g.n(p + "v51.rh_w", (4, nh), 0.3) if awake else np.zeros((4, nh), np.float32)
            w[p + "v51.rh_r"] = g.n(p + "v51.rh_r", (4, nh), 0.3) if awake else np.zeros((4, nh), np.float32)
        if cfg.get("dopamine") and i > 0:
            w[p + "v51.da_w"] = g.n(p + "v51.da_w", (d,), 0.5) if awake else np.zeros(d, np.float32)
            w[p + "v51.da_c"] = g.n(p + "v51.da_c", (d,), 0.1) if awake else np.zeros(d, np.float32)
        if cfg.get("mood") and i > 0:
            w[p + "v51.mood_g"] = g.n(p + "v51.mood_g", (cfg["mood"], d), 0.3) if awake else np.zeros((cfg["mood"], d), np.float32)
        w[p + "mlp.norm"] = ones("mlp.norm")
        w[p + "mlp.w1"] = g.q8(p + "mlp.w1", d, H, gain(d))
        w[p + "mlp.w2"] = g.q8(p + "mlp.w2", H, d, gain(cfg["kwta_k"], 0.25))
        if cfg["dense"]:
            w[p + "dense"] = g.n(p + "dense", (i + 2,), 0.05) if awake else np.zeros(i + 2, np.float32)
    return w


def token_ids(vocab: int, rows: int, t: int, seed0: int = 0) -> np.ndarray:
    """ids [rows, t] uniform over the vocabulary; row r draws from SplitMix64(seed0 + r)."""
    out = np.empty((rows, t), np.uint32)
    for r in range(rows):
        out[r] = np.minimum((uniform(seed0 + r, t) * vocab).astype(np.uint32), vocab - 1)
    return out


def weight_bytes(cfg: dict) -> int:
    """int8 weight bytes one step streams: every block's matrices and the head (scales not counted)."""
    d, H, V, L = cfg["d"], cfg["hidden"], cfg["vocab"], cfg["n_blocks"]
    per_block = (2 + ((5 + (1 if cfg["out_gate"] else 0)) if cfg["fast_mem"] else 0)) * d * d + 2 * d * H
    eng = 4 * d * d if cfg["eng_block"] >= 0 else 0
    return L * per_block + eng + V * d
