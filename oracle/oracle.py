"""ctypes binding of the CPU oracle (libava_oracle.so).

TEST INFRASTRUCTURE ONLY.  The oracle is the checker the CUDA engine is compared with; only the tests, the smoke
check and the benchmark's CPU-baseline leg may import this module.  Nothing in the product package does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libava_oracle.so")

FN1 = C.CFUNCTYPE(C.c_float, C.c_float)


class OrcConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "vocab", "d", "n_blocks", "hidden", "kwta_k", "head_size", "eng_block", "eng_head_size", "eng_store_bf16",
        "eng_cap", "gate_rank", "spikes", "alif", "theta", "lif_scale", "value_residual", "relu2", "dense",
        "out_gate", "fast_mem", "dendrite", "neuromod", "stp", "dopamine", "mood", "cb_units", "letters", "rhythm", "thalamus")] + [("mem_momentum", C.c_float), ("slope", C.c_float)]


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe beside it (g++ only) and return the library's path."""
    srcs = [os.path.join(_HERE, n) for n in ("ava_oracle.cpp", "ava_chunk.cpp", "ava_oracle.h", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(os.path.getmtime(p) > os.path.getmtime(_LIB_PATH) for p in srcs)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s", "clean"])
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        build()
    L = C.CDLL(_LIB_PATH)
    fp = C.POINTER(C.c_float)
    i8p = C.POINTER(C.c_int8)
    L.orc_set_math.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    L.orc_set_trig.argtypes = [C.c_void_p, C.c_void_p]
    L.orc_set_threads.argtypes = [C.c_int]
    L.orc_set_simd.argtypes = [C.c_int]
    L.orc_set_event_max.argtypes = [C.c_double]
    L.orc_quantize_int8.argtypes = [fp, C.c_int, C.c_int, i8p, fp]
    L.orc_q8_matmul.argtypes = [fp, C.c_int, i8p, fp, C.c_int, C.c_int, fp]
    L.orc_last_event_rows.restype = C.c_int
    L.orc_rmsnorm.argtypes = [fp, fp, C.c_int, fp]
    L.orc_l2_heads.argtypes = [fp, C.c_int, C.c_int]
    L.orc_head_norm.argtypes = [fp, C.c_int, C.c_int]
    L.orc_sigmoid.argtypes = [C.c_float]
    L.orc_sigmoid.restype = C.c_float
    L.orc_log_sigmoid.argtypes = [C.c_float]
    L.orc_log_sigmoid.restype = C.c_float
    L.orc_gemv.argtypes = [fp, C.c_int, fp, C.c_int, fp]
    L.orc_stp.argtypes = [fp] * 7 + [C.c_int] + [fp] * 4
    L.orc_stp.restype = None
    L.orc_model_set_token_bytes.argtypes = [C.c_void_p, C.POINTER(C.c_uint8), C.POINTER(C.c_int64)]
    L.orc_model_set_token_bytes.restype = C.c_int
    L.orc_cb_wiring.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_uint32), fp]
    L.orc_cb_wiring.restype = None
    L.orc_lif.argtypes = [fp, fp, fp, fp, fp, C.c_int, C.c_float, fp, fp, fp, C.c_int, fp, fp, fp]
    L.orc_kth_largest.argtypes = [fp, C.c_int, C.c_int]
    L.orc_kth_largest.restype = C.c_float
    L.orc_kwta.argtypes = [fp, C.c_int, C.c_int, C.c_int, fp]
    L.orc_attend.argtypes = [fp, fp, fp, C.c_int, C.c_int, C.c_float, fp]
    L.orc_head_rows.argtypes = [C.c_int, fp, fp, fp, fp, fp, fp, C.c_float, C.c_float, C.c_float, C.c_float,
                                C.c_float, fp, fp, fp, fp, fp, fp, fp]
    L.orc_delta_plain.argtypes = [C.c_int, fp, fp, fp, fp, C.c_float, C.c_float, fp, fp]
    L.orc_inv_unit_lower.argtypes = [fp, C.c_int, fp]
    L.orc_delta_rule_from.argtypes = [C.c_int, C.c_int, fp, fp, fp, fp, fp, fp, fp, fp]
    L.orc_delta_rec.argtypes = [C.c_int, C.c_int, C.c_int, fp, fp, fp, fp, fp, fp, C.c_float, fp, fp, C.c_float, fp, fp, fp]
    L.orc_delta_chunk.argtypes = [C.c_int, C.c_int, C.c_int, fp, fp, fp, fp, fp, fp, C.c_float, fp, fp, fp, fp, fp]
    L.orc_bf16_round.argtypes = [C.c_float]
    L.orc_bf16_round.restype = C.c_float
    L.orc_model_new.argtypes = [C.POINTER(OrcConfig)]
    L.orc_model_new.restype = C.c_void_p
    L.orc_model_free.argtypes = [C.c_void_p]
    L.orc_model_set_f32.argtypes = [C.c_void_p, C.c_char_p, fp, C.c_int64]
    L.orc_model_set_q8.argtypes = [C.c_void_p, C.c_char_p, i8p, fp, C.c_int, C.c_int]
    L.orc_model_set_q8_from_f32.argtypes = [C.c_void_p, C.c_char_p, fp, C.c_int, C.c_int]
    L.orc_model_check.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    L.orc_state_new.argtypes = [C.c_void_p, C.c_int]
    L.orc_state_new.restype = C.c_void_p
    L.orc_state_free.argtypes = [C.c_void_p]
    L.orc_state_rows.argtypes = [C.c_void_p]
    L.orc_state_select.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int]
    L.orc_state_select.restype = C.c_void_p
    L.orc_state_len.argtypes = [C.c_void_p, C.c_int, C.c_char_p]
    L.orc_state_len.restype = C.c_int64
    L.orc_state_get.argtypes = [C.c_void_p, C.c_int, C.c_char_p, fp]
    L.orc_state_put.argtypes = [C.c_void_p, C.c_int, C.c_char_p, fp, C.c_int64]
    L.orc_state_seen.argtypes = [C.c_void_p, C.c_int]
    L.orc_state_seen.restype = C.c_int64
    L.orc_step.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32), fp]
    L.orc_forward.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.c_int, fp]
    L.orc_trace_enable.argtypes = [C.c_int]
    L.orc_trace_len.argtypes = [C.c_char_p, C.c_int]
    L.orc_trace_len.restype = C.c_int64
    L.orc_trace_get.argtypes = [C.c_char_p, C.c_int, fp]
    _lib = L
    return L


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


_keep_math = []


def set_math(expf=None, logf=None, rsqrtf=None, sinf=None, cosf=None):
    """Plug in other exp / ln / x^-0.5 / sin / cos (ctypes function pointers or addresses); None keeps the current one."""
    def addr(f):
        if f is None:
            return None
        _keep_math.append(f)
        return C.cast(f, C.c_void_p)
    lib().orc_set_math(addr(expf), addr(logf), addr(rsqrtf))
    lib().orc_set_trig(addr(sinf), addr(cosf))


def reset_math():
    lib().orc_reset_math()


# ------------------------------------------------------------------------------------------------ op level
def quantize_int8(w):
    w, wp = _f(w)
    rows, cols = w.shape
    q = np.empty((rows, cols), np.int8)
    sc = np.empty(cols, np.float32)
    lib().orc_quantize_int8(wp, rows, cols, q.ctypes.data_as(C.POINTER(C.c_int8)), _fp(sc))
    return q, sc


def q8_matmul(x, q, scale):
    x, xp = _f(x)
    x2 = x.reshape(-1, x.shape[-1])
    q = np.ascontiguousarray(q, np.int8)
    scale, sp = _f(scale)
    din, dout = q.shape
    y = np.empty((x2.shape[0], dout), np.float32)
    lib().orc_q8_matmul(xp, x2.shape[0], q.ctypes.data_as(C.POINTER(C.c_int8)), sp, din, dout, _fp(y))
    return y.reshape(x.shape[:-1] + (dout,))


def rmsnorm(x, g):
    x, xp = _f(x)
    g, gp = _f(g)
    y = np.empty_like(x)
    lib().orc_rmsnorm(xp, gp, x.size, _fp(y))
    return y


def l2_heads(x, hs):
    x = np.array(x, np.float32, copy=True)
    lib().orc_l2_heads(_fp(x), x.size, hs)
    return x


def head_norm(x, hs):
    x = np.array(x, np.float32, copy=True)
    lib().orc_head_norm(_fp(x), x.size, hs)
    return x


def gemv(x, w):
    x, xp = _f(x)
    w, wp = _f(w)
    out = np.empty(w.shape[1], np.float32)
    lib().orc_gemv(xp, x.size, wp, w.shape[1], _fp(out))
    return out


def lif(cur, beta, v0, s0, theta=None, rho=None, gain=None, a0=None, spikes=2, slope=4.0):
    cur, cp = _f(cur)
    d = cur.size
    arrs = [np.ascontiguousarray(a, np.float32) if a is not None else None for a in (beta, theta, rho, gain, v0, s0, a0)]
    beta, theta, rho, gain, v0, s0, a0 = arrs
    s1 = np.empty(d, np.float32)
    v1 = np.empty(d, np.float32)
    a1 = np.empty(d, np.float32) if rho is not None else None
    lib().orc_lif(cp, _fp(beta), _fp(theta), _fp(rho), _fp(gain), spikes, slope, _fp(v0), _fp(s0), _fp(a0), d,
                  _fp(s1), _fp(v1), _fp(a1))
    return s1, v1, a1


def stp(s, u_param, f_param, d_param, mix, u0, x0):
    """(out, u1, x1, efficacy) of one step of the short-term-plastic synapse."""
    s, sp = _f(s)
    arrs = [_f(a) for a in (u_param, f_param, d_param, mix, u0, x0)]
    out, u1, x1, eff = (np.empty_like(s) for _ in range(4))
    L = lib()
    L.orc_stp(sp, *[a[1] for a in arrs], s.size, _fp(out), _fp(u1), _fp(x1), _fp(eff))
    return out, u1, x1, eff


def cb_wiring(inputs: int, g: int):
    idx, w = np.empty(g * 4, np.uint32), np.empty(g * 4, np.float32)
    lib().orc_cb_wiring(inputs, g, idx.ctypes.data_as(C.POINTER(C.c_uint32)), _fp(w))
    return idx.reshape(g, 4), w.reshape(g, 4)


def kth_largest(u, k):
    u, up = _f(u)
    return float(lib().orc_kth_largest(up, u.size, k))


def kwta(u, k, relu2):
    u, up = _f(u)
    a = np.empty_like(u)
    lib().orc_kwta(up, u.size, k, int(relu2), _fp(a))
    return a


def attend(q, kc, vc, scale):
    q, qp = _f(q)
    kc, kp = _f(kc)
    vc, vp = _f(vc)
    n, hs = kc.shape
    out = np.empty(hs, np.float32)
    lib().orc_attend(qp, kp, vp, n, hs, scale, _fp(out))
    return out


def head_rows(e, v, w, ah, qg, ex, qw, qa, f0, ke=0.0, tinv=1.0, mom=0.0, qs=None, p2=None, s0=None):
    hs = len(e)
    arrs = [np.ascontiguousarray(a, np.float32) if a is not None else None for a in (e, v, w, ah, qg, ex, qs, p2, f0, s0)]
    e, v, w, ah, qg, ex, qs, p2, f0, s0 = arrs
    y = np.empty(hs, np.float32)
    f1 = np.empty((hs, hs), np.float32)
    s1 = np.empty((hs, hs), np.float32) if mom > 0 else None
    lib().orc_head_rows(hs, _fp(e), _fp(v), _fp(w), _fp(ah), _fp(qg), _fp(ex), qw, qa, ke, tinv, mom, _fp(qs), _fp(p2),
                        _fp(f0), _fp(s0), _fp(y), _fp(f1), _fp(s1))
    return y, f1, s1


def inv_unit_lower(a):
    """(I + A)^-1 for strictly lower-triangular A [c, c] (src/model.rs:720-742)."""
    a = np.ascontiguousarray(a, np.float32)
    c = a.shape[0]
    out = np.empty((c, c), np.float32)
    lib().orc_inv_unit_lower(_fp(a), c, _fp(out))
    return out


def delta_rule_from(q, k, v, la, beta, f0=None):
    """One head of `delta_rule_from` (src/model.rs:761-799): y [t, hs] and the fast weights after the window."""
    q, k, v = (np.ascontiguousarray(x, np.float32) for x in (q, k, v))
    la, beta = np.ascontiguousarray(la, np.float32), np.ascontiguousarray(beta, np.float32)
    t, hs = q.shape
    y, f1 = np.empty((t, hs), np.float32), np.empty((hs, hs), np.float32)
    f0 = None if f0 is None else np.ascontiguousarray(f0, np.float32)
    lib().orc_delta_rule_from(t, hs, _fp(q), _fp(k), _fp(v), _fp(la), _fp(beta), _fp(f0) if f0 is not None else None, _fp(y), _fp(f1))
    return y, f1


def _delta_args(q, k, e, v, la, b, f0, s0):
    q, k, e, v = (np.ascontiguousarray(x, np.float32) for x in (q, k, e, v))
    t, hs = q.shape
    la = np.ascontiguousarray(la, np.float32).reshape(t, -1)
    b = np.ascontiguousarray(b, np.float32).reshape(t, -1)
    g = la.shape[1]
    assert g in (1, hs) and b.shape[1] == g
    f0 = None if f0 is None else np.ascontiguousarray(f0, np.float32)
    s0 = None if s0 is None else np.ascontiguousarray(s0, np.float32)
    return q, k, e, v, la, b, f0, s0, t, hs, g


def delta_rec(q, k, e, v, la, b, m=0.0, f0=None, s0=None, cap=1e5):
    """One head of `delta_rec` (src/arch.rs:1091-1136), the token loop: y, F and (with momentum) S."""
    q, k, e, v, la, b, f0, s0, t, hs, g = _delta_args(q, k, e, v, la, b, f0, s0)
    y, f1, s1 = np.empty((t, hs), np.float32), np.empty((hs, hs), np.float32), np.zeros((hs, hs), np.float32)
    lib().orc_delta_rec(t, hs, g, _fp(q), _fp(k), _fp(e), _fp(v), _fp(la), _fp(b), m, _fp(f0) if f0 is not None else None,
                        _fp(s0) if s0 is not None else None, cap, _fp(y), _fp(f1), _fp(s1))
    return y, f1, (s1 if m > 0 else None)


def delta_chunk(q, k, e, v, la, b, m=0.0, f0=None, s0=None):
    """One head of `delta_chunk` / `chunk_core` (src/arch.rs:1151-1173, 1243-1327): the same rule in chunks."""
    q, k, e, v, la, b, f0, s0, t, hs, g = _delta_args(q, k, e, v, la, b, f0, s0)
    y, f1, s1 = np.empty((t, hs), np.float32), np.empty((hs, hs), np.float32), np.zeros((hs, hs), np.float32)
    lib().orc_delta_chunk(t, hs, g, _fp(q), _fp(k), _fp(e), _fp(v), _fp(la), _fp(b), m, _fp(f0) if f0 is not None else None,
                          _fp(s0) if s0 is not None else None, _fp(y), _fp(f1), _fp(s1))
    return y, f1, (s1 if m > 0 else None)


def delta_plain(f0, k, v, q, al, b):
    f0, fp0 = _f(f0)
    k, kp = _f(k)
    v, vp = _f(v)
    q, qp = _f(q)
    hs = k.size
    f1 = np.empty((hs, hs), np.float32)
    y = np.empty(hs, np.float32)
    lib().orc_delta_plain(hs, fp0, kp, vp, qp, al, b, _fp(f1), _fp(y))
    return f1, y


def bf16_round(x):
    return float(lib().orc_bf16_round(float(x)))


# ------------------------------------------------------------------------------------------------ model level
class OracleModel:
    """The oracle's model: configuration + weights by their reference names."""

    def __init__(self, cfg: dict, weights: dict | None = None):
        self.cfg = dict(cfg)
        c = OrcConfig(**{k: cfg[k] for k, _ in OrcConfig._fields_})
        self._c = c
        self.h = lib().orc_model_new(C.byref(c))
        if not self.h:
            raise ValueError("oracle: bad configuration")
        if weights is not None:
            self.load(weights)

    def load(self, weights: dict):
        """weights: name -> f32 array, or name -> (int8 [din, dout], f32 scale [dout])."""
        L = lib()
        for name, w in weights.items():
            if name == "token_bytes":
                data, off = np.ascontiguousarray(w[0], np.uint8), np.ascontiguousarray(w[1], np.int64)
                rc = L.orc_model_set_token_bytes(self.h, data.ctypes.data_as(C.POINTER(C.c_uint8)), off.ctypes.data_as(C.POINTER(C.c_int64)))
            elif isinstance(w, tuple):
                q, sc = w
                q = np.ascontiguousarray(q, np.int8)
                sc = np.ascontiguousarray(sc, np.float32)
                rc = L.orc_model_set_q8(self.h, name.encode(), q.ctypes.data_as(C.POINTER(C.c_int8)), _fp(sc),
                                        q.shape[0], q.shape[1])
            else:
                w = np.ascontiguousarray(w, np.float32)
                rc = L.orc_model_set_f32(self.h, name.encode(), _fp(w), w.size)
                if rc != 0 and w.ndim == 2:
                    # an f32 matrix of a checkpoint: quantised per output column (nn/parts/src/quant.rs:18-31)
                    rc = L.orc_model_set_q8_from_f32(self.h, name.encode(), _fp(w), w.shape[0], w.shape[1])
            if rc != 0:
                raise ValueError(f"oracle: tensor {name!r} refused (unknown name or wrong size)")
        if "head" not in weights:
            e = np.ascontiguousarray(weights["tok_emb"], np.float32)
            et = np.ascontiguousarray(e.T)
            L.orc_model_set_q8_from_f32(self.h, b"head", _fp(et), et.shape[0], et.shape[1])
        buf = C.create_string_buffer(128)
        if L.orc_model_check(self.h, buf, 128) != 0:
            raise ValueError(f"oracle: missing tensor {buf.value.decode()!r}")

    def state(self, rows: int) -> "OracleState":
        return OracleState(self, lib().orc_state_new(self.h, rows))

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_model_free(self.h)
            self.h = None


class OracleState:
    def __init__(self, model: OracleModel, h):
        self.m = model
        self.h = h

    @property
    def rows(self) -> int:
        return lib().orc_state_rows(self.h)

    def select(self, idx) -> "OracleState":
        idx = np.ascontiguousarray(idx, np.int32)
        h = lib().orc_state_select(self.h, idx.ctypes.data_as(C.POINTER(C.c_int32)), idx.size)
        if not h:
            raise IndexError("oracle: row out of range")
        return OracleState(self.m, h)

    def get(self, row: int, name: str) -> np.ndarray:
        n = lib().orc_state_len(self.h, row, name.encode())
        if n < 0:
            raise KeyError(name)
        out = np.empty(n, np.float32)
        lib().orc_state_get(self.h, row, name.encode(), _fp(out))
        return out

    def put(self, row: int, name: str, a):
        a = np.ascontiguousarray(a, np.float32)
        if lib().orc_state_put(self.h, row, name.encode(), _fp(a), a.size) != 0:
            raise KeyError(name)

    def seen(self, row: int) -> int:
        return lib().orc_state_seen(self.h, row)

    def step(self, tok) -> np.ndarray:
        tok = np.ascontiguousarray(tok, np.uint32).reshape(-1)
        assert tok.size == self.rows
        logits = np.empty((self.rows, self.m.cfg["vocab"]), np.float32)
        rc = lib().orc_step(self.m.h, self.h, tok.ctypes.data_as(C.POINTER(C.c_uint32)), _fp(logits))
        if rc < 0:
            raise RuntimeError(f"oracle step failed: {rc}")
        self.last_status = rc
        return logits

    def forward(self, ids, last_only=False) -> np.ndarray:
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, t = ids.shape
        assert rows == self.rows
        V = self.m.cfg["vocab"]
        logits = np.empty((rows, V) if last_only else (rows, t, V), np.float32)
        rc = lib().orc_forward(self.m.h, self.h, ids.ctypes.data_as(C.POINTER(C.c_uint32)), t, int(last_only), _fp(logits))
        if rc < 0:
            raise RuntimeError(f"oracle forward failed: {rc}")
        self.last_status = rc
        return logits

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_state_free(self.h)
            self.h = None


def trace_enable(on: bool):
    lib().orc_trace_enable(int(on))


def trace(name: str, block: int) -> np.ndarray:
    n = lib().orc_trace_len(name.encode(), block)
    if n < 0:
        raise KeyError((name, block))
    out = np.empty(n, np.float32)
    lib().orc_trace_get(name.encode(), block, _fp(out))
    return out


def set_threads(n: int):
    lib().orc_set_threads(n)


def set_simd(on: bool):
    lib().orc_set_simd(int(on))


def set_event_max(v: float):
    lib().orc_set_event_max(v)


def last_event_rows() -> int:
    return lib().orc_last_event_rows()
