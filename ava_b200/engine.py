"""Python mirror of the reference's model/engine interface over the C ABI (include/ava_engine.h).

`Model` / `State` carry the reference's method names (`Model::state`, `Model::step`, `Model::forward_with_state`,
`State::select`, `State::cat`; design-tests/nn/gpu/src/model.rs:1260, src/state.rs:129,207,593,684).  Everything goes
through libava_engine.so with ctypes; there is no other compute path: without the library or without a CUDA device
these calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import config as _config

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libava_engine.so")

OK, NOT_APPLICABLE = 0, 1
ERR_ARG, ERR_CUDA, ERR_STATE, ERR_NONFINITE, ERR_MISSING, ERR_CAPACITY = -1, -2, -3, -4, -5, -6


class AvaConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in _config.FIELDS_I32] + [(n, C.c_float) for n in _config.FIELDS_F32]


class EngineError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"ava engine error {code}: {msg}")
        self.code = code


class NotApplicable(RuntimeError):
    """The engine does not cover this configuration (the reference's `Ok(None)` convention)."""


_lib = None
fp = C.POINTER(C.c_float)
i8p = C.POINTER(C.c_int8)
u32p = C.POINTER(C.c_uint32)
i32p = C.POINTER(C.c_int32)
PICK_FN = C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.c_int32, fp, C.c_int32)
STOP_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int32, u32p, C.c_int32)


def lib() -> C.CDLL:
    """The C-ABI library.  Raises when it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m ava_b200.build` (no CPU fallback exists)")
    L = C.CDLL(LIB_PATH)
    vp = C.c_void_p
    sig = {
        "ava_engine_create": ([C.POINTER(AvaConfig), C.c_int, C.POINTER(vp)], C.c_int),
        "ava_engine_destroy": ([vp], None),
        "ava_last_error": ([vp], C.c_char_p),
        "ava_engine_set_f32": ([vp, C.c_char_p, fp, C.c_int64], C.c_int),
        "ava_engine_set_token_bytes": ([vp, C.POINTER(C.c_uint8), C.POINTER(C.c_int64)], C.c_int),
        "ava_engine_set_q8": ([vp, C.c_char_p, i8p, fp, C.c_int32, C.c_int32], C.c_int),
        "ava_engine_set_q8_from_f32": ([vp, C.c_char_p, fp, C.c_int32, C.c_int32], C.c_int),
        "ava_engine_finalize": ([vp], C.c_int),
        "ava_engine_blocker": ([vp], C.c_char_p),
        "ava_state_new": ([vp, C.c_int32, C.c_int32, C.POINTER(vp)], C.c_int),
        "ava_state_destroy": ([vp], None),
        "ava_state_rows": ([vp], C.c_int32),
        "ava_state_select": ([vp, i32p, C.c_int32, C.POINTER(vp)], C.c_int),
        "ava_state_cat": ([C.POINTER(vp), C.c_int32, C.POINTER(vp)], C.c_int),
        "ava_state_seen": ([vp, C.c_int32], C.c_int64),
        "ava_state_len": ([vp, C.c_int32, C.c_char_p], C.c_int64),
        "ava_state_export": ([vp, C.c_int32, C.c_char_p, fp], C.c_int),
        "ava_state_import": ([vp, C.c_int32, C.c_char_p, fp, C.c_int64], C.c_int),
        "ava_step": ([vp, vp, u32p, fp], C.c_int),
        "ava_step_greedy": ([vp, vp, u32p, u32p], C.c_int),
        "ava_forward_with_state": ([vp, vp, u32p, C.c_int32, C.c_int32, fp], C.c_int),
        "ava_step_device": ([vp, vp, vp, vp, vp], C.c_int),
        "ava_prefill_device": ([vp, vp, vp, C.c_int32, C.c_int32, vp, vp], C.c_int),
        "ava_state_set_kv_shard": ([vp, C.c_int32, C.c_int32, C.c_int64, C.c_int64], C.c_int),
        "ava_shard_parts": ([vp, vp], C.c_int32),
        "ava_split_step_begin": ([vp, vp, vp, vp], C.c_int),
        "ava_shard_partial": ([vp, vp, vp, vp], C.c_int),
        "ava_split_step_end": ([vp, vp, vp, C.c_int32, vp, vp], C.c_int),
        "ava_sync": ([vp], C.c_int),
        "ava_engine_stream": ([vp], vp),
        "ava_engine_launches": ([vp], C.c_int64),
        "ava_engine_bytes": ([vp], C.c_int64),
        "ava_state_bytes": ([vp], C.c_int64),
        "ava_engine_set_segmented_read": ([vp, C.c_int32], C.c_int),
        "ava_engine_set_fast_products": ([vp, C.c_int32], C.c_int),
        "ava_engine_set_lanes": ([vp, C.c_int32], C.c_int),
        "ava_state_set_commit_at_end": ([vp, C.c_int32], C.c_int),
        "ava_split_step": ([vp, vp, vp, C.c_int32, C.c_int32, vp, vp, vp, vp, vp, vp], C.c_int),
        "ava_nccl_unique_id": ([C.c_char_p], C.c_int),
        "ava_nccl_comm_init": ([vp, C.c_int32, C.c_int32, C.c_char_p, C.POINTER(vp)], C.c_int),
        "ava_nccl_comm_destroy": ([vp], C.c_int),
        "ava_nccl_version": ([C.POINTER(C.c_int32)], C.c_int),
        "ava_split_wait": ([vp, vp, C.c_int32], C.c_int),
        "ava_engine_set_chunked_memory": ([vp, C.c_int32], C.c_int),
        "ava_engine_chunked_memory_counts": ([vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)], C.c_int),
        "ava_step_trace": ([vp, vp, C.c_uint32, fp, C.POINTER(vp)], C.c_int),
        "ava_trace_get": ([vp, C.c_char_p, C.c_int32, fp, C.c_int64], C.c_int64),
        "ava_trace_free": ([vp], None),
        "ava_prof_enable": ([vp, C.c_int32], C.c_int),
        "ava_prof_read": ([vp, C.c_char_p, C.POINTER(C.c_int64), C.POINTER(C.c_double)], C.c_int),
        "ava_prof_names": ([vp, C.c_char_p, C.c_int32], C.c_int),
        "ava_debug_keep": ([vp, C.c_int32], C.c_int),
        "ava_debug_width": ([vp, C.c_char_p], C.c_int64),
        "ava_debug_get": ([vp, C.c_char_p, C.c_int32, fp], C.c_int),
        "ava_op_q8_matmul": ([C.c_int, fp, C.c_int32, i8p, fp, C.c_int32, C.c_int32, fp], C.c_int),
        "ava_engine_fingerprint": ([vp], C.c_uint64),
        "ava_state_engine": ([vp], vp),
        "ava_state_set_seen": ([vp, C.c_int32, C.c_int64], C.c_int),
        "ava_state_save": ([vp, C.c_char_p], C.c_int),
        "ava_state_load": ([vp, C.c_char_p, C.c_int32, C.POINTER(vp)], C.c_int),
        "ava_ckpt_read_u32": ([vp, C.c_int32, u32p, C.c_int64], C.c_int),
        "ava_conv_path": ([C.c_char_p, C.c_char_p, C.c_char_p, C.c_int64], C.c_int),
        "ava_conv_save": ([C.c_char_p, C.c_char_p, vp], C.c_int),
        "ava_conv_load": ([vp, C.c_char_p, C.c_char_p, C.c_int32, C.POINTER(vp), i32p], C.c_int),
        "ava_step_sample": ([vp, vp, u32p, C.c_float, C.c_int32, C.POINTER(C.c_double), u32p], C.c_int),
        "ava_generate_sampled": ([vp, u32p, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_uint32, C.c_float, C.c_int32,
                                  C.POINTER(C.c_uint64), STOP_FN, vp, u32p, C.POINTER(C.c_int32)], C.c_int),
        "ava_op_sample": ([C.c_int, fp, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.POINTER(C.c_double), u32p], C.c_int),
        "ava_engine_device": ([vp], C.c_int),
        "ava_engine_config": ([vp], C.POINTER(AvaConfig)),
        "ava_splitmix64_next": ([C.POINTER(C.c_uint64)], C.c_uint64),
        "ava_pick": ([fp, C.c_int32, C.c_float, C.c_int32, C.POINTER(C.c_uint64), u32p, fp, fp], C.c_int),
        "ava_generate": ([vp, u32p, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_uint32, PICK_FN, STOP_FN, vp, u32p,
                          C.POINTER(C.c_int32)], C.c_int),
        "ava_loader_error": ([], C.c_char_p),
        "ava_ckpt_open": ([C.c_char_p, C.POINTER(vp)], C.c_int),
        "ava_ckpt_close": ([vp], None),
        "ava_ckpt_count": ([vp], C.c_int32),
        "ava_ckpt_find": ([vp, C.c_char_p], C.c_int32),
        "ava_ckpt_tensor": ([vp, C.c_int32, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), C.POINTER(C.c_int32), C.POINTER(C.c_int64)], C.c_int),
        "ava_ckpt_read_f32": ([vp, C.c_int32, fp, C.c_int64], C.c_int),
        "ava_arch_flags": ([C.c_char_p, C.POINTER(AvaConfig)], C.c_int),
        "ava_config_from_ckpt": ([vp, C.c_char_p, C.c_char_p, C.POINTER(AvaConfig)], C.c_int),
        "ava_engine_load_ckpt": ([vp, vp], C.c_int),
        "ava_op_q8_event_matmul": ([C.c_int, fp, C.c_int32, i8p, fp, C.c_int32, C.c_int32, fp], C.c_int),
        "ava_op_q8_tc_matmul": ([C.c_int, fp, C.c_int32, i8p, fp, C.c_int32, C.c_int32, fp, C.c_int32, fp], C.c_int),
        "ava_op_rmsnorm": ([C.c_int, fp, fp, C.c_int32, C.c_int32, fp], C.c_int),
        "ava_op_lif": ([C.c_int, fp, fp, fp, fp, fp, C.c_int32, fp, fp, fp, C.c_int32, C.c_int32, fp, fp, fp], C.c_int),
        "ava_op_kwta": ([C.c_int, fp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, fp], C.c_int),
        "ava_op_mem_heads": ([C.c_int, C.c_int32, C.c_int32, fp, fp, fp, fp, fp, fp, fp, fp, fp, fp], C.c_int),
        "ava_op_mem_chunk": ([C.c_int, C.c_int32, C.c_int32, C.c_int32, fp, fp, fp, fp, fp, fp, fp, fp, C.POINTER(C.c_int32)], C.c_int),
        "ava_op_engram_chunk": ([C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, fp, fp, fp, fp], C.c_int),
        "ava_op_q8_spike_tc_matmul": ([C.c_int, fp, C.c_int32, i8p, fp, C.c_int32, C.c_int32, fp], C.c_int),
        "ava_op_tc_bgemm": ([C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_int32, fp, fp, fp, fp, fp], C.c_int),
        "ava_debug_mem_heads_wait_runs_out": ([C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_uint32, C.POINTER(C.c_int32)], C.c_int),
        "ava_mem_heads_static": ([C.c_int, vp, C.c_int32, C.c_int32] + [vp] * 10, C.c_int),
        "ava_static_last_error": ([], C.c_char_p),
        "ava_op_attend": ([C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_int32, fp, fp, fp, fp], C.c_int),
        "ava_host_expf": ([C.c_float], C.c_float),
        "ava_host_logf": ([C.c_float], C.c_float),
        "ava_host_rsqrtf": ([C.c_float], C.c_float),
        "ava_host_sinf": ([C.c_float], C.c_float),
        "ava_host_cosf": ([C.c_float], C.c_float),
        "ava_op_math": ([C.c_int, C.c_int32, fp, C.c_int64, fp], C.c_int),
    }
    for name, (args, res) in sig.items():
        f = getattr(L, name)
        f.argtypes = args
        f.restype = res
    _lib = L
    return L


EXPORTS = ("ava_engine_create ava_engine_destroy ava_last_error ava_engine_set_f32 ava_engine_set_token_bytes ava_engine_set_q8 "
           "ava_engine_set_q8_from_f32 ava_engine_finalize ava_engine_blocker ava_state_new ava_state_destroy "
           "ava_state_rows ava_state_select ava_state_cat ava_state_seen ava_state_len ava_state_export "
           "ava_state_import ava_step ava_step_greedy ava_forward_with_state ava_step_device ava_prefill_device ava_state_set_kv_shard ava_shard_parts ava_split_step_begin ava_shard_partial ava_split_step_end ava_sync "
           "ava_engine_stream ava_engine_launches ava_engine_bytes ava_state_bytes ava_debug_keep ava_debug_width "
           "ava_debug_get ava_engine_set_segmented_read ava_engine_set_fast_products ava_engine_set_lanes ava_state_set_commit_at_end ava_split_step ava_nccl_unique_id ava_nccl_comm_init ava_nccl_comm_destroy ava_nccl_version ava_split_wait ava_engine_set_chunked_memory ava_engine_chunked_memory_counts ava_prof_enable ava_prof_read ava_prof_names ava_engine_fingerprint ava_state_engine ava_state_set_seen ava_state_save ava_state_load ava_ckpt_read_u32 ava_conv_path ava_conv_save ava_conv_load ava_step_sample ava_generate_sampled ava_op_sample ava_engine_device ava_engine_config ava_splitmix64_next ava_pick ava_generate ava_loader_error ava_ckpt_open ava_ckpt_close ava_ckpt_count ava_ckpt_find ava_ckpt_tensor ava_ckpt_read_f32 ava_arch_flags ava_config_from_ckpt ava_engine_load_ckpt ava_op_q8_matmul ava_op_q8_event_matmul ava_op_q8_tc_matmul ava_debug_mem_heads_wait_runs_out ava_op_tc_bgemm ava_op_q8_spike_tc_matmul ava_op_engram_chunk ava_op_mem_chunk ava_op_rmsnorm ava_op_lif ava_op_kwta ava_op_mem_heads ava_mem_heads_static ava_static_last_error ava_op_attend "
           "ava_host_expf ava_host_logf ava_host_rsqrtf ava_host_sinf ava_host_cosf ava_op_math ava_step_trace ava_trace_get ava_trace_free").split()


def _f32(a):
    return np.ascontiguousarray(a, np.float32)


def _p(a, t=fp):
    return a.ctypes.data_as(t) if a is not None else None


def host_math():
    """(expf, logf, rsqrtf, sinf, cosf) of the engine as C function addresses, for a checker that wants the same arithmetic."""
    L = lib()
    return tuple(C.cast(getattr(L, n), C.c_void_p) for n in ("ava_host_expf", "ava_host_logf", "ava_host_rsqrtf", "ava_host_sinf", "ava_host_cosf"))


class Rng:
    """SplitMix64 as the reference's tools use it (design-tests/nn/data/src/rng.rs:7-31), stepped by the library."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def next_u64(self) -> int:
        return int(lib().ava_splitmix64_next(C.byref(self.state)))


def pick(logits, temperature: float, top_k: int, rng: Rng | None, traced: bool = False):
    """`diary::pick` on one row of logits; traced: (token, ln p under the model, ln p under the sampler)."""
    a = _f32(logits).reshape(-1)
    tok, lp, slp = C.c_uint32(), C.c_float(), C.c_float()
    rc = lib().ava_pick(_p(a), a.size, temperature, top_k, C.byref(rng.state) if rng is not None else None, C.cast(C.byref(tok), u32p),
                        C.cast(C.byref(lp), fp), C.cast(C.byref(slp), fp))
    if rc != OK:
        raise EngineError(rc, "ava_pick: bad argument")
    return (tok.value, lp.value, slp.value) if traced else tok.value


def op_sample(logits, temperature: float, top_k: int, uniform, device: int = 0) -> np.ndarray:
    """The device sampler on rows of host logits (one uniform number per row)."""
    a = _f32(logits)
    a2 = a.reshape(-1, a.shape[-1])
    u = np.ascontiguousarray(uniform, np.float64).reshape(-1)
    out = np.empty(a2.shape[0], np.uint32)
    _rc(lib().ava_op_sample(device, _p(a2), a2.shape[0], a2.shape[1], temperature, top_k, _p(u, C.POINTER(C.c_double)), _p(out, u32p)))
    return out


def _loader_check(rc):
    if rc == NOT_APPLICABLE:
        raise NotApplicable(lib().ava_loader_error().decode())
    if rc != OK:
        raise EngineError(rc, lib().ava_loader_error().decode())


def _config_dict(c: "AvaConfig") -> dict:
    return {k: (float(getattr(c, k)) if k in _config.FIELDS_F32 else int(getattr(c, k))) for k in _config.FIELDS_I32 + _config.FIELDS_F32}


def arch_flags(flags: str, cfg: dict) -> dict:
    """`Arch::from_flags` on top of cfg: the configuration with an arch.txt line applied."""
    c = AvaConfig(**{k: cfg[k] for k in _config.FIELDS_I32 + _config.FIELDS_F32})
    _loader_check(lib().ava_arch_flags(flags.encode(), C.byref(c)))
    return _config_dict(c)


class Checkpoint:
    """A .safetensors file opened by the library's loader (host side; needs no GPU)."""

    def __init__(self, path: str):
        h = C.c_void_p()
        _loader_check(lib().ava_ckpt_open(str(path).encode(), C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            lib().ava_ckpt_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self):
        return lib().ava_ckpt_count(self.h)

    def info(self, i: int):
        name, dt, rank = C.c_char_p(), C.c_char_p(), C.c_int32()
        dims = (C.c_int64 * 4)()
        _loader_check(lib().ava_ckpt_tensor(self.h, i, C.byref(name), C.byref(dt), C.byref(rank), dims))
        return name.value.decode(), dt.value.decode(), tuple(dims[k] for k in range(rank.value))

    def names(self):
        return [self.info(i)[0] for i in range(len(self))]

    def get(self, name: str) -> np.ndarray:
        i = lib().ava_ckpt_find(self.h, name.encode())
        if i < 0:
            raise KeyError(name)
        _, dt, shape = self.info(i)
        if dt == "U32":
            out = np.empty(shape, np.uint32)
            _loader_check(lib().ava_ckpt_read_u32(self.h, i, _p(out, u32p), out.size))
            return out
        out = np.empty(shape, np.float32)
        _loader_check(lib().ava_ckpt_read_f32(self.h, i, _p(out), out.size))
        return out

    def config(self, kind: str, flags: str | None = None) -> dict:
        """`ckpt::detect` + the arch.txt line: the configuration the file was saved with."""
        c = AvaConfig()
        _loader_check(lib().ava_config_from_ckpt(self.h, kind.encode(), (flags or "").encode(), C.byref(c)))
        return _config_dict(c)


class ConvStore:
    """`ConvStore` of the reference: one saved state per conversation in a folder."""

    def __init__(self, folder: str):
        self.dir = str(folder)

    def path(self, conv_id: str) -> str:
        buf = C.create_string_buffer(4096)
        rc = lib().ava_conv_path(self.dir.encode(), conv_id.encode(), buf, 4096)
        if rc != OK:
            raise EngineError(rc, "conversation path")
        return buf.value.decode()

    def save(self, conv_id: str, state: "State"):
        state.m._check(lib().ava_conv_save(self.dir.encode(), conv_id.encode(), state.h))

    def load(self, conv_id: str, model: "Model", max_ctx: int = 4096):
        """("fresh", None), ("resumed", State) or ("stale", None)."""
        h, found = C.c_void_p(), C.c_int32()
        model._check(lib().ava_conv_load(model.h, self.dir.encode(), conv_id.encode(), max_ctx, C.byref(h), C.byref(found)))
        return ("fresh", "resumed", "stale")[found.value], (State(model, h) if found.value == 1 else None)


class Model:
    """`Model` of the reference for the one-token step: configuration + weights on one GPU."""

    def __init__(self, cfg: dict, weights: dict | None = None, device: int = 0):
        self.cfg = dict(cfg)
        self.device = device
        c = AvaConfig(**{k: cfg[k] for k in _config.FIELDS_I32 + _config.FIELDS_F32})
        h = C.c_void_p()
        rc = lib().ava_engine_create(C.byref(c), device, C.byref(h))
        if rc != OK:
            raise EngineError(rc, lib().ava_last_error(None).decode())
        self.h = h
        if weights is not None:
            self.load(weights)

    def _check(self, rc):
        if rc == NOT_APPLICABLE:
            why = lib().ava_engine_blocker(self.h)
            raise NotApplicable(why.decode() if why else "not applicable")
        if rc != OK:
            raise EngineError(rc, lib().ava_last_error(self.h).decode())

    def load(self, weights: dict):
        """weights: name -> f32 array, or (int8 [din, dout], f32 scale [dout]); then `set_int8` + `set_fused`."""
        L = lib()
        for name, w in weights.items():
            if name == "token_bytes":   # --letters: the tokens' spellings (data u8, offsets i64 [vocab + 1])
                self.set_token_bytes(*w)
            elif isinstance(w, tuple):
                q = np.ascontiguousarray(w[0], np.int8)
                sc = _f32(w[1])
                self._check(L.ava_engine_set_q8(self.h, name.encode(), _p(q, i8p), _p(sc), q.shape[0], q.shape[1]))
            else:
                a = _f32(w)
                self._check(L.ava_engine_set_f32(self.h, name.encode(), _p(a), a.size))
        self._check(L.ava_engine_finalize(self.h))

    def set_token_bytes(self, data, offsets):
        """--letters: every token's spelling, data[offsets[t]:offsets[t + 1]] (the reference reads its tokenizer's file)."""
        data = np.ascontiguousarray(data, np.uint8)
        offsets = np.ascontiguousarray(offsets, np.int64)
        if offsets.size != self.cfg["vocab"] + 1:
            raise ValueError("offsets: vocab + 1 values")
        self._check(lib().ava_engine_set_token_bytes(self.h, data.ctypes.data_as(C.POINTER(C.c_uint8)), offsets.ctypes.data_as(C.POINTER(C.c_int64))))

    @classmethod
    def from_checkpoint(cls, path: str, kind: str, flags: str | None = None, device: int = 0, token_bytes=None, **overrides) -> "Model":
        """`ckpt::load_auto` + `set_int8` + `set_fused`: the model a .safetensors file holds (`flags`: the arch.txt line
        beside it).  overrides: configuration fields the file does not fix (eng_cap, eng_store_bf16, ...)."""
        ck = Checkpoint(path)
        try:
            cfg = ck.config(kind, flags)
            cfg.update(overrides)
            m = cls(cfg, None, device)
            if token_bytes is not None:
                m.set_token_bytes(*token_bytes)
            rc = lib().ava_engine_load_ckpt(m.h, ck.h)
            if rc != OK:
                _loader_check(rc)
            m._check(lib().ava_engine_finalize(m.h))
            return m
        finally:
            ck.close()

    def generate(self, prompts, max_new: int, batch_rows: int = 256, eos: int = 256, pick_fn=None, stop_fn=None, max_ctx: int = 0):
        """`state::generate`: continuations of every prompt (lists of ids).  pick_fn(prompt_index, logits) -> token
        (None: greedy, taken on the device); stop_fn(prompt_index, tokens) -> bool.  Returns one list of ids per prompt."""
        lens = np.array([len(p) for p in prompts], np.int32)
        flat = np.ascontiguousarray(np.concatenate([np.asarray(p, np.uint32) for p in prompts]) if len(prompts) else np.zeros(0, np.uint32))
        out = np.zeros((len(prompts), max(max_new, 1)), np.uint32)
        out_len = np.zeros(len(prompts), np.int32)
        V = self.cfg["vocab"]
        errors = []

        def _pick(_user, r, lg, n):
            try:
                return int(pick_fn(r, np.ctypeslib.as_array(lg, shape=(n,)))) & 0xFFFFFFFF
            except Exception as ex:   # an exception must not cross the C frames
                errors.append(ex)
                return eos

        def _stop(_user, r, toks, n):
            try:
                return int(bool(stop_fn(r, [int(toks[i]) for i in range(n)])))
            except Exception as ex:
                errors.append(ex)
                return 1

        cp = PICK_FN(_pick) if pick_fn is not None else C.cast(None, PICK_FN)
        cs = STOP_FN(_stop) if stop_fn is not None else C.cast(None, STOP_FN)
        rc = lib().ava_generate(self.h, _p(flat, u32p), _p(lens, i32p), len(prompts), max_new, batch_rows, max_ctx, eos, cp, cs, None,
                                _p(out, u32p), _p(out_len, i32p))
        if errors:
            raise errors[0]
        self._check(rc)
        assert V > 0
        return [out[r, :out_len[r]].tolist() for r in range(len(prompts))]

    @property
    def fingerprint(self) -> int:
        return int(lib().ava_engine_fingerprint(self.h))

    def load_state(self, path: str, max_ctx: int = 4096) -> "State":
        """`State::load`: a state `State.save` wrote for this model."""
        h = C.c_void_p()
        rc = lib().ava_state_load(self.h, str(path).encode(), max_ctx, C.byref(h))
        if rc != OK:
            raise EngineError(rc, lib().ava_last_error(self.h).decode() or lib().ava_loader_error().decode() or "not a state of this model")
        return State(self, h)

    def fused_blocker(self):
        why = lib().ava_engine_blocker(self.h)
        return why.decode() if why else None

    def state(self, rows: int, max_ctx: int = 4096) -> "State":
        h = C.c_void_p()
        self._check(lib().ava_state_new(self.h, rows, max_ctx, C.byref(h)))
        return State(self, h)

    def step(self, st: "State", tok) -> np.ndarray:
        tok = np.ascontiguousarray(tok, np.uint32).reshape(-1)
        assert tok.size == st.rows
        logits = np.empty((st.rows, self.cfg["vocab"]), np.float32)
        self._check(lib().ava_step(self.h, st.h, _p(tok, u32p), _p(logits)))
        return logits

    def step_sample(self, st: "State", tok, temperature: float, top_k: int, uniform) -> np.ndarray:
        """One step with every row's next token drawn on the device (`diary::pick` with the row's uniform number)."""
        tok = np.ascontiguousarray(tok, np.uint32).reshape(-1)
        u = np.ascontiguousarray(uniform, np.float64).reshape(-1)
        assert tok.size == st.rows == u.size
        nxt = np.empty(st.rows, np.uint32)
        self._check(lib().ava_step_sample(self.h, st.h, _p(tok, u32p), temperature, top_k, _p(u, C.POINTER(C.c_double)), _p(nxt, u32p)))
        return nxt

    def generate_sampled(self, prompts, max_new: int, temperature: float, top_k: int, rng: "Rng", batch_rows: int = 256, eos: int = 256,
                         stop_fn=None, max_ctx: int = 0):
        """`state::generate` with `diary::pick(logits, temperature, top_k, rng)` as the pick, the draws taken on the device."""
        lens = np.array([len(p) for p in prompts], np.int32)
        flat = np.ascontiguousarray(np.concatenate([np.asarray(p, np.uint32) for p in prompts]))
        out = np.zeros((len(prompts), max(max_new, 1)), np.uint32)
        out_len = np.zeros(len(prompts), np.int32)
        errors = []

        def _stop(_user, r, toks, n):
            try:
                return int(bool(stop_fn(r, [int(toks[i]) for i in range(n)])))
            except Exception as ex:
                errors.append(ex)
                return 1

        cs = STOP_FN(_stop) if stop_fn is not None else C.cast(None, STOP_FN)
        rc = lib().ava_generate_sampled(self.h, _p(flat, u32p), _p(lens, i32p), len(prompts), max_new, batch_rows, max_ctx, eos, temperature, top_k,
                                        C.byref(rng.state), cs, None, _p(out, u32p), _p(out_len, i32p))
        if errors:
            raise errors[0]
        self._check(rc)
        return [out[r, :out_len[r]].tolist() for r in range(len(prompts))]

    def step_trace(self, st: "State", tok: int):
        """`Model::step_trace`: one token of a one-row state; (logits [vocab], get(name, block) -> f32 array)."""
        L = lib()
        logits = np.empty(self.cfg["vocab"], np.float32)
        h = C.c_void_p()
        self._check(L.ava_step_trace(self.h, st.h, int(tok), _p(logits), C.byref(h)))
        rec = {}

        def get(name: str, block: int) -> np.ndarray:
            n = L.ava_trace_get(h, name.encode(), block, None, 0)
            if n < 0:
                raise KeyError((name, block))
            a = np.empty(n, np.float32)
            L.ava_trace_get(h, name.encode(), block, _p(a), n)
            return a
        try:
            for blk in range(-1, self.cfg["n_blocks"]):
                for name in ("input_rms", "spikes", "winners", "hidden", "mem_write", "mem_read", "mem_keep", "mem_gate", "engram_attn", "engram_read"):
                    try:
                        rec[(name, blk)] = get(name, blk)
                    except KeyError:
                        pass
        finally:
            L.ava_trace_free(h)
        return logits, rec

    def step_greedy(self, st: "State", tok) -> np.ndarray:
        tok = np.ascontiguousarray(tok, np.uint32).reshape(-1)
        nxt = np.empty(st.rows, np.uint32)
        self._check(lib().ava_step_greedy(self.h, st.h, _p(tok, u32p), _p(nxt, u32p)))
        return nxt

    def forward_with_state(self, ids, st: "State", last_only: bool = False) -> np.ndarray:
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, t = ids.shape
        assert rows == st.rows
        V = self.cfg["vocab"]
        logits = np.empty((rows, V) if last_only else (rows, t, V), np.float32)
        self._check(lib().ava_forward_with_state(self.h, st.h, _p(ids, u32p), t, int(last_only), _p(logits)))
        return logits

    # device-resident form: raw device addresses (ints), nothing copied, nothing synchronised
    def step_device(self, st: "State", tok_ptr: int, logits_ptr: int | None, next_ptr: int | None):
        self._check(lib().ava_step_device(self.h, st.h, tok_ptr, logits_ptr, next_ptr))

    def prefill_device(self, st: "State", tok_ptr: int, t: int, chunk: int, logits_ptr: int | None, next_ptr: int | None):
        """tok_ptr: device u32 [t][rows] (time-major); queued on the engine's stream."""
        self._check(lib().ava_prefill_device(self.h, st.h, tok_ptr, t, chunk, logits_ptr, next_ptr))

    def sync(self):
        self._check(lib().ava_sync(self.h))

    @property
    def stream(self) -> int:
        return lib().ava_engine_stream(self.h)

    @property
    def launches(self) -> int:
        return lib().ava_engine_launches(self.h)

    @property
    def nbytes(self) -> int:
        return lib().ava_engine_bytes(self.h)

    def set_segmented_read(self, seg_len: int):
        """seg_len > 0: the engram is always read in segments of that many keys (the long-context / split-store path)."""
        self._check(lib().ava_engine_set_segmented_read(self.h, seg_len))

    def set_lanes(self, lanes: int):
        self._check(lib().ava_engine_set_lanes(self.h, int(lanes)))

    def set_chunked_memory(self, on: bool):
        """With fast products: prompt chunks read the fast-weight memory in its chunk-parallel form (default on)."""
        self._check(lib().ava_engine_set_chunked_memory(self.h, int(on)))

    def chunked_memory_counts(self):
        """(block, chunk) passes of the fast-weight memory in the chunk form, those that fell back to the token loop, and
        the chunks whose engram read took the causal pass."""
        a, b, c = C.c_int64(0), C.c_int64(0), C.c_int64(0)
        self._check(lib().ava_engine_chunked_memory_counts(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def set_fast_products(self, on: bool):
        """Dense products on the tensor cores: exact products, the tensor core's summation order (about 1e-6 of each
        sum's magnitudes from the reference's ordered sums; off by default)."""
        self._check(lib().ava_engine_set_fast_products(self.h, int(on)))

    def prof_enable(self, on: bool):
        self._check(lib().ava_prof_enable(self.h, int(on)))

    def prof_read(self) -> dict:
        """kernel -> (launches, total ms) since the section clock was switched on."""
        buf = C.create_string_buffer(4096)
        self._check(lib().ava_prof_names(self.h, buf, 4096))
        out = {}
        for name in buf.value.decode().split():
            n, ms = C.c_int64(), C.c_double()
            self._check(lib().ava_prof_read(self.h, name.encode(), C.byref(n), C.byref(ms)))
            out[name] = (n.value, ms.value)
        return out

    def debug_keep(self, on: bool):
        self._check(lib().ava_debug_keep(self.h, int(on)))

    def debug_get(self, name: str, block: int, rows: int) -> np.ndarray:
        w = lib().ava_debug_width(self.h, name.encode())
        if w < 0:
            raise KeyError(name)
        out = np.empty((rows, w), np.float32)
        self._check(lib().ava_debug_get(self.h, name.encode(), block, _p(out)))
        return out

    def close(self):
        if getattr(self, "h", None):
            lib().ava_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class State:
    """`State` of the reference: the carried membranes, traces, fast weights and engram store of `rows` rows."""

    def __init__(self, model: Model, h):
        self.m = model
        self.h = h

    @property
    def rows(self) -> int:
        return lib().ava_state_rows(self.h)

    @property
    def nbytes(self) -> int:
        return lib().ava_state_bytes(self.h)

    def select(self, idx) -> "State":
        idx = np.ascontiguousarray(idx, np.int32)
        h = C.c_void_p()
        self.m._check(lib().ava_state_select(self.h, _p(idx, i32p), idx.size, C.byref(h)))
        return State(self.m, h)

    @staticmethod
    def cat(parts) -> "State":
        arr = (C.c_void_p * len(parts))(*[p.h for p in parts])
        h = C.c_void_p()
        parts[0].m._check(lib().ava_state_cat(arr, len(parts), C.byref(h)))
        return State(parts[0].m, h)

    def save(self, path: str):
        """`State::save`: a safetensors file under the reference's tensor names (whole or absent: tmp + rename)."""
        self.m._check(lib().ava_state_save(self.h, str(path).encode()))

    def set_commit_at_end(self, on: bool):
        """A host-facing call that fails after work was queued puts the state back as it was (twice the fast-weight memory)."""
        self.m._check(lib().ava_state_set_commit_at_end(self.h, int(on)))

    def seen(self, row: int) -> int:
        return lib().ava_state_seen(self.h, row)

    def get(self, row: int, name: str) -> np.ndarray:
        n = lib().ava_state_len(self.h, row, name.encode())
        if n < 0:
            raise KeyError(name)
        out = np.empty(n, np.float32)
        if n:
            self.m._check(lib().ava_state_export(self.h, row, name.encode(), _p(out)))
        return out

    def put(self, row: int, name: str, a):
        a = _f32(a)
        self.m._check(lib().ava_state_import(self.h, row, name.encode(), _p(a), a.size))

    def close(self):
        if getattr(self, "h", None) and getattr(self.m, "h", None):
            lib().ava_state_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------------------------- single operators
def _rc(rc):
    if rc == NOT_APPLICABLE:
        raise NotApplicable("operator shape not covered")
    if rc != OK:
        raise EngineError(rc, "operator failed")


def op_q8_matmul(x, q, scale, device=0, event=False):
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    q = np.ascontiguousarray(q, np.int8)
    scale = _f32(scale)
    y = np.empty((x2.shape[0], q.shape[1]), np.float32)
    f = lib().ava_op_q8_event_matmul if event else lib().ava_op_q8_matmul
    _rc(f(device, _p(x2), x2.shape[0], _p(q, i8p), _p(scale), q.shape[0], q.shape[1], _p(y)))
    return y.reshape(x.shape[:-1] + (q.shape[1],))


def op_q8_tc_matmul(x, q, scale, device=0, reps=0):
    """The product on the tensor cores (exact products, the tensor core's summation order).  With reps > 0 also
    returns the milliseconds per launch of the product kernel alone: (y, ms)."""
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    q = np.ascontiguousarray(q, np.int8)
    scale = _f32(scale)
    y = np.empty((x2.shape[0], q.shape[1]), np.float32)
    ms = C.c_float(0.0)
    _rc(lib().ava_op_q8_tc_matmul(device, _p(x2), x2.shape[0], _p(q, i8p), _p(scale), q.shape[0], q.shape[1], _p(y), reps,
                                  C.cast(C.byref(ms), fp)))
    y = y.reshape(x.shape[:-1] + (q.shape[1],))
    return (y, ms.value) if reps > 0 else y


def op_rmsnorm(x, gain, device=0):
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    y = np.empty_like(x2)
    g = _f32(gain)
    _rc(lib().ava_op_rmsnorm(device, _p(x2), _p(g), x2.shape[0], x2.shape[1], _p(y)))
    return y.reshape(x.shape)


def op_lif(cur, beta, v0, s0, theta=None, rho=None, gain=None, a0=None, spikes=2, device=0):
    cur = _f32(cur)
    m, d = cur.shape
    arrs = [_f32(a) if a is not None else None for a in (beta, theta, rho, gain, v0, s0, a0)]
    beta, theta, rho, gain, v0, s0, a0 = arrs
    s1, v1 = np.empty((m, d), np.float32), np.empty((m, d), np.float32)
    a1 = np.empty((m, d), np.float32) if rho is not None else None
    _rc(lib().ava_op_lif(device, _p(cur), _p(beta), _p(theta), _p(rho), _p(gain), spikes, _p(v0), _p(s0), _p(a0), m, d,
                         _p(s1), _p(v1), _p(a1)))
    return s1, v1, a1


def op_kwta(u, k, relu2, device=0):
    u = _f32(u)
    m, n = u.shape
    a = np.empty_like(u)
    _rc(lib().ava_op_kwta(device, _p(u), m, n, k, int(relu2), _p(a)))
    return a


def op_tc_bgemm(a, b, colscale=None, c_in=None, device=0):
    """c[i] = a[i] . b[i]^T (+ colscale[i][n] * c_in[i]) on the tensor cores with three bf16 limbs per operand."""
    a, b = _f32(a), _f32(b)
    batch, m, k = a.shape
    n = b.shape[1]
    c = np.zeros((batch, m, n), np.float32) if c_in is None else _f32(c_in).copy()
    limb_sum = np.zeros_like(c) if colscale is not None else None
    cs = None if colscale is None else _f32(colscale)
    _rc(lib().ava_op_tc_bgemm(device, batch, m, n, k, _p(a), _p(b), _p(cs) if cs is not None else None, _p(c), _p(limb_sum) if limb_sum is not None else None))
    return (c, limb_sum) if colscale is not None else c


def op_q8_spike_tc_matmul(x, q, scale, y, device=0):
    """y + (x . q) * scale for rows x of small integers, on the tensor cores (exact)."""
    x, scale = _f32(x), _f32(scale)
    q = np.ascontiguousarray(q, np.int8)
    m, din = x.shape
    dout = q.shape[1]
    out = np.array(y, np.float32, copy=True)
    _rc(lib().ava_op_q8_spike_tc_matmul(device, _p(x), m, _p(q, i8p), _p(scale), din, dout, _p(out)))
    return out


def op_engram_chunk(qkv, k_prev, v_prev, start=0, device=0):
    """The engram's causal read over a chunk: qkv [t][rows][3 d], k_prev / v_prev [rows][d // 64][n0][64]; returns o [t][rows][d]."""
    qkv = _f32(qkv)
    t, rows, d3 = qkv.shape
    d = d3 // 3
    k_prev, v_prev = _f32(k_prev), _f32(v_prev)
    n0 = k_prev.shape[2]
    o = np.zeros((t, rows, d), np.float32)
    _rc(lib().ava_op_engram_chunk(device, rows, t, n0, start, d, _p(qkv), _p(k_prev) if n0 else None, _p(v_prev) if n0 else None, _p(o)))
    return o


def op_mem_chunk(qn, e, w, ah, v, la, f, device=0):
    """The chunk-parallel fast-weight memory over t tokens: inputs [t][hb][hs], f [hb][hs][hs]; returns (y, f', out_of_range)."""
    qn, e, w, ah, v, la = map(_f32, (qn, e, w, ah, v, la))
    t, hb, hs = qn.shape
    f = np.array(f, np.float32, copy=True).reshape(hb, hs, hs)
    y = np.zeros((t, hb, hs), np.float32)
    oor = C.c_int32(0)
    _rc(lib().ava_op_mem_chunk(device, t, hb, hs, _p(qn), _p(e), _p(w), _p(ah), _p(v), _p(la), _p(f), _p(y), C.byref(oor)))
    return y, f, bool(oor.value)


def op_mem_heads(e, v, w, ah, qg, ex, qw, qa, f, device=0):
    e, v, w, ah, qg, ex, qw, qa = map(_f32, (e, v, w, ah, qg, ex, qw, qa))
    m, hs = e.shape
    f = np.array(f, np.float32, copy=True).reshape(m, hs, hs)
    y = np.empty((m, hs), np.float32)
    _rc(lib().ava_op_mem_heads(device, m, hs, _p(e), _p(v), _p(w), _p(ah), _p(qg), _p(ex), _p(qw), _p(qa), _p(f), _p(y)))
    return y, f


def op_attend(q, kc, vc, bf16_store=False, device=0):
    q, kc, vc = _f32(q), _f32(kc), _f32(vc)
    m, n, hs = kc.shape
    out = np.empty((m, hs), np.float32)
    _rc(lib().ava_op_attend(device, m, n, hs, int(bf16_store), _p(q), _p(kc), _p(vc), _p(out)))
    return out


def op_math(which, x, device=0):
    x = _f32(x).reshape(-1)
    y = np.empty_like(x)
    _rc(lib().ava_op_math(device, which, _p(x), x.size, _p(y)))
    return y
