//! Rust binding of libava_engine.so (include/ava_engine.h) for the reference's crate `ava_gpu`
//! (design-tests/nn/gpu).  NOT COMPILED in the environment this repository was built in (no Rust tool chain there):
//! it is the text a maintainer would add as `src/b200.rs`, written against the C header line by line.
//!
//! It gives the engine the reference's own method names so that the callers of the one-token path
//! (`ava_live`, `generate_gpu`, `talk_bench`, `int8_bench`, `state::generate`) switch by changing a type:
//!   Model::state(rows)                  -> B200Model::state(rows, max_ctx)
//!   Model::step(&mut Stream, tok)       -> B200Model::step(&mut B200State, &[tok]) (one token per row)
//!   Model::forward_with_state(ids, st)  -> B200Model::forward_with_state(ids, t, &mut st, last_only)
//!   State::select / State::cat          -> B200State::select / B200State::cat
//! `Ok(None)` of the reference's fused step ("this fast path does not apply") is status 1 here.

use std::ffi::{c_char, c_int, c_void, CStr, CString};

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct AvaConfig {
    pub vocab: i32,
    pub d: i32,
    pub n_blocks: i32,
    pub hidden: i32,
    pub kwta_k: i32,
    pub head_size: i32,
    pub eng_block: i32,
    pub eng_head_size: i32,
    pub eng_store_bf16: i32,
    pub eng_cap: i32,
    pub gate_rank: i32,
    pub spikes: i32,
    pub alif: i32,
    pub theta: i32,
    pub lif_scale: i32,
    pub value_residual: i32,
    pub relu2: i32,
    pub dense: i32,
    pub out_gate: i32,
    pub fast_mem: i32,
    pub dendrite: i32,
    pub neuromod: i32,
    pub stp: i32,
    pub thalamus: i32,
    pub dopamine: i32,
    pub mood: i32,
    pub cb_units: i32,
    pub letters: i32,
    pub rhythm: i32,
    pub mem_momentum: f32,
    pub slope: f32,
}

#[repr(C)]
pub struct AvaEngine { _p: [u8; 0] }
#[repr(C)]
pub struct AvaState { _p: [u8; 0] }
#[repr(C)]
pub struct AvaCkpt { _p: [u8; 0] }
#[repr(C)]
pub struct AvaTrace { _p: [u8; 0] }

#[link(name = "ava_engine")]
extern "C" {
    // ---- begin: generated from include/ava_engine.h by bindings/gen_extern.py
    pub fn ava_engine_create(cfg: *const AvaConfig, device: c_int, out: *mut *mut AvaEngine) -> c_int;
    pub fn ava_engine_destroy(e: *mut AvaEngine);
    pub fn ava_last_error(e: *const AvaEngine) -> *const c_char;
    pub fn ava_engine_set_f32(e: *mut AvaEngine, name: *const c_char, data: *const f32, n: i64) -> c_int;
    pub fn ava_engine_set_token_bytes(e: *mut AvaEngine, bytes: *const u8, offsets: *const i64) -> c_int;
    pub fn ava_engine_set_q8(e: *mut AvaEngine, name: *const c_char, q: *const i8, scale: *const f32, din: i32, dout: i32) -> c_int;
    pub fn ava_engine_set_q8_from_f32(e: *mut AvaEngine, name: *const c_char, w: *const f32, din: i32, dout: i32) -> c_int;
    pub fn ava_engine_finalize(e: *mut AvaEngine) -> c_int;
    pub fn ava_engine_blocker(e: *const AvaEngine) -> *const c_char;
    pub fn ava_state_new(e: *mut AvaEngine, rows: i32, max_ctx: i32, out: *mut *mut AvaState) -> c_int;
    pub fn ava_state_destroy(s: *mut AvaState);
    pub fn ava_state_rows(s: *const AvaState) -> i32;
    pub fn ava_state_select(s: *const AvaState, idx: *const i32, n: i32, out: *mut *mut AvaState) -> c_int;
    pub fn ava_state_cat(parts: *const *const AvaState, n: i32, out: *mut *mut AvaState) -> c_int;
    pub fn ava_state_seen(s: *const AvaState, row: i32) -> i64;
    pub fn ava_state_len(s: *const AvaState, row: i32, name: *const c_char) -> i64;
    pub fn ava_state_export(s: *const AvaState, row: i32, name: *const c_char, out: *mut f32) -> c_int;
    pub fn ava_state_import(s: *mut AvaState, row: i32, name: *const c_char, in_: *const f32, n: i64) -> c_int;
    pub fn ava_step(e: *mut AvaEngine, s: *mut AvaState, tok: *const u32, logits: *mut f32) -> c_int;
    pub fn ava_step_greedy(e: *mut AvaEngine, s: *mut AvaState, tok: *const u32, next: *mut u32) -> c_int;
    pub fn ava_forward_with_state(e: *mut AvaEngine, s: *mut AvaState, ids: *const u32, t: i32, last_only: i32, logits: *mut f32) -> c_int;
    pub fn ava_state_set_commit_at_end(s: *mut AvaState, on: i32) -> c_int;
    pub fn ava_step_device(e: *mut AvaEngine, s: *mut AvaState, tok_device: *const u32, logits_device: *mut f32, next_device: *mut u32) -> c_int;
    pub fn ava_prefill_device(e: *mut AvaEngine, s: *mut AvaState, tok_device: *const u32, t: i32, chunk: i32, logits_device: *mut f32, next_device: *mut u32) -> c_int;
    pub fn ava_sync(e: *mut AvaEngine) -> c_int;
    pub fn ava_engine_stream(e: *mut AvaEngine) -> *mut c_void;
    pub fn ava_engine_launches(e: *const AvaEngine) -> i64;
    pub fn ava_engine_bytes(e: *const AvaEngine) -> i64;
    pub fn ava_state_bytes(s: *const AvaState) -> i64;
    pub fn ava_engine_set_segmented_read(e: *mut AvaEngine, seg_len: i32) -> c_int;
    pub fn ava_engine_set_lanes(e: *mut AvaEngine, lanes: i32) -> c_int;
    pub fn ava_engine_set_fast_products(e: *mut AvaEngine, on: i32) -> c_int;
    pub fn ava_engine_set_chunked_memory(e: *mut AvaEngine, on: i32) -> c_int;
    pub fn ava_engine_chunked_memory_counts(e: *const AvaEngine, chunked: *mut i64, token_loop: *mut i64, engram_chunks: *mut i64) -> c_int;
    pub fn ava_state_set_kv_shard(s: *mut AvaState, rank: i32, world: i32, block: i64, position: i64) -> c_int;
    pub fn ava_shard_parts(e: *const AvaEngine, s: *const AvaState) -> i32;
    pub fn ava_split_step_begin(e: *mut AvaEngine, s: *mut AvaState, tok_device: *const u32, qkv_device: *mut f32) -> c_int;
    pub fn ava_shard_partial(e: *mut AvaEngine, s: *mut AvaState, qkv_device: *const f32, partial_device: *mut f32) -> c_int;
    pub fn ava_split_step_end(e: *mut AvaEngine, s: *mut AvaState, gathered_device: *const f32, world: i32, logits_device: *mut f32, next_device: *mut u32) -> c_int;
    pub fn ava_split_step(e: *mut AvaEngine, s: *mut AvaState, nccl_comm: *mut c_void, rank: i32, world: i32, tok_device: *const u32, qkv_device: *mut f32, partial_device: *mut f32, gathered_device: *mut f32, logits_device: *mut f32, next_device: *mut u32) -> c_int;
    pub fn ava_nccl_unique_id(id128: *mut u8) -> c_int;
    pub fn ava_nccl_comm_init(e: *mut AvaEngine, world: i32, rank: i32, id128: *const u8, comm: *mut *mut c_void) -> c_int;
    pub fn ava_nccl_comm_destroy(comm: *mut c_void) -> c_int;
    pub fn ava_nccl_version(version: *mut i32) -> c_int;
    pub fn ava_split_wait(e: *mut AvaEngine, nccl_comm: *mut c_void, timeout_ms: i32) -> c_int;
    pub fn ava_step_trace(e: *mut AvaEngine, s: *mut AvaState, tok: u32, logits: *mut f32, out: *mut *mut AvaTrace) -> c_int;
    pub fn ava_trace_get(t: *const AvaTrace, name: *const c_char, block: i32, out: *mut f32, cap: i64) -> i64;
    pub fn ava_trace_free(t: *mut AvaTrace);
    pub fn ava_prof_enable(e: *mut AvaEngine, on: i32) -> c_int;
    pub fn ava_prof_read(e: *mut AvaEngine, kernel: *const c_char, launches: *mut i64, ms: *mut f64) -> c_int;
    pub fn ava_prof_names(e: *mut AvaEngine, out: *mut c_char, cap: i32) -> c_int;
    pub fn ava_debug_keep(e: *mut AvaEngine, on: i32) -> c_int;
    pub fn ava_debug_width(e: *const AvaEngine, name: *const c_char) -> i64;
    pub fn ava_debug_get(e: *mut AvaEngine, name: *const c_char, block: i32, out: *mut f32) -> c_int;
    pub fn ava_loader_error() -> *const c_char;
    pub fn ava_ckpt_open(path: *const c_char, out: *mut *mut AvaCkpt) -> c_int;
    pub fn ava_ckpt_close(c: *mut AvaCkpt);
    pub fn ava_ckpt_count(c: *const AvaCkpt) -> i32;
    pub fn ava_ckpt_find(c: *const AvaCkpt, name: *const c_char) -> i32;
    pub fn ava_ckpt_tensor(c: *const AvaCkpt, i: i32, name: *mut *const c_char, dtype: *mut *const c_char, rank: *mut i32, dims: *mut i64) -> c_int;
    pub fn ava_ckpt_read_f32(c: *const AvaCkpt, i: i32, out: *mut f32, n: i64) -> c_int;
    pub fn ava_ckpt_read_u32(c: *const AvaCkpt, i: i32, out: *mut u32, n: i64) -> c_int;
    pub fn ava_arch_flags(flags: *const c_char, cfg: *mut AvaConfig) -> c_int;
    pub fn ava_config_from_ckpt(c: *const AvaCkpt, kind: *const c_char, arch_flags: *const c_char, out: *mut AvaConfig) -> c_int;
    pub fn ava_engine_load_ckpt(e: *mut AvaEngine, c: *const AvaCkpt) -> c_int;
    pub fn ava_engine_fingerprint(e: *const AvaEngine) -> u64;
    pub fn ava_state_engine(s: *const AvaState) -> *mut AvaEngine;
    pub fn ava_state_set_seen(s: *mut AvaState, row: i32, seen: i64) -> c_int;
    pub fn ava_state_save(s: *const AvaState, path: *const c_char) -> c_int;
    pub fn ava_state_load(e: *mut AvaEngine, path: *const c_char, max_ctx: i32, out: *mut *mut AvaState) -> c_int;
    pub fn ava_conv_path(dir: *const c_char, id: *const c_char, out: *mut c_char, n: i64) -> c_int;
    pub fn ava_conv_save(dir: *const c_char, id: *const c_char, s: *const AvaState) -> c_int;
    pub fn ava_conv_load(e: *mut AvaEngine, dir: *const c_char, id: *const c_char, max_ctx: i32, out: *mut *mut AvaState, found: *mut i32) -> c_int;
    pub fn ava_engine_config(e: *const AvaEngine) -> *const AvaConfig;
    pub fn ava_engine_device(e: *const AvaEngine) -> c_int;
    pub fn ava_splitmix64_next(state: *mut u64) -> u64;
    pub fn ava_pick(logits: *const f32, vocab: i32, temperature: f32, top_k: i32, rng_state: *mut u64, token: *mut u32, logp: *mut f32, sample_logp: *mut f32) -> c_int;
    pub fn ava_step_sample(e: *mut AvaEngine, s: *mut AvaState, tok: *const u32, temperature: f32, top_k: i32, uniform: *const f64, next: *mut u32) -> c_int;
    pub fn ava_generate(e: *mut AvaEngine, prompts: *const u32, prompt_len: *const i32, n_prompts: i32, max_new: i32, batch_rows: i32, max_ctx: i32, eos: u32, pick: Option<extern "C" fn(*mut c_void, i32, *const f32, i32) -> u32>, stop: Option<extern "C" fn(*mut c_void, i32, *const u32, i32) -> c_int>, user: *mut c_void, out: *mut u32, out_len: *mut i32) -> c_int;
    pub fn ava_generate_sampled(e: *mut AvaEngine, prompts: *const u32, prompt_len: *const i32, n_prompts: i32, max_new: i32, batch_rows: i32, max_ctx: i32, eos: u32, temperature: f32, top_k: i32, rng_state: *mut u64, stop: Option<extern "C" fn(*mut c_void, i32, *const u32, i32) -> c_int>, user: *mut c_void, out: *mut u32, out_len: *mut i32) -> c_int;
    pub fn ava_op_q8_matmul(device: c_int, x: *const f32, m: i32, q: *const i8, scale: *const f32, din: i32, dout: i32, y: *mut f32) -> c_int;
    pub fn ava_op_q8_event_matmul(device: c_int, x: *const f32, m: i32, q: *const i8, scale: *const f32, din: i32, dout: i32, y: *mut f32) -> c_int;
    pub fn ava_op_q8_tc_matmul(device: c_int, x: *const f32, m: i32, q: *const i8, scale: *const f32, din: i32, dout: i32, y: *mut f32, reps: i32, ms_per_launch: *mut f32) -> c_int;
    pub fn ava_op_sample(device: c_int, logits: *const f32, m: i32, vocab: i32, temperature: f32, top_k: i32, uniform: *const f64, next: *mut u32) -> c_int;
    pub fn ava_op_rmsnorm(device: c_int, x: *const f32, gain: *const f32, m: i32, n: i32, y: *mut f32) -> c_int;
    pub fn ava_op_lif(device: c_int, cur: *const f32, beta: *const f32, theta: *const f32, rho: *const f32, gain: *const f32, spikes: i32, v0: *const f32, s0: *const f32, a0: *const f32, m: i32, d: i32, s1: *mut f32, v1: *mut f32, a1: *mut f32) -> c_int;
    pub fn ava_op_kwta(device: c_int, u: *const f32, m: i32, n: i32, k: i32, relu2: i32, a: *mut f32) -> c_int;
    pub fn ava_op_mem_heads(device: c_int, m: i32, hs: i32, e: *const f32, v: *const f32, w: *const f32, ah: *const f32, qg: *const f32, ex: *const f32, qw: *const f32, qa: *const f32, f: *mut f32, y: *mut f32) -> c_int;
    pub fn ava_op_q8_spike_tc_matmul(device: c_int, x: *const f32, m: i32, q: *const i8, scale: *const f32, din: i32, dout: i32, y: *mut f32) -> c_int;
    pub fn ava_mem_heads_static(device: c_int, stream: *mut c_void, m: i32, hs: i32, e: *const f32, v: *const f32, w: *const f32, ah: *const f32, qg: *const f32, ex: *const f32, qw: *const f32, qa: *const f32, f: *mut f32, y: *mut f32) -> c_int;
    pub fn ava_static_last_error() -> *const c_char;
    pub fn ava_op_attend(device: c_int, m: i32, n: i32, hs: i32, bf16_store: i32, q: *const f32, kc: *const f32, vc: *const f32, out: *mut f32) -> c_int;
    pub fn ava_op_engram_chunk(device: c_int, rows: i32, t: i32, n0: i32, start: i32, d: i32, qkv: *const f32, k_prev: *const f32, v_prev: *const f32, o: *mut f32) -> c_int;
    pub fn ava_op_tc_bgemm(device: c_int, batch: i32, m: i32, n: i32, k: i32, a: *const f32, b: *const f32, colscale: *const f32, c: *mut f32, c_limb_sum: *mut f32) -> c_int;
    pub fn ava_op_mem_chunk(device: c_int, t: i32, hb: i32, hs: i32, qn: *const f32, e: *const f32, w: *const f32, ah: *const f32, v: *const f32, la: *const f32, f: *mut f32, y: *mut f32, out_of_range: *mut i32) -> c_int;
    pub fn ava_debug_mem_heads_wait_runs_out(device: c_int, m: i32, hs: i32, chunk: i32, poll_limit: u32, state_changed: *mut i32) -> c_int;
    pub fn ava_host_expf(x: f32) -> f32;
    pub fn ava_host_logf(x: f32) -> f32;
    pub fn ava_host_rsqrtf(x: f32) -> f32;
    pub fn ava_host_sinf(x: f32) -> f32;
    pub fn ava_host_cosf(x: f32) -> f32;
    pub fn ava_op_math(device: c_int, which: i32, x: *const f32, n: i64, y: *mut f32) -> c_int;
    // ---- end: generated
}

#[derive(Debug)]
pub enum B200Error {
    /// status 1: the engine does not cover this configuration (the reference's `Ok(None)`), with the reason
    NotApplicable(String),
    Failed(i32, String),
}

pub struct B200Model {
    h: *mut AvaEngine,
    pub vocab: usize,
}
pub struct B200State {
    h: *mut AvaState,
}

impl B200Model {
    fn check(&self, rc: c_int) -> Result<(), B200Error> {
        match rc {
            0 => Ok(()),
            1 => {
                let p = unsafe { ava_engine_blocker(self.h) };
                let why = if p.is_null() { String::new() } else { unsafe { CStr::from_ptr(p) }.to_string_lossy().into_owned() };
                Err(B200Error::NotApplicable(why))
            }
            rc => Err(B200Error::Failed(rc, unsafe { CStr::from_ptr(ava_last_error(self.h)) }.to_string_lossy().into_owned())),
        }
    }

    /// `Model::new` + `set_int8(true)` + `set_fused(true)`: `f32s` are (tensor name, values), `q8s` (name, W [din, dout]
    /// f32 row-major) are quantised by the engine exactly as `ava_parts::quant::quantize_int8`.
    pub fn new(cfg: &AvaConfig, device: i32, f32s: &[(&str, &[f32])], q8s: &[(&str, &[f32], usize, usize)]) -> Result<B200Model, B200Error> {
        let mut h = std::ptr::null_mut();
        let rc = unsafe { ava_engine_create(cfg, device, &mut h) };
        if rc != 0 {
            return Err(B200Error::Failed(rc, unsafe { CStr::from_ptr(ava_last_error(std::ptr::null())) }.to_string_lossy().into_owned()));
        }
        let m = B200Model { h, vocab: cfg.vocab as usize };
        for (name, v) in f32s {
            let n = CString::new(*name).unwrap();
            m.check(unsafe { ava_engine_set_f32(m.h, n.as_ptr(), v.as_ptr(), v.len() as i64) })?;
        }
        for (name, w, din, dout) in q8s {
            let n = CString::new(*name).unwrap();
            m.check(unsafe { ava_engine_set_q8_from_f32(m.h, n.as_ptr(), w.as_ptr(), *din as i32, *dout as i32) })?;
        }
        m.check(unsafe { ava_engine_finalize(m.h) })?;
        Ok(m)
    }

    /// `Model::state(rows)`
    pub fn state(&self, rows: usize, max_ctx: usize) -> Result<B200State, B200Error> {
        let mut s = std::ptr::null_mut();
        self.check(unsafe { ava_state_new(self.h, rows as i32, max_ctx as i32, &mut s) })?;
        Ok(B200State { h: s })
    }

    /// `Model::step`: one token per row, logits [rows, vocab]
    pub fn step(&self, st: &mut B200State, tok: &[u32]) -> Result<Vec<f32>, B200Error> {
        let rows = unsafe { ava_state_rows(st.h) } as usize;
        assert_eq!(tok.len(), rows);
        let mut logits = vec![0f32; rows * self.vocab];
        self.check(unsafe { ava_step(self.h, st.h, tok.as_ptr(), logits.as_mut_ptr()) })?;
        Ok(logits)
    }

    /// `Model::forward_with_state(ids [rows, t], &mut State)`
    pub fn forward_with_state(&self, ids: &[u32], t: usize, st: &mut B200State, last_only: bool) -> Result<Vec<f32>, B200Error> {
        let rows = unsafe { ava_state_rows(st.h) } as usize;
        assert_eq!(ids.len(), rows * t);
        let mut logits = vec![0f32; rows * self.vocab * if last_only { 1 } else { t }];
        self.check(unsafe { ava_forward_with_state(self.h, st.h, ids.as_ptr(), t as i32, last_only as i32, logits.as_mut_ptr()) })?;
        Ok(logits)
    }
}

impl B200State {
    /// `State::select`
    pub fn select(&self, idx: &[i32]) -> Option<B200State> {
        let mut s = std::ptr::null_mut();
        (unsafe { ava_state_select(self.h, idx.as_ptr(), idx.len() as i32, &mut s) } == 0).then_some(B200State { h: s })
    }
    /// `State::cat`
    pub fn cat(parts: &[&B200State]) -> Option<B200State> {
        let ps: Vec<*const AvaState> = parts.iter().map(|p| p.h as *const AvaState).collect();
        let mut s = std::ptr::null_mut();
        (unsafe { ava_state_cat(ps.as_ptr(), ps.len() as i32, &mut s) } == 0).then_some(B200State { h: s })
    }
    pub fn seen(&self, row: usize) -> i64 {
        unsafe { ava_state_seen(self.h, row as i32) }
    }
}

impl Drop for B200State {
    fn drop(&mut self) {
        unsafe { ava_state_destroy(self.h) }
    }
}
impl Drop for B200Model {
    fn drop(&mut self) {
        unsafe { ava_engine_destroy(self.h) }
    }
}
