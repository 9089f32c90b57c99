"""Benchmark of the block step: batch-256 decode of the Ava-0.4-shaped model on N B200s.

A "step" is one decoded token for every resident sequence (256 per GPU; sequences are independent, so each rank steps
its own 256 with no data-path collective: weak scaling).  Workload = benchmark configuration 1: each sequence has read a
prompt and is decoding with its membranes, thresholds, 12 fast-synapse 768x768 f32 matrices and the block-6 bf16 KV
store resident in HBM.  The KV length over the timed steps is centred on the configuration's mean decode context
(1024-token prompt + 1024 decode tokens: mean 1535.5), reached by untimed steps.

  value      tokens/s over all ranks, inputs resident in HBM, CUDA events on the engine's stream, max over ranks
  e2e        the same through ava_step (host token ids in, host logits out, copies inside the timed region)
  roofline   the fast-weight state pass (mem_heads kernel): algorithmic bytes per launch / its mean launch time
  cpu_baseline / --impl reference
             the CPU oracle (a restatement of the reference's int8 CPU engine; the reference itself needs a Rust tool
             chain and cannot be built here) on the host cores, on a bounded sample of the same workload
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tokens/s (batch 256 per GPU, Ava-0.4-shaped int8 model)"
UNIT = "tokens/s"
ROWS_PER_GPU = 256
TRAFFIC_PER_STATE_BYTE = 0.813  # ncu: DRAM bytes moved per algorithmic byte of the state pass (capture of a 64-row lane, profiles/)
MEAN_CTX = 1536  # mean KV length of the decode phase of configuration 1 (1024 prompt + 1024 decode)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class Clocks:
    """Samples the SM clock and the throttle reasons while the steps run: NVML from a thread every 10 ms (reading only),
    or nvidia-smi's own loop when the NVML module is missing.  start() before the warm-up steps, mark() when the timed
    region begins: the summary is over the samples from the mark on (over all of them when the region was too short
    to hold three)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.p = None
        self.thread = None
        self.samples = []   # (time, sm MHz, reasons bitmask)
        self.t_mark = None
        self.stop_flag = False
        self.max_mhz = None

    def _loop(self, nv, h):
        while not self.stop_flag:
            try:
                self.samples.append((time.perf_counter(), float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                     int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            # NVML counts physical GPUs; CUDA_VISIBLE_DEVICES may renumber them for this process
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            ent = vis.split(",")[self.gpu].strip() if vis else str(self.gpu)
            h = nv.nvmlDeviceGetHandleByUUID(ent) if ent.startswith("GPU-") else nv.nvmlDeviceGetHandleByIndex(int(ent))
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._loop, args=(nv, h), daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        try:  # nvidia-smi's own loop beside it: the summary falls back to it when the thread got too few samples
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.gpu)],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    def mark(self):
        self.t_mark = time.perf_counter()

    def stop(self) -> dict:
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            timed = [x for x in self.samples if self.t_mark is not None and x[0] >= self.t_mark]
            use, window = (timed, "timed steps") if len(timed) >= 3 else (self.samples, "warm-up and timed steps")
            mask = 0
            for x in use:
                mask |= x[2]
            reasons = sorted(name for bit, name in self.BITS.items() if mask & bit)
            if len(use) >= 3:
                if self.p is not None:
                    self.p.terminate()
                    self.p.communicate()
                return {"sm_mhz": float(np.median([x[1] for x in use])) if use else None, "sm_max_mhz": self.max_mhz, "samples": len(use),
                        "window": window, "source": "NVML, every 10 ms", "reasons": reasons}
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out, _ = self.p.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "window": "warm-up and timed steps", "source": "nvidia-smi, every 50 ms", "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------- CPU baseline
def cpu_reference(cfg, weights, steps: int, warmup: int, rows: int, threads: int):
    """The CPU oracle stepping `rows` sequences of the workload from a fresh state: tokens/s and what was run."""
    from oracle import oracle
    from ava_b200 import synth
    oracle.build()
    oracle.set_threads(threads)
    oracle.set_simd(True)
    m = oracle.OracleModel(cfg, weights)
    st = m.state(rows)
    ids = synth.token_ids(cfg["vocab"], rows, warmup + steps)
    for t in range(warmup):
        st.step(ids[:, t])
    t0 = time.perf_counter()
    for t in range(warmup, warmup + steps):
        st.step(ids[:, t])
    dt = time.perf_counter() - t0
    sample = (f"{rows} of the {ROWS_PER_GPU} sequences, {steps} steps after {warmup} warm-up steps from a fresh state "
              f"(KV length {warmup}..{warmup + steps}), AVX2+FMA tile kernel, {threads} threads")
    return rows * steps / dt, dt / steps * 1e3, sample


def run_reference(args, cfg, rank):
    if rank != 0:
        return
    from ava_b200 import synth
    rows = 16
    w = synth.model(cfg, 0, "bench")
    # the port's threading does not always gain from every core of a large host: a short trial at all, 16 and 8 threads
    # picks the count the timed run uses (the fastest), and the line says which
    allc = os.cpu_count() or 1
    tried = {}
    for th in sorted({allc, min(allc, 16), min(allc, 8)}, reverse=True):
        tried[th] = cpu_reference(cfg, w, 6, 2, rows, th)[0]
    threads = max(tried, key=tried.get)
    val, ms, sample = cpu_reference(cfg, w, args.steps, args.warmup, rows, threads)
    line = {"metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations x int8 weights",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": "benchmark configuration 1 (Ava-0.4-shaped decode), bounded CPU sample", "rows": rows},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                             "threads_tried": {str(k): v for k, v in tried.items()}, "host_cores": allc},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def waves_note(total: int, world: int, rows: int) -> dict:
    """Sequences are independent, so a job larger than the GPUs' memory runs as waves of world x rows resident sequences,
    each wave from its prompt to its last token before the next starts; tokens/s is that of one wave."""
    if total <= 0:
        return {}
    return {"sequences_total": total, "waves": -(-total // (world * rows)), "wave_schedule": "waves of gpus x rows_per_gpu resident sequences run one after "
            "another (no state leaves the GPU); value is the rate while a wave runs"}


def prefill_tensor_flops(cfg, tokens):
    """Tensor-core FLOPs per prompt token of the tolerance mode's chunked pass: (executed, algorithmic).  Executed counts
    every limb product the kernels issue (3 per dense product: three activation limbs x one exact bf16 weight; 6 per
    product of the chunk-parallel memory: three limbs each side, i + j <= 2; the engram's scores 3 twice and its mix 2);
    algorithmic counts each product once (and the scores once)."""
    d, H, L, hs = cfg["d"], cfg["hidden"], cfg["n_blocks"], cfg["head_size"]
    nh = d // hs
    dense = d * d * (1 + 4 + (1 if cfg["out_gate"] else 0) + 1) + 2 * d * H          # W_in, q|k|v|e(|g), W_o, W_1, W_2 (W_out is the event sum)
    gate_cols = 2 * cfg["gate_rank"] + 2 * nh
    mem = nh * (128 * 128 * hs + 2 * 128 * hs * hs) / 64.0                           # per token: the Gram, the state read and the state update of a 64-token chunk
    eng_dense = 4 * d * d if cfg["eng_block"] >= 0 else 0
    mean_keys = (tokens + 1) / 2.0 + 32                                              # causal, in tiles of 64 keys
    attn = d * mean_keys if cfg["eng_block"] >= 0 else 0                             # one product of a query with its keys, all heads
    algorithmic = 2.0 * (L * (dense + d * gate_cols + mem) + eng_dense + 2 * attn)
    executed = 2.0 * (L * (3 * dense + 6 * d * gate_cols + 6 * mem) + 3 * eng_dense + 8 * attn)
    return executed, algorithmic


def tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained: the pass runs for seconds)"
    return 1400.0, "fallback (1.4 PFLOP/s sustained, earlier measurement on this pool)"


def measure_prefill(model, cfg, local, world, dist, rows, tokens, chunk, seed0, fast=False):
    """Chunked prompt reading through ava_prefill_device: tokens/s over all ranks, device-timed, ids resident."""
    import torch
    from ava_b200 import synth
    ids = synth.token_ids(cfg["vocab"], rows, tokens, seed0=seed0)
    tok = torch.from_numpy(np.ascontiguousarray(ids.T).astype(np.int32)).to(f"cuda:{local}")
    logits = torch.empty(rows, cfg["vocab"], dtype=torch.float32, device=f"cuda:{local}")
    stream = torch.cuda.ExternalStream(model.stream, device=local)
    warm = model.state(rows, chunk + 8)
    model.prefill_device(warm, tok.data_ptr(), chunk, chunk, logits.data_ptr(), None)
    model.sync()
    warm.close()
    st = model.state(rows, tokens + 8)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    l0 = model.launches
    c0 = model.chunked_memory_counts()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    model.prefill_device(st, tok.data_ptr(), tokens, chunk, logits.data_ptr(), None)
    ev1.record(stream)
    model.sync()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    st.close()
    if fast:
        executed, algorithmic = prefill_tensor_flops(cfg, tokens)
        tps = rows * tokens / (ms * 1e-3)   # per GPU
        peak, src = tensor_peak()
        after = model.chunked_memory_counts()
        return {"value": world * tps, "unit": "tokens/s", "rows_per_gpu": rows, "tokens_per_row": tokens, "chunk": chunk, "ms": ms,
                "gpu_launches": int(model.launches - l0),
                "what": "benchmark configuration 2 in the tolerance mode: dense products, the chunk-parallel fast-weight memory (chunks of 64) and "
                        "the engram's causal read on tcgen05 tensor cores; agrees with the sequential reference to rounding, not bit for bit",
                "memory_passes": {"chunk_form": after[0] - c0[0], "token_loop": after[1] - c0[1], "engram_chunks": after[2] - c0[2]},
                "roofline": {"bound": "tensor", "achieved": executed * tps / 1e12, "peak": peak, "unit": "TFLOP/s", "frac": executed * tps / 1e12 / peak,
                             "of": src, "counts": "limb products issued (executed FLOPs)", "algorithmic_tflops": algorithmic * tps / 1e12,
                             "flops_per_token": {"executed": executed, "algorithmic": algorithmic}, "traffic": None}}
    return {"value": world * rows * tokens / (ms * 1e-3), "unit": "tokens/s", "rows_per_gpu": rows, "tokens_per_row": tokens, "chunk": chunk,
            "ms": ms, "gpu_launches": int(model.launches - l0),
            "what": "chunked prompt reading, bit-identical to stepping (CUDA-core products in k order, LIF time scan, one streaming pass of the "
                    "fast weights per token, engram read token by token); config 2 is 8192 tokens per row, this is its first part"}


# ------------------------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--rows", type=int, default=ROWS_PER_GPU, help="sequences per GPU")
    ap.add_argument("--ctx", type=int, default=MEAN_CTX, help="KV length the timed steps are centred on")
    ap.add_argument("--small", action="store_true", help="a small model and batch (profiling captures, not a bench value)")
    ap.add_argument("--scaled", action="store_true", help="benchmark configuration 3: 24 blocks, d 2048, wide 8192, vocab 32768 (use --rows 128: an 8-GPU share of 1024 sequences)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--total-sequences", type=int, default=0, help="the job's sequences over all GPUs when they do not all fit at once (configuration 3 "
                    "on 1 or 2 GPUs): they run as waves of gpus x rows resident sequences, one wave after another; the line states the waves")
    ap.add_argument("--parts", action="store_true", help="the same workload with the nine Ava-0.4 parts switched on (their cost; not the headline configuration)")
    ap.add_argument("--prefill-tokens", type=int, default=1024, help="tokens per row of the exact prompt-reading sample (config 2 is 8192: about half a minute)")
    ap.add_argument("--fast-prefill-tokens", type=int, default=8192, help="tokens per row of the tolerance mode's prompt-reading leg (config 2: 8192)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    from ava_b200 import config, synth
    cfg = config.ava04_shaped()
    if args.small:
        cfg = config.make(4096, 768, 2, head_size=768, eng_block=1, eng_head_size=64, eng_store_bf16=1)
    if args.scaled:
        cfg = config.ava04_shaped(scaled=True)
    if args.parts:
        cfg = dict(cfg, stp=1, neuromod=3, dendrite=1, letters=1, dopamine=1, mood=4, rhythm=1, thalamus=1, cb_units=12288)

    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return

    import torch
    import torch.distributed as dist
    from ava_b200 import engine

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the engine has no CPU path)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    weights = synth.model(cfg, 0, "bench")
    model = engine.Model(cfg, weights, device=local)
    rows, K, W = args.rows, args.steps, args.warmup
    e2e_steps = K
    # untimed steps bring the KV length to ctx - K/2, so that the timed steps straddle the mean decode context
    prompt = max(1, args.ctx - K // 2 - W)
    max_ctx = prompt + W + K + 2 * (e2e_steps + W) + 16 + K + W + 8   # decode, end to end (two calls), section clock, fast-products leg
    state = model.state(rows, max_ctx)
    stream = torch.cuda.ExternalStream(model.stream, device=local)

    from ava_b200 import shard
    first, last = shard.block(world * rows, world, rank)                           # this rank's sequences (weak scaling)
    assert last - first == rows
    ids = synth.token_ids(cfg["vocab"], rows, prompt, seed0=first)                 # sequence r reads SplitMix64(r)
    ids_dev = torch.from_numpy(np.ascontiguousarray(ids.T).astype(np.int32)).to(f"cuda:{local}")  # [prompt, rows]
    tok = [torch.zeros(rows, dtype=torch.int32, device=f"cuda:{local}") for _ in range(2)]
    logits_dev = torch.empty(rows, cfg["vocab"], dtype=torch.float32, device=f"cuda:{local}")
    torch.cuda.synchronize()

    # the prompt, token by token (untimed; no output head)
    for t in range(prompt - 1):
        model.step_device(state, ids_dev[t].data_ptr(), None, None)
    model.step_device(state, ids_dev[prompt - 1].data_ptr(), logits_dev.data_ptr(), tok[0].data_ptr())
    model.sync()

    def decode(n, cur):
        for _ in range(n):
            model.step_device(state, tok[cur].data_ptr(), logits_dev.data_ptr(), tok[cur ^ 1].data_ptr())
            cur ^= 1
        return cur

    # the clock sampler starts before the warm-up steps (a short timed region would otherwise end before its first
    # sample): its samples cover warm-up and timed steps, both under the same load
    clocks = Clocks(local)
    clocks.start()
    cur = decode(W, 0)
    model.sync()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks.mark()
    l0 = model.launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    cur = decode(K, cur)
    ev1.record(stream)
    model.sync()
    torch.cuda.synchronize()
    launches = model.launches - l0
    ms = ev0.elapsed_time(ev1)
    clk = clocks.stop()
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    value = world * rows * K / (ms * 1e-3)

    # ---- end to end: the reference-facing call with host buffers (pinned), copies inside the timed region
    # the ids each step sends are uniform draws prepared beforehand (picking the next token from the returned logits is
    # the caller's work, not the engine's; which token is fed does not change the step's cost)
    e2e_ids = torch.from_numpy(synth.token_ids(cfg["vocab"], W + e2e_steps, rows, seed0=10_000 + first).astype(np.int32)).pin_memory()
    logits_host = torch.empty(rows, cfg["vocab"], dtype=torch.float32).pin_memory()
    L = engine.lib()
    import ctypes as C
    e2e_at = [0]

    def host_step():
        tok_ptr = e2e_ids[e2e_at[0]].data_ptr()
        e2e_at[0] += 1
        rc = L.ava_step(model.h, state.h, C.cast(tok_ptr, engine.u32p), C.cast(logits_host.data_ptr(), engine.fp))
        if rc != 0:
            raise RuntimeError(L.ava_last_error(model.h).decode())

    for _ in range(W):
        host_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = world * rows * e2e_steps / e2e_s

    # the same through the greedy call (host token ids in, host token ids out: what a generation loop moves per step)
    nxt_host = torch.empty(rows, dtype=torch.int32).pin_memory()
    cur_host = e2e_ids[0].clone().pin_memory()

    def greedy_step():
        rc = L.ava_step_greedy(model.h, state.h, C.cast(cur_host.data_ptr(), engine.u32p), C.cast(nxt_host.data_ptr(), engine.u32p))
        if rc != 0:
            raise RuntimeError(L.ava_last_error(model.h).decode())
        cur_host.copy_(nxt_host)

    for _ in range(W):
        greedy_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        greedy_step()
    torch.cuda.synchronize()
    greedy_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([greedy_s], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        greedy_s = float(t.item())
    e2e_greedy = world * rows * e2e_steps / greedy_s

    # ---- the dominant kernel under the section clock: a few more steps with every launch bracketed by events
    model.prof_enable(True)
    cur2 = decode(4, cur)
    prof = model.prof_read()
    model.prof_enable(False)
    total_ms = sum(v[1] for v in prof.values()) or 1.0
    n_mh, ms_mh = prof.get("mem_heads", (0, 0.0))
    state_bytes = rows * 2 * 4 * cfg["d"] * cfg["head_size"]        # read once + written once, f32, per launch
    peak, peak_src = peaks()
    achieved = state_bytes / (ms_mh / max(n_mh, 1) * 1e-3) / 1e9 if n_mh else 0.0
    # DRAM bytes one launch moved under ncu (the state pass over a 64-row lane of 768x768 matrices, from the capture
    # summarised under profiles/): a constant of that profile, scaled by the state a launch streams, not something this
    # run measures
    traffic = TRAFFIC_PER_STATE_BYTE * state_bytes
    # the whole step against the HBM roofline: algorithmic bytes per decoded token (state + weights/rows + KV + LIF)
    kv_bytes = args.ctx * 2 * cfg["d"] * 2 if cfg["eng_block"] >= 0 else 0
    tok_bytes = (2 * 4 * cfg["n_blocks"] * cfg["d"] * cfg["head_size"] + synth.weight_bytes(cfg) / rows + kv_bytes
                 + 2 * 4 * 3 * cfg["n_blocks"] * cfg["d"])
    step_frac = (value / world) * tok_bytes / 1e9 / peak

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations x int8 weights, f32 state, bf16 KV",
        "data": "synthetic",
        "config": {"workload": "benchmark configuration 1: Ava-0.4-shaped decode (12 blocks, d 768, wide 3072, kWTA 768, vocab 16384, one 768x768 f32 "
                               "fast-synapse matrix per block, bf16 engram of 12x64 in block 6)" if not (args.small or args.scaled) else
                   ("small profiling case" if args.small else "benchmark configuration 3: scaled Ava (24 blocks, d 2048, wide 8192, kWTA 2048, vocab 32768, one "
                    "2048x2048 f32 fast-synapse matrix per block)"),
                   "parts": "the nine Ava-0.4 parts on (stp, neuromod 3, dendrite, letters, dopamine, mood, rhythm, thalamus, cerebellum head 12288)" if args.parts else "none",
                   "rows_per_gpu": rows, **waves_note(args.total_sequences, world, rows), "kv_len_timed": [prompt + W, prompt + W + K], "l2": "per-step inputs (state "
                   f"{state.nbytes / 1e9:.2f} GB per GPU) are larger than L2", "sequences": "independent, sharded by rank, no collective"},
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": rows * 4, "d2h_bytes_per_step": rows * cfg["vocab"] * 4,
                "steps": e2e_steps, "call": "ava_step (host token ids in, host logits out, pinned buffers)",
                "greedy": {"value": e2e_greedy, "unit": UNIT, "h2d_bytes_per_step": rows * 4, "d2h_bytes_per_step": rows * 4,
                           "call": "ava_step_greedy (host token ids in, host token ids out; the arg-max on the device)"}},
        "gpu_launches": int(launches),
        "clocks": clk,
        "roofline": {"bound": "hbm", "kernel": "mem_heads (fast-weight state pass)", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "of": peak_src, "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read + write)", "traffic_source": "profile constant (ncu capture under profiles/), scaled by the bytes a launch streams; not measured in this run",
                     "bytes_per_launch": state_bytes,
                     "mean_launch_ms": ms_mh / max(n_mh, 1), "launches_timed": n_mh,
                     "step_bytes_per_token": tok_bytes, "step_frac_of_hbm_roofline": step_frac},
        "kernel_share": {k: round(v[1] / total_ms, 4) for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])},
        "kernel_ms_per_step": {k: round(v[1] / 4, 4) for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])},
    }
    # ---- the same decode with the dense products on the tensor cores (opt-in: exact products, another summation
    # order, so results agree with the reference's to rounding and not bit for bit; the headline above is the exact mode)
    model.set_fast_products(True)
    cur2 = decode(W, cur2)
    model.sync()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    l0 = model.launches
    ev0.record(stream)
    cur2 = decode(K, cur2)
    ev1.record(stream)
    model.sync()
    torch.cuda.synchronize()
    fast_launches = model.launches - l0
    fast_ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([fast_ms], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        fast_ms = float(t.item())
    model.prof_enable(True)
    cur2 = decode(4, cur2)
    fprof = model.prof_read()
    model.prof_enable(False)
    fast_prefill = None
    if not args.small and not args.scaled:
        fast_prefill = measure_prefill(model, cfg, local, world, dist, rows=64, tokens=args.fast_prefill_tokens, chunk=1024, seed0=50_000 + first, fast=True)
    model.set_fast_products(False)
    line["fast_products"] = {"prefill": fast_prefill, "value": world * rows * K / (fast_ms * 1e-3), "unit": UNIT, "ms_per_step": fast_ms / K, "gpu_launches": int(fast_launches),
                             "parity": "dense products on tcgen05 tensor cores: exact products (3 bf16 limbs x bf16 weights), f32 sums in the "
                                       "tensor core's order; agrees with the reference to ~2e-6 of each sum's magnitudes, not bit for bit",
                             "kernel_ms_per_step": {k: round(v[1] / 4, 4) for k, v in sorted(fprof.items(), key=lambda kv: -kv[1][1])}}
    # ---- prompt reading (benchmark configuration 2's shape: 64 rows per GPU, chunks of 256 tokens), a bounded sample of it
    if not args.small and not args.scaled:
        line["prefill"] = measure_prefill(model, cfg, local, world, dist, rows=64, tokens=args.prefill_tokens, chunk=256, seed0=50_000 + first)
    # ---- configuration 0's shape on the GPU: one sequence alone (256-token prompt, then decode), exact mode
    if rank == 0 and not args.small and not args.scaled:
        one = model.state(1, 512)
        ids1 = torch.from_numpy(np.ascontiguousarray(synth.token_ids(cfg["vocab"], 1, 256 + 3, seed0=0).T).astype(np.int32)).to(f"cuda:{local}")
        lg1 = torch.empty(1, cfg["vocab"], dtype=torch.float32, device=f"cuda:{local}")
        nx = [torch.zeros(1, dtype=torch.int32, device=f"cuda:{local}") for _ in range(2)]
        for t in range(256):
            model.step_device(one, ids1[t].data_ptr(), lg1.data_ptr(), nx[0].data_ptr())
        model.sync()
        ev0.record(stream)
        for t in range(64):
            model.step_device(one, nx[t & 1].data_ptr(), lg1.data_ptr(), nx[(t & 1) ^ 1].data_ptr())
        ev1.record(stream)
        model.sync()
        torch.cuda.synchronize()
        one_ms = ev0.elapsed_time(ev1) / 64
        line["config0_batch1"] = {"value": 1e3 / one_ms, "unit": UNIT, "ms_per_token": one_ms,
                                  "what": "one sequence alone on the GPU (greedy feedback on the device, KV length 256..320), exact mode; the CPU's figure "
                                          "for the same case is cpu_baseline.config0_batch1"}
        one.close()
    if rank == 0 and not args.no_cpu and not args.small:
        threads = os.cpu_count() or 1
        val, _, sample = cpu_reference(cfg, weights, 128, 4, 16, threads)
        # the same sample at fewer threads (bounded: a few seconds each), and configuration 0's own case: one sequence
        sweep = {str(threads): val}
        for th in (1, 4, 8):
            if th < threads:
                sweep[str(th)] = cpu_reference(cfg, weights, 8 * th, 2, 16, th)[0]
        one, one_ms, one_sample = cpu_reference(cfg, weights, 64, 4, 1, threads)
        best = max(sweep, key=sweep.get)
        line["cpu_baseline"] = {"value": sweep[best], "unit": UNIT, "cores": int(best), "kind": "port", "sample": sample.replace(f"{threads} threads", f"{best} threads (the fastest of those tried)"),
                                "by_threads": sweep,
                                "config0_batch1": {"value": one, "unit": UNIT, "ms_per_token": one_ms, "sample": one_sample}}
    elif rank == 0:
        line["cpu_baseline"] = None
    if rank == 0:
        print(json.dumps(line), flush=True)
    del cur2
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
