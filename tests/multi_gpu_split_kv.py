"""Run under torchrun on 2+ GPUs (one process per GPU, NCCL):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        tests/multi_gpu_split_kv.py [--prompt 2048] [--decode 32]

One long sequence (benchmark configuration 4 at a reduced prompt length): rank 0 reads the prompt, the engram store is
dealt out by position, then every decoded token takes a broadcast of q,k,v and an all-gather of the partial softmax
statistics.  Rank 0 checks its logits against the CPU oracle's one-pass read (1e-4 relative) and prints a JSON line
with the decode rate.  Not collected by pytest (no test_ prefix): the single-GPU emulation of the same path is
tests/test_gpu_split_kv.py.
"""
import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=32)
    ap.add_argument("--full", action="store_true", help="the Ava-0.4-shaped model instead of the small one")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--seg-len", type=int, default=512, help="keys per segment of the partial read (one block of threads sums a segment in key order)")
    ap.add_argument("--import-keys", type=int, default=0, help="no prompt is read: the store starts with this many positions of seeded random keys and "
                    "values (bf16-exact), dealt out by position, and the membranes and fast weights start fresh (benchmark configuration 4 at its full 131072)")
    ap.add_argument("--torch-exchange", action="store_true", help="the two collectives through torch.distributed instead of the library's own call")
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    from ava_b200 import config, engine, longctx, synth

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = config.ava04_shaped() if args.full else config.tiny(eng_head_size=64, eng_store_bf16=1, vocab=512)
    w = synth.model(cfg, 0, "bench" if args.full else "awake")
    model = engine.Model(cfg, w, device=local)
    P, D = (args.import_keys or args.prompt), args.decode
    block = -(-P // world)
    cap = block + D + 8
    sk = longctx.SplitKV(model, 1, cap, rank, world, dist=dist, seg_len=args.seg_len)
    if not args.torch_exchange:
        sk.make_comm()   # a communicator made through the C ABI; every token is then one call of the library
    ids = synth.token_ids(cfg["vocab"], 1, P + D, seed0=7)
    heads, hs = cfg["d"] // cfg["eng_head_size"], cfg["eng_head_size"]
    dev = torch.device("cuda", local)
    kv = torch.empty((2, heads, P, hs) if not args.import_keys else (1,), dtype=torch.float32, device=dev)
    carried = []
    prompt_s = 0.0

    def bf16_exact(a):
        u = np.ascontiguousarray(a, np.float32).view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)

    if args.import_keys:
        rng = np.random.default_rng(11)   # the same draw on every rank: nothing to send
        kvh = np.stack([bf16_exact(rng.standard_normal((heads, P, hs), dtype=np.float32)) for _ in range(2)])
        sk.take_prompt_store(kvh[0], kvh[1], P, block)
    if rank == 0 and not args.import_keys:
        full = model.state(1, P + 8)
        t0 = time.perf_counter()
        model.forward_with_state(ids[:, :P], full, last_only=True)
        prompt_s = time.perf_counter() - t0
        kv[0] = torch.from_numpy(full.get(0, "eng.k").reshape(heads, P, hs)).to(dev)
        kv[1] = torch.from_numpy(full.get(0, "eng.v").reshape(heads, P, hs)).to(dev)
        names = [f"lif.{i}.{k}" for i in range(cfg["n_blocks"]) for k in "vsa"] + [f"mem.{i}.f" for i in range(cfg["n_blocks"])]
        for n in names:
            sk.state.put(0, n, full.get(0, n))
        full.close()
    if not args.import_keys:
        dist.broadcast(kv, src=0)                       # the prompt's keys and values, once
        kvh = kv.cpu().numpy()
        sk.take_prompt_store(kvh[0], kvh[1], P, block)
    del kv
    logits = torch.empty(1, cfg["vocab"], dtype=torch.float32, device=dev)
    toks = torch.from_numpy(ids[0, P:].astype(np.int32)).to(dev)
    torch.cuda.synchronize()
    dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = []
    ev0.record(sk.stream)
    for t in range(D):
        (sk.step if args.torch_exchange else sk.step_c)(toks[t:t + 1].data_ptr() if rank == 0 else None, logits.data_ptr() if rank == 0 else None, None)
        if rank == 0 and not args.no_check:
            model.sync()
            out.append(logits.cpu().numpy().copy())
    ev1.record(sk.stream)
    if not args.torch_exchange:
        sk.wait(60000)
    model.sync()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    t_ms = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    counts = [None] * world
    dist.all_gather_object(counts, sk.state.get(0, "eng.k").size // cfg["d"])
    if rank == 0:
        line = {"what": "one sequence, engram store split by position", "world": world, "prompt": P, "decode": D,
                "tokens_per_rank": counts, "ms_per_token": float(t_ms.item()) / D, "seg_len": args.seg_len, "exchange": "torch.distributed" if args.torch_exchange else "ava_split_step (NCCL by dlopen, own communicator)", "prompt_read_s": prompt_s, "checked": not args.no_check}
        assert sum(counts) == P + D, counts
        if not args.no_check:
            from oracle import oracle
            oracle.build()
            oracle.set_math(*engine.host_math())
            oracle.set_threads(os.cpu_count() or 1)
            om = oracle.OracleModel(cfg, w)
            os_ = om.state(1)
            if args.import_keys:
                os_.put(0, "eng.k", kvh[0])
                os_.put(0, "eng.v", kvh[1])
            else:
                os_.forward(ids[:, :P], last_only=True)
            want0 = os_.step(ids[:, P:P + 1])
            err = float(np.abs(out[0] - want0).max() / max(1.0, np.abs(want0).max()))
            line["first_token_rel_err"] = err
            assert err <= 1e-4, err
        print(json.dumps(line), flush=True)
    dist.barrier()
    sk.close_comm()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
