"""The N > 1 path on CPU: two gloo ranks each step their own block of sequences (here with the CPU oracle standing in
for the GPU engine: the host-side sharding logic is what is under test) and together reproduce the single-process
batch bit for bit, with no collective on the data path."""
import os
import subprocess
import sys
import textwrap

import numpy as np

from ava_b200 import shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_blocks_partition_the_rows():
    for total in (1, 7, 256, 1024, 1025):
        for world in (1, 2, 3, 4, 8):
            spans = [shard.block(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
            for row in (0, total // 2, total - 1):
                a, b = shard.block(total, world, shard.owner(total, world, row))
                assert a <= row < b


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r})
    import numpy as np, torch, torch.distributed as dist
    from ava_b200 import config, shard, synth
    from oracle import oracle
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = config.tiny()
    m = oracle.OracleModel(cfg, synth.model(cfg, 0, "awake"))
    total, T = 5, 6
    ids = synth.token_ids(cfg["vocab"], total, T)
    a, b = shard.block(total, world, rank)
    st = m.state(b - a)
    mine = st.forward(ids[a:b], last_only=True)            # no collective on the data path
    slow = shard.max_over_ranks(float(rank + 1), dist)     # the measurement's only reduction
    assert slow == 2.0
    out = [None, None]
    dist.all_gather_object(out, (a, b, mine))              # the host gathers outputs
    if rank == 0:
        full = np.concatenate([o[2] for o in sorted(out, key=lambda o: o[0])])
        np.save({out!r}, full)
    dist.barrier()
    dist.destroy_process_group()
""")


def test_two_ranks_reproduce_the_single_process_batch(tmp_path, orc):
    from ava_b200 import config, synth
    out = str(tmp_path / "full.npy")
    port = 29500 + os.getpid() % 2000
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT, port=port, out=out))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    logs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    cfg = config.tiny()
    m = orc.OracleModel(cfg, synth.model(cfg, 0, "awake"))
    ids = synth.token_ids(cfg["vocab"], 5, 6)
    want = m.state(5).forward(ids, last_only=True)
    got = np.load(out)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
