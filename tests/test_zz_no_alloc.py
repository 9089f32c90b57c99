"""The entry point for callers that cannot allocate device memory (ava_mem_heads_static).

Some users of this library run where cudaMalloc is off limits: inside a host callback or a latency-critical thread
that must not wait on the allocator, in a process whose GPU memory was all handed out at start-up, or in a region that
may not allocate until an earlier stream capture ends.  For them the fast-weight update + read exists in a form that
takes device pointers and keeps its scratch in a fixed array inside the library.  This test drives it through the C
ABI with buffers the TEST allocates (the entry point itself allocates nothing) and checks it against the ordinary
entry point, ava_op_mem_heads, bit for bit, on two calls in a row: the second call reuses the shared scratch that the
first one left behind and continues from the state the first one wrote.

The file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from ava_b200 import build, engine

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def make_inputs(rng, m, hs):
    unit = lambda x: (x / np.sqrt((x * x).sum(-1, keepdims=True))).astype(np.float32)
    e, k, q = (unit(rng.normal(size=(m, hs))) for _ in range(3))
    v = rng.normal(size=(m, hs)).astype(np.float32)
    ex = rng.uniform(0.9, 1.0, (m, hs)).astype(np.float32)
    be = rng.uniform(0.05, 1.5, (m, hs)).astype(np.float32)
    return dict(e=e, v=v, w=k * be, ah=e * (be * ex), qg=q * ex, ex=ex, qw=rng.normal(size=m).astype(np.float32),
                qa=rng.normal(size=m).astype(np.float32))


@pytest.mark.parametrize("m,hs", [(3, 768), (16, 64)])
def test_static_entry_matches_the_allocating_one_twice(m, hs):
    import torch
    build.build()
    L = engine.lib()
    rng = np.random.default_rng(hs + m)
    f0 = rng.normal(0, 0.3, (m, hs, hs)).astype(np.float32)
    calls = [make_inputs(rng, m, hs), make_inputs(rng, m, hs)]

    # reference results from the existing entry point (host buffers, allocates its own temporaries)
    want, f_ref = [], f0
    for inp in calls:
        y, f_ref = engine.op_mem_heads(inp["e"], inp["v"], inp["w"], inp["ah"], inp["qg"], inp["ex"], inp["qw"], inp["qa"], f_ref)
        want.append((y, f_ref))

    dev = torch.device("cuda", 0)
    f_dev = torch.from_numpy(f0.copy()).to(dev)
    y_dev = torch.empty(m, hs, dtype=torch.float32, device=dev)
    for i, inp in enumerate(calls):
        t = {k: torch.from_numpy(v).to(dev) for k, v in inp.items()}
        torch.cuda.synchronize()
        rc = L.ava_mem_heads_static(0, None, m, hs, *[C.c_void_p(t[k].data_ptr()) for k in ("e", "v", "w", "ah", "qg", "ex", "qw", "qa")],
                                    C.c_void_p(f_dev.data_ptr()), C.c_void_p(y_dev.data_ptr()))
        assert rc == 0, L.ava_static_last_error().decode()
        assert np.array_equal(bits(y_dev.cpu().numpy()), bits(want[i][0])), f"read of call {i}"
        assert np.array_equal(bits(f_dev.cpu().numpy()), bits(want[i][1])), f"state after call {i}"


def test_static_entry_refuses_what_does_not_fit():
    import torch
    build.build()
    L = engine.lib()
    hs = 768
    m = 4194304 // (hs * hs) + 1          # one head more than the built-in scratch holds
    z = torch.zeros(8, device="cuda:0")
    p = C.c_void_p(z.data_ptr())
    rc = L.ava_mem_heads_static(0, None, m, hs, p, p, p, p, p, p, p, p, p, p)
    assert rc == engine.ERR_CAPACITY
    msg = L.ava_static_last_error().decode()
    assert "4194304" in msg and "scratch" in msg
