"""CPU checks of the C-ABI library: it loads, exports every symbol the header declares, its host arithmetic is what the
kernels use, and without a GPU it fails loudly instead of falling back to anything."""
import ctypes as C
import math
import os
import re

import numpy as np
import pytest

from ava_b200 import build, config, engine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    build.build()
    return engine.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ava_engine.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ava_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(L):
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(L, n), n
    assert set(names) == set(engine.EXPORTS)


def test_each_entry_point_cites_the_reference():
    text = open(os.path.join(ROOT, "include", "ava_engine.h")).read()
    assert text.count("src/") >= 20


def test_host_math_is_close_to_libm(L):
    xs = np.concatenate([np.linspace(-100, 88, 4001), np.array([0.0, -0.0, 1e-30, -1e-30, 88.7, -103.9])]).astype(np.float32)
    for x in xs:
        got, want = L.ava_host_expf(float(x)), math.exp(float(x))
        if want > 1e-37:
            assert abs(got - want) <= 2.5e-7 * want, (x, got, want)
        else:
            assert abs(got - want) < 1e-38
    assert L.ava_host_expf(float("inf")) == float("inf") and L.ava_host_expf(float("-inf")) == 0.0
    assert math.isnan(L.ava_host_expf(float("nan")))
    for x in np.concatenate([np.logspace(-38, 38, 3001), np.linspace(0.5, 2.5, 2001)]).astype(np.float32):
        got, want = L.ava_host_logf(float(x)), math.log(float(x))
        assert abs(got - want) <= 2.5e-7 * max(abs(want), 0.3), (x, got, want)
    assert L.ava_host_logf(1.0) == 0.0 and L.ava_host_logf(0.0) == float("-inf") and math.isnan(L.ava_host_logf(-1.0))
    for x in np.logspace(-30, 30, 2001).astype(np.float32):
        got, want = L.ava_host_rsqrtf(float(x)), float(x) ** -0.5
        assert abs(got - want) <= 1.3e-7 * want


def test_oracle_accepts_the_engines_math(L, orc):
    """The checker can run on the engine's exp / ln / x^-1/2, and doing so only moves results by rounding."""
    cfg = config.tiny()
    from ava_b200 import synth
    m = orc.OracleModel(cfg, synth.model(cfg, 0, "awake"))
    ids = synth.token_ids(cfg["vocab"], 1, 4)
    a = m.state(1).forward(ids)
    try:
        orc.set_math(*engine.host_math())
        m2 = orc.OracleModel(cfg, synth.model(cfg, 0, "awake"))
        b = m2.state(1).forward(ids)
    finally:
        orc.reset_math()
    np.testing.assert_allclose(a[0, 0], b[0, 0], rtol=0, atol=1e-5)


def test_no_gpu_means_an_error_not_a_fallback(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(engine.EngineError) as ei:
        engine.Model(config.tiny())
    assert ei.value.code == engine.ERR_CUDA and "no CPU path" in str(ei.value)
    x = np.zeros((1, 16), np.float32)
    with pytest.raises(engine.EngineError):
        engine.op_q8_matmul(x, np.zeros((16, 4), np.int8), np.ones(4, np.float32))


def test_split_step_calls_refuse_missing_arguments_before_any_cuda_call(L):
    """The split step's entry points check their arguments first (no engine, a negative time limit): an error code, no
    CUDA call, so this runs without a GPU."""
    ERR_ARG = -1
    assert L.ava_split_wait(None, None, 10) == ERR_ARG
    assert L.ava_nccl_unique_id(None) == ERR_ARG
    assert L.ava_nccl_comm_destroy(None) == ERR_ARG


def test_product_does_not_touch_the_oracle():
    """Nothing under the package may import, link or name the oracle."""
    pkg = os.path.join(ROOT, "ava_b200")
    for dp, _, files in os.walk(pkg):
        if os.path.basename(dp) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dp, f)).read()
                assert "oracle" not in text.lower().replace("a checker", ""), os.path.join(dp, f)
    out = os.popen(f"ldd {engine.LIB_PATH}").read()
    assert "oracle" not in out


def test_static_entry_refuses_an_unaligned_vector_before_any_launch(L):
    """ava_mem_heads_static reads six of its inputs with bulk copies, which fault on a source that is not 16-byte
    aligned; the entry point must refuse such a pointer with AVA_ERR_ARG before it touches the device (so this runs
    without a GPU: the check comes before the first CUDA call)."""
    buf = (C.c_float * 4096)()
    base = C.addressof(buf)
    base += (-base) % 16
    ok = C.c_void_p(base)
    off4 = C.c_void_p(base + 4)     # a 4-byte-aligned view into the buffer, as a caller slicing a larger array would pass
    off2 = C.c_void_p(base + 2)
    for i in range(6):              # e, v, w, ah, qg, ex
        args = [ok] * 10
        args[i] = off4
        rc = L.ava_mem_heads_static(0, None, 1, 64, *args)
        assert rc == engine.ERR_ARG, i
        assert b"16-byte aligned" in L.ava_static_last_error()
    for i in range(6, 10):          # qw, qa, f, y: 4-byte alignment is enough, 2 is not
        args = [ok] * 10
        args[i] = off2
        assert L.ava_mem_heads_static(0, None, 1, 64, *args) == engine.ERR_ARG


def test_rust_binding_declares_exactly_the_headers_entry_points():
    """bindings/ava_engine.rs: the names in its extern "C" block are the header's, and the block is what
    bindings/gen_extern.py writes from the header today (so a new entry point cannot be forgotten there)."""
    import subprocess
    import sys
    rs = open(os.path.join(ROOT, "bindings", "ava_engine.rs")).read()
    block = rs[rs.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    in_rs = sorted(set(re.findall(r"pub fn (ava_[a-z0-9_]+)\s*\(", block)))
    assert in_rs == declared_symbols()
    assert subprocess.run([sys.executable, os.path.join(ROOT, "bindings", "gen_extern.py"), "--check"]).returncode == 0
