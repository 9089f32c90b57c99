"""One long sequence with its engram store split by position over several GPUs (benchmark configuration 4).

One process per GPU, each with its own engine (replicated weights).  The membranes and the fast-synapse state live on
rank 0 and are stepped there; every rank keeps the keys and values of the positions it owns and, per decoded token,
contributes the partial softmax statistics (max, sum, mix) of its part.  The exchange is two small NCCL collectives per
token: a broadcast of the engram's q,k,v [rows, 3 d] from rank 0 and an all-gather of the partials
[rows, heads, parts, 2 + head size]; rank 0 merges them in position order and finishes the step.

The reference has no counterpart (single device, design-tests/nn/gpu/src/memory.rs:664-692); the merged read is checked
against a one-pass softmax on the CPU to rounding.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import engine, shard


class SplitKV:
    """This rank's part of a long sequence.  `dist` is torch.distributed (initialised, NCCL) or None for one rank."""

    def __init__(self, model: engine.Model, rows: int, capacity: int, rank: int, world: int, dist=None, seg_len: int = 2048):
        import torch
        self.torch = torch
        self.m, self.rank, self.world, self.dist = model, rank, world, dist
        self.rows = rows
        model.set_segmented_read(seg_len)
        self.state = model.state(rows, capacity)
        self.dev = torch.device("cuda", model.device)
        cfg = model.cfg
        self.parts = engine.lib().ava_shard_parts(model.h, self.state.h)
        heads = cfg["d"] // cfg["eng_head_size"]
        self.qkv = torch.empty(rows, 3 * cfg["d"], dtype=torch.float32, device=self.dev)
        self.partial = torch.empty(rows, heads, self.parts, 2 + cfg["eng_head_size"], dtype=torch.float32, device=self.dev)
        self.gathered = torch.empty((world,) + tuple(self.partial.shape), dtype=torch.float32, device=self.dev)
        self.stream = torch.cuda.ExternalStream(model.stream, device=self.dev)

    def take_prompt_store(self, k_full, v_full, prompt_len: int, block: int):
        """k_full, v_full: [heads, prompt_len, hs] f32 of row 0 (what rank 0's prompt reading exported).  This rank keeps
        the positions it owns; ownership of later positions follows the same rule."""
        lo = min(self.rank * block, prompt_len)
        hi = prompt_len if self.rank == self.world - 1 else min((self.rank + 1) * block, prompt_len)
        for r in range(self.rows):
            if hi > lo:
                self.state.put(r, "eng.k", np.ascontiguousarray(k_full[:, lo:hi]))
                self.state.put(r, "eng.v", np.ascontiguousarray(v_full[:, lo:hi]))
            else:
                self.state.put(r, "eng.k", np.zeros(0, np.float32))
                self.state.put(r, "eng.v", np.zeros(0, np.float32))
        rc = engine.lib().ava_state_set_kv_shard(self.state.h, self.rank, self.world, block, prompt_len)
        self.m._check(rc)
        assert shard.kv_owner(prompt_len, block, self.world) == self.world - 1 or prompt_len < block * self.world

    # ---- one decoded token, as the three calls a rank makes around the two collectives
    def begin(self, tok_ptr: int):
        """rank 0: the blocks up to the engram's q,k,v."""
        self.m._check(engine.lib().ava_split_step_begin(self.m.h, self.state.h, tok_ptr, self.qkv.data_ptr()))

    def partial_read(self):
        """every rank, after q,k,v arrived: append if this rank owns the position, then its part's statistics."""
        self.m._check(engine.lib().ava_shard_partial(self.m.h, self.state.h, self.qkv.data_ptr(), self.partial.data_ptr()))

    def end(self, logits_ptr, next_ptr):
        """rank 0, after the partials were gathered: merge in position order and finish the step."""
        self.m._check(engine.lib().ava_split_step_end(self.m.h, self.state.h, self.gathered.data_ptr(), self.world, logits_ptr, next_ptr))

    # ---- the exchange behind the C ABI: a communicator of the engine's own, NCCL loaded by the library itself
    def make_comm(self):
        """Collective over `dist` (any backend): rank 0 draws the id, everyone joins.  After it, step_c is the whole token."""
        ident = C.create_string_buffer(128)
        if self.rank == 0:
            self.m._check(engine.lib().ava_nccl_unique_id(ident))
        if self.world > 1:
            box = [ident.raw if self.rank == 0 else None]
            self.dist.broadcast_object_list(box, src=0)
            ident = C.create_string_buffer(box[0], 128)
        comm = C.c_void_p()
        self.m._check(engine.lib().ava_nccl_comm_init(self.m.h, self.world, self.rank, ident, C.byref(comm)))
        self.comm = comm

    def close_comm(self):
        if getattr(self, "comm", None):
            engine.lib().ava_nccl_comm_destroy(self.comm)
            self.comm = None

    def step_c(self, tok_ptr: int | None, logits_ptr=None, next_ptr=None):
        """One token as one call of the library (ava_split_step): both collectives inside, on the engine's stream."""
        comm = getattr(self, "comm", None)
        self.m._check(engine.lib().ava_split_step(self.m.h, self.state.h, comm, self.rank, self.world, tok_ptr, self.qkv.data_ptr(),
                                                  self.partial.data_ptr(), self.gathered.data_ptr(), logits_ptr, next_ptr))

    def wait(self, timeout_ms: int = 10000):
        """Bounded host wait for the token (ava_split_wait).  On a NCCL error or when the time runs out the library has
        aborted the communicator: it is dropped here, and the error is raised."""
        comm = getattr(self, "comm", None)
        rc = engine.lib().ava_split_wait(self.m.h, comm, timeout_ms)
        if rc != 0:
            self.comm = None
        self.m._check(rc)

    def step(self, tok_ptr: int | None, logits_ptr=None, next_ptr=None):
        """One token with torch.distributed doing the exchange on the engine's stream."""
        torch, dist = self.torch, self.dist
        with torch.cuda.stream(self.stream):
            if self.rank == 0:
                self.begin(tok_ptr)
            if self.world > 1:
                dist.broadcast(self.qkv, src=0)
            self.partial_read()
            if self.world > 1:
                dist.all_gather_into_tensor(self.gathered.view(-1), self.partial.view(-1))
            else:
                self.gathered.copy_(self.partial.unsqueeze(0))
            if self.rank == 0:
                self.end(logits_ptr, next_ptr)
