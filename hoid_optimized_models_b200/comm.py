"""Peer-memory link for the fused tensor-parallel decode path (one process per GPU).

Each rank allocates one small communication buffer with cudaMalloc at set-up time, the ranks
exchange CUDA IPC handles through torch.distributed and map each other's buffers; the decode
kernels then exchange partial sums with plain peer stores over NVLink (see b200_gemv_bf16_tp in
include/b200ops.h).  No collective library call is made on the decode path.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check


class PeerLink:
    def __init__(self, group, rank: int, world: int, hidden: int):
        lib = _lib.lib()
        nbytes = lib.b200_tp_buffer_bytes(world, hidden)
        own = C.c_void_p()
        handle = C.create_string_buffer(64)
        check(lib.b200_tp_alloc(C.byref(own), handle, nbytes), "b200_tp_alloc")
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw, group=group)
        bufs = (C.c_void_p * world)()
        for p in range(world):
            if p == rank:
                bufs[p] = own.value
            else:
                q = C.c_void_p()
                check(lib.b200_tp_open(C.byref(q), handles[p]), "b200_tp_open")
                bufs[p] = q.value
        ctx = lib.b200_tp_create(bufs, world, rank, hidden)
        if ctx < 0:
            check(ctx, "b200_tp_create")
        self.ctx, self.rank, self.world = ctx, rank, world
        torch.cuda.synchronize()
        dist.barrier(group=group)     # every rank has mapped every buffer before first use
