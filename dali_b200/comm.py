"""Brings up the library's communicator (include/dali_b200.h, "ranks and collectives") from a launcher
that already has torch.distributed running -- harness only: the collectives themselves, the peer exchange
and the sharding rules live in libdali_b200.so.

  init_from_torch(lib, device)   one process per GPU (torchrun): rank 0 draws the NCCL id, torch.distributed
                                 carries its 128 bytes to the other ranks, every rank joins.  world == 1
                                 needs no process group at all.
  init_host_from_torch(lib)      the library's collectives run through torch.distributed on HOST buffers
                                 (gloo on CPU in the tests; any backend that reduces CPU tensors).
"""
import ctypes

import numpy as np

_NP = {0: np.float32, 1: np.float64, 2: np.int32}


def init_from_torch(lib, device):
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        lib.comm_init_rank(device, 1, 0, None)
        return
    world, rank = dist.get_world_size(), dist.get_rank()
    on_gpu = dist.get_backend() == "nccl"
    ident = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        ident = torch.frombuffer(bytearray(lib.comm_unique_id()), dtype=torch.uint8).clone()
    if on_gpu:
        ident = ident.cuda()
    dist.broadcast(ident, 0)
    lib.comm_init_rank(device, world, rank, bytes(ident.cpu().numpy().tobytes()))


def init_host_from_torch(lib):
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(), dist.get_rank()
    ops = {0: dist.ReduceOp.SUM, 1: dist.ReduceOp.PRODUCT, 2: dist.ReduceOp.MAX, 3: dist.ReduceOp.MIN}

    def view(address, count, np_dtype):
        size = count * np.dtype(np_dtype).itemsize
        raw = (ctypes.c_char * size).from_address(address)
        return np.frombuffer(raw, dtype=np_dtype, count=count)

    def allreduce(address, n, dtype, op):
        a = view(address, n, _NP[dtype])
        t = torch.from_numpy(a.copy())
        dist.all_reduce(t, op=ops[op])
        a[:] = t.numpy()

    def allgather(send, recv, nbytes):
        mine = torch.from_numpy(view(send, nbytes, np.uint8).copy())
        parts = [torch.empty(nbytes, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(parts, mine)
        out = view(recv, nbytes * world, np.uint8)
        for r, part in enumerate(parts):
            out[r * nbytes:(r + 1) * nbytes] = part.numpy()

    lib.comm_init_host(world, rank, allreduce, allgather)
