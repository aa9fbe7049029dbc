"""Shared pieces of the data-parallel tests: the worker both the CPU (gloo + oracle) and the
GPU (libvolta_b200 + NCCL) tests run in every rank."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = [96, 160, 128, 1]
GLOBAL_BATCH = 64
STEPS = 4


def inputs(cfg_act="silu"):
    from volta_b200 import synth
    x = synth.rows("uniform", 1234, 0, GLOBAL_BATCH, LAYERS[0])
    y = synth.rows("normal", 4321, 0, GLOBAL_BATCH, LAYERS[-1])
    ws, bs = synth.kaiming_uniform_weights(LAYERS, 42)
    return x, y, ws, bs


def oracle_shard_worker(rank, world, port, opt, real, out_dir, act="silu", dropout_p=0.0):
    """One CPU rank: oracle on its row shard, gradients summed over ranks with gloo in rank
    order, identical update everywhere.  Writes its final parameters and loss trace."""
    import torch
    import torch.distributed as dist
    from oracle.oracle import Oracle

    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    x, y, ws, bs = inputs()
    B = GLOBAL_BATCH // world
    xs, ys = x[rank * B:(rank + 1) * B], y[rank * B:(rank + 1) * B]
    o = Oracle(LAYERS, act, opt, B, real=real, dropout_p=dropout_p)
    o.set_global_batch(GLOBAL_BATCH)
    o.set_shard_row0(rank * B)      # the mask stream is the single-process one; this rank draws its rows' slice
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    losses = []
    for _ in range(STEPS):
        o.grad_step(xs, ys)
        gw, gb = o.grad_views()
        for g in gw + gb:
            t = torch.from_numpy(g)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        lt = torch.tensor([o.loss()], dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        losses.append(float(lt.item()))
        o.update(0.01)
    pw, pb = o.get_params()
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), losses=np.array(losses),
             **{"w%d" % i: w for i, w in enumerate(pw)}, **{"b%d" % i: b for i, b in enumerate(pb)})
    dist.destroy_process_group()


def gpu_shard_worker(rank, world, port, opt, out_dir, repeat, fused=False, act="silu", options=None):
    """One GPU rank: libvolta_b200 handle on its row shard; the unique id travels over gloo.  fused: False (NCCL),
    True / "fused" (the peer-memory kernel) or "copy" (pushes by the copy engines + local sum)."""
    import torch
    import torch.distributed as dist
    from volta_b200 import TrainHandle
    from volta_b200.train import dp_unique_id

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    x, y, ws, bs = inputs()
    B = GLOBAL_BATCH // world
    xs, ys = np.ascontiguousarray(x[rank * B:(rank + 1) * B]), np.ascontiguousarray(y[rank * B:(rank + 1) * B])
    for rep in range(repeat):
        box = [dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        h = TrainHandle(LAYERS, act, opt, B, global_batch=GLOBAL_BATCH, world_size=world, rank=rank, unique_id=box[0],
                        dp_exchange="peer_copy" if fused == "copy" else "nccl", **(options or {}))
        if fused:
            handles = [None] * world
            dist.all_gather_object(handles, h.ipc_handle())
            h.attach_peers(handles)
        for i, (w, b) in enumerate(zip(ws, bs)):
            h.set_params(i, w, b)
        losses = []
        for _ in range(STEPS):
            h.step(xs, ys, 0.01)
            losses.append(h.loss())
        pw, pb = h.get_params()
        np.savez(os.path.join(out_dir, "rank%d_rep%d.npz" % (rank, rep)), losses=np.array(losses, dtype=np.float32),
                 **{"w%d" % i: w for i, w in enumerate(pw)}, **{"b%d" % i: b for i, b in enumerate(pb)})
        h.free()
        dist.barrier()
    dist.destroy_process_group()


def gpu_missing_rank_worker(rank, world, port, out_dir, wait_ms=200, exchange="nccl"):
    """Two ranks on the fused peer-memory path take two steps together; then rank 1 sits a step out (alive,
    its arena still mapped, nothing of its own in flight) while rank 0 steps alone with a short wait limit.
    Rank 0 records what it saw: the error code, and its parameters before and after the lonely step."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from volta_b200 import TrainHandle, VoltaB200Error
    from volta_b200.train import dp_unique_id

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    x, y, ws, bs = inputs()
    B = GLOBAL_BATCH // world
    xs, ys = np.ascontiguousarray(x[rank * B:(rank + 1) * B]), np.ascontiguousarray(y[rank * B:(rank + 1) * B])
    box = [dp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    h = TrainHandle(LAYERS, "silu", "adam", B, global_batch=GLOBAL_BATCH, world_size=world, rank=rank, unique_id=box[0],
                    device_wait_ms=wait_ms, dp_exchange=exchange)
    handles = [None] * world
    dist.all_gather_object(handles, h.ipc_handle())
    h.attach_peers(handles)
    for i, (w, b) in enumerate(zip(ws, bs)):
        h.set_params(i, w, b)
    for _ in range(2):
        h.step(xs, ys, 0.01)
        h.loss()
    before = sum(h.get_params(), [])
    dist.barrier()                       # both ranks idle, nothing in flight
    if rank == 0:
        code, msg = 0, ""
        h.step(xs, ys, 0.01)             # rank 1 never joins this one
        try:
            h.loss()
        except VoltaB200Error as e:
            code, msg = e.code, str(e)
        fp = C.POINTER(C.c_float)
        wo, bo = (fp * h.n)(), (fp * h.n)()
        rc = h.lib.volta_b200_get_params(h.h, wo, bo)
        after = [np.ctypeslib.as_array(wo[i], shape=(LAYERS[i], LAYERS[i + 1])).copy() for i in range(h.n)] + \
                [np.ctypeslib.as_array(bo[i], shape=(LAYERS[i + 1],)).copy() for i in range(h.n)]
        refused = 0
        try:
            h.step(xs, ys, 0.01)
        except VoltaB200Error as e:
            refused = e.code
        np.savez(os.path.join(out_dir, "rank0.npz"), code=code, msg=msg, get_params_rc=rc, refused=refused,
                 **{"before%d" % i: a for i, a in enumerate(before)}, **{"after%d" % i: a for i, a in enumerate(after)})
    dist.barrier()                       # rank 1 learns on the host that the step is over
    h.free()
    dist.barrier()
    dist.destroy_process_group()
