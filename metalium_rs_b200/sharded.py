"""The reference's multi-chip product on GPUs of one box: a GEMM split along N with K whole.

`Fabric::matmul_resident` (crates/tt-kernels/src/shard.rs:348-458; Burn side
`MeshEngine::matmul_dram`, crates/burn-tt/src/server.rs:5408) replicates A, gives every
chip a run of B's columns (`per = ceil(ceil(N/32)/chips)` tiles, shard.rs:398-405), multiplies
on each chip and gathers the column slices on chip 0.  K is never split, so every element is
the same sum as on one chip, bit for bit (shard.rs:11-16).

Here: one process a GPU, each with its own engine.  Rank r holds A and columns
[r*per, (r+1)*per) of B and runs the engine's product on its slice.  `PeerStoreMatmul` has the
product's epilogue store every tile into every rank's C (its peers' through CUDA IPC mappings, over
NVLink); `ShardedMatmul` multiplies into a buffer of its own and lets an NCCL all-gather
(torch.distributed) and one strided copy build the row-major C.  No kernel reads another GPU's
memory, and no TMA copy touches it.
"""
from __future__ import annotations

import json
import os
from typing import List, Tuple

import numpy as np


def partition(n: int, world: int, tile: int = 32) -> List[Tuple[int, int]]:
    """Column runs [first, last) per rank: whole tiles, dealt in order (shard.rs:398-405).
    Trailing ranks may get nothing."""
    tiles = -(-n // tile)
    per = -(-tiles // world) * tile
    return [(min(r * per, n), min((r + 1) * per, n)) for r in range(world)]


def gather_columns(local, world: int, group=None):
    """All-gather the ranks' [M, per] column slices into [world, M, per] (torch tensors, CPU with
    gloo or CUDA with NCCL).  Every rank's slice must have the same shape."""
    import torch
    import torch.distributed as dist
    m, per = local.shape
    out = torch.empty((world * m, per), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    return out.view(world, m, per)


def interleave(staged, n: int):
    """[world, M, per] -> row-major [M, n] (torch; the CPU twin of the engine's copy_blocks)."""
    world, m, per = staged.shape
    return staged.permute(1, 0, 2).reshape(m, world * per)[:, :n].contiguous()


class MeshExecution:
    """Completion evidence of the sharded products, the reference's `FabricExecution`
    (crates/tt-kernels/src/shard.rs:139-145; `Engine::mesh_execution`, crates/burn-tt/src/server.rs:587):
    how many products each rank has completed and how much it has handed to its peers.  A rank counts
    a step once its exchange has been ordered behind the product (the gather waited for, or the
    all-reduce behind the peer stores enqueued); `report()` synchronises, gathers the ranks' counts and
    returns them with the transfers and bytes this rank sent."""

    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world
        self.completed = 0
        self.transfers = 0
        self.bytes = 0

    def count(self, transfers: int, nbytes: int):
        self.completed += 1
        self.transfers += transfers
        self.bytes += nbytes

    def report(self, sync=None, group=None) -> dict:
        import torch.distributed as dist
        if sync:
            sync()
        counts = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(counts, self.completed, group=group)
        else:
            counts = [self.completed]
        return {"completed_matmuls": counts, "acknowledged_transfers": self.transfers, "acknowledged_bytes": self.bytes}


class ShardedMatmul:
    """C = A B on `world` GPUs, B's columns split.  A [M,K] and the local B slice [K,per] are
    engine buffers that stay resident; `run()` returns a new buffer holding the full row-major C.

    The product is cut in `panels` row panels.  Each panel's product is launched on the engine's
    stream and its all-gather is issued asynchronously behind it, so NCCL moves panel p over
    NVLink while the tensor cores work on panel p+1; one strided copy at the end lays the
    gathered [panel, rank, rows, per] blocks side by side as the row-major C."""

    def __init__(self, eng, rank: int, world: int, m: int, k: int, n: int, a_buf: int, b_slice_buf: int, bf16=True,
                 panels: int = 0, comm_sms: int = -1):
        """panels: row panels (0: B200TT_SHARD_PANELS or 8).  comm_sms: SMs the products leave free for
        the all-gather running beside them (-1: B200TT_SHARD_COMM_SMS or 0).  Measured on four B200s at
        16384^3: 8 panels 3,531 TFLOP/s against 3,321 with 4; leaving 16 or 32 SMs free made it slower
        (3,097 and 3,212) -- NCCL's blocks share the SMs with the persistent product's mostly waiting
        warps well enough -- so the default keeps every SM on the product."""
        import torch
        from . import BF16, F32
        panels = panels or int(os.environ.get("B200TT_SHARD_PANELS", "8"))
        comm_sms = comm_sms if comm_sms >= 0 else int(os.environ.get("B200TT_SHARD_COMM_SMS", "0"))
        self.eng, self.rank, self.world = eng, rank, world
        self.m, self.k, self.n = m, k, n
        self.parts = partition(n, world)
        self.per = self.parts[0][1] - self.parts[0][0]
        if any(hi - lo != self.per for lo, hi in self.parts):
            raise ValueError(f"{n} columns do not split evenly over {world} ranks in whole tiles")
        while panels > 1 and (m % panels or (m // panels) % 256):
            panels -= 1
        self.panels, self.mp = panels, m // panels
        self.a, self.b = a_buf, b_slice_buf
        self.bf16 = bf16
        self.dt = torch.int16 if bf16 else torch.float32
        self.elem = BF16 if bf16 else F32
        dev = torch.device("cuda", torch.cuda.current_device())
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.sm_limit = max(2, sms - comm_sms) if (world > 1 and comm_sms > 0) else 0
        # torch owns the exchange buffer; the engine adopts it so its copy kernel reads it
        self.staged = torch.empty((panels * world * self.mp, self.per), dtype=self.dt, device=dev)
        self.staged_buf = eng.adopt(self.staged.data_ptr(), panels * world * self.mp, self.per, self.elem)
        self.stream = torch.cuda.ExternalStream(eng.stream())
        self.a_panels = [eng.slice_rows(a_buf, p * self.mp, self.mp)[0] for p in range(panels)] if panels > 1 else [a_buf]
        self.moves = [(((p * world + r) * self.mp, 0), (p * self.mp, r * self.per), (self.mp, self.per), False)
                      for p in range(panels) for r in range(world)]
        self.mesh = MeshExecution(rank, world)

    def run(self) -> int:
        import torch
        import torch.distributed as dist
        eng, g, mp = self.eng, self.world, self.mp
        mm = eng.matmul_dram_bf16 if self.bf16 else eng.matmul_dram
        pending = []
        eng.set_matmul_sm_limit(self.sm_limit)
        with torch.cuda.stream(self.stream):
            for p in range(self.panels):
                out, _ = mm(self.a_panels[p], False, self.b, False)
                ptr, _ = eng.device_ptr(out)
                src = _as_tensor(ptr, (mp, self.per), self.dt)
                dst = self.staged[p * g * mp:(p + 1) * g * mp]
                if self.bf16:  # NCCL has no 16-bit integer type: name the same bits BF16
                    src, dst = src.view(torch.bfloat16), dst.view(torch.bfloat16)
                pending.append((dist.all_gather_into_tensor(dst, src, async_op=True), out))
            for work, out in pending:
                work.wait()      # the engine's stream waits for the gather; the panel may then be reused
                eng.free(out)
        eng.set_matmul_sm_limit(0)
        self.mesh.count(self.panels, self.m * self.per * (2 if self.bf16 else 4) * (g - 1))
        full, _ = eng.copy_blocks(self.staged_buf, self.moves, (self.m, self.n))
        return full  # the caller gives it back with release()

    def release(self, buf: int):
        self.eng.free(buf)

    def mesh_execution(self) -> dict:
        return self.mesh.report(self.eng.sync)

    def close(self):
        pass

    describe = "row panels: NCCL all-gather of panel p overlapped with the product of panel p+1, then one strided copy into row-major C"


class _Shared:
    """A [rows, cols] BF16 matrix every rank can store into, in two alternating copies.  How a rank reaches the
    other ranks' copies, best first (`B200TT_EXCHANGE` = multicast | peer | ipc forces one):

      multicast  the copies are symmetric memory bound to one NVLS multicast object (torch.distributed's
                 symmetric memory does the driver calls); a store to the multicast address is delivered by the
                 NVSwitch to every rank, so a rank sends each piece once;
      peer       the same memory, reached through each peer's own address: one store a peer;
      ipc        pool blocks of the engine exchanged as CUDA IPC handles: one store a peer.

    With plain peer stores the destinations are taken in the order rank + 1, rank + 2, ... so that the ranks do not
    all store into the same peer at the same moment.  `dst[i]` is the address list for `matmul_into` /
    `store_block_into` (own copy first); `mc[i]` the multicast address, or 0."""

    def __init__(self, eng, rank: int, world: int, rows: int, cols: int):
        import torch
        import torch.distributed as dist
        self.eng, self.rank, self.world = eng, rank, world
        self.bufs, self.dst, self.mc, self.opened, self.keep = [], [], [], [], []
        want = os.environ.get("B200TT_EXCHANGE", "")
        order = [(rank + i) % world for i in range(1, world)]
        self.how = "ipc"
        if want != "ipc":
            try:
                import torch.distributed._symmetric_memory as symm
                from . import BF16
                dev = torch.device("cuda", torch.cuda.current_device())
                for _ in range(2):
                    t = symm.empty((rows, cols), dtype=torch.bfloat16, device=dev)
                    t.zero_()
                    h = symm.rendezvous(t, dist.group.WORLD)
                    ptrs = [int(x) for x in h.buffer_ptrs]
                    mc = int(h.multicast_ptr) if (want != "peer" and h.has_multicast_support) else 0
                    self.keep.append((t, h))
                    self.bufs.append(eng.adopt(t.data_ptr(), rows, cols, BF16))
                    self.dst.append([ptrs[rank]] + [ptrs[r] for r in order])
                    self.mc.append(mc)
                self.how = "multicast" if all(self.mc) else "peer"
                if not all(self.mc):
                    self.mc = [0, 0]
                torch.cuda.synchronize()
            except Exception as ex:        # no symmetric memory on this box: the IPC form below
                if want in ("multicast", "peer"):
                    raise
                self._why_not = str(ex)[:200]
                for b in self.bufs:
                    eng.free(b)
                self.bufs, self.dst, self.mc, self.keep = [], [], [], []
        agree = [None] * world
        dist.all_gather_object(agree, self.how)
        if len(set(agree)) != 1:           # every rank takes the same form, or all fall back together
            for b in self.bufs:
                eng.free(b)
            self.bufs, self.dst, self.mc, self.keep, self.how = [], [], [], [], "ipc"
        if self.how == "ipc":
            for _ in range(2):
                c, _ = eng.zeros_dram((rows, cols), bf16=True)
                mine, _ = eng.device_ptr(c)
                handles = [None] * world
                dist.all_gather_object(handles, eng.ipc_export(c))
                peers = [eng.ipc_open(handles[r]) for r in order]
                self.bufs.append(c)
                self.opened += peers
                self.dst.append([mine] + peers)
                self.mc.append(0)

    def close(self):
        import torch.distributed as dist
        self.eng.sync()
        dist.barrier()
        for p in self.opened:
            self.eng.ipc_close(p)
        dist.barrier()                               # every mapping is closed before an owner frees its copy
        for c in self.bufs:
            self.eng.free(c)
        self.opened, self.bufs, self.keep = [], [], []


class PeerStoreMatmul:
    """The same sharded product with the exchange inside the product: every rank keeps a whole C that every
    rank can store into (`_Shared`), and a rank's product stores each finished tile of its column slice into every
    rank's C from its epilogue -- once, at the NVLS multicast address (`b200_matmul_into_multicast`: the NVSwitch
    replicates it), or, where no multicast object can be had, once a rank over NVLink (`b200_matmul_into`).  No
    staging buffer, no collective on the data, no final copy.

    Ordering is on the device: a one-element NCCL all-reduce is enqueued on the engine's stream behind
    the product, so it completes on a rank only when every rank's product -- and with it every store
    into this rank's C -- has completed; whatever the caller enqueues next reads a whole C.  Two C
    buffers alternate, so the product of step i+1 never writes what a reader of step i may still
    read; a reader must be done with step i's C before step i+2 is issued.

    `run()` returns the buffer that holds this step's C; it belongs to this object (release() does
    nothing)."""

    def __init__(self, eng, rank: int, world: int, m: int, k: int, n: int, a_buf: int, b_slice_buf: int, bf16=True):
        import torch
        import torch.distributed as dist
        self.eng, self.rank, self.world = eng, rank, world
        self.m, self.k, self.n = m, k, n
        self.parts = partition(n, world)
        self.per = self.parts[0][1] - self.parts[0][0]
        if any(hi - lo != self.per for lo, hi in self.parts):
            raise ValueError(f"{n} columns do not split evenly over {world} ranks in whole tiles")
        if not bf16:
            raise ValueError("the peer-store product is BF16")
        self.a, self.b = a_buf, b_slice_buf
        self.shared = _Shared(eng, rank, world, m, n)
        self.c = self.shared.bufs
        if self.shared.how == "multicast" and (self.per * 2) % 128:
            raise ValueError("a multicast slice must be whole 128-byte row segments")
        self.step = 0
        self.panels = 1
        self.stream = torch.cuda.ExternalStream(eng.stream())
        self.flag = torch.zeros(1, device=torch.device("cuda", torch.cuda.current_device()))
        self.mesh = MeshExecution(rank, world)
        self.describe = {"multicast": "each rank's product stores its tiles once at an NVLS multicast address from its epilogue "
                                      "(multimem.st; the NVSwitch delivers them to every rank's C)",
                         "peer": "each rank's product stores its tiles into every rank's C from its epilogue (peer stores over NVLink "
                                 "into symmetric memory)",
                         "ipc": "each rank's product stores its tiles into every rank's C from its epilogue (peer stores over NVLink "
                                "through CUDA IPC mappings)"}[self.shared.how] + \
            "; a one-element all-reduce behind it orders the ranks; no collective on the data"
        dist.barrier()

    def run(self) -> int:
        import torch
        import torch.distributed as dist
        which = self.step & 1
        self.step += 1
        first = self.parts[self.rank][0]
        if self.shared.mc[which]:
            self.eng.matmul_into_multicast(self.a, self.b, self.shared.mc[which], (self.m, self.n), first, True)
        else:
            self.eng.matmul_into(self.a, self.b, self.shared.dst[which], (self.m, self.n), first, True)
        with torch.cuda.stream(self.stream):
            dist.all_reduce(self.flag)               # behind the product on the engine's stream: a device-side barrier
        sent = 1 if self.shared.mc[which] else self.world - 1
        self.mesh.count(sent, self.m * self.per * 2 * sent)
        return self.c[which]

    def run_from_host(self, a_rows_host: int, b_slice_host: int, c_rows_host: int) -> None:
        """One step with host operands and a host result, the work of bringing them in shared by the ranks: this
        rank uploads ITS row block of A ([m / world, k]) and its column slice of B from pinned host memory, the row
        blocks are all-gathered over NVLink into every rank's A, the product runs, and this rank downloads ITS row
        block of C ([m / world, n]) -- so across the ranks A and B go up once and one C comes down
        (`Fabric::matmul_resident` leaves one C, on chip 0: crates/tt-kernels/src/shard.rs:444-452).  The three
        arguments are host addresses; returns when this rank's rows of C are in host memory."""
        import torch
        import torch.distributed as dist
        e, g, r = self.eng, self.world, self.rank
        rows = self.m // g
        assert self.m % g == 0
        if not hasattr(self, "_a_rows"):     # views of this rank's row blocks (`slice_rows`: no copy)
            self._a_rows = e.slice_rows(self.a, r * rows, rows)[0]
            self._c_rows = [e.slice_rows(c, r * rows, rows)[0] for c in self.c]
            a_ptr, _ = e.device_ptr(self.a)
            self._a_t = _as_tensor(a_ptr, (self.m, self.k), torch.int16).view(torch.bfloat16)
        which = self.step & 1
        e.write_ptr(self._a_rows, a_rows_host, rows * self.k, 2)
        e.write_ptr(self.b, b_slice_host, self.k * self.per, 2)
        with torch.cuda.stream(self.stream):
            dist.all_gather_into_tensor(self._a_t, self._a_t[r * rows:(r + 1) * rows])   # in place: the row blocks are contiguous
        self.run()
        e.download_into(self._c_rows[which], c_rows_host, rows * self.n, 2)

    def release(self, buf: int):
        pass

    def mesh_execution(self) -> dict:
        return self.mesh.report(self.eng.sync)

    def close(self):
        if hasattr(self, "_a_rows"):
            for v in [self._a_rows] + self._c_rows:
                self.eng.free(v)
        self.shared.close()
        self.c = []


class TpMlp:
    """The tensor-parallel MLP of the attention-shaped workload: x [m, hidden]; gate and up
    [hidden, ff] column-sharded (rank r holds its ff/g columns of each, side by side); silu(gate)*up
    local; the hidden activation [m, ff] gathered on every rank; down [ff, hidden] column-sharded;
    the output [m, hidden] gathered on every rank.  K is never split (shard.rs:11-16), so every
    element is the one-GPU sum.  Both gathers are owner stores over NVLink: the activation slice by
    `b200_store_block_into`, the output slice from the down product's epilogue (`b200_matmul_into`);
    a one-element all-reduce behind each orders the ranks on the device."""

    def __init__(self, eng, rank: int, world: int, m: int, hidden: int, ff: int, x_buf: int, wgu_slice: int, wdown_slice: int):
        import torch
        import torch.distributed as dist
        assert ff % world == 0 and hidden % world == 0
        self.eng, self.rank, self.world = eng, rank, world
        self.m, self.hidden, self.ff = m, hidden, ff
        self.pf, self.ph = ff // world, hidden // world
        self.x, self.wgu, self.wd = x_buf, wgu_slice, wdown_slice
        self.hid = _Shared(eng, rank, world, m, ff)
        self.out = _Shared(eng, rank, world, m, hidden)
        self.step = 0
        self.stream = torch.cuda.ExternalStream(eng.stream())
        self.flag = torch.zeros(1, device=torch.device("cuda", torch.cuda.current_device()))
        dist.barrier()

    def run(self) -> int:
        import torch
        import torch.distributed as dist
        from . import EltwiseOp, kinds
        e, m, pf = self.eng, self.m, self.pf
        which = self.step & 1
        self.step += 1
        gu, _ = e.matmul_dram_bf16(self.x, False, self.wgu, False)                      # [m, gate_r | up_r]
        act, _ = e.eltwise_blocks_as(EltwiseOp(kinds.SILU_MUL, 0.0, 0.0), (gu, (0, 0), (m, pf)), (gu, (0, pf), (m, pf)), None, True)
        e.free(gu)
        if self.hid.mc[which]:
            e.store_block_into_multicast((act, (0, 0), (m, pf)), self.hid.mc[which], (m, self.ff), self.rank * pf)
        else:
            e.store_block_into((act, (0, 0), (m, pf)), self.hid.dst[which], (m, self.ff), self.rank * pf)
        e.free(act)
        with torch.cuda.stream(self.stream):
            dist.all_reduce(self.flag)          # every rank's slice of the activation is here
        if self.out.mc[which]:
            e.matmul_into_multicast(self.hid.bufs[which], self.wd, self.out.mc[which], (m, self.hidden), self.rank * self.ph, True)
        else:
            e.matmul_into(self.hid.bufs[which], self.wd, self.out.dst[which], (m, self.hidden), self.rank * self.ph, True)
        with torch.cuda.stream(self.stream):
            dist.all_reduce(self.flag)          # every rank's slice of the output is here
        return self.out.bufs[which]

    def flops(self) -> float:
        return 6.0 * self.m * self.hidden * self.ff

    def close(self):
        self.hid.close()
        self.out.close()


def tp_mlp_bench(eng, rank, world, dev, steps=5):
    """x [4096, 8192], ff 28672 (the attention-shaped workload's MLP).  Returns (ms a step, validated)."""
    import torch
    import torch.distributed as dist
    from . import BF16, EltwiseOp, kinds
    m, hidden, ff = 4096, 8192, 28672
    pf, ph = ff // world, hidden // world
    g = torch.Generator(device=dev)
    g.manual_seed(0xC0F5)
    rnd = lambda r, c, s: ((torch.rand((r, c), generator=g, device=dev) * 2 - 1) * s).to(torch.bfloat16)
    x_t = rnd(m, hidden, 1.0)
    wg, wu, wd = rnd(hidden, ff, 0.02), rnd(hidden, ff, 0.02), rnd(ff, hidden, 0.02)
    lo_f, lo_h = rank * pf, rank * ph
    wgu_t = torch.cat([wg[:, lo_f:lo_f + pf], wu[:, lo_f:lo_f + pf]], 1).contiguous()
    wd_t = wd[:, lo_h:lo_h + ph].contiguous()
    x_buf = eng.adopt(x_t.data_ptr(), m, hidden, BF16)
    wgu_buf = eng.adopt(wgu_t.data_ptr(), hidden, 2 * pf, BF16)
    wd_buf = eng.adopt(wd_t.data_ptr(), ff, ph, BF16)
    torch.cuda.synchronize()
    mlp = TpMlp(eng, rank, world, m, hidden, ff, x_buf, wgu_buf, wd_buf)
    for _ in range(3):
        out = mlp.run()
    eng.sync()
    # validation: the first 256 rows computed whole on this GPU, bit for bit
    rows = 256
    xp = eng.adopt(x_t.data_ptr(), rows, hidden, BF16)
    wfull = torch.cat([wg, wu], 1).contiguous()
    wfull_buf = eng.adopt(wfull.data_ptr(), hidden, 2 * ff, BF16)
    wd_full = eng.adopt(wd.data_ptr(), ff, hidden, BF16)
    gu, _ = eng.matmul_dram_bf16(xp, False, wfull_buf, False)
    act, _ = eng.eltwise_blocks_as(EltwiseOp(kinds.SILU_MUL, 0.0, 0.0), (gu, (0, 0), (rows, ff)), (gu, (0, ff), (rows, ff)), None, True)
    ref, _ = eng.matmul_dram_bf16(act, False, wd_full, False)
    eng.sync()
    op, _ = eng.device_ptr(out)
    rp, _ = eng.device_ptr(ref)
    same = bool(torch.equal(_as_tensor(op, (m, hidden), torch.int16)[:rows], _as_tensor(rp, (rows, hidden), torch.int16)))
    finite = bool(torch.isfinite(_as_tensor(op, (m, hidden), torch.int16).view(torch.bfloat16).float()).all())
    for b in (gu, act, ref):
        eng.free(b)
    okt = torch.tensor([1.0 if (same and finite) else 0.0], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    dist.barrier()
    eng.sync()
    eng.timer_start()
    for _ in range(steps):
        mlp.run()
    ms = eng.timer_stop() / steps
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops = mlp.flops()
    mlp.close()
    del wfull, wg, wu, wd
    return float(t.item()), okt.item() >= 1.0, flops


def _as_tensor(ptr: int, shape, dtype):
    """A torch view of device memory the engine owns."""
    import torch

    class _Iface:
        pass
    it = _Iface()
    code = {torch.int16: "<i2", torch.float32: "<f4"}[dtype]
    it.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": code, "data": (ptr, False), "version": 3,
                                   "strides": None}
    return torch.as_tensor(it, device=torch.device("cuda", torch.cuda.current_device()))


def bench_main(args, metric, unit, size, workload_name, peaks, ClockSampler, cheap_bf16):
    """`bench.py --gpus N` under torchrun: the 16384^3 BF16 product column-sharded over N ranks."""
    import torch
    import torch.distributed as dist
    from . import BF16, CudaEngine, build

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if rank == 0:
        build.build()
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dist.barrier()
    eng = CudaEngine(local_rank, bf16_matmul_mode=2)
    m = k = n = args.size or size
    parts = partition(n, world)
    lo, hi = parts[rank]
    per = hi - lo
    dev = torch.device("cuda", local_rank)

    # Same A and B on every rank (same seed), generated on the device; B is then cut.
    g = torch.Generator(device=dev)
    g.manual_seed(0xC0F2)
    a_t = (torch.rand((m, k), generator=g, device=dev) * 2 - 1).to(torch.bfloat16)
    b_full = (torch.rand((k, n), generator=g, device=dev) * 2 - 1).to(torch.bfloat16)
    b_t = b_full[:, lo:hi].contiguous()
    a_buf = eng.adopt(a_t.data_ptr(), m, k, BF16)
    b_buf = eng.adopt(b_t.data_ptr(), k, per, BF16)
    torch.cuda.synchronize()
    # The exchange: peer stores from the product's epilogue, or (B200TT_SHARD=nccl, or where CUDA IPC is
    # refused) an NCCL all-gather in row panels.
    sm, how = None, os.environ.get("B200TT_SHARD", "peer")
    if how != "nccl":
        try:
            sm = PeerStoreMatmul(eng, rank, world, m, k, n, a_buf, b_buf)
        except Exception as ex:   # every rank fails alike (same box, same driver): fall back together
            if rank == 0:
                print(f"peer-store product unavailable ({ex}); using the NCCL all-gather", flush=True)
            sm = None
    agree = torch.tensor([1.0 if sm is not None else 0.0], device=dev)
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    if agree.item() < 1.0:
        if sm is not None:
            sm.close()
        sm = ShardedMatmul(eng, rank, world, m, k, n, a_buf, b_buf)
    fused = isinstance(sm, PeerStoreMatmul)

    for _ in range(max(args.warmup, 3)):
        sm.release(sm.run())
    full = sm.run()
    eng.sync()
    torch.cuda.synchronize()
    fp, _ = eng.device_ptr(full)
    full_t = _as_tensor(fp, (m, n), torch.int16)

    # validity: 32 sampled elements against F64 dot products, and (shard.rs:11-16) the sharded
    # result equals the one-GPU product bit for bit on a 2048-column probe of this rank's slice
    c = full_t.view(torch.bfloat16)
    rng = np.random.default_rng(rank)
    worst = 0.0
    for i, j in zip(rng.integers(0, m, 32), rng.integers(0, n, 32)):
        ai = a_t[int(i)].double()
        bj = b_full[:, int(j)].double()
        t = float(ai @ bj)
        s = float(ai.abs() @ bj.abs())
        worst = max(worst, abs(float(c[int(i), int(j)]) - t) / s)
    ok = worst <= 2.0 ** -8
    probe_cols = min(2048, n)
    pb = b_full[:, :probe_cols].contiguous()
    pb_buf = eng.adopt(pb.data_ptr(), k, probe_cols, BF16)
    single, _ = eng.matmul_dram_bf16(a_buf, False, pb_buf, False)
    sp, _ = eng.device_ptr(single)
    eng.sync()
    same = bool(torch.equal(_as_tensor(sp, (m, probe_cols), torch.int16), full_t[:, :probe_cols]))
    eng.free(single)
    sm.release(full)
    flags = torch.tensor([0.0, worst], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    okt = torch.tensor([1.0 if (ok and same) else 0.0], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if okt.item() < 1.0:
        if rank == 0:
            print(json.dumps({"metric": metric, "error": "sharded product failed validation",
                              "max_err_over_S": float(flags[1].item())}))
        dist.destroy_process_group()
        raise SystemExit(1)

    launches0 = eng.device_traffic().launches
    sampler = ClockSampler(local_rank) if rank == 0 else None
    dist.barrier()
    torch.cuda.synchronize()
    eng.sync()
    eng.timer_start()
    for _ in range(args.steps):
        sm.release(sm.run())
    ms = eng.timer_stop()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    launches = eng.device_traffic().launches - launches0

    # completion evidence (the reference's `FabricExecution`): every rank's completed products, this rank's transfers
    mesh = sm.mesh_execution()

    # product alone (no exchange), to show what the exchange costs.  The two legs run one after the other under a
    # power cap that moves, so each carries the SM clock sampled while it ran: compare time x median MHz.
    for _ in range(3):
        o, _ = eng.matmul_dram_bf16(a_buf, False, b_buf, False)
        eng.free(o)
    sampler2 = ClockSampler(local_rank) if rank == 0 else None
    dist.barrier()
    eng.sync()
    eng.timer_start()
    for _ in range(args.steps):
        o, _ = eng.matmul_dram_bf16(a_buf, False, b_buf, False)
        eng.free(o)
    ms_mm = eng.timer_stop()
    clocks_mm = sampler2.stop() if sampler2 else None
    t2 = torch.tensor([ms_mm], device=dev)
    dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    ms_mm = float(t2.item())

    # the attention-shaped workload's tensor-parallel MLP on the same ranks (owner stores for both gathers)
    tp = None
    if fused and os.environ.get("B200TT_TP_MLP", "1") == "1":
        try:
            tp_ms, tp_ok, tp_flops = tp_mlp_bench(eng, rank, world, dev)
            tp = {"ms_per_step": tp_ms, "tflops": tp_flops / (tp_ms * 1e-3) / 1e12, "equals_single_gpu_bits": bool(tp_ok),
                  "shape": "x [4096, 8192] BF16, ff 28672: gate|up and down column-sharded, both gathers by owner stores",
                  "exchange": sm.shared.how}
        except Exception as ex:
            tp = {"error": str(ex)[:200]}

    # end to end: A and the B slice from pinned host memory, the sharded product, C back to the host
    e2e = None
    if not args.no_e2e:
        import time
        steps = 3
        if fused and m % world == 0:
            # every rank brings in its row block of A and its column slice of B and takes out its row block of C:
            # across the ranks the operands go up once and one C comes down
            rows = m // world
            a_host = a_t[rank * rows:(rank + 1) * rows].view(torch.int16).cpu().pin_memory()
            b_host = b_t.view(torch.int16).cpu().pin_memory()
            c_host = torch.empty((rows, n), dtype=torch.int16).pin_memory()
            sm.run_from_host(a_host.data_ptr(), b_host.data_ptr(), c_host.data_ptr())      # warm-up
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                sm.run_from_host(a_host.data_ptr(), b_host.data_ptr(), c_host.data_ptr())
            dt = torch.tensor([(time.perf_counter() - t0) * 1e3 / steps], device=dev)
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            e2e_ms = float(dt.item())
            same = torch.equal(c_host, full_t[rank * rows:(rank + 1) * rows].cpu())          # the rows that came down are C's
            okh = torch.tensor([1.0 if same else 0.0], device=dev)
            dist.all_reduce(okh, op=dist.ReduceOp.MIN)
            e2e = {"value": 2.0 * m * n * k / (e2e_ms * 1e-3) / 1e12, "unit": unit, "ms_per_step": e2e_ms,
                   "h2d_bytes_per_step": (m * k + k * n) * 2, "d2h_bytes_per_step": m * n * 2,
                   "call": "PeerStoreMatmul.run_from_host: a rank uploads its rows of A and its columns of B, the rows are "
                           "all-gathered over NVLink, the product runs, the rank downloads its rows of C",
                   "host_result_equals_device_result": bool(okh.item() >= 1.0)}
        else:
            a_host = a_t.view(torch.int16).cpu().pin_memory()
            b_host = b_t.view(torch.int16).cpu().pin_memory()
            c_host = torch.empty((m, n), dtype=torch.int16).pin_memory()
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                eng.write_ptr(a_buf, a_host.data_ptr(), m * k, 2)
                eng.write_ptr(b_buf, b_host.data_ptr(), k * per, 2)
                full = sm.run()
                eng.download_into(full, c_host.data_ptr(), m * n, 2)
                sm.release(full)
            dt = torch.tensor([(time.perf_counter() - t0) * 1e3 / steps], device=dev)
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            e2e_ms = float(dt.item())
            e2e = {"value": 2.0 * m * n * k / (e2e_ms * 1e-3) / 1e12, "unit": unit, "ms_per_step": e2e_ms,
                   "h2d_bytes_per_step": world * (m * k + k * per) * 2, "d2h_bytes_per_step": world * m * n * 2}

    if rank == 0:
        flops = 2.0 * m * n * k
        ms_step = ms / args.steps
        value = flops / (ms_step * 1e-3) / 1e12
        pk, which = peaks()
        peak = float(pk.get("bf16_tflops", 1590.0)) * world
        gather_bytes = (world - 1) / world * m * n * 2
        line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": workload_name(world) if m == size else f"bf16 gemm {m}^3 column-sharded over {world}",
                           "m": m, "n": n, "k": k, "columns_per_rank": per,
                           "l2": "operands exceed the 126 MB L2; no flush needed",
                           "collective": (f"{sm.panels} " if not fused else "") + sm.describe},
                "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
                "roofline": {"bound": "tensor", "kernel": ("gemm_tc2_kernel storing to " + sm.shared.how) if fused else "gemm_tc_kernel + ncclAllGather",
                             "achieved": value, "peak": peak,
                             "unit": unit, "frac": value / peak, "peak_source": f"{which} cuBLAS bf16 burst x {world}",
                             "traffic": None, "product_only_ms": ms_mm / args.steps,
                             "product_only_clocks": clocks_mm,
                             "step_ms_x_mhz": (ms_step * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None,
                             "product_only_ms_x_mhz": (ms_mm / args.steps * clocks_mm["sm_mhz"]) if clocks_mm and clocks_mm.get("sm_mhz") else None,
                             "exchange": getattr(getattr(sm, "shared", None), "how", "nccl all-gather"),
                             "bytes_received_per_rank": gather_bytes,
                             "bytes_sent_per_rank": (m * per * 2) if getattr(getattr(sm, "shared", None), "how", "") == "multicast" else gather_bytes,
                             "receive_floor_ms_at_770GBs": gather_bytes / 770e9 * 1e3},
                "validated": {"max_err_over_S": float(flags[1].item()), "sharded_equals_single_gpu_bits": True},
                "tp_mlp": tp, "mesh_execution": mesh}
        print(json.dumps(line))
    dist.barrier()
    sm.close()
    eng.close()
    dist.destroy_process_group()
