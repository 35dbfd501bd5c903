"""Multi-GPU wave scheduling (one process per GPU, torch.distributed for the plumbing).

Two ways to spread a plan over the GPUs of one box:

* **column replicas** — the plan is replicated and every rank owns its own columns (batch entries or whole
  sequences). Columns never interact, so there is no data-path collective at all; `column_slice` only tells a
  rank which columns are its own.
* **neuron sharding** — for plans whose weights do not fit one GPU. Rank r keeps only rows
  [r*cout/n, (r+1)*cout/n) of every wave (weights, bias, gather lists of those groups); the canvas is
  replicated. After a wave each rank holds its block of the wave's output rows, which is one contiguous
  slab of the canvas, so the exchange is an in-place all-gather of `cout*pitch` FP16 elements on the
  canvas region itself. The next wave then gathers from a complete canvas in the rank's own HBM.

The reference is single-GPU; nothing here has a counterpart in it.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Callable, List, Optional, Tuple

import numpy as np

from .plan import Plan, Wave


def column_slice(total_columns: int, rank: int, world: int, granule: int = 1) -> Tuple[int, int]:
    """Columns [c0, c1) owned by `rank`; blocks are multiples of `granule` (e.g. one whole sequence) except
    possibly the last."""
    units = (total_columns + granule - 1) // granule
    per = (units + world - 1) // world
    c0 = min(total_columns, rank * per * granule)
    c1 = min(total_columns, (rank + 1) * per * granule)
    return c0, c1


def row_block(cout: int, group: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [r0, r1) of a wave owned by `rank`. Blocks are equal (the in-place all-gather needs that) and made of
    whole neuron groups."""
    if cout % world:
        raise ValueError(f"{cout} rows cannot be cut into {world} equal blocks")
    blk = cout // world
    if blk % group or blk % 16:
        raise ValueError(f"row block of {blk} is not made of whole groups of {group} neurons (and multiples of 16 rows)")
    return rank * blk, (rank + 1) * blk


def shard_wave(w: Wave, pitch: int, rank: int, world: int) -> Wave:
    """The part of wave `w` that `rank` computes: its rows, their weights / bias / gather lists, and the output
    (and residual) offsets moved to the block's first row."""
    if w.cout_map is not None:
        raise ValueError("waves with an output-row map cannot be neuron-sharded")
    r0, r1 = row_block(w.cout, w.group, rank, world)
    g0, g1 = r0 // w.group, r1 // w.group
    log0 = min(max(w.logical_cout - r0, 0), r1 - r0)
    return replace(
        w, cout=r1 - r0, logical_cout=log0 if log0 else (r1 - r0), idx=w.idx[g0:g1].copy(), weights=w.weights[r0:r1].copy(),
        bias=None if w.bias is None else w.bias[r0:r1].copy(), y_off=w.y_off + r0 * pitch,
        res_off=(w.res_off + r0 * pitch) if w.has_residual else w.res_off, name=f"{w.name}[{rank}/{world}]")


def shard_plan(plan: Plan, rank: int, world: int) -> Plan:
    return replace(plan, waves=[shard_wave(w, plan.pitch, rank, world) for w in plan.waves], name=f"{plan.name}[{rank}/{world}]")


def allgather_bytes(plan: Plan, world: int) -> List[int]:
    """Bytes each rank receives per wave: (n-1)/n of the wave's output rows."""
    return [w.cout * plan.pitch * 2 * (world - 1) // world for w in plan.waves]


class NeuronShardedRunner:
    """Runs a neuron-sharded plan: `compute(i)` produces this rank's rows of wave i on the local canvas, then the
    rows of all ranks are exchanged in place.

    `canvas` is a 1-D torch tensor of FP16 elements (CUDA for NCCL, CPU for gloo); `compute` is
    `NativePlan.execute_wave` in production. The collective runs on the current stream after the wave, so stream
    order makes wave i+1 see the complete rows.
    """

    def __init__(self, full_plan: Plan, rank: int, world: int, canvas, compute: Callable[[int], None], group=None):
        self.plan, self.rank, self.world, self.canvas, self.compute, self.group = full_plan, rank, world, canvas, compute, group
        self.regions = []
        for w in full_plan.waves:
            r0, r1 = row_block(w.cout, w.group, rank, world)
            self.regions.append((w.y_off, w.cout * full_plan.pitch, (r1 - r0) * full_plan.pitch))

    def exchange(self, i: int) -> None:
        import torch.distributed as dist
        y_off, total, blk = self.regions[i]
        out = self.canvas[y_off: y_off + total]
        mine = out[self.rank * blk: (self.rank + 1) * blk]
        if self.world == 1:
            return
        if self.canvas.is_cuda:
            dist.all_gather_into_tensor(out, mine, group=self.group)       # in place: `mine` is a view into `out`
        else:
            import torch
            raw = out.view(torch.uint8)                                     # gloo: ship the rows as plain bytes
            nb = 2 * blk
            parts = [raw[r * nb: (r + 1) * nb] for r in range(self.world)]
            dist.all_gather(parts, raw[self.rank * nb: (self.rank + 1) * nb].clone(), group=self.group)

    def run(self) -> None:
        for i in range(len(self.plan.waves)):
            self.compute(i)
            self.exchange(i)


def connect_peers(native_plan, rank: int, world: int):
    """Exchange the CUDA IPC handles of every rank's canvas and sync block over the default process group and hand
    them to the library: from then on the wave kernels store their rows into all canvases and order their launches
    against the peers' themselves, so a step needs no collective call (and can be one CUDA graph). Returns, per launch of a
    step, how many of the launches just before it the launch need not wait for on the peers (None if the ranks' plans
    do not have the same number of launches, in which case every launch waits for all earlier ones)."""
    import torch.distributed as dist
    mine = native_plan.ipc_handles()
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    native_plan.set_peers_ipc(rank, world, [h[0] for h in everyone], [h[1] for h in everyone])
    # order launches by the rows they touch: every rank learns which canvas intervals each launch of every rank reads and
    # writes, so that a launch waits only for the peers' launches it really depends on
    hulls = [None] * world
    dist.all_gather_object(hulls, native_plan.launch_hulls())
    slack = None
    if len({h.shape for h in hulls}) == 1:
        from .native import compute_peer_slack
        native_plan.set_peer_hulls(np.stack(hulls))
        slack = compute_peer_slack(np.stack(hulls))
    dist.barrier()          # every rank has its mappings before anybody launches
    return slack
