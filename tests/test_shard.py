"""Multi-rank host logic on CPU (gloo, world size 2): neuron sharding of a plan, the per-wave in-place
all-gather, and the column split. The per-rank wave computation is done by the oracle here (the CUDA path
needs a GPU); what is under test is the partitioning and the exchange."""
import os
import socket

import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import shard, synth
from snntome_b200.plan import ACT_RELU


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_plan():
    return synth.sparse_plan(seed=71, input_rows=1024, waves=3, cout=512, runs=8, run_len=16, columns=64, group=128, act=ACT_RELU)


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = _make_plan()
        x = synth.random_input(plan, 72)
        mine = shard.shard_plan(plan, rank, world)
        canvas_np = O.make_canvas(plan, x)
        canvas = torch.from_numpy(canvas_np.view(np.int16)).view(torch.float16)

        def compute(i):                      # oracle stands in for the device kernel on this rank's rows
            O.wave_forward(canvas_np, mine.waves[i], mine)

        runner = shard.NeuronShardedRunner(plan, rank, world, canvas, compute)
        runner.run()
        np.save(os.path.join(out_dir, f"canvas{rank}.npy"), canvas_np)
    finally:
        dist.destroy_process_group()


def test_neuron_sharded_plan_matches_single_rank(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    plan = _make_plan()
    want = O.run_plan(plan, synth.random_input(plan, 72))
    for r in range(world):
        got = np.load(tmp_path / f"canvas{r}.npy")
        assert np.array_equal(got, want), f"rank {r} canvas differs from the unsharded run"


def test_shard_wave_partitions_rows_exactly():
    plan = _make_plan()
    w = plan.waves[1]
    parts = [shard.shard_wave(w, plan.pitch, r, 4) for r in range(4)]
    assert [p.cout for p in parts] == [128] * 4
    assert np.array_equal(np.concatenate([p.weights for p in parts]), w.weights)
    assert np.array_equal(np.concatenate([p.idx for p in parts]), w.idx)
    assert np.array_equal(np.concatenate([p.bias for p in parts]), w.bias)
    assert [p.y_off for p in parts] == [w.y_off + r * 128 * plan.pitch for r in range(4)]
    with pytest.raises(ValueError):
        shard.shard_wave(w, plan.pitch, 0, 8)          # 64-row blocks would cut a 128-neuron group
    with pytest.raises(ValueError):
        shard.shard_wave(w, plan.pitch, 0, 3)
    assert shard.allgather_bytes(plan, 4) == [512 * 64 * 2 * 3 // 4] * 3


def test_column_slice_covers_all_columns_once():
    for total, world, granule in [(512, 8, 1), (8 * 4096, 8, 4096), (8 * 4096, 3, 4096), (100, 8, 1), (64, 2, 64)]:
        seen = np.zeros(total, dtype=int)
        for r in range(world):
            c0, c1 = shard.column_slice(total, r, world, granule)
            assert c0 % granule == 0
            seen[c0:c1] += 1
        assert (seen == 1).all()


def _slack_reference(hulls):
    """The ordering rule restated: union the intervals over the ranks; launch n may skip waiting for the launches just before
    it until it meets one (cyclically, the step before included) whose writes meet its reads, whose reads meet its writes, or
    whose writes meet its writes."""
    world, L, _ = hulls.shape
    u = []
    for n in range(L):
        r = [(int(h[n, 0]), int(h[n, 1])) for h in hulls if h[n, 0] < h[n, 1]]
        w = [(int(h[n, 2]), int(h[n, 3])) for h in hulls if h[n, 2] < h[n, 3]]
        u.append(((min(a for a, _ in r), max(b for _, b in r)) if r else None, (min(a for a, _ in w), max(b for _, b in w)) if w else None))
    meet = lambda a, b: a is not None and b is not None and a[0] < b[1] and b[0] < a[1]
    out = []
    for n in range(L):
        s = 0
        for back in range(1, L + 1):
            m = u[(n - back) % L]
            if meet(m[1], u[n][0]) or meet(m[0], u[n][1]) or meet(m[1], u[n][1]):
                break
            s += 1
        out.append(min(s, L - 1))
    return np.array(out, dtype=np.uint32)


def test_launch_ordering_rule_matches_its_restatement_and_a_decoder_layer_by_hand():
    from snntome_b200.native import compute_peer_slack
    rng = np.random.default_rng(17)
    for _ in range(200):
        world, L = int(rng.integers(1, 5)), int(rng.integers(1, 12))
        lo = rng.integers(0, 50, size=(world, L, 2)) * 64
        ln = rng.integers(0, 6, size=(world, L, 2)) * 64              # empty intervals occur
        hulls = np.stack([lo[..., 0], lo[..., 0] + ln[..., 0], lo[..., 1], lo[..., 1] + ln[..., 1]], axis=-1).astype(np.uint64)
        assert np.array_equal(compute_peer_slack(hulls), _slack_reference(hulls))
    # one decoder layer, tensors x, q|k|v, h, g, u, y as disjoint row ranges: launches qkv, o, gate, up, down
    T = {name: (i * 1000, i * 1000 + 1000) for i, name in enumerate(["x", "qkv", "h", "g", "u", "y"])}
    span = lambda *names: (min(T[n][0] for n in names), max(T[n][1] for n in names))
    launches = [(span("x"), span("qkv")), (span("x", "qkv"), span("h")), (span("h"), span("g")), (span("h"), span("u")), (span("h", "g"), span("y"))]
    hulls = np.array([[[r[0], r[1], w[0], w[1]] for r, w in launches]] * 2, dtype=np.uint64)
    slack = compute_peer_slack(hulls)
    assert slack[1] == 0 and slack[2] == 0          # o reads q, gate reads h: each waits for the launch just before it
    assert slack[3] == 1                            # up reads h (written two launches earlier) and touches nothing of gate's
    assert slack[4] == 1                            # down reads g and h: gate wrote g two launches back; up only read h and wrote u
    assert slack[0] == 3                            # qkv overwrites q|k|v, which o (four launches back, cyclically) reads
