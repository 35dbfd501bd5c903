"""Neuron sharding with direct stores into the peers' canvases, checked on one GPU: the ranks' plans live on the same
device, point at each other's canvas and sync block, and their launches are queued strictly in the order
wave 0 of every rank, wave 1 of every rank, ... on one stream. In that order every launch finds the launch counts it
waits for already published (nothing ever waits for a launch that is queued behind it), so the addressing, the
last-CTA election and the counting are exercised without two kernels having to run at the same time."""
import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import shard, synth
from snntome_b200.native import NativeError, NativePlan, PATH_FMA
from snntome_b200.plan import ACT_RELU, ACT_SILU

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-3


def run_sharded_on_one_gpu(plan, x, world, reps=2):
    import torch
    plans = [NativePlan.from_plan(shard.shard_plan(plan, r, world), device=0) for r in range(world)]
    canvases = [p.canvas_tensor() for p in plans]
    xt = torch.from_numpy(np.ascontiguousarray(x).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    for c in canvases:
        c[plan.input_off: plan.input_off + xt.numel()] = xt
    cps, sps = [p.canvas_ptr for p in plans], [p.sync_ptr for p in plans]
    for r, p in enumerate(plans):
        p.set_peers_raw(r, world, cps, sps)
    for _ in range(reps):
        for i in range(len(plan.waves)):
            for p in plans:
                p.execute_wave(i)
    out = []
    for p, c in zip(plans, canvases):
        assert p.status() == 0
        out.append(c.cpu().numpy().view(np.uint16))
    for p in plans:
        p.close()
    return out


@pytest.mark.parametrize("world", [2, 4])
def test_streaming_waves_store_to_every_canvas(world):
    plan = synth.sparse_plan(seed=91, input_rows=2048, waves=3, cout=1024 * world // 2, runs=8, run_len=32, columns=128, group=128, act=ACT_RELU)
    x = synth.random_input(plan, 92)
    want = O.run_plan(plan, x)
    got = run_sharded_on_one_gpu(plan, x, world)
    for r in range(world):
        for w in plan.waves:
            a, b = w.y_off, w.y_off + w.cout * plan.pitch
            ok, err, k = O.compare(got[r][a:b], want[a:b], RTOL, ATOL)
            assert ok, (r, w.name, err, k)
        assert np.array_equal(got[r], got[0])


def test_streaming_waves_send_their_tiles_with_tensor_copies():
    """More 128-neuron tiles per rank than SMs: the persistent streaming kernel, whose epilogue hands each 128 x 64 output block
    to the copy engine once per canvas (own and peers'). 160 tiles per rank, a partial last column block of valid columns, a
    residual on the second wave."""
    plan = synth.sparse_plan(seed=191, input_rows=2048, waves=2, cout=2 * 80 * 128, runs=4, run_len=32, columns=100, group=128, act=ACT_SILU)
    plan.waves[1].has_residual, plan.waves[1].res_off = True, plan.waves[0].y_off
    x = synth.random_input(plan, 192)
    want = O.run_plan(plan, x)
    got = run_sharded_on_one_gpu(plan, x, 2)
    for r in range(2):
        for w in plan.waves:
            a, b = w.y_off, w.y_off + w.cout * plan.pitch
            ok, err, k = O.compare(got[r][a:b], want[a:b], RTOL, ATOL)
            assert ok, (r, w.name, err, k)
    assert np.array_equal(got[0], got[1])


def test_small_waves_with_residual_store_to_every_canvas():
    """Dense chain at decode size: every wave runs on the cluster kernel (K splits reduced through distributed shared
    memory); the second wave adds a residual that a peer produced."""
    plan = synth.dense_chain(seed=93, dims=[512, 512, 512, 256], columns=64, act=ACT_SILU, weight_std=0.05, residual_from={2: 1})
    x = synth.random_input(plan, 94, dist="normal")
    want = O.run_plan(plan, x)
    got = run_sharded_on_one_gpu(plan, x, 2)
    for r in range(2):
        for w in plan.waves:
            a, b = w.y_off, w.y_off + w.cout * plan.pitch
            ok, err, k = O.compare(got[r][a:b], want[a:b], RTOL, ATOL)
            assert ok, (r, w.name, err, k)
    assert np.array_equal(got[0], got[1])


@pytest.mark.parametrize("world,group", [(2, 32), (4, 16), (2, 64)])
def test_small_group_waves_store_to_every_canvas(world, group):
    """Groups of 16 / 32 / 64 neurons run on the mma.sync kernel, which speaks the same protocol: bounded wait for the peers'
    launch counts, every output pair stored into every canvas, launch count published by the last CTA. The last wave gathers
    scattered single rows (index table instead of a run table)."""
    plan = synth.sparse_plan(seed=99 + group, input_rows=1024, waves=3, cout=64 * world, runs=8, run_len=16, columns=100, group=group, act=ACT_SILU)
    rng = np.random.default_rng(group)
    plan.waves[2].idx = (rng.integers(0, 1024 + 2 * 64 * world, size=plan.waves[2].idx.shape) * plan.pitch).astype(np.uint32)
    x = synth.random_input(plan, 96, dist="normal")
    want = O.run_plan(plan, x)
    got = run_sharded_on_one_gpu(plan, x, world)
    for r in range(world):
        for w in plan.waves:
            a, b = w.y_off, w.y_off + w.cout * plan.pitch
            ok, err, k = O.compare(got[r][a:b], want[a:b], RTOL, ATOL)
            assert ok, (r, w.name, err, k)
        assert np.array_equal(got[r], got[0])


def test_plans_with_fma_path_waves_are_rejected():
    plan = synth.sparse_plan(seed=95, input_rows=512, waves=1, cout=256, runs=8, run_len=32, columns=64, group=128, act=ACT_RELU)
    p0 = NativePlan.from_plan(shard.shard_plan(plan, 0, 2), device=0, force_path=PATH_FMA)
    p1 = NativePlan.from_plan(shard.shard_plan(plan, 1, 2), device=0)
    with pytest.raises(NativeError, match="stores to peers"):
        p0.set_peers_raw(0, 2, [p0.canvas_ptr, p1.canvas_ptr], [p0.sync_ptr, p1.sync_ptr])
    p0.close(); p1.close()


def test_missing_peer_ends_the_wait_with_a_status_bit(monkeypatch):
    """A rank whose peer never shows up: its second launch waits for the peer's first launch count, the bounded wait
    (shortened to 200 ms here) runs out, the kernel records status bit 5 and returns, and the context stays usable —
    a plan executed afterwards on the same GPU still matches the oracle. Nothing faults or hangs: the flag is simply
    never written."""
    import torch
    monkeypatch.setenv("K44B_WAIT_MS", "200")
    plan = synth.sparse_plan(seed=97, input_rows=1024, waves=2, cout=512, runs=8, run_len=32, columns=64, group=128, act=ACT_RELU)
    x = synth.random_input(plan, 98)
    p0 = NativePlan.from_plan(shard.shard_plan(plan, 0, 2), device=0)
    p1 = NativePlan.from_plan(shard.shard_plan(plan, 1, 2), device=0)      # never executes
    cps, sps = [p0.canvas_ptr, p1.canvas_ptr], [p0.sync_ptr, p1.sync_ptr]
    p0.set_peers_raw(0, 2, cps, sps)
    p1.set_peers_raw(1, 2, cps, sps)
    xt = torch.from_numpy(np.ascontiguousarray(x).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    p0.canvas_tensor()[plan.input_off: plan.input_off + xt.numel()] = xt
    p0.execute_wave(0)                    # needs nothing from the peer
    torch.cuda.synchronize()
    assert p0.status() == 0
    p0.execute_wave(1)                    # needs the peer's launch 0, which never comes
    torch.cuda.synchronize()
    with pytest.raises(NativeError) as ei:
        p0.status()
    assert "0x20" in str(ei.value) or "peer" in str(ei.value).lower()
    p0.close(); p1.close()
    monkeypatch.delenv("K44B_WAIT_MS")
    small = synth.config0(group=128)                                       # the context is still healthy
    xs = synth.random_input(small, 11)
    npn = NativePlan.from_plan(small, device=0)
    c = npn.canvas_tensor()
    c[small.input_off: small.input_off + xs.size] = torch.from_numpy(xs.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    npn.execute()
    assert npn.status() == 0
    want = O.run_plan(small, xs)
    got = c.cpu().numpy().view(np.uint16)
    for w in small.waves:
        a, b = w.y_off, w.y_off + w.cout * small.pitch
        ok, err, k = O.compare(got[a:b], want[a:b], RTOL, ATOL)
        assert ok, (w.name, err, k)
    npn.close()


def test_missing_peer_on_the_small_group_kernel_costs_one_wait_period(monkeypatch):
    """The mma.sync kernel's grid is not persistent: a rank's half of a group-16 wave of 65536 neurons x 2 column tiles is 4096 CTAs. With a
    peer that never shows up the CTAs resident first wait out the (shortened) bound together; every later CTA sees the status
    bit and neither waits nor touches the canvas. The launch therefore ends after about one wait period, not one per batch of
    resident CTAs, and writes nothing."""
    import time
    import torch
    monkeypatch.setenv("K44B_WAIT_MS", "200")
    plan = synth.sparse_plan(seed=131, input_rows=2048, waves=2, cout=65536, runs=4, run_len=16, columns=128, group=16, act=ACT_RELU)
    p0 = NativePlan.from_plan(shard.shard_plan(plan, 0, 2), device=0)
    p1 = NativePlan.from_plan(shard.shard_plan(plan, 1, 2), device=0)      # never executes
    assert p0.wave_info(1).path == 3
    cps, sps = [p0.canvas_ptr, p1.canvas_ptr], [p0.sync_ptr, p1.sync_ptr]
    p0.set_peers_raw(0, 2, cps, sps)
    p1.set_peers_raw(1, 2, cps, sps)
    x = synth.random_input(plan, 132)
    xt = torch.from_numpy(np.ascontiguousarray(x).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    p0.canvas_tensor()[plan.input_off: plan.input_off + xt.numel()] = xt
    p0.execute_wave(0)
    torch.cuda.synchronize()
    assert p0.status() == 0
    w1 = shard.shard_plan(plan, 0, 2).waves[1]
    before = p0.canvas_tensor()[w1.y_off: w1.y_off + w1.cout * plan.pitch].clone()
    t0 = time.perf_counter()
    p0.execute_wave(1)                    # 4096 CTAs on this rank; needs the peer's launch 0, which never comes
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    with pytest.raises(NativeError) as ei:
        p0.status()
    assert "peer" in str(ei.value).lower()
    assert dt < 1.5, f"launch with a missing peer took {dt:.2f} s: CTAs waited batch after batch"
    after = p0.canvas_tensor()[w1.y_off: w1.y_off + w1.cout * plan.pitch]
    assert torch.equal(before, after)     # a launch that gave up stores nothing
    p0.close(); p1.close()


def test_split_k_plan_is_clean_again_after_a_timeout(monkeypatch):
    """Split-K waves (partial sums in a global FP32 scratch, K44B_CLUSTER=0) on two ranks: rank 0 runs ahead, its second launch
    gives up on the missing peer, the status read puts scratch, arrival counters and the launch bookkeeping back to their
    between-launches state; then the peer catches up and the whole plan, run in order on both ranks, matches the oracle."""
    import torch
    monkeypatch.setenv("K44B_WAIT_MS", "200")
    monkeypatch.setenv("K44B_CLUSTER", "0")
    plan = synth.dense_chain(seed=133, dims=[1024, 512, 512], columns=64, act=ACT_SILU, weight_std=0.04)
    x = synth.random_input(plan, 134, dist="normal")
    want = O.run_plan(plan, x)
    plans = [NativePlan.from_plan(shard.shard_plan(plan, r, 2), device=0) for r in range(2)]
    assert plans[0].wave_info(0).k_splits > 1
    xt = torch.from_numpy(np.ascontiguousarray(x).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    for p in plans:
        p.canvas_tensor()[plan.input_off: plan.input_off + xt.numel()] = xt
    cps, sps = [p.canvas_ptr for p in plans], [p.sync_ptr for p in plans]
    for r, p in enumerate(plans):
        p.set_peers_raw(r, 2, cps, sps)
    plans[0].execute_wave(0)
    plans[0].execute_wave(1)              # waits for the peer's first launch: times out
    torch.cuda.synchronize()
    with pytest.raises(NativeError):
        plans[0].status()
    plans[1].execute_wave(0)              # the peer catches up: both ranks have now issued two launches
    plans[1].execute_wave(1)
    torch.cuda.synchronize()
    assert plans[1].status() == 0
    for i in range(len(plan.waves)):      # and the plan runs in order on both
        for p in plans:
            p.execute_wave(i)
    got = []
    for p in plans:
        assert p.status() == 0
        got.append(p.canvas_tensor().cpu().numpy().view(np.uint16))
    for r in range(2):
        for w in plan.waves:
            a, b = w.y_off, w.y_off + w.cout * plan.pitch
            ok, err, k = O.compare(got[r][a:b], want[a:b], RTOL, ATOL)
            assert ok, (r, w.name, err, k)
    for p in plans:
        p.close()
