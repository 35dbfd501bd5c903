"""Two-GPU checks of neuron sharding with the real kernels: each rank runs its rows of every wave on its own GPU;
the rows are either all-gathered in place over NCCL, or stored by the wave kernels straight into the peer's canvas
(CUDA IPC mappings, launch ordering by one counter word per peer). Skipped where fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import shard, synth
from snntome_b200.plan import ACT_RELU

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _plan(group=128):
    return synth.sparse_plan(seed=81, input_rows=2048, waves=3, cout=1024, runs=8, run_len=32, columns=128, group=group, act=ACT_RELU)


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from snntome_b200.native import NativePlan
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        plan = _plan()
        x = synth.random_input(plan, 82)
        mine = shard.shard_plan(plan, rank, world)
        npn = NativePlan.from_plan(mine, device=rank)
        canvas = npn.canvas_tensor()
        xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
        canvas[: xt.numel()] = xt
        runner = shard.NeuronShardedRunner(plan, rank, world, canvas, lambda i: npn.execute_wave(i))
        runner.run()
        assert npn.status() == 0
        np.save(os.path.join(out_dir, f"canvas{rank}.npy"), canvas.cpu().numpy().view(np.uint16))
        npn.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_neuron_sharding_matches_oracle(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    plan = _plan()
    want = O.run_plan(plan, synth.random_input(plan, 82))
    for r in range(2):
        got = np.load(tmp_path / f"canvas{r}.npy")
        for w in plan.waves:
            a, b = w.y_off, w.y_off + w.cout * plan.pitch
            ok, err, k = O.compare(got[a:b], want[a:b], 2e-3, 1e-3)
            assert ok, (r, w.name, err, k)
    assert np.array_equal(np.load(tmp_path / "canvas0.npy"), np.load(tmp_path / "canvas1.npy"))


def _worker_fused(rank, world, port, out_dir, group):
    import torch
    import torch.distributed as dist
    from snntome_b200.native import NativePlan
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        plan = _plan(group)
        x = synth.random_input(plan, 82)
        npn = NativePlan.from_plan(shard.shard_plan(plan, rank, world), device=rank)
        canvas = npn.canvas_tensor()
        xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
        canvas[: xt.numel()] = xt
        torch.cuda.synchronize()
        shard.connect_peers(npn, rank, world)
        for _ in range(3):                     # the same graph replayed: launch counts keep running across steps
            npn.execute_graph()
        torch.cuda.synchronize()
        st = npn.status()
        dist.barrier()                         # nobody frees its canvas while a peer may still store into it
        assert st == 0
        np.save(os.path.join(out_dir, f"fused{rank}.npy"), canvas.cpu().numpy().view(np.uint16))
        npn.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("group", [128, 32])
def test_two_gpu_peer_stores_match_oracle(tmp_path, group):
    """group 128: tcgen05 kernels; group 32: the mma.sync kernel — both store their rows into the peer's canvas themselves."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker_fused, args=(2, _free_port(), str(tmp_path), group), nprocs=2, join=True)
    plan = _plan(group)
    want = O.run_plan(plan, synth.random_input(plan, 82))
    for r in range(2):
        got = np.load(tmp_path / f"fused{r}.npy")
        for w in plan.waves:
            a, b = w.y_off, w.y_off + w.cout * plan.pitch
            ok, err, k = O.compare(got[a:b], want[a:b], 2e-3, 1e-3)
            assert ok, (r, w.name, err, k)
    assert np.array_equal(np.load(tmp_path / "fused0.npy"), np.load(tmp_path / "fused1.npy"))


def _worker_pruned(rank, world, port, out_dir, layers):
    import sys
    import torch
    import torch.distributed as dist
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path[:0] = [here, os.path.dirname(here)]
    os.environ["K44B_WAIT_MS"] = "500"               # if a rank stops, its peer's launches give up quickly instead of after 2 s each
    import bench
    import pruned_check
    from snntome_b200.native import fill_normal_f16
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        plan, info = bench.build_pruned_plan(layers, rank, rank, world)
        canvas = plan.canvas_tensor()
        fill_normal_f16(canvas[: info["cfg"]["hidden"] * info["pitch"]], 4242, 1.0)
        torch.cuda.synchronize()
        shard.connect_peers(plan, rank, world)
        picks = set(pruned_check.sampled_waves(plan.num_waves))
        worst = 0.0
        for wi in range(plan.num_waves):
            plan.execute_wave(wi)
            if wi in picks:                          # both ranks stop at the same waves
                st = plan.status_code()
                assert st == 0, f"rank {rank}: kernel status {st:#x} at wave {wi}"
                worst = max(worst, pruned_check.check_wave(plan, info, wi, canvas, seed=rank))
                dist.barrier()
        # then whole steps as one graph (grouped launches, region-ordered waits): every replica of the canvas must end up identical
        for _ in range(3):
            plan.execute_graph()
        torch.cuda.synchronize()
        st = plan.status_code()
        dist.barrier()
        assert st == 0, f"rank {rank}: kernel status {st:#x} after the graph steps"
        lo = info["rows"]["logits"] * info["pitch"]
        logits = canvas[lo: lo + info["vocab_rows"] * info["pitch"]]
        digest = torch.stack([logits.view(torch.int16).to(torch.int64).sum(), logits.float().abs().sum().to(torch.int64)])
        both = [torch.zeros_like(digest) for _ in range(world)]
        dist.all_gather(both, digest)
        assert all(torch.equal(b, both[0]) for b in both), f"replicas of the logits differ: {both}"
        assert bool(torch.isfinite(logits.float()).all())
        with open(os.path.join(out_dir, f"pruned{rank}.txt"), "w") as f:
            f.write(f"{worst}\n")
        dist.barrier()
        plan.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_pruned_8b_chain_sampled_groups_and_identical_replicas(tmp_path):
    """BASELINE configs[4], neuron-sharded over two GPUs with the wave kernels exchanging the rows themselves: sampled groups of
    sampled waves against the oracle on every rank (each rank checks rows it computed, from inputs that include rows its peer
    stored), then three steps as one CUDA graph with grouped launches, after which the logits of both replicas must be equal
    bit for bit."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    layers = int(os.environ.get("K44B_TEST_LAYERS", "32"))
    mp.spawn(_worker_pruned, args=(2, _free_port(), str(tmp_path), layers), nprocs=2, join=True)
    for r in range(2):
        assert float((tmp_path / f"pruned{r}.txt").read_text()) < 0.1
