#!/usr/bin/env python
"""Benchmark of the wave-executor hot path on the ultra-sparse plan.

Workload (synthetic, seeded; stands in for the benchmark text's "ultra-sparse large plan"): FP16 substrate
with 40,000,000 input rows of 64 columns, 4 waves x 1,048,576 neurons, fan-in 4096 = 64 runs of 64 consecutive
rows with uniform aligned starts over the input and earlier waves, groups of 128 neurons sharing their runs,
weights N(0, 1/4096), no bias, ReLU, 64 columns (batch) per GPU. One step = one pass of all 4 waves.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scale S]

Under torchrun each rank runs its own replica on its own 64 columns (weak scaling, no data-path
collective); time is the maximum over ranks, value the aggregate over all ranks.

Prints one JSON line: metric = effective synaptic TFLOP/s (2 * synapses * columns / s).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEED = 2024
NCU_TRAFFIC_RATIO = 0.928      # measured DRAM traffic / algorithmic bytes of k44_wave_umma_kernel<64> (see profiles/)
FULL = dict(input_rows=40_000_000, waves=4, cout=1 << 20, runs=64, run_len=64, columns=64, group=128)


def workload(scale: float) -> dict:
    """scale < 1 shrinks rows and neurons proportionally (development only; the default is the full plan)."""
    w = dict(FULL)
    if scale != 1.0:
        w["input_rows"] = max(65536, int(FULL["input_rows"] * scale) // 64 * 64)
        w["cout"] = max(1024, int(FULL["cout"] * scale) // 128 * 128)
    return w


def algorithmic_bytes_per_wave(w: dict) -> float:
    """Weights once + run table + every group's gathered rows once + output rows (no bias in this plan)."""
    fan_in = w["runs"] * w["run_len"]
    groups = w["cout"] // w["group"]
    return (w["cout"] * fan_in * 2 + groups * w["runs"] * 8 + groups * fan_in * w["columns"] * 2 + w["cout"] * w["columns"] * 2)


def flops_per_wave(w: dict) -> float:
    return 2.0 * w["cout"] * w["runs"] * w["run_len"] * w["columns"]


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def host_threads() -> int:
    """CPU threads this process may use. (torch.distributed.run exports OMP_NUM_THREADS=1 to its children; the CPU arm sets
    its own thread count from this instead.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return max(1, os.cpu_count() or 1)


def gpu_numa_cpus(device: int) -> list[int]:
    """CPUs of the NUMA node the GPU hangs off (from sysfs), restricted to the CPUs this process may use; empty if unknown."""
    try:
        import torch
        props = torch.cuda.get_device_properties(device)
        if hasattr(props, "pci_bus_id"):
            addr = f"{getattr(props, 'pci_domain_id', 0):04x}:{props.pci_bus_id:02x}:{getattr(props, 'pci_device_id', 0):02x}.0"
        else:       # older bindings: ask the driver tool (the index is the visible-device ordinal only without a device mask)
            out = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(device)],
                                 capture_output=True, text=True, timeout=10).stdout.strip().lower()
            addr = out[-12:]                            # "00000000:1b:00.0" -> "0000:1b:00.0"
        node = int(Path(f"/sys/bus/pci/devices/{addr}/numa_node").read_text().strip())
        if node < 0:
            return []
        cpus: list[int] = []
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            a, _, b = part.partition("-")
            cpus += list(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0)
        return [c for c in cpus if c in allowed]
    except Exception:
        return []


def pinned_near_gpu(n_elems: int, device: int):
    """Pinned FP16 host buffer whose pages are first touched by a thread running on the GPU's own NUMA node, so that with
    several ranks per host the uploads do not all cross the socket interconnect. Returns (tensor, node cpus used or None)."""
    import torch
    cpus = gpu_numa_cpus(device)
    before = None
    if cpus:
        try:
            before = os.sched_getaffinity(0)
            os.sched_setaffinity(0, cpus)
        except OSError:
            before = None
    try:
        t = torch.empty(n_elems, dtype=torch.float16).pin_memory()
        t.zero_()
    finally:
        if before is not None:
            os.sched_setaffinity(0, before)
    return t, (len(cpus) if before is not None else None)


def init_nccl(dist, local_rank: int) -> None:
    """NCCL process group with this rank's GPU. NCCL writes its version banner to stdout while the first communicator is set
    up; stdout carries one JSON line and nothing else, so file descriptor 1 points at stderr until a first collective is through."""
    import torch
    sys.stdout.flush()
    saved = os.dup(1)
    try:
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def run_starts_table(wave: int, w: dict) -> np.ndarray:
    from snntome_b200 import synth
    rows_avail = w["input_rows"] + wave * w["cout"]
    return synth.run_starts(SEED, wave, w["cout"] // w["group"], w["runs"], w["run_len"], rows_avail).astype(np.uint32)


def build_device_plan(w: dict, device: int):
    """Plan built in memory: weights are generated on the device wave by wave (row-major), packed by the
    library, and the row-major copy is dropped."""
    import torch
    from snntome_b200._lib import WaveDesc
    from snntome_b200.native import NativePlan, fill_normal_f16
    pitch = 64
    fan_in = w["runs"] * w["run_len"]
    total_rows = w["input_rows"] + w["waves"] * w["cout"]
    plan = NativePlan.create(total_rows * pitch, pitch, w["columns"], device=device)
    scratch = torch.empty((w["cout"], fan_in), dtype=torch.float16, device=f"cuda:{device}")
    for wi in range(w["waves"]):
        fill_normal_f16(scratch, SEED * 1000 + wi, (1.0 / fan_in) ** 0.5)
        torch.cuda.synchronize()
        starts = run_starts_table(wi, w)
        d = WaveDesc()
        d.cout = d.logical_cout = w["cout"]
        d.cin = w["input_rows"] + wi * w["cout"]
        d.group, d.fan_in, d.fan_in_raw, d.act, d.has_residual = w["group"], fan_in, fan_in, 1, 0
        d.y_off = (w["input_rows"] + wi * w["cout"]) * pitch
        d.run_rows, d.run_len = starts.ctypes.data, w["run_len"]
        d.weights, d.weights_on_device = scratch.data_ptr(), 1
        d.name = f"wave{wi}".encode()
        plan.add_wave_desc(d)
    del scratch
    torch.cuda.empty_cache()
    plan.set_io(0, w["input_rows"], (w["input_rows"] + (w["waves"] - 1) * w["cout"]) * pitch, w["cout"], w["columns"])
    return plan


def cpu_baseline(w: dict, seconds_target: float = 15.0, threads: int | None = None) -> dict:
    """The oracle (a port: the reference has no CPU implementation of this path) timed on this host on a bounded
    sample: whole 128-neuron groups of one wave with the full fan-in and 64 columns, gathering from a reduced
    substrate."""
    from oracle import oracle as O
    from snntome_b200 import synth
    from snntome_b200.plan import Plan, Wave, expand_runs
    L = O.lib()
    L.k44o_set_num_threads(threads or host_threads())
    cores = L.k44o_num_threads()
    fan_in = w["runs"] * w["run_len"]
    rows = 1 << 20                                   # 128 MiB substrate sample (far beyond the CPU caches)
    groups = max(1, min(64, int(2 * cores)))
    cout = groups * w["group"]
    rng = np.random.default_rng(SEED)
    starts = synth.run_starts(SEED, 0, groups, w["runs"], w["run_len"], rows)
    wave = Wave(cout=cout, group=w["group"], fan_in=fan_in, idx=expand_runs(starts, w["run_len"], 64),
                weights=synth.f16_bits(rng.normal(0, (1.0 / fan_in) ** 0.5, (cout, fan_in))), bias=None, y_off=rows * 64, act=1)
    plan = Plan(canvas_elems=(rows + cout) * 64, pitch=64, columns=64, input_off=0, input_c=rows, output_off=rows * 64,
                output_c=cout, waves=[wave])
    canvas = np.zeros(plan.canvas_elems, dtype=np.uint16)
    canvas[: rows * 64] = synth.f16_bits(rng.normal(0, 1, rows * 64).astype(np.float32))
    O.wave_forward(canvas, wave, plan, rows=(0, w["group"]))          # warm-up on one group
    t0 = time.perf_counter()
    reps = 0
    while True:
        O.wave_forward(canvas, wave, plan)
        reps += 1
        if time.perf_counter() - t0 > seconds_target / 2 or reps >= 400:
            break
    dt = (time.perf_counter() - t0) / reps
    flops = 2.0 * cout * fan_in * 64
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port", "seconds_per_rep": dt,
            "sample": f"{cout} neurons ({groups} groups of {w['group']}) of one wave, fan-in {fan_in}, 64 columns, "
                      f"substrate sample of {rows} rows; double accumulation, OpenMP over neurons"}



# ------------------------------------------------------------------------------------------------------------
# second workload: dense decoder compiled to waves (Llama-3.2-1B shapes), decode batch 64
# ------------------------------------------------------------------------------------------------------------
DECODER = dict(hidden=2048, layers=16, heads=32, kv_heads=8, head_dim=64, ffn=8192, vocab=128256, columns=64)


def build_decoder_plan(cfg: dict, device: int, seed: int = 7, full: bool = False, ctx: int = 512):
    """Every linear of the decoder is one wave whose neurons gather the full input width (one run). Weights
    N(0, 0.01^2) generated on the device. With full=False only the wave chain is built (`o` reads the q rows and
    `down` the gate rows as stand-ins of the same shape); with full=True the element-wise and attention commands
    sit between the waves as in the model: RMSNorm (scale 1, folded) before q/k/v and before the MLP, rotary
    embedding + attention of the new token against a key / value cache of `ctx` positions per sequence (filled
    with N(0,1), the new token written at the last position), SwiGLU product, final RMSNorm."""
    import torch
    from snntome_b200._lib import WaveDesc
    from snntome_b200.native import NativePlan, fill_normal_f16
    H, F, V = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    KV = cfg["kv_heads"] * cfg["head_dim"]
    pitch = 64
    rows = {}
    cur = 0
    names = [("x0", H), ("x1", H), ("q", H), ("k", KV), ("v", KV), ("h", H), ("g", F), ("u", F), ("logits", V)]
    if full:
        names += [("n", H), ("att", H), ("f", F)] + [(f"{c}cache{l}", KV * ctx) for l in range(cfg["layers"]) for c in "kv"]
    for name, n in names:
        rows[name] = cur
        cur += n
    plan = NativePlan.create(cur * pitch, pitch, cfg["columns"], device=device)
    scratch = torch.empty(max(V * H, F * H), dtype=torch.float16, device=f"cuda:{device}")
    params = 0
    counter = [0]

    def add(name, src, dst, cin, cout, act=0, res=None):
        nonlocal params
        wv = scratch[: cout * cin]
        fill_normal_f16(wv, seed * 100003 + counter[0], 0.01)
        counter[0] += 1
        torch.cuda.synchronize()
        groups = cout // 128
        starts = np.full((groups, 1), rows[src], dtype=np.uint32)
        d = WaveDesc()
        d.cout = d.logical_cout = cout
        d.cin, d.group, d.fan_in, d.fan_in_raw, d.act = cin, 128, cin, cin, act
        d.has_residual = 1 if res else 0
        d.y_off = rows[dst] * pitch
        d.src_off = rows[src] * pitch
        d.res_off = rows[res] * pitch if res else 0
        d.run_rows, d.run_len = starts.ctypes.data, cin
        d.weights, d.weights_on_device = wv.data_ptr(), 1
        d.name = name.encode()
        plan.add_wave_desc(d)
        params += cout * cin

    x_in, x_out = "x0", "x1"
    off = lambda name: rows[name] * pitch
    if full:        # token ids in: embedding rows gathered into the first activation tensor
        plan.embedding_table = torch.empty(V * H, dtype=torch.float16, device=f"cuda:{device}")
        fill_normal_f16(plan.embedding_table, seed * 17 + 3, 1.0)
        plan.add_embedding(plan.embedding_table.data_ptr(), V, H, off("x0"))
    for layer in range(cfg["layers"]):
        if full:
            plan.add_rmsnorm(off(x_in), off("n"), H, 1e-5, None, name=f"L{layer}.norm1")
        src = "n" if full else x_in
        add(f"L{layer}.q", src, "q", H, H)
        add(f"L{layer}.k", src, "k", H, KV)
        add(f"L{layer}.v", src, "v", H, KV)
        if full:
            plan.add_decode_attn(off("q"), off("k"), off("v"), off("att"), off(f"kcache{layer}"), off(f"vcache{layer}"), cfg["heads"],
                                 cfg["kv_heads"], cfg["head_dim"], ctx, 500000.0, True, name=f"L{layer}.attn")
        add(f"L{layer}.o", "att" if full else "q", "h", H, H, res=x_in)
        if full:
            plan.add_rmsnorm(off("h"), off("n"), H, 1e-5, None, name=f"L{layer}.norm2")
        src = "n" if full else "h"
        add(f"L{layer}.gate", src, "g", H, F, act=3)
        add(f"L{layer}.up", src, "u", H, F)
        if full:
            plan.add_swiglu(off("g"), off("u"), off("f"), F, name=f"L{layer}.swiglu")
        add(f"L{layer}.down", "f" if full else "g", x_out, F, H, res="h")
        x_in, x_out = x_out, x_in
    if full:
        plan.add_rmsnorm(off(x_in), off("n"), H, 1e-5, None, name="final_norm")
    add("lm_head", "n" if full else x_in, "logits", H, V)
    if full:
        plan.add_argmax(off("logits"), V)                 # greedy next token per sequence, read back by the host
        canvas = plan.canvas_tensor()
        c0 = off("kcache0")
        fill_normal_f16(canvas[c0: c0 + 2 * cfg["layers"] * KV * ctx * pitch], seed * 31 + 5, 1.0)
        plan.set_decode_pos(ctx - 1)
        torch.cuda.synchronize()
    del scratch
    torch.cuda.empty_cache()
    plan.set_io(0, H, rows["logits"] * pitch, V, cfg["columns"])
    return plan, params, rows


def reference_call_e2e(device: int, steps: int = 5, layers: int | None = None, tokens: int = 64) -> dict:
    """End to end through the reference's own execution call, `wavec_gpu_infer_f32` (wavec/k44_wave_executor.cu:972-986): a
    decoder of the 1B shape built with the reference's graph-builder calls the way its LLM example does (RMSNorm, q/k/v/o,
    rotary + causal grouped-query attention, gated MLP, residuals, final norm, lm_head), one sequence of 64 tokens, dense
    host FP32 [2048][1][64] in and [128256][1][64] out per call, blocking. The ultra-sparse plan itself cannot go through this
    call: its input tensor has 2.56e9 elements and the call's `int in_elems` stops at 2^31 - 1. Weights: one random FP16
    block per distinct shape, reused by every layer (the call's cost does not depend on the values)."""
    import torch
    from snntome_b200.wavec import WaveGraph
    cfg = dict(DECODER, layers=layers or DECODER["layers"])
    H, F, V, HQ, HKV, HD = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    rng = np.random.default_rng(31)
    blk = lambda o, i: (rng.standard_normal((o, i), dtype=np.float32) * 0.02).astype(np.float16)
    wq, wkv, wgu, wd, wlm = blk(H, H), blk(HKV * HD, H), blk(F, H), blk(H, F), blk(V, H)
    ones = np.ones(H, dtype=np.float32)
    t_build = time.perf_counter()
    g = WaveGraph(max_B_per_wave=F, default_S=64, fold_rmsnorm_gamma=True, reuse_canvas=True)
    g.add_input("x0", c=H, h=1, w=tokens, is_1d=True)
    x = "x0"
    for l in range(cfg["layers"]):
        g.add_rmsnorm(f"L{l}.n1", x, f"L{l}.a", H, ones, eps=1e-5)
        g.add_linear(f"L{l}.q", f"L{l}.a", f"L{l}.qv", H, H, wq, act="none")
        g.add_linear(f"L{l}.k", f"L{l}.a", f"L{l}.kv", H, HKV * HD, wkv, act="none")
        g.add_linear(f"L{l}.v", f"L{l}.a", f"L{l}.vv", H, HKV * HD, wkv, act="none")
        g.add_rope_gqa_attn(f"L{l}.att", f"L{l}.qv", f"L{l}.kv", f"L{l}.vv", f"L{l}.ao", HQ, HKV, HD, rope_theta=500000.0, llama3_scaling=True)
        g.add_linear(f"L{l}.o", f"L{l}.ao", f"L{l}.h", H, H, wq, act="none", res_blob=x)
        g.add_rmsnorm(f"L{l}.n2", f"L{l}.h", f"L{l}.b", H, ones, eps=1e-5)
        g.add_linear(f"L{l}.gate", f"L{l}.b", f"L{l}.g", H, F, wgu, act="silu")
        g.add_linear(f"L{l}.up", f"L{l}.b", f"L{l}.u", H, F, wgu, act="none")
        g.add_swiglu(f"L{l}.sw", f"L{l}.g", f"L{l}.u", f"L{l}.f", F)
        g.add_linear(f"L{l}.down", f"L{l}.f", f"L{l}.x", F, H, wd, act="none", res_blob=f"L{l}.h")
        x = f"L{l}.x"
    g.add_rmsnorm("final_norm", x, "xn", H, ones, eps=1e-5)
    g.add_linear("lm_head", "xn", "logits", H, V, wlm, act="none")
    g.set_output("logits")
    plan = g.compile()
    plan.init_gpu(device=device)
    build_s = time.perf_counter() - t_build
    xin = (rng.standard_normal((H, 1, tokens)) * 0.5).astype(np.float32)
    out, _ = plan.infer_f32(xin)                       # warm-up (also allocates the staging buffers)
    torch.cuda.synchronize()
    gpu_ms = []
    t0 = time.perf_counter()
    for _ in range(steps):
        out, ms = plan.infer_f32(xin)
        gpu_ms.append(ms)
    wall_ms = (time.perf_counter() - t0) * 1e3 / steps
    summ = plan.summary
    res = {"api": "wavec_gpu_infer_f32 (dense host FP32 in and out, blocking; graph built with wavec_add_* and wavec_compile)",
           "workload": f"1B-shape decoder, {cfg['layers']} layers + final norm + lm_head, one sequence of {tokens} tokens "
                       f"({summ.get('num_waves')} waves, {summ.get('num_cmds')} commands)",
           "value": tokens / (wall_ms * 1e-3), "unit": "tok/s", "ms_per_call": wall_ms, "gpu_ms_waves_only": float(np.mean(gpu_ms)),
           "steps": steps, "h2d_bytes_per_step": int(xin.nbytes), "d2h_bytes_per_step": int(out.nbytes),
           "build_and_upload_s": build_s, "finite": bool(np.isfinite(out).all()), "checksum": float(np.abs(out[:64]).sum())}
    plan.release_gpu()
    return res


def decode_main(args) -> None:
    import torch
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        init_nccl(dist, local_rank)
    cfg = dict(DECODER, layers=args.layers)
    full = args.workload == "decode-full"
    ctx = 512
    from snntome_b200.native import fill_normal_f16
    plan, params, rows = build_decoder_plan(cfg, local_rank, full=full, ctx=ctx)
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: cfg["hidden"] * 64], 99 + rank, 1.0)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    nw = plan.num_waves
    warmup = max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warmup):
        plan.execute_graph(stream)
    assert plan.status() == 0
    # weights (2.47 GB) exceed the 126 MB L2, so every step streams them from HBM again
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    l0 = plan.launch_count
    t0.record(stream)
    for _ in range(args.steps):
        plan.execute_graph(stream)
    t1.record(stream)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    launches = plan.launch_count - l0
    assert plan.status() == 0
    ms = t0.elapsed_time(t1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    # per-wave breakdown with direct launches (not part of the timed region)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(nw + 1)]
    for rep in range(2):
        ev[0].record(stream)
        for i in range(nw):
            plan.execute_wave(i, stream)
            ev[i + 1].record(stream)
    torch.cuda.synchronize()
    wave_us = [ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(nw)]
    # end to end through the public API: token ids host -> device, one graph replay, next token ids device -> host
    e2e = None
    if full:
        toks = np.random.default_rng(5).integers(0, cfg["vocab"], size=cfg["columns"]).astype(np.int32)
        e_steps = max(5, min(args.steps, 20))
        plan.set_tokens(toks, stream); plan.execute_graph(stream); toks = plan.next_tokens(cfg["columns"], stream)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e_steps):
            plan.set_tokens(toks, stream)
            plan.execute_graph(stream)
            toks = plan.next_tokens(cfg["columns"], stream)        # synchronises: the host holds the ids before the next step
        e1.record(stream)
        torch.cuda.synchronize()
        e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - w0) * 1e3)
        if dist is not None:
            t = torch.tensor([e_ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); e_ms = float(t.item())
        e2e = {"value": cfg["columns"] * world / (e_ms / e_steps * 1e-3), "unit": "tok/s", "ms_per_step": e_ms / e_steps, "steps": e_steps,
               "h2d_bytes_per_step": 4 * cfg["columns"], "d2h_bytes_per_step": 4 * cfg["columns"],
               "api": "k44b_plan_set_tokens + k44b_execute_graph + k44b_plan_get_next_tokens (greedy, one token per sequence and step)",
               "checksum": int(toks.astype(np.int64).sum())}
    clocks = sampler.stop()
    peak, kind = measured_peaks()
    kv_bytes = 2.0 * cfg["layers"] * cfg["kv_heads"] * cfg["head_dim"] * ctx * 64 * 2 if full else 0.0      # K and V of every layer, read once
    bytes_step = params * 2.0 + kv_bytes
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    infos = [plan.wave_info(i) for i in range(nw)]
    if rank == 0:
        line = {"metric": ("decode tok/s (1B dense decoder, whole layer stack with attention over a 512-position cache, batch 64 per GPU)" if full else
                           "decode tok/s (wave chain of a 1B dense decoder, batch 64 per GPU)"), "value": cfg["columns"] * world / (ms_step * 1e-3),
                "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                "config": {"workload": "dense decoder as waves: hidden 2048, 32/8 heads x 64, FFN 8192, vocab 128256, one wave per linear, "
                                       "64 columns per GPU; " + ("RMSNorm, rotary + attention against a key/value cache of 512 positions per sequence, SwiGLU product between the waves"
                                                                 if full else "wave chain only (no attention / norm / rope kernels)"),
                           "layers": cfg["layers"], "commands_per_step": nw, "params": params, "kv_cache_bytes_read_per_step": kv_bytes, "launch": "one CUDA graph per step",
                           "l2_policy": "2.47 GB of weights per step exceed the 126 MB L2; no explicit flush"},
                "roofline": {"bound": "hbm", "kernel": "whole step (k44_wave_umma_kernel<64> small-wave and streaming variants)", "achieved": achieved,
                             "peak": peak, "peak_kind": f"of {kind}", "unit": "GB/s", "frac": achieved / peak, "algorithmic_bytes_per_step": bytes_step,
                             "traffic": None},
                "per_wave_us_direct_launch": {"layer0": wave_us[:12 if full else 7], "lm_head": wave_us[-1], "sum": sum(wave_us)},
                "k_splits": {"layer0": [i.k_splits for i in infos[:12 if full else 7]], "lm_head": infos[-1].k_splits},
                "cpu_baseline": None, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------------
# third workload: cluster-pruned 8B decoder, neuron-sharded per wave with an all-gather of the wave's rows
# ------------------------------------------------------------------------------------------------------------
PRUNED = dict(hidden=4096, layers=32, kv=1024, ffn=14336, vocab=128256, columns=256, cluster=32, keep=0.10)


def build_pruned_plan(layers: int, rank: int, local_rank: int, world: int):
    """The cluster-pruned 8B wave chain, this rank's share: Llama-3-8B shaped linears (q, k, v, o, gate, up, down per layer,
    dense lm_head); every 128-neuron group keeps 10 % of its 32-row input clusters (uniform, seeded); rank r holds rows
    [r*cout/n, (r+1)*cout/n) of every wave and only their weights; the canvas is replicated. Returns (plan, info): info has
    the tensors' first rows (`rows`), per wave (output offset of the whole wave, its elements, this rank's block elements)
    in `waves`, per wave the run-start table of this rank's groups and the run length in `tables`, and the kept parameter
    count."""
    import torch
    from snntome_b200 import synth
    from snntome_b200._lib import WaveDesc
    from snntome_b200.native import NativePlan, fill_normal_f16
    cfg = dict(PRUNED, layers=layers)
    H, F, V, KV, C = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["kv"], cfg["columns"]
    V = -(-V // (world * 128)) * world * 128      # vocabulary rows padded to whole 128-neuron groups per rank (128256 -> 128512 at 4 and 8 ranks)
    pitch = C
    rows, cur = {}, 0
    for name, n in [("x0", H), ("x1", H), ("q", H), ("k", KV), ("v", KV), ("h", H), ("g", F), ("u", F), ("logits", V)]:
        rows[name] = cur; cur += n
    plan = NativePlan.create(cur * pitch, pitch, C, device=local_rank)
    waves = []       # (y_off, cout_total, block_elems)
    tables = []      # (run starts [groups, runs], run_len, first row of this rank's block, residual tensor's first row or None, act)
    kept_params = 0
    scratch = torch.empty(max(V // world * H, 1), dtype=torch.float16, device="cuda")

    def add(name, wi, src, dst, cin, cout, act=0, res=None, dense=False):
        nonlocal kept_params
        blk = cout // world
        assert cout % world == 0 and blk % 128 == 0, f"{name}: {cout} rows do not split into {world} blocks of whole 128-neuron groups"
        r0 = rank * blk
        groups = blk // 128
        if dense:
            fan_in, run_len = cin, cin
            starts = np.full((groups, 1), rows[src], dtype=np.uint32)
        else:
            clusters = cin // cfg["cluster"]
            keep = max(2, int(round(cfg["keep"] * clusters / 2)) * 2)
            fan_in, run_len = keep * cfg["cluster"], cfg["cluster"]
            ctr = (np.arange(groups * keep, dtype=np.uint64) + np.uint64((r0 // 128) * keep))
            starts = (rows[src] + synth.uniform_int(SEED + 5, wi, ctr, clusters).astype(np.int64) * cfg["cluster"]).astype(np.uint32).reshape(groups, keep)
            starts.sort(axis=1)
        wv = scratch[: blk * fan_in]
        fill_normal_f16(wv, SEED * 7919 + wi * 64 + rank, 0.01)
        torch.cuda.synchronize()
        d = WaveDesc()
        d.cout = d.logical_cout = blk
        d.cin, d.group, d.fan_in, d.fan_in_raw, d.act = cin, 128, fan_in, fan_in, act
        d.has_residual = 1 if res else 0
        d.y_off = (rows[dst] + r0) * pitch
        d.src_off = rows[src] * pitch
        d.res_off = (rows[res] + r0) * pitch if res else 0
        d.run_rows, d.run_len = starts.ctypes.data, run_len
        d.weights, d.weights_on_device = wv.data_ptr(), 1
        d.name = name.encode()
        plan.add_wave_desc(d)
        waves.append((rows[dst] * pitch, cout * pitch, blk * pitch))
        tables.append((starts, run_len, rows[dst] + r0, (rows[res] + r0) if res else None, act))
        kept_params += cout * fan_in

    x_in, x_out, wi = "x0", "x1", 0
    for layer in range(cfg["layers"]):
        for name, src, dst, cin, cout, act, res in [("q", x_in, "q", H, H, 0, None), ("k", x_in, "k", H, KV, 0, None), ("v", x_in, "v", H, KV, 0, None),
                                                    ("o", "q", "h", H, H, 0, x_in), ("gate", "h", "g", H, F, 3, None), ("up", "h", "u", H, F, 0, None),
                                                    ("down", "g", x_out, F, H, 0, "h")]:
            add(f"L{layer}.{name}", wi, src, dst, cin, cout, act, res); wi += 1
        x_in, x_out = x_out, x_in
    add("lm_head", wi, x_in, "logits", H, V, dense=True)
    del scratch
    torch.cuda.empty_cache()
    return plan, {"rows": rows, "waves": waves, "tables": tables, "kept_params": kept_params, "cfg": cfg, "vocab_rows": V, "pitch": pitch}


def sharded_measure(layers: int, steps: int, warmup: int, rank: int, local_rank: int, world: int, breakdown: bool = True) -> dict:
    """The cluster-pruned 8B wave chain (see build_pruned_plan), neuron-sharded: the rows of every wave reach all replicas of
    the canvas (see K44B_SHARD_MODE below). The default process group must already exist when world > 1. Every rank returns
    the same result line (a dict); a kernel status other than zero on any rank is reported in it as "error" instead of
    raised, so that all ranks keep taking the same path."""
    import torch
    import torch.distributed as dist
    from snntome_b200 import shard
    from snntome_b200.native import fill_normal_f16
    plan, info = build_pruned_plan(layers, rank, local_rank, world)
    rows, waves, kept_params, cfg, V, pitch = info["rows"], info["waves"], info["kept_params"], info["cfg"], info["vocab_rows"], info["pitch"]
    H, C = cfg["hidden"], cfg["columns"]
    canvas = plan.canvas_tensor()
    stream = torch.cuda.current_stream()
    nw = plan.num_waves
    mode = os.environ.get("K44B_SHARD_MODE", "peer")
    slack, signal = None, None
    if world > 1 and mode == "peer":
        slack = shard.connect_peers(plan, rank, world)
        # what one dependent launch costs at least: ranks 0 and 1 bounce a count word (alone, and behind a 16 KiB payload — one
        # 128 x 64 output block — stored into the peer's canvas and a system-scope fence), before the input is written
        try:
            if rank < 2:
                rt0 = plan.peer_latency(1 - rank, rank == 0, 2000, 0, stream)
                rt16 = plan.peer_latency(1 - rank, rank == 0, 2000, 16384, stream)
                signal = {"round_trip_us_word_only": rt0 / 1e3, "round_trip_us_16KiB_block_fence_word": rt16 / 1e3}
        except Exception as exc:
            signal = {"error": str(exc)}
        dist.barrier()
    fill_normal_f16(canvas[: H * pitch], 4242, 1.0)       # same input on every rank (replicated canvas)
    torch.cuda.synchronize()

    def eager_step():
        st = torch.cuda.current_stream()
        for i in range(nw):
            plan.execute_wave(i, st)
            y_off, total, blk = waves[i]
            if world > 1 and blk != total:
                out = canvas[y_off: y_off + total]
                dist.all_gather_into_tensor(out, out[rank * blk: (rank + 1) * blk])

    # How the ranks exchange rows (K44B_SHARD_MODE):
    #   peer  (default) the wave kernels store their rows into every canvas themselves (peer-mapped memory) and order
    #         their launches against the peers' through counter words; a step is one CUDA graph, no collective call;
    #   nccl  one in-place all-gather per wave after its launch (the plain baseline); nccl-graph: the same, captured.
    graph = None
    if world > 1 and mode == "nccl-graph":
        eager_step()                      # NCCL communicator set-up and lazy initialisation happen outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            eager_step()

    def step():
        if graph is not None:
            graph.replay()
        elif world == 1 or mode == "peer":
            plan.execute_graph(stream)
        else:
            eager_step()

    def all_status() -> int:              # the kernels' status word, worst over the ranks (every rank calls this at the same points)
        st = plan.status_code()
        if world > 1:
            t = torch.tensor([st], device="cuda", dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            st = int(t.item())
        return st

    warmup = max(3, warmup)
    sampler = ClockSampler(local_rank); sampler.start()
    for _ in range(warmup):
        step()
    status = all_status()
    ms_step, launches = float("nan"), 0
    if status == 0:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        l0 = plan.launch_count
        t0.record(stream)
        for _ in range(steps):
            step()
        t1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        status = all_status()
        launches = plan.launch_count - l0
        ms = t0.elapsed_time(t1)
        if world > 1:
            t = torch.tensor([ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
        ms_step = ms / steps
    clocks = sampler.stop()
    checksum = float(canvas[rows["logits"] * pitch: rows["logits"] * pitch + 4096].float().abs().sum().item())
    # per-wave breakdown with one launch per wave (outside the timed region; with peers it includes waiting for them)
    wave_us = None
    if breakdown and status == 0 and (world == 1 or mode == "peer"):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(nw + 1)]
        for _ in range(2):
            if world > 1:
                dist.barrier()
            ev[0].record(stream)
            for i in range(nw):
                plan.execute_wave(i, stream)
                ev[i + 1].record(stream)
            torch.cuda.synchronize()
        us = [ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(nw)]
        wave_us = {"layer0": [round(v, 1) for v in us[:7]], "lm_head": round(us[-1], 1), "sum": round(sum(us), 1)}
        status = all_status()
    gather_bytes = sum(total * 2 * (world - 1) // world for (_, total, blk) in waves if blk != total)
    peak, kind = measured_peaks()
    line = {"metric": "decode tok/s (cluster-pruned 8B wave chain, neuron-sharded, batch 256)", "value": C / (ms_step * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
            "config": {"workload": "Llama-3-8B shaped wave chain, 90 % of 32-row input clusters removed per 128-neuron group, dense lm_head, "
                                   "batch 256; rows of every wave split over the ranks, canvas replicated",
                       "layers": cfg["layers"], "waves_per_step": nw, "kept_params": kept_params, "lm_head_rows": V,
                       "exchange": ("none (one GPU)" if world == 1 else {"peer": "direct stores into the peers' canvases from the wave kernels, counter-word launch ordering, one CUDA graph per step",
                                                                    "nccl": "in-place NCCL all-gather after every wave", "nccl-graph": "in-place NCCL all-gather after every wave, captured in one CUDA graph"}[mode]),
                       "exchange_mode": "none" if world == 1 else mode,
                       "bytes_received_per_rank_per_step": gather_bytes,
                       "nvlink_time_bound_ms": gather_bytes / 770e9 * 1e3,
                       "launches_per_step": int(launches // max(steps, 1)) if launches else None,
                       "launches_that_wait_for_the_launch_before": int((slack == 0).sum()) if slack is not None else None,
                       "signal": signal},
            "roofline": {"bound": "hbm", "kernel": "whole step", "achieved": kept_params * 2.0 / world / (ms_step * 1e-3) / 1e9, "peak": peak,
                         "peak_kind": f"of {kind}", "unit": "GB/s", "frac": kept_params * 2.0 / world / (ms_step * 1e-3) / 1e9 / peak, "traffic": None},
            "per_wave_us_direct_launch": wave_us,
            "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches), "checksum": checksum, "clocks": clocks}
    if status != 0:
        line["error"] = f"kernel status {status:#x} on at least one rank"
    if world > 1:
        dist.barrier()                  # no rank frees its canvas while a peer may still store into it
        graph = None
        torch.cuda.synchronize()
    plan.close()
    return line


def sharded_main(args) -> None:
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0")); local_rank = int(os.environ.get("LOCAL_RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        init_nccl(dist, local_rank)
    line = sharded_measure(args.layers if args.layers != 16 else PRUNED["layers"], args.steps, args.warmup, rank, local_rank, world)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------------
# fourth workload: receptive-field token shift (tensor-pipe bound)
# ------------------------------------------------------------------------------------------------------------
SHIFT = dict(sequences=8, tokens=4096, input_channels=2048, waves=4, cout=8192, runs=32, run_len=16, group=128, max_shift=7)


def build_shift_plan(c: dict, device: int):
    """Token-shift plan built in memory (weights generated on the device); returns the plan and, per wave, the run
    starts [groups, runs] and shifts [groups, runs] it was built from."""
    import torch
    from snntome_b200 import synth
    from snntome_b200._lib import WaveDesc
    from snntome_b200.native import NativePlan, fill_normal_f16
    pitch = c["sequences"] * c["tokens"]
    fan_in = c["runs"] * c["run_len"]
    total_rows = c["input_channels"] + c["waves"] * c["cout"]
    plan = NativePlan.create(total_rows * pitch, pitch, pitch, device=device)
    scratch = torch.empty((c["cout"], fan_in), dtype=torch.float16, device=f"cuda:{device}")
    tables = []
    for wi in range(c["waves"]):
        fill_normal_f16(scratch, SEED * 1000 + 500 + wi, (1.0 / fan_in) ** 0.5)
        torch.cuda.synchronize()
        groups = c["cout"] // c["group"]
        avail = c["input_channels"] + wi * c["cout"]
        starts = synth.run_starts(SEED + 1, wi, groups, c["runs"], c["run_len"], avail).astype(np.uint32)
        shifts = synth.uniform_int(SEED + 2, 2000 + wi, np.arange(groups * c["runs"], dtype=np.uint64), c["max_shift"] + 1).astype(np.uint8)
        shifts = np.ascontiguousarray(shifts.reshape(groups, c["runs"]))
        tables.append((starts, shifts))
        d = WaveDesc()
        d.cout = d.logical_cout = c["cout"]
        d.cin = avail
        d.group, d.fan_in, d.fan_in_raw, d.act, d.has_residual = c["group"], fan_in, fan_in, int(c.get("act", 5)), 0
        d.y_off = avail * pitch
        d.run_rows, d.run_len = starts.ctypes.data, c["run_len"]
        d.shifts, d.frame_len = shifts.ctypes.data, c["tokens"]
        d.weights, d.weights_on_device = scratch.data_ptr(), 1
        d.name = f"shift{wi}".encode()
        plan.add_wave_desc(d)
    del scratch
    plan.set_io(0, c["input_channels"], (total_rows - c["cout"]) * pitch, c["cout"], pitch)
    return plan, tables


def shift_main(args) -> None:
    """8 sequences x 4096 tokens as one row of 32768 columns per channel; 4 waves x 8192 neurons, fan-in 512 = 32 runs of
    16 channels, every run read 0..7 tokens earlier with zero padding at the start of each sequence; GELU."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        init_nccl(dist, local_rank)
    from snntome_b200.native import fill_normal_f16
    c = dict(SHIFT)
    c["max_shift"] = max(0, min(8, args.max_shift))
    c["act"] = args.shift_act
    if args.scale != 1.0:
        c["sequences"] = max(1, int(round(c["sequences"] * args.scale)))
    plan, _tables = build_shift_plan(c, local_rank)
    pitch = c["sequences"] * c["tokens"]
    fan_in = c["runs"] * c["run_len"]
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: c["input_channels"] * pitch], SEED + 177 + rank, 1.0)
    torch.cuda.synchronize()
    nw = plan.num_waves
    infos = [plan.wave_info(i) for i in range(nw)]
    stream = torch.cuda.current_stream()
    warmup = max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warmup):
        plan.execute(stream)
    assert plan.status() == 0
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(nw + 1)] for _ in range(args.steps)]
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    l0 = plan.launch_count
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for s_ in range(args.steps):
        ev[s_][0].record(stream)
        for i in range(nw):
            plan.execute_wave(i, stream)
            ev[s_][i + 1].record(stream)
    t1.record(stream)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    launches = plan.launch_count - l0
    assert plan.status() == 0
    ms = t0.elapsed_time(t1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    clocks = sampler.stop()
    per_wave = [float(np.mean([ev[s_][i].elapsed_time(ev[s_][i + 1]) for s_ in range(args.steps)])) for i in range(nw)]
    flops_wave = 2.0 * c["cout"] * fan_in * pitch
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    kind = "measured (sustained dense bf16)" if peaks else "fallback"
    achieved = flops_wave / (float(np.mean(per_wave)) * 1e-3) / 1e12
    if rank == 0:
        line = {"metric": "effective synaptic TFLOP/s (2*synapses*columns/s)", "value": flops_wave * nw * world / (ms_step * 1e-3) / 1e12,
                "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                "config": {"workload": "token-shift receptive fields: sequences x 4096 tokens per GPU, 2048 input channels, 4 waves x 8192 neurons, "
                                       "fan-in 512 = 32 runs of 16 channels, shift 0..7 tokens per run, groups of 128, " + {0: "no activation", 1: "ReLU", 2: "sigmoid", 3: "SiLU", 4: "leaky ReLU", 5: "GELU"}.get(c["act"], "?"),
                           "sequences_per_gpu": c["sequences"], "columns_per_gpu": pitch, "scale": args.scale, "max_shift": c["max_shift"],
                           "l2_policy": "substrate (0.13 - 2.3 GB) exceeds the 126 MB L2; no explicit flush"},
                "roofline": {"bound": "tensor", "kernel": (("k44_wave_umma_shift_ws_kernel" if infos[0].weights_in_tmem else f"k44_wave_umma_shift_kernel<{infos[0].n_tile}>") if c["max_shift"] else f"k44_wave_umma_kernel<{infos[0].n_tile}>") if infos[0].path == 1 else ("k44_wave_mma_kernel" if infos[0].path == 3 else "k44_wave_fma_kernel"),
                             "achieved": achieved, "peak": peak, "peak_kind": f"of {kind}", "unit": "TFLOP/s", "frac": achieved / peak,
                             "flops_per_launch": flops_wave, "per_wave_ms": per_wave, "traffic": None},
                "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches), "kernel_paths": [i.path for i in infos], "clocks": clocks}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------------
# fifth workload: the reference benchmark's own regime (large neuron groups, 512 columns, tensor-bound)
# ------------------------------------------------------------------------------------------------------------
# (group, fan-in, neurons per wave, columns) of the two rows the reference's benchmark calls its fastest
# (whitepaper/sparse_wmma_kernel/tests/benchmark_whitepaper_k44.cpp:191-197); one pass = 16 independent waves over one
# substrate, cycling through 256 MiB of weights (benchmark_common.cuh:401-442).
WHITEPAPER_ROWS = {"g512_b2048_c4096": dict(group=512, fan_in=2048, cout=4096, columns=512),
                   "g256_b1024_c8192": dict(group=256, fan_in=1024, cout=8192, columns=512)}
WHITEPAPER_WAVES = 16


def build_whitepaper_plan(row: dict, cin: int, device: int, gen: str, merged: bool):
    """One pass of the reference benchmark as a plan: `WHITEPAPER_WAVES` waves that all gather from the same `cin` substrate
    rows and write their own output rows. merged: the 16 waves become one wave of 16 x cout neurons (same arithmetic: the
    waves are independent and share the substrate), so that one launch fills the GPU. gen "rows": the reference's generator —
    every group draws fan_in single rows uniformly and sorts them; gen "runs": runs of 64 consecutive rows instead.
    Returns (plan, tables): tables[i] = (rows [groups, entries], run_len, first output row, neurons)."""
    import torch
    from snntome_b200 import synth
    from snntome_b200._lib import WaveDesc
    from snntome_b200.native import NativePlan, fill_normal_f16
    pitch, B, G = row["columns"], row["fan_in"], row["group"]
    n_waves = 1 if merged else WHITEPAPER_WAVES
    cout = row["cout"] * (WHITEPAPER_WAVES if merged else 1)
    plan = NativePlan.create((cin + n_waves * cout) * pitch, pitch, pitch, device=device)
    scratch = torch.empty((cout, B), dtype=torch.float16, device=f"cuda:{device}")
    tables = []
    for wi in range(n_waves):
        fill_normal_f16(scratch, SEED * 31 + wi, (1.0 / B) ** 0.5)
        torch.cuda.synchronize()
        groups = cout // G
        if gen == "rows":
            rows = synth.uniform_int(SEED + 9, 5000 + wi, np.arange(groups * B, dtype=np.uint64), cin).astype(np.uint32).reshape(groups, B)
            rows.sort(axis=1)
            run_len = 1
        else:
            rows = synth.run_starts(SEED + 9, 5000 + wi, groups, B // 64, 64, cin).astype(np.uint32)
            run_len = 64
        rows = np.ascontiguousarray(rows)
        d = WaveDesc()
        d.cout = d.logical_cout = cout
        d.cin, d.group, d.fan_in, d.fan_in_raw, d.act, d.has_residual = cin, G, B, B, 0, 0
        d.y_off = (cin + wi * cout) * pitch
        d.run_rows, d.run_len = rows.ctypes.data, run_len
        d.weights, d.weights_on_device = scratch.data_ptr(), 1
        d.name = f"pass_wave{wi}".encode()
        plan.add_wave_desc(d)
        tables.append((rows, run_len, cin + wi * cout, cout))
    del scratch
    torch.cuda.empty_cache()
    plan.set_io(0, 1, cin * pitch, 1, pitch)
    return plan, tables


def whitepaper_main(args) -> None:
    """The reference's own Blackwell regime: neurons in groups of 512 / 256 sharing their gather list, 512 columns, substrate of
    80 M rows (82 GB), one pass = 16 waves. Tensor-bound. Reported against the measured sustained dense rate; the reference's
    published figure for its sm_100a kernel (522.4 TSyn/s HBM-streaming at 80 M substrate rows, shape unstated) is context."""
    import torch
    from snntome_b200.native import fill_normal_f16
    rank = int(os.environ.get("RANK", "0")); local_rank = int(os.environ.get("LOCAL_RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        init_nccl(dist, local_rank)
    row = WHITEPAPER_ROWS[args.wp_row]
    cin = max(1 << 16, int(80_000_000 * args.scale))
    plan, _ = build_whitepaper_plan(row, cin, local_rank, args.wp_gen, not args.wp_unmerged)
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: cin * row["columns"]], SEED + 300 + rank, 1.0)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    nw = plan.num_waves
    info = plan.wave_info(0)
    warmup = max(3, args.warmup)
    sampler = ClockSampler(local_rank); sampler.start()
    for _ in range(warmup):
        plan.execute(stream)
    assert plan.status() == 0
    # a pass takes a fraction of a millisecond: time blocks of 100 passes, about two seconds in all, so that the clock
    # sampler sees the GPU under load more than once
    inner = 100
    blocks = max(args.steps, 10) * 10
    steps = blocks * inner
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    l0 = plan.launch_count
    ev[0].record(stream)
    for i in range(blocks):
        for _ in range(inner):
            plan.execute(stream)
        ev[i + 1].record(stream)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    launches = plan.launch_count - l0
    assert plan.status() == 0
    ms = ev[0].elapsed_time(ev[blocks])
    if dist is not None:
        t = torch.tensor([ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
    ms_step = ms / steps
    per_pass = [ev[i].elapsed_time(ev[i + 1]) / inner for i in range(blocks)]
    clocks = sampler.stop()
    syn = float(row["cout"]) * WHITEPAPER_WAVES * row["fan_in"] * row["columns"]
    flops = 2.0 * syn
    groups = row["cout"] * WHITEPAPER_WAVES // row["group"]
    bytes_alg = (row["cout"] * WHITEPAPER_WAVES * row["fan_in"] * 2 + groups * row["fan_in"] * 4 + groups * row["fan_in"] * row["columns"] * 2
                 + row["cout"] * WHITEPAPER_WAVES * row["columns"] * 2)
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    achieved = flops / (ms_step * 1e-3) / 1e12
    if rank == 0:
        line = {"metric": "effective synaptic TFLOP/s (2*synapses*columns/s)", "value": achieved * world, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                "tsyn_per_s": syn * world / (ms_step * 1e-3) / 1e12,
                # the run is long enough for the power cap to pull the clocks down; the fastest block of 100 passes shows the rate before that
                "burst": {"tflops": flops / (float(np.min(per_pass)) * 1e-3) / 1e12, "tsyn_per_s": syn / (float(np.min(per_pass)) * 1e-3) / 1e12,
                          "what": "fastest block of 100 consecutive passes"},
                "config": {"workload": f"reference benchmark regime: groups of {row['group']} neurons, fan-in {row['fan_in']}, {row['cout']} neurons per wave, "
                                       f"{row['columns']} columns, {cin} substrate rows, one pass = {WHITEPAPER_WAVES} waves"
                                       + (" launched as one wave of 16 x the neurons" if not args.wp_unmerged else " launched one by one"),
                           "gather_table": "one sorted uniform random row per synapse (the reference's generator)" if args.wp_gen == "rows" else "runs of 64 consecutive rows",
                           "substrate_bytes": cin * row["columns"] * 2, "scale": args.scale,
                           "l2_policy": "weights (268 MB per pass) and gathered rows (268 MB per pass out of the substrate) exceed the 126 MB L2; no explicit flush",
                           "reference_published": "522.4 TSyn/s HBM-streaming at 80 M substrate rows, 612.7 in-cache, on B200 with the reference's own tcgen05 kernel; shape not stated (whitepaper main.pdf p.14)"},
                "roofline": {"bound": "tensor", "kernel": f"k44_wave_umma_kernel<{info.n_tile}>" if info.path == 1 else ("k44_wave_mma_kernel" if info.path == 3 else "k44_wave_fma_kernel"),
                             "achieved": achieved, "peak": peak, "peak_kind": "of measured (sustained dense bf16)" if peaks else "of fallback", "unit": "TFLOP/s",
                             "frac": achieved / peak, "flops_per_launch": flops / nw, "per_pass_ms_min_median": [float(np.min(per_pass)), float(np.median(per_pass))],
                             "hbm_algorithmic_bytes_per_pass": bytes_alg, "hbm_gbs_algorithmic": bytes_alg / (ms_step * 1e-3) / 1e9,
                             "hbm_frac_of_measured_copy_rate": bytes_alg / (ms_step * 1e-3) / 1e9 / hbm, "traffic": None},
                "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches), "kernel_paths": [plan.wave_info(i).path for i in range(nw)],
                "rows_per_box": info.box_rows, "clocks": clocks}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def tiny_main(args) -> None:
    """The tiny correctness plan (2 waves x 1024 neurons, fan-in 256 as 16 runs of 16 rows, 32 columns): launch-latency
    bound, reported as microseconds per wave of a replayed CUDA graph."""
    import torch
    from snntome_b200 import synth
    from snntome_b200.native import NativePlan
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    plan = synth.config0(group=128)
    npn = NativePlan.from_plan(plan, device=torch.cuda.current_device())
    x = synth.random_input(plan, 11)
    canvas = npn.canvas_tensor()
    canvas[plan.input_off: plan.input_off + x.size] = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    stream = torch.cuda.current_stream()
    reps = max(200, args.steps)
    for _ in range(20):
        npn.execute_graph(stream)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record(stream)
    for _ in range(reps):
        npn.execute_graph(stream)
    t1.record(stream)
    torch.cuda.synchronize()
    assert npn.status() == 0
    us_step = t0.elapsed_time(t1) * 1e3 / reps
    nw = npn.num_waves
    print(json.dumps({"metric": "microseconds per wave (tiny correctness plan, CUDA graph replay)", "value": us_step / nw, "unit": "us/wave",
                      "n_gpus": 1, "steps": reps, "warmup": 20, "ms_per_step": us_step / 1e3, "higher_is_better": False, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                      "config": {"workload": "tiny plan: 4096 input rows, 2 waves x 1024 neurons, fan-in 256 = 16 runs of 16 rows, groups of 128, ReLU, 32 columns",
                                 "l2_policy": "0.7 MB per wave: L2-resident, launch-latency bound by construction"},
                      "kernel_paths": [npn.wave_info(i).path for i in range(nw)], "k_splits": [npn.wave_info(i).k_splits for i in range(nw)],
                      "roofline": None, "cpu_baseline": None, "e2e": None, "gpu_launches": int(npn.launch_count)}))


def build_image_graph(size: int = 640, width: float = 1.0, seed: int = 7, frames: int = 1):
    """A detector backbone + two neck stages in the style of the reference's image example (wavec/examples/example_yolov8.py):
    3 x size x size input; 3x3 / stride-2 convolutions down to size / 32; C2f blocks (1x1, slice, n bottlenecks of two 3x3 with a
    shortcut, concat, 1x1) of 32 / 64 / 128 / 256 channels; SPPF; nearest upsampling + concat + C2f back up to size / 8. SiLU
    everywhere, random weights N(0, 1 / fan-in). Built with the reference's graph-builder calls."""
    from snntome_b200.wavec import WaveGraph
    rng = np.random.default_rng(seed)
    ch = lambda c: max(16, int(round(c * width / 16)) * 16)

    def wt(cout, cin, k):
        return (rng.standard_normal((cout, cin, k, k)) * (1.0 / (cin * k * k)) ** 0.5).astype(np.float32), (rng.standard_normal(cout) * 0.02).astype(np.float32)

    g = WaveGraph(max_B_per_wave=288, reuse_canvas=False, batch_size=frames)    # every tensor its own zero-initialised region: no halo clears between the waves
    g.add_input("images", c=3, h=size, w=size, is_1d=False)
    uid = [0]

    def conv(x, cin, cout, k, stride=1, act="silu", res=None):
        uid[0] += 1
        y = f"t{uid[0]}"
        w, b = wt(cout, cin, k)
        g.add_conv2d(f"conv{uid[0]}", x, y, cin, cout, k, k, w, b, stride=stride, pad=k // 2, act=act, res_blob=res)
        return y

    def c2f(x, cin, cout, n, shortcut):
        c = cout // 2
        y = conv(x, cin, 2 * c, 1)
        uid[0] += 1
        a, b = f"t{uid[0]}a", f"t{uid[0]}b"
        g.add_slice(f"split{uid[0]}", y, [a, b], [c, c])
        parts, last = [a, b], b
        for _ in range(n):
            h = conv(last, c, c, 3)
            last = conv(h, c, c, 3, res=last if shortcut else None)
            parts.append(last)
        uid[0] += 1
        cat = f"t{uid[0]}"
        g.add_concat(f"cat{uid[0]}", parts, cat)
        return conv(cat, (2 + n) * c, cout, 1)

    def sppf(x, c):
        y = conv(x, c, c // 2, 1)
        pools, last = [y], y
        for i in range(3):
            uid[0] += 1
            p = f"t{uid[0]}"
            g.add_maxpool(f"pool{uid[0]}", last, p, kernel_size=5, stride=1, pad=2)
            pools.append(p); last = p
        uid[0] += 1
        cat = f"t{uid[0]}"
        g.add_concat(f"cat{uid[0]}", pools, cat)
        return conv(cat, 2 * c, c, 1)

    def up_cat(x, skip):
        uid[0] += 1
        u, cat = f"t{uid[0]}u", f"t{uid[0]}c"
        g.add_upsample2x(f"up{uid[0]}", x, u)
        g.add_concat(f"cat{uid[0]}", [u, skip], cat)
        return cat

    c1, c2, c3, c4, c5 = ch(16), ch(32), ch(64), ch(128), ch(256)
    x = conv("images", 3, c1, 3, stride=2)                 # size / 2
    x = conv(x, c1, c2, 3, stride=2)                       # size / 4
    x = c2f(x, c2, c2, 1, True)
    x = conv(x, c2, c3, 3, stride=2)                       # size / 8
    p3 = c2f(x, c3, c3, 2, True)
    x = conv(p3, c3, c4, 3, stride=2)                      # size / 16
    p4 = c2f(x, c4, c4, 2, True)
    x = conv(p4, c4, c5, 3, stride=2)                      # size / 32
    x = c2f(x, c5, c5, 1, True)
    p5 = sppf(x, c5)
    x = c2f(up_cat(p5, p4), c5 + c4, c4, 1, False)         # size / 16
    out = c2f(up_cat(x, p3), c4 + c3, c3, 1, False)        # size / 8
    g.set_output(out)
    return g, rng


def image_main(args) -> None:
    """The 2-D image path: one detector-style network per inference through the reference-facing builder API. `value` times the
    compiled plan replayed as one CUDA graph with the image resident in the canvas; `e2e` is `wavec_gpu_infer_f32` with a dense
    host FP32 image in and the feature map out."""
    import torch
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    size = max(128, int(round(640 * args.scale / 128)) * 128)      # every stride-2 convolution needs an input width that is a multiple of 8
    t_build = time.perf_counter()
    frames = max(1, args.frames)
    g, rng = build_image_graph(size, frames=frames)
    plan = g.compile()
    plan.init_gpu(device=local_rank)
    build_s = time.perf_counter() - t_build
    summ = plan.summary
    x = rng.standard_normal((frames, 3, size, size) if frames > 1 else (3, size, size)).astype(np.float32)
    out, _ = plan.infer_f32(x)                               # fills the canvas with a real image, warms everything up
    assert np.isfinite(out).all()
    npn = plan.native
    stream = torch.cuda.current_stream()
    steps = args.steps if args.steps else 200
    warmup = max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warmup):
        npn.execute_graph(stream)
    torch.cuda.synchronize()
    l0 = npn.launch_count
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(steps):
        npn.execute_graph(stream)
    t1.record(stream)
    torch.cuda.synchronize()
    assert npn.status() == 0
    ms_step = t0.elapsed_time(t1) / steps
    launches = npn.launch_count - l0
    clocks = sampler.stop()
    e_steps = max(5, min(steps, 50))
    t_e = time.perf_counter()
    for _ in range(e_steps):
        out, _ = plan.infer_f32(x)
    e_ms = (time.perf_counter() - t_e) * 1e3 / e_steps
    gflop = float(summ.get("total_gflops", 0.0))
    kinds = {}
    for c in summ.get("cmds", []):
        kinds[c["type"]] = kinds.get(c["type"], 0) + 1
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops", 1590.0))
    achieved = gflop / ms_step            # GFLOP / ms = TFLOP/s
    print(json.dumps({"metric": f"images/s (detector backbone + neck, {frames} image{'s' if frames > 1 else ''} per inference)", "value": frames * 1e3 / ms_step, "unit": "images/s", "n_gpus": 1,
                      "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                      "config": {"workload": f"3 x {size} x {size} image; stride-2 3x3 convolutions to 1/32, C2f blocks of 32 / 64 / 128 / 256 channels, SPPF, two upsample + concat + C2f "
                                             f"stages; SiLU; built with wavec_add_conv2d / _maxpool / _upsample2x / _slice / _concat", "image_size": size, "frames_per_inference": frames,
                                 "commands": kinds, "gflop_per_image": gflop, "canvas_bytes": int(summ.get("canvas_bytes", 0)),
                                 "l2_policy": "the whole canvas fits L2 at one frame: launch- and latency-bound by construction"},
                      "roofline": {"bound": "tensor", "kernel": "k44_wave_mma_kernel (image tiles)", "achieved": achieved, "peak": peak,
                                   "peak_kind": "of measured (burst dense bf16)" if peaks else "of fallback", "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None},
                      "cpu_baseline": None,
                      "e2e": {"value": frames * 1e3 / e_ms, "unit": "images/s", "ms_per_step": e_ms, "steps": e_steps, "h2d_bytes_per_step": int(x.nbytes), "d2h_bytes_per_step": int(out.nbytes),
                              "api": "wavec_gpu_infer_f32 (dense host FP32 image in, feature map out, blocking)"},
                      "gpu_launches": int(launches), "build_and_upload_s": build_s, "clocks": clocks}))
    plan.release_gpu()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default: 10; 2000 / 1000 / 500 for the decode, decode-full and token-shift workloads, whose steps are 1 - 2 ms, so that the clock sampler sees the timed region)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scale", type=float, default=float(os.environ.get("K44B_BENCH_SCALE", "1.0")))
    ap.add_argument("--workload", default="ultra-sparse", choices=["ultra-sparse", "decode", "decode-full", "pruned-sharded", "token-shift", "tiny", "whitepaper", "image"])
    ap.add_argument("--wp-row", default="g512_b2048_c4096", choices=sorted(WHITEPAPER_ROWS), help="whitepaper workload: which of the reference benchmark's rows")
    ap.add_argument("--wp-gen", default="rows", choices=["rows", "runs"], help="whitepaper workload: single sorted random rows (the reference's generator) or runs of 64 rows")
    ap.add_argument("--wp-unmerged", action="store_true", help="whitepaper workload: launch the 16 waves of a pass one by one instead of as one wave")
    ap.add_argument("--layers", type=int, default=16, help="decode workload: decoder layers (16 = the 1B shape)")
    ap.add_argument("--columns", type=int, default=64, help="ultra-sparse workload: valid columns (batch) per GPU, 1..64")
    ap.add_argument("--group", type=int, default=128, choices=[16, 32, 64, 128],
                    help="ultra-sparse workload: neurons sharing one gather list (below 128: the general mma.sync kernel)")
    ap.add_argument("--shift-act", type=int, default=5, help="token-shift workload: activation code of its waves (5 = GELU as the configuration names; 0 = none, to separate the epilogue's share)")
    ap.add_argument("--max-shift", type=int, default=7, help="token-shift workload: largest token shift drawn per run (0 = unshifted runs)")
    ap.add_argument("--frames", type=int, default=1, help="image workload: images per inference (wavec_set_batch_size; at most 9 at 640 x 640)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-pipeline", action="store_true", help="end to end with one blocking k44b_infer_f16 call per step only")
    ap.add_argument("--no-sharded", action="store_true", help="with several GPUs: skip the neuron-sharded sub-measurement")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = {"decode": 2000, "decode-full": 1000, "token-shift": 500, "image": 500}.get(args.workload, 10)
    if args.workload in ("decode", "decode-full"):
        return decode_main(args)
    if args.workload == "pruned-sharded":
        return sharded_main(args)
    if args.workload == "token-shift":
        return shift_main(args)
    if args.workload == "tiny":
        return tiny_main(args)
    if args.workload == "whitepaper":
        return whitepaper_main(args)
    if args.workload == "image":
        return image_main(args)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = workload(args.scale)
    w["columns"] = max(1, min(64, args.columns))
    w["group"] = args.group
    warmup = max(3, args.warmup)
    cfg = {"workload": f"ultra-sparse plan: {w['input_rows'] / 1e6:g}M-row FP16 substrate, {w['waves']} waves x {w['cout']} neurons, fan-in "
                       f"{w['runs'] * w['run_len']} as {w['runs']} runs of {w['run_len']} rows, groups of {w['group']}, ReLU, {w['columns']} columns per GPU",
           "input_rows": w["input_rows"], "neurons_per_wave": w["cout"], "waves": w["waves"], "fan_in": w["runs"] * w["run_len"],
           "run_len": w["run_len"], "group": w["group"], "columns_per_gpu": w["columns"], "global_columns": w["columns"] * world,
           "parallelism": f"column replicas x{world} (plan replicated, no collective)",
           "l2_policy": "weights streamed per step (34 GB) exceed the 126 MB L2; no explicit flush", "scale": args.scale}

    if args.impl == "reference":
        # The reference has no CPU implementation of this path and may not be compiled or run; the timed CPU arm is
        # the oracle port with all host threads, on rank 0 only.
        if rank != 0:
            return
        steps = max(1, min(args.steps, 3))
        cb = cpu_baseline(w, seconds_target=20.0, threads=host_threads())     # all host threads, whatever OMP_NUM_THREADS says
        line = {"impl": "reference", "metric": "effective synaptic TFLOP/s (2*synapses*columns/s)", "value": cb["value"], "unit": "TFLOP/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": cb["seconds_per_rep"] * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16 operands, f64 accumulate (CPU)", "data": "synthetic", "config": cfg,
                "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        init_nccl(dist, local_rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    from snntome_b200.native import fill_normal_f16
    plan = build_device_plan(w, local_rank)
    canvas = plan.canvas_tensor()
    in_elems = w["input_rows"] * 64
    fill_normal_f16(canvas[:in_elems], SEED + 77 + rank, 1.0)
    torch.cuda.synchronize()
    nw = plan.num_waves
    paths = [plan.wave_info(i).path for i in range(nw)]
    stream = torch.cuda.current_stream()

    # ---- device-resident throughput ----
    sampler = ClockSampler(local_rank)       # started before the warm-up: nvidia-smi needs ~0.1 s to deliver its first sample
    sampler.start()
    for _ in range(warmup):
        plan.execute(stream)
    assert plan.status() == 0
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(nw + 1)] for _ in range(args.steps)]
    barrier()
    l0 = plan.launch_count
    t_start = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for s in range(args.steps):
        ev[s][0].record(stream)
        for i in range(nw):
            plan.execute_wave(i, stream)
            ev[s][i + 1].record(stream)
    t_end.record(stream)
    barrier()
    launches = plan.launch_count - l0
    assert plan.status() == 0
    total_ms = t_start.elapsed_time(t_end)
    wave_ms = [[ev[s][i].elapsed_time(ev[s][i + 1]) for i in range(nw)] for s in range(args.steps)]
    if dist is not None:
        t = torch.tensor([total_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    flops_step = flops_per_wave(w) * nw
    value = flops_step * world / (ms_per_step * 1e-3) / 1e12
    bytes_wave = algorithmic_bytes_per_wave(w)
    avg_wave_ms = float(np.mean(wave_ms))
    peak, peak_kind = measured_peaks()
    achieved = bytes_wave / (avg_wave_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": f"k44_wave_umma_kernel<{plan.wave_info(0).n_tile}>" if paths[0] == 1 else ("k44_wave_mma_kernel" if paths[0] == 3 else "k44_wave_fma_kernel"),
                "achieved": achieved, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                "algorithmic_bytes_per_launch": bytes_wave, "avg_launch_ms": avg_wave_ms,
                "per_wave_ms": [float(np.mean([wave_ms[s][i] for s in range(args.steps)])) for i in range(nw)],
                # dram__bytes_read + dram__bytes_write per launch of this kernel: not measured in this run. The figure is the
                # ratio (DRAM bytes / algorithmic bytes = 0.928) of an ncu capture of the same kernel on the same plan at 1/20
                # size, times this run's algorithmic bytes; at 1/20 size part of the 256 MB substrate stays in L2, so at full
                # size the true figure is nearer the algorithmic bytes.
                "traffic": NCU_TRAFFIC_RATIO * bytes_wave if (w["columns"] == 64 and w["group"] == 128) else None,
                "traffic_kind": "scaled: ncu capture at 1/20 size (ratio 0.928 of algorithmic bytes) x this run's algorithmic bytes"
                                if (w["columns"] == 64 and w["group"] == 128) else None}

    # ---- end to end through the C ABI with host buffers (pinned FP16 in canvas layout) ----
    e2e = None
    if not args.no_e2e:
        out_rows = w["cout"]
        h_in, numa_cpus = pinned_near_gpu(in_elems, local_rank)
        h_in.copy_(canvas[:in_elems])
        h_out, _ = pinned_near_gpu(out_rows * 64, local_rank)
        e_steps = max(2, min(args.steps, 5))
        plan.infer_f16(h_in.data_ptr(), h_out.data_ptr(), stream)      # warm-up
        # the bound the host side sets: the same upload alone, all ranks at once (host memory and PCIe are shared by the ranks)
        barrier()
        c0 = torch.cuda.Event(enable_timing=True); c1 = torch.cuda.Event(enable_timing=True)
        c0.record(stream)
        canvas[:in_elems].copy_(h_in, non_blocking=True)
        c1.record(stream)
        barrier()
        copy_ms = c0.elapsed_time(c1)
        if dist is not None:
            t = torch.tensor([copy_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            copy_ms = float(t.item())
        barrier()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(e_steps):
            plan.infer_f16(h_in.data_ptr(), h_out.data_ptr(), stream)
        t1.record(stream)
        barrier()
        serial_ms = t0.elapsed_time(t1)
        # the same steps with every step's upload running under the waves of the step before it (k44b_infer_f16_begin / _next):
        # the first upload is outside the timed region, the upload started by the last timed step is inside it and waited for,
        # so the region holds e_steps uploads, e_steps executions and e_steps downloads (host clock around blocking calls)
        pipe_ms = None
        if not args.no_pipeline:
            plan.infer_f16_begin(h_in.data_ptr())
            plan.infer_f16_next(h_in.data_ptr(), h_out.data_ptr(), stream)          # warm-up of the staging path; leaves one input staged
            barrier()
            w0 = time.perf_counter()
            for _ in range(e_steps):
                plan.infer_f16_next(h_in.data_ptr(), h_out.data_ptr(), stream)
            torch.cuda.synchronize()                                                # the upload started by the last step (the plan's copy stream)
            pipe_ms = (time.perf_counter() - w0) * 1e3
            plan.infer_f16_next(0, 0, stream)                                       # outside the region: consume the staged input
        e_ms = serial_ms if pipe_ms is None else min(serial_ms, pipe_ms)
        pipelined = pipe_ms is not None and pipe_ms < serial_ms
        if dist is not None:
            t = torch.tensor([e_ms, serial_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms, serial_ms = float(t[0].item()), float(t[1].item())
        e2e = {"value": flops_step * world / (e_ms / e_steps * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms / e_steps,
               "steps": e_steps, "h2d_bytes_per_step": in_elems * 2, "d2h_bytes_per_step": out_rows * 64 * 2,
               "api": ("k44b_infer_f16_begin / k44b_infer_f16_next (host FP16 rows in, last wave's rows out, pinned memory; each step's upload runs under the previous step's waves)"
                       if pipelined else "k44b_infer_f16 (host FP16 rows in, last wave's rows out, pinned memory)"),
               "ms_per_step_one_blocking_call_per_step": serial_ms / e_steps,
               "host_copy_bound": {"upload_ms_alone_max_over_ranks": copy_ms, "upload_gbs_per_rank": in_elems * 2 / (copy_ms * 1e-3) / 1e9,
                                   "bound_ms_per_step": (max(copy_ms, ms_per_step) if pipelined else copy_ms + ms_per_step),
                                   "frac_of_bound": (max(copy_ms, ms_per_step) if pipelined else copy_ms + ms_per_step) / (e_ms / e_steps),
                                   "pinned_on_gpu_numa_node": numa_cpus is not None},
               "checksum": float(h_out[: 64 * 1024].float().abs().sum().item())}
        del h_in, h_out

    clocks = sampler.stop()                  # samples span warm-up, the timed steps and the end-to-end steps
    cb = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb = cpu_baseline(w)
    plan.close()
    del canvas
    torch.cuda.empty_cache()
    # the reference's own execution call (wavec_gpu_infer_f32: dense host FP32 in and out) on a workload whose tensors fit its
    # `int` element counts; one GPU only
    ref_call = None
    if rank == 0 and world == 1 and not args.no_e2e and args.scale == 1.0:
        try:
            ref_call = reference_call_e2e(local_rank, steps=max(3, min(args.steps, 10)))
        except Exception as exc:      # reported, never fatal for the main line
            ref_call = {"error": f"{type(exc).__name__}: {exc}"}
    # neuron sharding (rows of every wave split over the ranks, rows exchanged by the wave kernels): strong scaling of one
    # batch, reported beside the column-replica result whenever there is more than one GPU
    sharded = None
    if world > 1 and not args.no_sharded:
        try:
            sh = sharded_measure(PRUNED["layers"], steps=10, warmup=3, rank=rank, local_rank=local_rank, world=world, breakdown=False)
            sharded = {k: sh[k] for k in ("metric", "value", "unit", "ms_per_step", "scaling", "steps", "gpu_launches", "checksum") if k in sh}
            sharded.update({"exchange_mode": sh["config"]["exchange_mode"], "exchange": sh["config"]["exchange"],
                            "bytes_received_per_rank_per_step": sh["config"]["bytes_received_per_rank_per_step"],
                            "nvlink_time_bound_ms": sh["config"]["nvlink_time_bound_ms"], "workload": sh["config"]["workload"],
                            "launches_per_step": sh["config"]["launches_per_step"], "signal": sh["config"]["signal"],
                            "launches_that_wait_for_the_launch_before": sh["config"]["launches_that_wait_for_the_launch_before"],
                            "waves_per_step": sh["config"]["waves_per_step"]})
            if "error" in sh:
                sharded["error"] = sh["error"]
        except Exception as exc:
            sharded = {"error": f"{type(exc).__name__}: {exc}"}
    if rank == 0:
        line = {"metric": "effective synaptic TFLOP/s (2*synapses*columns/s)", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic", "config": cfg,
                "hbm_gbs_algorithmic": bytes_wave * nw * world / (ms_per_step * 1e-3) / 1e9, "roofline": roofline, "cpu_baseline": cb,
                "e2e": e2e, "e2e_reference_call": ref_call, "sharded": sharded, "gpu_launches": int(launches), "kernel_paths": paths, "clocks": clocks}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
