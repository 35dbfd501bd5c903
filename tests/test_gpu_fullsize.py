"""Parity at benchmark size and on the benchmark workloads' structure.

* the ultra-sparse plan at its full size (40 M substrate rows, 4 x 1 M neurons, fan-in 4096; about 40 GB on the
  device): the oracle cannot run all of it, so whole neuron groups are sampled per wave and recomputed by the oracle
  from the device's own inputs (the rows the group gathers, read back from the canvas) and weights (unpacked from the
  device's packed copy);
* the token-shift plan at its full size (8 sequences x 4096 tokens, 4 waves x 8192 neurons, fan-in 512 as 32 shifted
  runs of 16 channels): sampled (group, sequence) pairs are recomputed by the oracle from the device's inputs and weights;
* a small dense decoder wave chain (same structure as the 1B benchmark: q,k,v / o+residual / gate,up / down+residual
  per layer, lm_head) replayed as a CUDA graph with grouped launches, against the oracle in full.
"""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from oracle import oracle as O
from snntome_b200 import synth
from snntome_b200.native import NativePlan, PATH_UMMA
from snntome_b200.plan import ACT_GELU, ACT_NONE, ACT_RELU, ACT_SILU, Plan, Wave

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-3


def test_ultra_sparse_plan_full_size_sampled_groups():
    import torch
    import bench
    free, _ = torch.cuda.mem_get_info()
    scale = float(os.environ.get("K44B_TEST_SCALE", "1.0"))
    if free < 60e9 * scale:
        pytest.skip("not enough free device memory for the full-size plan")
    w = bench.workload(scale)
    plan = bench.build_device_plan(w, 0)
    from snntome_b200.native import fill_normal_f16
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: w["input_rows"] * 64], 5, 1.0)
    plan.execute()
    assert plan.status() == 0
    rng = np.random.default_rng(3)
    fan_in = w["runs"] * w["run_len"]
    cv2 = canvas.view(-1, 64)
    for wi in range(w["waves"]):
        assert plan.wave_info(wi).path == PATH_UMMA and plan.wave_info(wi).box_rows == 64
        starts = bench.run_starts_table(wi, w)                          # [groups, runs]
        wrm = plan.weights_rowmajor(wi)                                   # device, [cout, fan_in] int16
        groups = rng.choice(starts.shape[0], size=6, replace=False)
        row0 = w["input_rows"] + wi * w["cout"]
        for g in groups:
            rows = (torch.from_numpy(starts[g].astype(np.int64))[:, None] + torch.arange(w["run_len"])[None, :]).reshape(-1).cuda()
            x = cv2[rows].cpu().numpy().view(np.uint16)                 # [fan_in, 64] gathered rows as the device saw them
            wg = wrm[g * 128:(g + 1) * 128].cpu().numpy().view(np.uint16)
            got = cv2[row0 + g * 128: row0 + (g + 1) * 128].cpu().numpy().view(np.uint16)
            idx = (np.arange(fan_in, dtype=np.uint32) * 64)[None, :]
            wave = Wave(cout=128, group=128, fan_in=fan_in, idx=idx, weights=wg, bias=None, y_off=fan_in * 64, act=ACT_RELU)
            mini = Plan(canvas_elems=(fan_in + 128) * 64, pitch=64, columns=64, input_off=0, input_c=fan_in, output_off=fan_in * 64,
                        output_c=128, waves=[wave])
            want = O.run_plan(mini, x)[fan_in * 64:]
            ok, err, k = O.compare(got.reshape(-1), want, RTOL, ATOL)
            assert ok, f"wave {wi} group {g}: max abs err {err} at {k}"
        del wrm
        torch.cuda.empty_cache()
    plan.close()


def test_token_shift_plan_full_size_sampled_groups():
    import torch
    import bench
    from snntome_b200.native import fill_normal_f16
    c = dict(bench.SHIFT)
    plan, tables = bench.build_shift_plan(c, 0)
    T, pitch = c["tokens"], c["sequences"] * c["tokens"]
    fan_in = c["runs"] * c["run_len"]
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: c["input_channels"] * pitch], 6, 1.0)
    plan.execute()
    assert plan.status() == 0
    rng = np.random.default_rng(4)
    cv2 = canvas.view(-1, pitch)
    for wi in range(c["waves"]):
        info = plan.wave_info(wi)
        assert info.path == PATH_UMMA and info.n_tile == 128 and info.weights_in_tmem > 0      # fan-in 512: the kernel that keeps the weight tile in tensor memory
        starts, shifts = tables[wi]
        wrm = plan.weights_rowmajor(wi)
        row0 = c["input_channels"] + wi * c["cout"]
        for g, f in zip(rng.choice(starts.shape[0], size=3, replace=False), rng.choice(c["sequences"], size=3, replace=True)):
            rows = (torch.from_numpy(starts[g].astype(np.int64))[:, None] + torch.arange(c["run_len"])[None, :]).reshape(-1).cuda()
            x = cv2[rows][:, f * T:(f + 1) * T].contiguous().cpu().numpy().view(np.uint16)     # this sequence's columns of the gathered rows
            wg = wrm[g * 128:(g + 1) * 128].cpu().numpy().view(np.uint16)
            got = cv2[row0 + g * 128: row0 + (g + 1) * 128, f * T:(f + 1) * T].contiguous().cpu().numpy().view(np.uint16)
            idx = (np.arange(fan_in, dtype=np.uint32) * T)[None, :]
            sh = np.repeat(shifts[g], c["run_len"])[None, :]
            wave = Wave(cout=128, group=128, fan_in=fan_in, idx=idx, weights=wg, bias=None, y_off=fan_in * T, act=ACT_GELU, shifts=sh, frame_len=T)
            mini = Plan(canvas_elems=(fan_in + 128) * T, pitch=T, columns=T, input_off=0, input_c=fan_in, output_off=fan_in * T,
                        output_c=128, waves=[wave])
            want = O.run_plan(mini, x)[fan_in * T:]
            ok, err, k = O.compare(got.reshape(-1), want, RTOL, ATOL)
            assert ok, f"wave {wi} group {g} sequence {f}: max abs err {err} at {k}"
        del wrm
    plan.close()


def test_dense_decoder_chain_full_size_sampled_rows():
    """The 113-wave chain of the 1B decoder at its benchmark size (2.47 GB of weights generated on the device): after one
    graph replay the last layer's tensors and the logits are still in the canvas, so sampled 128-row groups of its seven
    waves and of the lm_head are recomputed by the oracle from the device's own inputs and unpacked weights."""
    import torch
    import bench
    from snntome_b200.native import fill_normal_f16
    cfg = dict(bench.DECODER)
    plan, params, rows = bench.build_decoder_plan(cfg, 0)
    H, F, V, KV = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["kv_heads"] * cfg["head_dim"]
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: H * 64], 99, 1.0)
    plan.execute_graph()
    assert plan.status() == 0
    cv2 = canvas.view(-1, 64)
    rng = np.random.default_rng(8)
    nw = plan.num_waves
    last = nw - 8                                            # first wave of layer 15; it reads x1 and writes x0
    # (wave index, source tensor, destination tensor, fan-in, rows, activation, residual tensor)
    checks = [(last + 0, "x1", "q", H, H, ACT_NONE, None), (last + 1, "x1", "k", H, KV, ACT_NONE, None), (last + 2, "x1", "v", H, KV, ACT_NONE, None),
              (last + 3, "q", "h", H, H, ACT_NONE, "x1"), (last + 4, "h", "g", H, F, ACT_SILU, None), (last + 5, "h", "u", H, F, ACT_NONE, None),
              (last + 6, "g", "x0", F, H, ACT_NONE, "h"), (nw - 1, "x0", "logits", H, V, ACT_NONE, None)]
    for wi, src, dst, cin, cout, act, res in checks:
        wrm = plan.weights_rowmajor(wi)
        x = cv2[rows[src]: rows[src] + cin].cpu().numpy().view(np.uint16)
        for g in rng.choice(cout // 128, size=2, replace=False):
            wg = wrm[g * 128:(g + 1) * 128].cpu().numpy().view(np.uint16)
            got = cv2[rows[dst] + g * 128: rows[dst] + (g + 1) * 128].cpu().numpy().view(np.uint16)
            idx = (np.arange(cin, dtype=np.uint32) * 64)[None, :]
            extra = 128 if res else 0
            wave = Wave(cout=128, group=128, fan_in=cin, idx=idx, weights=wg, bias=None, y_off=(cin + extra) * 64, act=act,
                        has_residual=res is not None, res_off=cin * 64)
            mini = Plan(canvas_elems=(cin + extra + 128) * 64, pitch=64, columns=64, input_off=0, input_c=cin + extra, output_off=(cin + extra) * 64,
                        output_c=128, waves=[wave])
            xin = x if not res else np.concatenate([x, cv2[rows[res] + g * 128: rows[res] + (g + 1) * 128].cpu().numpy().view(np.uint16)])
            want = O.run_plan(mini, xin)[(cin + extra) * 64:]
            ok, err, k = O.compare(got.reshape(-1), want, RTOL, ATOL)
            assert ok, f"wave {wi} ({dst}) group {g}: max abs err {err} at {k}"
        del wrm
    plan.close()


def mini_decoder(seed=9, hidden=256, kv=64, ffn=768, vocab=1024, layers=2, columns=64):
    rng = np.random.default_rng(seed)
    pitch = 64
    rows, cur = {}, 0
    for name, n in [("x0", hidden), ("x1", hidden), ("q", hidden), ("k", kv), ("v", kv), ("h", hidden), ("g", ffn), ("u", ffn), ("logits", vocab)]:
        rows[name] = cur
        cur += n
    waves = []

    def add(name, src, dst, cin, cout, act=ACT_NONE, res=None):
        offs = ((rows[src] + np.arange(cin)) * pitch).astype(np.uint32)
        g = 128 if cout % 128 == 0 else 64
        waves.append(Wave(cout=cout, group=g, fan_in=cin, idx=np.tile(offs, (cout // g, 1)), weights=synth.f16_bits(rng.normal(0, 0.03, (cout, cin))),
                          bias=None, y_off=rows[dst] * pitch, act=act, has_residual=res is not None,
                          res_off=rows[res] * pitch if res else 0, name=name))

    x_in, x_out = "x0", "x1"
    for layer in range(layers):
        add(f"L{layer}.q", x_in, "q", hidden, hidden)
        add(f"L{layer}.k", x_in, "k", hidden, kv)
        add(f"L{layer}.v", x_in, "v", hidden, kv)
        add(f"L{layer}.o", "q", "h", hidden, hidden, res=x_in)
        add(f"L{layer}.gate", "h", "g", hidden, ffn, act=ACT_SILU)
        add(f"L{layer}.up", "h", "u", hidden, ffn)
        add(f"L{layer}.down", "g", x_out, ffn, hidden, res="h")
        x_in, x_out = x_out, x_in
    add("lm_head", x_in, "logits", hidden, vocab)
    return Plan(canvas_elems=cur * pitch, pitch=pitch, columns=columns, input_off=0, input_c=hidden, output_off=rows["logits"] * pitch,
                output_c=vocab, waves=waves)


@pytest.mark.parametrize("group_launches", [1, 0])
def test_decoder_wave_chain_graph_replay(group_launches, monkeypatch):
    import torch
    monkeypatch.setenv("K44B_GROUP", str(group_launches))
    plan = mini_decoder()
    x = synth.random_input(plan, 31, dist="normal")
    want = O.run_plan(plan, x)
    npn = NativePlan.from_plan(plan, force_path=PATH_UMMA)
    canvas = npn.canvas_tensor()
    xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    before = npn.launch_count
    for _ in range(3):
        canvas[: xt.numel()] = xt                            # the last layer writes its result over the input rows
        npn.execute_graph()
    assert npn.status() == 0
    per_step = (npn.launch_count - before) // 3
    assert per_step == (9 if group_launches else 15)        # {q,k,v} {o} {gate,up} {down} per layer + lm_head
    got = canvas.cpu().numpy().view(np.uint16)
    for w in plan.waves[-8:]:                                 # last layer and lm_head hold their final values
        a, b = w.y_off, w.y_off + w.cout * plan.pitch
        ok, err, k = O.compare(got[a:b], want[a:b], RTOL, ATOL)
        assert ok, (w.name, err, k)
    npn.close()


@pytest.mark.parametrize("path_name", ["auto", "fma"])
def test_more_than_65535_neuron_blocks_of_a_small_group(path_name):
    """A million neurons in groups of 16 (the full-size plan's neuron count): 65,538 neuron blocks per column tile, more than
    the y extent of a grid allows, so the general kernels index a one-dimensional grid. Sampled groups against the oracle,
    the last (partial-range) blocks included."""
    import torch
    from snntome_b200.native import PATH_AUTO, PATH_FMA, PATH_MMA
    from snntome_b200.plan import expand_runs
    force = PATH_AUTO if path_name == "auto" else PATH_FMA
    rng = np.random.default_rng(77)
    group, fan_in, pitch, rows_in = 16, 64, 64, 4096
    cout = 65536 * 16 + 32
    groups = cout // group
    starts = (rng.integers(0, rows_in // 16, size=(groups, 4)) * 16).astype(np.int64)          # four runs of 16 rows per group
    idx = expand_runs(starts, 16, pitch)
    wts = synth.f16_bits(rng.normal(0, 0.125, size=(cout, fan_in)).astype(np.float32))
    wave = Wave(cout=cout, group=group, fan_in=fan_in, idx=idx, weights=wts, bias=None, y_off=rows_in * pitch, act=ACT_RELU, name="wide")
    plan = Plan(canvas_elems=(rows_in + cout) * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=rows_in,
                output_off=rows_in * pitch, output_c=cout, waves=[wave])
    x = synth.random_input(plan, 78, dist="normal")
    npn = NativePlan.from_plan(plan, device=0, force_path=force)
    assert npn.wave_info(0).path == (PATH_MMA if path_name == "auto" else PATH_FMA)
    canvas = npn.canvas_tensor()
    canvas[: x.size] = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    npn.execute()
    assert npn.status() == 0
    got = canvas.cpu().numpy().view(np.uint16)
    npn.close()
    picks = np.concatenate([rng.integers(0, groups, size=48), [0, 4095, 4096, groups - 3, groups - 2, groups - 1]])
    xin = x.reshape(rows_in, pitch)
    for g in picks:
        g = int(g)
        sub = Wave(cout=group, group=group, fan_in=fan_in, idx=idx[g:g + 1].copy(), weights=wts[g * group:(g + 1) * group].copy(), bias=None,
                   y_off=rows_in * pitch, act=ACT_RELU, name="sample")
        sp = Plan(canvas_elems=(rows_in + group) * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=rows_in,
                  output_off=rows_in * pitch, output_c=group, waves=[sub])
        want = O.run_plan(sp, xin)[rows_in * pitch:]
        a = (rows_in + g * group) * pitch
        ok, err, k = O.compare(got[a:a + group * pitch], want, RTOL, ATOL)
        assert ok, (g, err, k)


def test_pruned_8b_chain_full_size_sampled_groups():
    """BASELINE configs[4] on one GPU at its full size (Llama-3-8B shapes, 32 layers, 90 % of the 32-row input clusters of every
    128-neuron group removed, dense lm_head, 256 columns): the chain is walked wave by wave and sampled groups of sampled
    waves — with and without residual, SiLU, the dense lm_head — are recomputed by the oracle from the device's own inputs."""
    import torch
    import bench
    import pruned_check
    from snntome_b200.native import fill_normal_f16
    layers = int(os.environ.get("K44B_TEST_LAYERS", "32"))
    plan, info = bench.build_pruned_plan(layers, 0, 0, 1)
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: info["cfg"]["hidden"] * info["pitch"]], 4242, 1.0)
    picks = set(pruned_check.sampled_waves(plan.num_waves))
    for wi in range(plan.num_waves):
        plan.execute_wave(wi)
        if wi in picks:
            assert plan.status() == 0
            pruned_check.check_wave(plan, info, wi, canvas)
    assert plan.status() == 0
    plan.close()


@pytest.mark.parametrize("gen,row", [("runs", "g512_b2048_c4096"), ("rows", "g512_b2048_c4096"), ("runs", "g256_b1024_c8192")])
def test_reference_benchmark_regime_sampled_groups(gen, row):
    """The reference benchmark's plan (groups of 512 / 256 neurons, fan-in 2048 / 1024, 512 columns, 16 waves merged into one)
    over a 2 M-row substrate (2 GB, beyond L2): run tables take the CTA-pair kernel (M = 256 MMAs), the reference's single
    scattered rows the row-fetching warps. Sampled groups against the oracle on the rows the device gathered."""
    import torch
    import bench
    from snntome_b200.native import fill_normal_f16
    spec = bench.WHITEPAPER_ROWS[row]
    cin = 2_000_000
    plan, tables = bench.build_whitepaper_plan(spec, cin, 0, gen, True)
    pitch, B, G = spec["columns"], spec["fan_in"], spec["group"]
    canvas = plan.canvas_tensor()
    fill_normal_f16(canvas[: cin * pitch], 21, 1.0)
    plan.execute()
    assert plan.status() == 0
    info = plan.wave_info(0)
    assert info.path == PATH_UMMA and info.n_tile == 256
    assert (info.cta_pairs == 1 and info.box_rows == 64) if gen == "runs" else info.box_rows == 1
    rows_tab, run_len, out_row0, cout = tables[0]
    wrm = plan.weights_rowmajor(0)
    cv2 = canvas.view(-1, pitch)
    rng = np.random.default_rng(8)
    for g in rng.choice(rows_tab.shape[0], size=3, replace=False):
        rows = (torch.from_numpy(rows_tab[g].astype(np.int64))[:, None] + torch.arange(run_len)[None, :]).reshape(-1).cuda()
        x = cv2[rows].cpu().numpy().view(np.uint16)                         # [B, pitch]
        j0 = int(g) * G + int(rng.integers(0, G // 128)) * 128              # one 128-neuron block of the group
        wg = wrm[j0: j0 + 128].cpu().numpy().view(np.uint16)
        got = cv2[out_row0 + j0: out_row0 + j0 + 128].cpu().numpy().view(np.uint16)
        idx = (np.arange(B, dtype=np.uint32) * pitch)[None, :]
        wave = Wave(cout=128, group=128, fan_in=B, idx=idx, weights=wg, bias=None, y_off=B * pitch, act=ACT_NONE)
        mini = Plan(canvas_elems=(B + 128) * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=B, output_off=B * pitch, output_c=128, waves=[wave])
        want = O.run_plan(mini, x)[B * pitch:]
        ok, err, k = O.compare(got.reshape(-1), want, RTOL, ATOL)
        assert ok, f"group {g}: max abs err {err} at {k}"
    del wrm
    plan.close()
    torch.cuda.empty_cache()
