"""GPU parity: the CUDA wave executor, called through the C ABI, against the CPU oracle on the same
seeded inputs. Tolerance for outputs is rtol 2e-3 / atol 1e-3 (FP16 operands, FP32 accumulation on
the device, double accumulation in the oracle); plan decoding, weight packing and container bytes
are compared exactly."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import native, synth
from snntome_b200.native import PATH_AUTO, PATH_FMA, PATH_MMA, PATH_UMMA, NativePlan
from snntome_b200.plan import ACT_GELU, ACT_LEAKY_RELU, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, Plan, Wave

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-3


def run_gpu(plan, x_bits, force_path=PATH_AUTO, expect_path=None):
    import torch
    npn = NativePlan.from_plan(plan, device=0, force_path=force_path)
    if expect_path is not None:
        for i in range(npn.num_waves):
            assert npn.wave_info(i).path == expect_path, f"wave {i} took path {npn.wave_info(i).path}"
    canvas = npn.canvas_tensor()
    x = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    canvas[plan.input_off: plan.input_off + x.numel()] = x
    npn.execute()
    assert npn.status() == 0
    out = canvas.cpu().numpy().view(np.uint16)
    npn.close()
    return out


def check(plan, got_canvas, want_canvas):
    for w in plan.waves:
        a, b = w.y_off, w.y_off + w.cout * plan.pitch
        ok, err, k = O.compare(got_canvas[a:b], want_canvas[a:b], RTOL, ATOL)
        assert ok, f"wave {w.name}: max abs err {err} at element {k} (row {k // plan.pitch}, col {k % plan.pitch})"


def check_per_wave(plan, got_canvas):
    """Every wave against the oracle run on what the device itself read: the final device canvas holds each wave's inputs (the
    waves of these plans write disjoint rows and read only rows written before them), so the oracle recomputes one wave at a
    time from it. Differences inside the tolerance of one wave then cannot add up through the waves that consume its rows —
    which they do, legitimately, in plans of ten million outputs per wave when the whole chain is computed on the oracle's side."""
    for w in plan.waves:
        c = got_canvas.copy()
        O.wave_forward(c, w, plan)
        a, b = w.y_off, w.y_off + w.cout * plan.pitch
        ok, err, k = O.compare(got_canvas[a:b], c[a:b], RTOL, ATOL)
        assert ok, f"wave {w.name}: max abs err {err} at element {k} (row {k // plan.pitch}, col {k % plan.pitch})"


@pytest.mark.parametrize("group", [128, 16])
def test_config0_fma_path(group):
    plan = synth.config0(group=group)
    x = synth.random_input(plan, 11)
    check(plan, run_gpu(plan, x, PATH_FMA, expect_path=PATH_FMA), O.run_plan(plan, x))


def test_config0_tensor_core_path():
    plan = synth.config0(group=128)
    x = synth.random_input(plan, 11)
    check(plan, run_gpu(plan, x, PATH_UMMA, expect_path=PATH_UMMA), O.run_plan(plan, x))


def test_config0_group16_takes_the_general_tensor_path_automatically():
    plan = synth.config0(group=16)
    x = synth.random_input(plan, 12)
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), O.run_plan(plan, x))


def test_ultra_sparse_rule_scaled_down():
    """Fan-in 4096 = 64 runs of 64 rows, groups of 128, ReLU, 64 columns — the benchmark plan's
    connectivity at a size the oracle finishes quickly."""
    plan = synth.config2_scaled(input_rows=32768, cout=1024, waves=2)
    x = synth.random_input(plan, 13, dist="normal")
    want = O.run_plan(plan, x)
    check(plan, run_gpu(plan, x, PATH_UMMA, expect_path=PATH_UMMA), want)
    check(plan, run_gpu(plan, x, PATH_FMA, expect_path=PATH_FMA), want)


@pytest.mark.parametrize("act", [ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, ACT_LEAKY_RELU, ACT_GELU])
@pytest.mark.parametrize("path", [PATH_FMA, PATH_UMMA])
def test_dense_chain_all_activations(act, path):
    plan = synth.dense_chain(seed=act + 20, dims=[192, 384, 200], columns=64, act=act, weight_std=0.08)
    x = synth.random_input(plan, 14)
    check(plan, run_gpu(plan, x, path, expect_path=path), O.run_plan(plan, x))


@pytest.mark.parametrize("act", [ACT_SIGMOID, ACT_SILU, ACT_GELU])
@pytest.mark.parametrize("path", [PATH_UMMA, PATH_MMA, PATH_FMA])
def test_smooth_activations_over_every_fp16_pre_activation(act, path):
    """Every finite FP16 value in [-24, 24] (subnormals and both zeros included) goes through the epilogue as the
    pre-activation: a wave whose neuron j copies input row j % 64 (one weight of 1.0). The tensor-core epilogue evaluates the
    smooth activations with fast exponentials and, for GELU, a fitted logit; the general kernels call expf / erff. All of them
    must stay inside rtol 2e-3 / atol 1e-3 of the oracle's double-precision exp / erf forms over the whole range, in particular
    on the negative tail where the result is tiny and only the absolute bound protects it."""
    bits = np.arange(0x10000, dtype=np.uint32).astype(np.uint16)
    vals = bits.view(np.float16).astype(np.float32)
    bits = bits[np.isfinite(vals) & (np.abs(vals) <= 24.0)]
    rows_in, cout = 64, 128
    pitch = (bits.size + rows_in * 64 - 1) // (rows_in * 64) * 64
    x = np.zeros((rows_in, pitch), dtype=np.uint16)
    x.reshape(-1)[: bits.size] = np.random.default_rng(3).permutation(bits)
    group = cout if path != PATH_MMA else 16               # groups of 16 with lists of their own: the general tensor kernel
    groups = cout // group
    idx = np.stack([np.roll(np.arange(64, dtype=np.uint32) * pitch, g) for g in range(groups)])      # group g lists row r at position (r + g) % 64
    w = np.zeros((cout, 64), dtype=np.float16)
    j = np.arange(cout)
    w[j, (j % 64 + j // group) % 64] = 1.0
    wave = Wave(cout=cout, group=group, fan_in=64, idx=idx, weights=w.view(np.uint16), bias=None, y_off=rows_in * pitch, act=act)
    plan = Plan(canvas_elems=(rows_in + cout) * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=rows_in,
                output_off=rows_in * pitch, output_c=cout, waves=[wave])
    want = O.run_plan(plan, x)
    got = run_gpu(plan, x, PATH_AUTO if path == PATH_MMA else path, expect_path=path)
    check(plan, got, want)


@pytest.mark.parametrize("path", [PATH_FMA, PATH_UMMA])
def test_ragged_sizes_and_tail_stage(path):
    # fan-in 96 (half-filled last stage), 80 output rows (partial 128-row tile), one group
    plan = synth.dense_chain(seed=31, dims=[96, 80, 130], columns=64, act=ACT_SILU, weight_std=0.1, group=0)
    for w in plan.waves:                      # single group per wave so the tensor-core path applies
        w.idx = w.idx[:1].copy()
        w.group = w.cout
    x = synth.random_input(plan, 15)
    check(plan, run_gpu(plan, x, path, expect_path=path), O.run_plan(plan, x))


@pytest.mark.parametrize("path", [PATH_FMA, PATH_UMMA])
@pytest.mark.parametrize("with_map", [False, True])
def test_residual_and_row_map(path, with_map):
    plan = synth.dense_chain(seed=41, dims=[128, 128, 128], columns=64, act=ACT_RELU, weight_std=0.1, residual_from={2: 1})
    if with_map:
        rng = np.random.default_rng(5)
        plan.waves[1].cout_map = rng.permutation(plan.waves[1].cout).astype(np.uint16)
    x = synth.random_input(plan, 16, dist="normal")
    check(plan, run_gpu(plan, x, path, expect_path=path), O.run_plan(plan, x))


@pytest.mark.parametrize("columns,n_tile", [(64, 64), (128, 128), (256, 256), (512, 256), (192, 64), (320, 64)])
def test_column_tiles(columns, n_tile, monkeypatch):
    monkeypatch.setenv("K44B_N_TILE", str(n_tile))
    plan = synth.sparse_plan(seed=51 + columns, input_rows=2048, waves=2, cout=256, runs=8, run_len=32, columns=columns,
                             group=128, act=ACT_RELU)
    x = synth.random_input(plan, 17)
    want = O.run_plan(plan, x)
    check(plan, run_gpu(plan, x, PATH_UMMA, expect_path=PATH_UMMA), want)
    check(plan, run_gpu(plan, x, PATH_FMA), want)


@pytest.mark.parametrize("run_len", [8, 16, 32, 64])
def test_run_lengths(run_len):
    plan = synth.sparse_plan(seed=60 + run_len, input_rows=4096, waves=1, cout=384, runs=256 // run_len, run_len=run_len,
                             columns=64, group=128, act=ACT_NONE)
    x = synth.random_input(plan, 18)
    check(plan, run_gpu(plan, x, PATH_UMMA, expect_path=PATH_UMMA), O.run_plan(plan, x))


def test_token_shift_offsets_use_general_path():
    """Element-granular gather offsets (a tap that is the same row read a few tokens earlier)."""
    rng = np.random.default_rng(70)
    pitch, rows_in, cout, B, group = 256, 64, 128, 64, 128
    shifts = rng.integers(0, 8, size=B)
    rows = rng.integers(1, rows_in, size=B)
    idx = (rows * pitch - shifts).astype(np.uint32)[None, :]
    w = synth.f16_bits(rng.normal(0, 0.2, (cout, B)))
    wave = Wave(cout=cout, group=group, fan_in=B, idx=idx, weights=w, bias=None, y_off=rows_in * pitch, act=ACT_GELU)
    plan = Plan(canvas_elems=(rows_in + cout) * pitch, pitch=pitch, columns=200, input_off=0, input_c=rows_in,
                output_off=rows_in * pitch, output_c=cout, waves=[wave])
    x = synth.random_input(plan, 19)
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), O.run_plan(plan, x))


@pytest.mark.parametrize("group,cout,tiles,residual,row_map", [(16, 96, 3, False, False), (32, 128, 2, True, False), (64, 192, 4, False, True),
                                                              (128, 384, 3, True, True), (128, 256, 5, False, False)])
def test_raw_offset_token_shifts_spread(group, cout, tiles, residual, row_map):
    """The reference's own token-shift form: gather offsets that are a row start minus a few elements, so that a shifted tap
    reads the tail of the previous canvas row at the start of its own (kernels/cuda/kernel44_cuda_pack.cuh:153-159) — no zero
    padding, no frames. Groups of 16 .. 128 neurons with their own lists, several column tiles, bias, residual added after
    or (with a row map) before the activation, on the general tensor kernel and on the FP32-FMA kernel."""
    rng = np.random.default_rng(7000 + group + cout)
    pitch, rows_in, B = 64 * tiles, 96, 96
    groups = cout // group
    shifts = rng.integers(0, 8, size=(groups, B))
    rows = rng.integers(1, rows_in, size=(groups, B))
    idx = (rows * pitch - shifts).astype(np.uint32)
    w = synth.f16_bits(rng.normal(0, 0.15, (cout, B)))
    bias = synth.f16_bits(rng.normal(0, 0.1, cout))
    res_off = (rows_in + cout) * pitch
    wave = Wave(cout=cout, group=group, fan_in=B, idx=idx, weights=w, bias=bias, y_off=rows_in * pitch, act=ACT_SILU,
                has_residual=residual, res_off=res_off if residual else 0)
    if row_map:
        wave.cout_map = rng.permutation(cout).astype(np.uint16)
    plan = Plan(canvas_elems=(rows_in + 2 * cout) * pitch, pitch=pitch, columns=pitch - 9, input_off=0, input_c=rows_in,
                output_off=rows_in * pitch, output_c=cout, waves=[wave])
    x = synth.random_input(plan, 33, dist="normal")
    canvas0 = np.zeros(plan.canvas_elems, dtype=np.uint16)
    canvas0[: x.size] = x.reshape(-1)
    if residual:
        canvas0[res_off: res_off + cout * pitch] = synth.f16_bits(rng.normal(0, 0.5, cout * pitch))
    want = canvas0.copy()
    O.wave_forward(want, wave, plan)
    for path, expect in ((PATH_AUTO, PATH_MMA), (PATH_FMA, PATH_FMA)):
        import torch
        npn = NativePlan.from_plan(plan, device=0, force_path=path)
        assert npn.wave_info(0).path == expect
        cv = npn.canvas_tensor()
        cv.copy_(torch.from_numpy(canvas0.view(np.int16)).cuda().view(torch.float16))
        npn.execute()
        assert npn.status() == 0
        got = cv.cpu().numpy().view(np.uint16)
        npn.close()
        check(plan, got, want)


def test_minimum_size_wave():
    plan = synth.dense_chain(seed=80, dims=[8, 3], columns=1, act=ACT_SIGMOID)
    assert plan.waves[0].cout == 16 and plan.waves[0].fan_in == 64
    x = synth.random_input(plan, 20)
    want = O.run_plan(plan, x)
    check(plan, run_gpu(plan, x, PATH_FMA), want)
    plan.waves[0].idx = plan.waves[0].idx[:1].copy()
    plan.waves[0].group = 16
    check(plan, run_gpu(plan, x, PATH_UMMA, expect_path=PATH_UMMA), want)


def test_weight_packing_is_bit_exact():
    import torch
    plan = synth.dense_chain(seed=90, dims=[160, 208], columns=64)
    npn = NativePlan.from_plan(plan)
    got = npn.weights_rowmajor(0).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, plan.waves[0].weights)
    # device-resident row-major source takes the other packer kernel
    w = plan.waves[0]
    dev = torch.from_numpy(w.weights.view(np.int16)).cuda()
    np2 = NativePlan.create(plan.canvas_elems, plan.pitch, plan.columns)
    np2.add_wave(w, device_weights_ptr=dev.data_ptr())
    assert np.array_equal(np2.weights_rowmajor(0).cpu().numpy().view(np.uint16), w.weights)


def test_run_table_form_equals_index_form():
    plan = synth.config0()
    x = synth.random_input(plan, 21)
    base = run_gpu(plan, x, PATH_UMMA)
    import torch
    npn = NativePlan.create(plan.canvas_elems, plan.pitch, plan.columns, force_path=PATH_UMMA)
    for wi, w in enumerate(plan.waves):
        starts = synth.run_starts(1234, wi, w.cout // w.group, 16, 16, 4096 + wi * 1024).astype(np.uint32)
        npn.add_wave(w, run_rows=starts, run_len=16)
        assert npn.wave_info(wi).box_rows == 16
    canvas = npn.canvas_tensor()
    xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    canvas[: xt.numel()] = xt
    npn.execute()
    assert npn.status() == 0
    assert np.array_equal(canvas.cpu().numpy().view(np.uint16), base)


def test_wavec_surface_end_to_end(tmp_path):
    """compile -> save .tcff -> fresh graph -> load -> infer_f32 through the reference-shaped API, and
    the same file through the native loader."""
    from snntome_b200.wavec import WaveGraph
    rng = np.random.default_rng(100)
    dims, cols = [256, 512, 128], 48
    ws = [rng.normal(0, 0.05, (dims[i + 1], dims[i])).astype(np.float32) for i in range(2)]
    bs = [rng.normal(0, 0.1, dims[i + 1]).astype(np.float32) for i in range(2)]

    def build(weights):
        g = WaveGraph(batch_size=cols)
        g.add_input("x", dims[0], 1, 1, is_1d=True)
        g.add_linear("fc1", "x", "h", dims[0], dims[1], weights[0], bs[0], act="silu")
        g.add_linear("fc2", "h", "y", dims[1], dims[2], weights[1], bs[1], act=None)
        g.set_output("y")
        return g

    g = build(ws)
    plan = g.compile()
    path = tmp_path / "mlp.tcff"
    plan.save_tcff(path)
    g2 = build([np.zeros_like(w) for w in ws])
    plan2 = g2.compile()
    plan2.load_tcff_weights(path)
    x = rng.uniform(-1, 1, (dims[0], 1, cols)).astype(np.float32)
    y, ms = plan2.infer_f32(x)
    assert y.shape == (dims[2], 1, cols) and ms > 0
    # oracle on the FP16-quantised operands
    xq = O.f16_to_f32(O.f32_to_f16(x[:, 0, :])).astype(np.float64)
    w1 = O.f16_to_f32(O.f32_to_f16(ws[0])).astype(np.float64)
    w2 = O.f16_to_f32(O.f32_to_f16(ws[1])).astype(np.float64)
    b1 = O.f16_to_f32(O.f32_to_f16(bs[0])).astype(np.float64)
    b2 = O.f16_to_f32(O.f32_to_f16(bs[1])).astype(np.float64)
    h = w1 @ xq + b1[:, None]
    h = O.f16_to_f32(O.f32_to_f16((h / (1 + np.exp(-h))).astype(np.float32))).astype(np.float64)
    want = O.f32_to_f16((w2 @ h + b2[:, None]).astype(np.float32))
    ok, err, k = O.compare(O.f32_to_f16(y[:, 0, :]), want, RTOL, ATOL)
    assert ok, (err, k)
    # native loader on the same file: no graph needed
    npn = NativePlan.from_tcff(path)
    assert npn.num_waves == 2
    y2, _ = npn.infer_f32(x, dims[2] * cols)
    # split-K partial sums are combined with FP32 atomics, whose order varies from run to run
    ok, err, k = O.compare(O.f32_to_f16(y2.reshape(dims[2], cols)), O.f32_to_f16(y[:, 0, :]), RTOL, ATOL)
    assert ok, (err, k)


def test_bad_plan_is_rejected_before_launch():
    plan = synth.config0()
    plan.waves[0].idx[3, 7] = plan.canvas_elems
    with pytest.raises(native.NativeError, match="leaves the canvas"):
        NativePlan.from_plan(plan)


def test_wave_that_gathers_its_own_output_rows_is_rejected():
    """A wave cannot run in place (CTAs of one launch would race; on a sharded plan a peer's stores would land in rows still
    being read): rejected when the wave is added. Residual rows equal to the output rows stay legal."""
    plan = synth.config0()
    w = plan.waves[1]
    w.idx[2, 5] = w.y_off + 3 * plan.pitch             # a real synapse pointing into the wave's own output rows
    with pytest.raises(native.NativeError, match="in place"):
        NativePlan.from_plan(plan)
    ok = synth.dense_chain(seed=3, dims=[256, 256, 256], columns=64, residual_from={2: 2})   # residual = own output rows
    NativePlan.from_plan(ok).close()


@pytest.mark.parametrize("cluster", [1, 0])
@pytest.mark.parametrize("splits", [0, 2, 3, 7, 32])
def test_split_k_small_waves(splits, cluster, monkeypatch):
    """Waves with fewer 128-neuron tiles than SMs cut their fan-in into K splits. Default: the splits of a tile
    form a thread-block cluster and add their partial sums through distributed shared memory. Fallback
    (K44B_CLUSTER=0): partial sums meet in an FP32 global scratch tile that must come back zeroed (repeated
    runs agree)."""
    import torch
    monkeypatch.setenv("K44B_CLUSTER", str(cluster))
    if splits:
        monkeypatch.setenv("K44B_SPLITS", str(splits))
    plan = synth.dense_chain(seed=110, dims=[2048, 320, 512, 200], columns=64, act=ACT_SILU, weight_std=0.03,
                             residual_from={3: 0})
    x = synth.random_input(plan, 22)
    want = O.run_plan(plan, x)
    npn = NativePlan.from_plan(plan, force_path=PATH_UMMA)
    infos = [npn.wave_info(i) for i in range(npn.num_waves)]
    assert all(i.path == PATH_UMMA for i in infos)
    if cluster:
        assert all(i.k_splits in (1, 2, 4, 8, 16) for i in infos)
        assert infos[0].k_splits == (8 if not splits else min(16, 1 << (min(splits, 32).bit_length() - 1)))
    else:
        assert infos[0].k_splits > 1
        if splits:
            assert infos[0].k_splits == -(-32 // -(-32 // min(splits, 32)))
    canvas = npn.canvas_tensor()
    xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    results = []
    for rep in range(3):
        canvas.zero_()
        canvas[: xt.numel()] = xt
        if rep == 2:
            npn.execute_graph()
        else:
            npn.execute()
        assert npn.status() == 0
        results.append(canvas.cpu().numpy().view(np.uint16))
        check(plan, results[-1], want)
    if cluster:      # the on-chip reduction adds the partial sums in a fixed order
        assert np.array_equal(results[0], results[1]) and np.array_equal(results[0], results[2])
    npn.close()


def test_graph_replay_equals_direct_launches():
    import torch
    plan = synth.config0()
    x = synth.random_input(plan, 23)
    npn = NativePlan.from_plan(plan)
    canvas = npn.canvas_tensor()
    xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    canvas[: xt.numel()] = xt
    npn.execute()
    assert npn.status() == 0
    a = canvas.cpu().numpy().view(np.uint16).copy()
    before = npn.launch_count
    for _ in range(3):
        canvas[xt.numel():].zero_()
        npn.execute_graph()
    assert npn.status() == 0
    assert npn.launch_count == before + 3 * npn.num_waves
    assert np.array_equal(canvas.cpu().numpy().view(np.uint16), a)


def shifted_plan(seed, *, rows_in=256, cout=256, runs=8, run_len=16, frames=2, frame_len=256, group=128, act=ACT_GELU, waves=2):
    """Token-shift receptive-field plan: every run of `run_len` rows is read 0..7 tokens earlier, with zero
    padding at the start of each frame (sequence)."""
    rng = np.random.default_rng(seed)
    pitch = frames * frame_len
    fan_in = runs * run_len
    ws, total = [], rows_in
    for wi in range(waves):
        groups = cout // group
        starts = synth.run_starts(seed, wi, groups, runs, run_len, total)
        from snntome_b200.plan import expand_runs
        idx = expand_runs(starts, run_len, pitch)
        sh_run = rng.integers(0, 8, size=(groups, runs)).astype(np.uint8)
        shifts = np.repeat(sh_run, run_len, axis=1)
        w = synth.f16_bits(rng.normal(0, (1.0 / fan_in) ** 0.5, (cout, fan_in)))
        ws.append(Wave(cout=cout, group=group, fan_in=fan_in, idx=idx, weights=w, bias=None, y_off=total * pitch, act=act,
                       shifts=shifts, frame_len=frame_len, name=f"shift{wi}"))
        total += cout
    return Plan(canvas_elems=total * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=rows_in,
                output_off=(total - cout) * pitch, output_c=cout, waves=ws)


@pytest.mark.parametrize("group", [128, 16])
def test_token_shift_plan_general_path(group):
    plan = shifted_plan(120, group=group)
    x = synth.random_input(plan, 24, dist="normal")
    check(plan, run_gpu(plan, x, PATH_FMA, expect_path=PATH_FMA), O.run_plan(plan, x))
    if group < 128:     # shifted runs of a small group: run table + funnel-shifted fetches on the mma.sync kernel
        check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), O.run_plan(plan, x))


@pytest.mark.parametrize("group,frames,frame_len", [(32, 2, 96), (64, 8, 40), (16, 3, 256)])
def test_token_shift_small_groups_and_odd_frames_on_the_general_tensor_path(group, frames, frame_len):
    plan = shifted_plan(150 + group, runs=8, run_len=16, frames=frames, frame_len=frame_len, cout=192, group=group)
    x = synth.random_input(plan, 27, dist="normal")
    want = O.run_plan(plan, x)
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), want)
    check(plan, run_gpu(plan, x, PATH_FMA, expect_path=PATH_FMA), want)



@pytest.mark.parametrize("n_tile,frames,frame_len,run_len", [(64, 3, 256, 16), (128, 2, 256, 16), (64, 4, 64, 32), (128, 3, 128, 64), (64, 1, 192, 16),
                                                             (256, 2, 256, 16), (256, 1, 512, 32)])
def test_token_shift_runs_on_tensor_cores(n_tile, frames, frame_len, run_len, monkeypatch):
    """Shifted runs (one table entry per run, shift in its top bits) execute on the tensor-core kernel whose aligner
    warps shift the rows on their way into the operand stage; frame starts read zero."""
    monkeypatch.setenv("K44B_N_TILE", str(n_tile))
    plan = shifted_plan(131 + n_tile + frame_len, runs=128 // run_len, run_len=run_len, frames=frames, frame_len=frame_len, cout=384)
    x = synth.random_input(plan, 25, dist="normal")
    want = O.run_plan(plan, x)
    check(plan, run_gpu(plan, x, PATH_UMMA, expect_path=PATH_UMMA), want)
    check(plan, run_gpu(plan, x, PATH_FMA, expect_path=PATH_FMA), want)


def test_token_shift_tensor_path_with_bias_residual_and_many_tiles():
    """More tiles than SMs (persistent walk over several items per CTA), bias, residual, a partial last neuron tile."""
    plan = shifted_plan(171, rows_in=512, runs=16, run_len=16, frames=4, frame_len=512, cout=1280 + 64, group=1280 + 64, waves=2, act=ACT_SILU)
    rng = np.random.default_rng(9)
    for w in plan.waves:
        w.bias = synth.f16_bits(rng.normal(0, 0.1, w.cout))
    w1 = plan.waves[1]
    w1.has_residual, w1.res_off = True, plan.waves[0].y_off
    x = synth.random_input(plan, 27, dist="normal")
    want = O.run_plan(plan, x)
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_UMMA), want)


@pytest.mark.parametrize("frames,frame_len,run_len,runs,cout,group,chunk", [(2, 256, 16, 8, 384, 128, 0), (1, 1024, 16, 32, 256, 128, 0), (3, 128, 32, 4, 208, 208, 0),
                                                                           (4, 512, 16, 32, 1280 + 64, 1280 + 64, 0), (2, 2048, 64, 8, 2560, 128, 3)])
def test_token_shift_with_the_weight_tile_in_tensor_memory(frames, frame_len, run_len, runs, cout, group, chunk, monkeypatch):
    """Fan-in up to 512: a work item is one neuron tile times a run of column tiles, its weights are copied shared memory ->
    tensor memory once (tcgen05.cp) and every MMA reads A from there. Cases: one and several items per CTA, fan-in 128 .. 512,
    a partial last neuron tile, a last run of column tiles shorter than the others, bias and residual."""
    monkeypatch.setenv("K44B_SHIFT_WS", "2")
    if chunk:
        monkeypatch.setenv("K44B_WS_CHUNK", str(chunk))      # 20 neuron tiles x 11 runs of column tiles: more work items than SMs
    plan = shifted_plan(900 + frame_len + run_len, rows_in=512, runs=runs, run_len=run_len, frames=frames, frame_len=frame_len, cout=cout, group=group, waves=2, act=ACT_SILU)
    rng = np.random.default_rng(19)
    for w in plan.waves:
        w.bias = synth.f16_bits(rng.normal(0, 0.1, w.cout))
    w1 = plan.waves[1]
    w1.has_residual, w1.res_off = True, plan.waves[0].y_off
    x = synth.random_input(plan, 29, dist="normal")
    want = O.run_plan(plan, x)
    npn = NativePlan.from_plan(plan, device=0)
    for i in range(npn.num_waves):
        info = npn.wave_info(i)
        assert info.path == PATH_UMMA and info.n_tile == 128 and info.weights_in_tmem > 0, (info.path, info.n_tile, info.weights_in_tmem)
    npn.close()
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_UMMA), want)
    monkeypatch.setenv("K44B_SHIFT_WS", "0")           # and the kernel that streams the weights through shared memory
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_UMMA), want)


def test_token_shift_frames_that_split_a_tile_fall_back():
    plan = shifted_plan(133, runs=8, run_len=16, frames=2, frame_len=96, cout=256)
    x = synth.random_input(plan, 25, dist="normal")
    check(plan, run_gpu(plan, x, PATH_UMMA, expect_path=PATH_MMA), O.run_plan(plan, x))


def test_token_shift_short_runs_fall_back():
    plan = shifted_plan(140, runs=16, run_len=8)
    x = synth.random_input(plan, 26, dist="normal")
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), O.run_plan(plan, x))


def test_independent_small_waves_share_a_launch():
    """q/k/v-style waves (same input rows, disjoint output rows) run as one grouped launch; a wave that reads one
    of them starts a new launch. Results are unchanged."""
    import torch
    rng = np.random.default_rng(150)
    pitch, d_in = 64, 512
    dims = [("q", 512, 0), ("k", 128, 0), ("v", 128, 0), ("o", 512, 1)]      # (name, rows, source tensor: 0 = x, 1 = q)
    rows0 = {"x": 0, "q": d_in, "k": d_in + 512, "v": d_in + 640, "o": d_in + 768}
    waves = []
    for name, cout, src in dims:
        src_row = rows0["x"] if src == 0 else rows0["q"]
        offs = ((src_row + np.arange(d_in)) * pitch).astype(np.uint32)
        waves.append(Wave(cout=cout, group=128, fan_in=d_in, idx=np.tile(offs, (cout // 128, 1)),
                          weights=synth.f16_bits(rng.normal(0, 0.05, (cout, d_in))), bias=synth.f16_bits(rng.normal(0, 0.1, cout)),
                          y_off=rows0[name] * pitch, act=ACT_NONE, name=name))
    total = d_in + 768 + 512
    plan = Plan(canvas_elems=total * pitch, pitch=pitch, columns=64, input_off=0, input_c=d_in, output_off=rows0["o"] * pitch,
                output_c=512, waves=waves)
    x = synth.random_input(plan, 27)
    want = O.run_plan(plan, x)
    npn = NativePlan.from_plan(plan, force_path=PATH_UMMA)
    canvas = npn.canvas_tensor()
    xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    canvas[: xt.numel()] = xt
    before = npn.launch_count
    npn.execute()
    assert npn.status() == 0
    assert npn.launch_count - before == 2            # {q, k, v} and {o}
    check(plan, canvas.cpu().numpy().view(np.uint16), want)
    npn.close()



@pytest.mark.parametrize("group", [16, 32, 64])
@pytest.mark.parametrize("act", [ACT_RELU, ACT_GELU])
def test_small_groups_on_the_general_tensor_path(group, act):
    """Groups of 16 / 32 / 64 neurons with their own gather lists (runs and scattered rows): too small for a tcgen05 tile,
    so the wave runs on the mma.sync kernel; the FP32-FMA kernel must agree with it."""
    plan = synth.sparse_plan(seed=500 + group, input_rows=2048, waves=2, cout=192, runs=12, run_len=16, columns=100, group=group, act=act)
    rng = np.random.default_rng(group)
    w1 = plan.waves[1]
    w1.idx = (rng.integers(0, 2048 + 192, size=w1.idx.shape) * plan.pitch).astype(np.uint32)      # scattered single rows
    x = synth.random_input(plan, 51, dist="normal")
    want = O.run_plan(plan, x)
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), want)
    check(plan, run_gpu(plan, x, PATH_FMA, expect_path=PATH_FMA), want)


def test_general_tensor_path_with_row_map_residual_and_partial_block():
    plan = synth.dense_chain(seed=61, dims=[96, 80, 80], columns=64, act=ACT_SILU, weight_std=0.1, residual_from={2: 1}, group=16)
    plan.waves[1].cout_map = np.random.default_rng(6).permutation(plan.waves[1].cout).astype(np.uint16)
    for w in plan.waves:                                   # distinct lists per group: rotate the synapse order
        w.idx = np.stack([np.roll(w.idx[g], g) for g in range(w.idx.shape[0])])
        w.weights = np.stack([np.roll(w.weights[j], j // w.group) for j in range(w.cout)])
        w.fan_in_raw = w.fan_in                            # the zero-weight padding slots moved with the roll
    x = synth.random_input(plan, 52, dist="normal")
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), O.run_plan(plan, x))


@pytest.mark.parametrize("rows_mode", [2, 1])
@pytest.mark.parametrize("columns,n_tile,cout", [(64, 64, 160 * 128), (256, 128, 80 * 128), (200, 256, 160 * 128), (512, 256, 75 * 128 + 64)])
def test_scattered_single_rows_on_the_streaming_tensor_kernel(columns, n_tile, cout, rows_mode, monkeypatch):
    """Gather tables the way the reference's benchmark draws them — one sorted random row per synapse, no runs — on waves with
    more 128-neuron tiles than SMs: the streaming tcgen05 kernel fetches the rows itself, four per gather-mode tensor copy
    (mode 2) or one by one with row-fetching warps (mode 1, the default). Tile widths 64 / 128 / 256, a partial last neuron
    tile, valid columns that do not fill the last tile, a second wave that gathers rows the first one wrote; the FP32-FMA
    kernel reads the same table as the cross-check."""
    monkeypatch.setenv("K44B_N_TILE", str(n_tile))
    monkeypatch.setenv("K44B_ROWS_MODE", str(rows_mode))
    plan = synth.scattered_rows_plan(seed=500 + n_tile + columns, input_rows=3000, waves=2, cout=cout, fan_in=160, columns=columns, group=cout if cout % 128 else 128,
                                     act=ACT_SILU)
    x = synth.random_input(plan, 501, dist="normal")
    want = O.run_plan(plan, x)
    import torch
    npn = NativePlan.from_plan(plan, device=0, force_path=PATH_AUTO)
    for i in range(npn.num_waves):
        info = npn.wave_info(i)
        assert info.path == PATH_UMMA and info.box_rows == 1 and info.n_tile == n_tile, (info.path, info.box_rows, info.n_tile)
    canvas = npn.canvas_tensor()
    canvas[plan.input_off: plan.input_off + x.size] = torch.from_numpy(np.ascontiguousarray(x).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    npn.execute()
    assert npn.status() == 0
    check(plan, canvas.cpu().numpy().view(np.uint16), want)
    npn.close()
    check(plan, run_gpu(plan, x, PATH_FMA, expect_path=PATH_FMA), want)


def test_scattered_rows_in_a_small_wave_stay_on_the_general_tensor_path():
    plan = synth.scattered_rows_plan(seed=601, input_rows=2000, waves=2, cout=1024, fan_in=128, columns=128, group=128)
    x = synth.random_input(plan, 602)
    check(plan, run_gpu(plan, x, PATH_AUTO, expect_path=PATH_MMA), O.run_plan(plan, x))


@pytest.mark.parametrize("mode", ["cta_pairs", "one_cta"])
@pytest.mark.parametrize("case", ["runs_groups_of_256", "scattered_rows_groups_of_512", "one_group_partial_last_block"])
def test_tiles_of_256_neurons_share_one_operand(case, mode, monkeypatch):
    """Waves with 256-column tiles whose neuron groups span an even number of 128-neuron blocks, with enough tiles to fill the
    GPU, run tiles of 256 neurons: two blocks with their own weights and accumulators on one gathered operand — by default on a
    pair of CTAs (M = 256 MMAs, each CTA staging half of the operand's columns), on request on one CTA. Run-structured and
    scattered-row gathers, bias, residual, GELU, a partial last 128-neuron block, a second wave reading the first."""
    import torch
    if mode == "one_cta":
        monkeypatch.setenv("K44B_PAIR", "0")
        monkeypatch.setenv("K44B_M_BLOCKS", "2")
    else:
        monkeypatch.setenv("K44B_PAIR", "1")
    if case == "runs_groups_of_256":
        plan = synth.sparse_plan(seed=701, input_rows=4096, waves=2, cout=2 * 128 * 74, runs=4, run_len=32, columns=512, group=256, act=ACT_GELU)
        plan.waves[1].has_residual, plan.waves[1].res_off = True, plan.waves[0].y_off
    elif case == "scattered_rows_groups_of_512":
        plan = synth.scattered_rows_plan(seed=702, input_rows=5000, waves=2, cout=512 * 37, fan_in=160, columns=512, group=512, act=ACT_SILU)
    else:
        cout = 2 * 128 * 148 - 64
        plan = synth.sparse_plan(seed=703, input_rows=2048, waves=1, cout=cout, runs=2, run_len=64, columns=200, group=cout, act=ACT_RELU)
    x = synth.random_input(plan, 704, dist="normal")
    want = O.run_plan(plan, x)
    npn = NativePlan.from_plan(plan, device=0)
    for i in range(npn.num_waves):
        info = npn.wave_info(i)
        assert info.path == PATH_UMMA and info.n_tile == 256 and info.m_blocks == 2, (info.path, info.n_tile, info.m_blocks)
        assert info.cta_pairs == (1 if mode == "cta_pairs" else 0)
    canvas = npn.canvas_tensor()
    canvas[plan.input_off: plan.input_off + x.size] = torch.from_numpy(np.ascontiguousarray(x).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    npn.execute()
    assert npn.status() == 0
    check(plan, canvas.cpu().numpy().view(np.uint16), want)
    npn.close()


def test_pipelined_host_io_gives_the_same_rows_as_blocking_calls():
    """k44b_infer_f16_begin / k44b_infer_f16_next: three different inputs in a row, each upload started while the inference before
    it runs; every output must equal what one blocking k44b_infer_f16 call returns for the same input, and the misuse cases
    (nothing staged, staging occupied) are refused."""
    import torch
    plan = synth.sparse_plan(seed=910, input_rows=2048, waves=2, cout=384, runs=8, run_len=32, columns=64, group=128, act=ACT_RELU)
    npn = NativePlan.from_plan(plan, device=0)
    in_elems, out_elems = plan.input_c * plan.pitch, plan.output_c * plan.pitch
    xs = [torch.from_numpy(synth.random_input(plan, 920 + i, dist="normal").view(np.int16).reshape(-1).copy()).pin_memory() for i in range(3)]
    outs = [torch.zeros(out_elems, dtype=torch.int16).pin_memory() for _ in range(3)]
    want = []
    for x in xs:
        o = torch.zeros(out_elems, dtype=torch.int16).pin_memory()
        npn.infer_f16(x.data_ptr(), o.data_ptr())
        want.append(o.clone())
        assert xs[0].numel() == in_elems
    with pytest.raises(native.NativeError, match="no staged input"):
        npn.infer_f16_next(0, outs[0].data_ptr())
    npn.infer_f16_begin(xs[0].data_ptr())
    with pytest.raises(native.NativeError, match="not been consumed"):
        npn.infer_f16_begin(xs[1].data_ptr())
    npn.infer_f16_next(xs[1].data_ptr(), outs[0].data_ptr())
    npn.infer_f16_next(xs[2].data_ptr(), outs[1].data_ptr())
    npn.infer_f16_next(0, outs[2].data_ptr())
    for got, w in zip(outs, want):
        assert torch.equal(got, w)
    assert not torch.equal(want[0], want[1])
    npn.close()
