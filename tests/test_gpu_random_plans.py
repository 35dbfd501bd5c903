"""GPU parity on seeded random plans: group size, run length (down to scattered single rows), fan-in tails, column
counts, activations, bias, residuals, row maps and token shifts are drawn per case; the executor picks its own kernel
for every wave (tcgen05, tcgen05 with aligners, small-wave clusters, mma.sync) and must match the CPU oracle within
rtol 2e-3 / atol 1e-3. The FP32-FMA kernel runs the same plans as a second witness."""
import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import synth
from snntome_b200.native import PATH_AUTO, PATH_FMA
from snntome_b200.plan import ACT_GELU, ACT_LEAKY_RELU, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU

from test_gpu_parity import check, check_per_wave, run_gpu

pytestmark = pytest.mark.gpu
ACTS = [ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, ACT_LEAKY_RELU, ACT_GELU]


def draw_plan(seed: int):
    rng = np.random.default_rng(9000 + seed)
    group = int(rng.choice([16, 32, 64, 128, 256]))
    cout = group * int(rng.integers(1, 4 if group >= 128 else 7))
    run_len = int(rng.choice([1, 8, 16, 32, 64]))
    fan_in = int(rng.choice([64, 96, 128, 160, 256, 320]))
    while fan_in % run_len:
        fan_in += 32
    columns = int(rng.choice([1, 7, 33, 64, 100, 128, 200]))
    waves = int(rng.integers(2, 4))
    plan = synth.sparse_plan(seed=seed, input_rows=int(rng.choice([512, 1024])), waves=waves, cout=cout, runs=fan_in // run_len,
                             run_len=run_len, columns=columns, group=group, act=int(rng.choice(ACTS)),
                             bias_scale=0.05 if rng.random() < 0.7 else 0.0)
    notes = [f"group {group}", f"cout {cout}", f"run_len {run_len}", f"fan_in {fan_in}", f"columns {columns}", f"waves {waves}"]
    for wi, w in enumerate(plan.waves):
        w.act = int(rng.choice(ACTS))
        if wi > 0 and rng.random() < 0.4:                          # residual: the previous wave's rows
            w.has_residual, w.res_off = True, plan.waves[wi - 1].y_off
            notes.append(f"residual@{wi}")
        if rng.random() < 0.25:
            w.cout_map = rng.permutation(cout).astype(np.uint16)
            notes.append(f"row map@{wi}")
        if run_len >= 8 and rng.random() < 0.35:                   # token shifts per run, causal zero padding per frame
            frames = [f for f in (plan.pitch, plan.pitch // 2, 64, 32, 24) if f and plan.pitch % f == 0]
            w.frame_len = int(rng.choice(frames))
            per_run = rng.integers(0, 8, size=(cout // group, fan_in // run_len)).astype(np.uint8)
            w.shifts = np.repeat(per_run, run_len, axis=1)
            notes.append(f"shifts@{wi} frame {w.frame_len}")
    return plan, ", ".join(notes)


@pytest.mark.parametrize("seed", range(60))
def test_random_plan_matches_the_oracle(seed):
    plan, notes = draw_plan(seed)
    x = synth.random_input(plan, 300 + seed, dist="normal")
    want = O.run_plan(plan, x)
    try:
        check(plan, run_gpu(plan, x, PATH_AUTO), want)
        if seed % 3 == 0:
            check(plan, run_gpu(plan, x, PATH_FMA), want)
    except AssertionError as e:
        raise AssertionError(f"{notes}: {e}") from None


@pytest.mark.parametrize("seed", range(16))
def test_random_token_shift_plan_on_the_kernel_with_weights_in_tensor_memory(seed, monkeypatch):
    """Seeded token-shift plans forced onto the kernel that keeps a work item's weight tile in tensor memory: neuron count
    (partial last tile included), group size, run length 16 / 32 / 64, fan-in 64 .. 512 (odd numbers of 64-synapse steps
    included), frames of 128 .. 1024 tokens, activation, bias, residual, and the number of column tiles per work item."""
    from snntome_b200.native import NativePlan, PATH_UMMA
    from test_gpu_parity import shifted_plan
    rng = np.random.default_rng(7000 + seed)
    run_len = int(rng.choice([16, 32, 64]))
    fan_in = int(rng.choice([64, 128, 192, 256, 320, 448, 512]))
    while fan_in % run_len:
        fan_in += 64
    fan_in = min(fan_in, 512)
    frame_len = int(rng.choice([128, 256, 384, 512, 1024]))
    frames = int(rng.integers(1, 4))
    group = int(rng.choice([128, 256]))
    cout = group * int(rng.integers(1, 5))
    if rng.random() < 0.4:
        cout_single = cout + int(rng.choice([16, 48, 80]))           # one group with a partial last 128-neuron tile
        cout = group = cout_single
    monkeypatch.setenv("K44B_SHIFT_WS", "2")
    monkeypatch.setenv("K44B_WS_CHUNK", str(int(rng.integers(1, 6))))
    monkeypatch.setenv("K44B_WS_GROUPS", str(int(rng.integers(1, 3))))
    plan = shifted_plan(8000 + seed, rows_in=int(rng.choice([256, 512])), runs=fan_in // run_len, run_len=run_len, frames=frames, frame_len=frame_len,
                        cout=cout, group=group, waves=2, act=int(rng.choice(ACTS)))
    for w in plan.waves:
        if rng.random() < 0.6:
            w.bias = synth.f16_bits(rng.normal(0, 0.1, w.cout))
    if rng.random() < 0.5:
        plan.waves[1].has_residual, plan.waves[1].res_off = True, plan.waves[0].y_off
    notes = f"cout {cout}, group {group}, fan-in {fan_in}, run_len {run_len}, {frames} x {frame_len} tokens"
    x = synth.random_input(plan, 400 + seed, dist="normal")
    want = O.run_plan(plan, x)
    npn = NativePlan.from_plan(plan, device=0)
    try:
        assert all(npn.wave_info(i).path == PATH_UMMA and npn.wave_info(i).weights_in_tmem > 0 for i in range(npn.num_waves)), notes
    finally:
        npn.close()
    try:
        check(plan, run_gpu(plan, x, PATH_AUTO), want)
    except AssertionError as e:
        raise AssertionError(f"{notes}: {e}") from None


@pytest.mark.parametrize("seed", range(10))
def test_random_plan_on_cta_pairs(seed):
    """Seeded plans large enough for tiles of 256 neurons x 256 columns on CTA pairs (cta_group::2): group size 256 / 512 /
    all neurons, run length 8 .. 64, fan-in 128 .. 512, 512 .. 1024 columns of which the last tile may be partly valid,
    activation, bias, a second wave that adds the first as residual."""
    from snntome_b200.native import NativePlan, PATH_UMMA
    rng = np.random.default_rng(7500 + seed)
    run_len = int(rng.choice([8, 16, 32, 64]))
    fan_in = int(rng.choice([128, 192, 256, 384, 512]))
    columns = int(rng.choice([512, 768, 1024]))
    blocks = -(-148 // (columns // 256)) + int(rng.integers(0, 6))          # 256-neuron blocks: at least one pair tile per SM
    group = int(rng.choice([256, 512]))
    blocks += (-blocks) % (group // 256)
    cout = 256 * blocks
    if rng.random() < 0.3:
        group = cout
    valid = columns - int(rng.choice([0, 0, 40, 63]))                      # the row pitch stays a whole number of 256-column tiles
    plan = synth.sparse_plan(seed=600 + seed, input_rows=4096, waves=2, cout=cout, runs=fan_in // run_len, run_len=run_len, columns=valid, group=group,
                             act=int(rng.choice(ACTS)), bias_scale=0.05 if rng.random() < 0.6 else 0.0)
    assert plan.pitch == columns
    if rng.random() < 0.5:
        plan.waves[1].has_residual, plan.waves[1].res_off = True, plan.waves[0].y_off
    notes = f"cout {cout}, group {group}, fan-in {fan_in}, run_len {run_len}, columns {valid} of {plan.pitch}"
    x = synth.random_input(plan, 500 + seed, dist="normal")
    npn = NativePlan.from_plan(plan, device=0)
    try:
        for i in range(npn.num_waves):
            info = npn.wave_info(i)
            assert info.path == PATH_UMMA and info.n_tile == 256 and info.cta_pairs == 1, (notes, info.path, info.n_tile, info.cta_pairs)
    finally:
        npn.close()
    try:
        check_per_wave(plan, run_gpu(plan, x, PATH_AUTO))
    except AssertionError as e:
        raise AssertionError(f"{notes}: {e}") from None


@pytest.mark.parametrize("seed", range(8))
def test_random_scattered_rows_plan_on_the_streaming_kernel(seed):
    """Seeded plans whose gather lists are single sorted random rows (the reference benchmark's generator), large enough for the
    streaming tcgen05 kernel with row-fetching warps: tile widths 64 / 128 / 256 by column count, groups of 128 / 256 / 512,
    fan-in 64 .. 320 (tails of a 64-synapse step included), bias, activation; every wave checked on what the device gathered."""
    from snntome_b200.native import NativePlan, PATH_UMMA
    rng = np.random.default_rng(7700 + seed)
    columns = int(rng.choice([64, 128, 256, 512]))
    group = int(rng.choice([128, 256, 512]))
    tiles_per_block = max(1, columns // 64)
    cout = group * max(1, -(-160 // (tiles_per_block * (group // 128))) + int(rng.integers(0, 3)))
    fan_in = int(rng.choice([64, 96, 160, 256, 320]))
    valid = columns - int(rng.choice([0, 0, 17]))
    plan = synth.scattered_rows_plan(seed=900 + seed, input_rows=int(rng.choice([3000, 8192])), waves=2, cout=cout, fan_in=fan_in, columns=valid, group=group,
                                     act=int(rng.choice(ACTS)))
    for w in plan.waves:
        if rng.random() < 0.5:
            w.bias = synth.f16_bits(rng.normal(0, 0.1, w.cout))
    notes = f"cout {cout}, group {group}, fan-in {fan_in}, columns {valid} of {plan.pitch}"
    x = synth.random_input(plan, 600 + seed, dist="normal")
    npn = NativePlan.from_plan(plan, device=0)
    try:
        for i in range(npn.num_waves):
            info = npn.wave_info(i)
            assert info.path == PATH_UMMA and info.box_rows == 1, (notes, info.path, info.box_rows)
    finally:
        npn.close()
    try:
        check_per_wave(plan, run_gpu(plan, x, PATH_AUTO))
    except AssertionError as e:
        raise AssertionError(f"{notes}: {e}") from None


@pytest.mark.parametrize("seed", range(8))
def test_random_token_shift_plan_with_weights_through_shared_memory(seed, monkeypatch):
    """Seeded token-shift plans on the aligner kernel that streams its weights through shared memory (the one that serves fan-in
    above 512): fan-in 128 .. 1024, tile widths 64 / 128 / 256, run lengths 16 / 32 / 64, bias, residual."""
    from snntome_b200.native import NativePlan, PATH_UMMA
    from test_gpu_parity import shifted_plan
    rng = np.random.default_rng(7900 + seed)
    run_len = int(rng.choice([16, 32, 64]))
    fan_in = int(rng.choice([128, 256, 576, 640, 768, 1024]))
    while fan_in % run_len:
        fan_in += 64
    n_tile = int(rng.choice([64, 128, 256]))
    frame_len = n_tile * int(rng.integers(1, 4))
    frames = int(rng.integers(1, 3))
    group = int(rng.choice([128, 256]))
    cout = group * int(rng.integers(1, 4))
    monkeypatch.setenv("K44B_SHIFT_WS", "0")
    monkeypatch.setenv("K44B_N_TILE", str(n_tile))
    plan = shifted_plan(8100 + seed, rows_in=1024, runs=fan_in // run_len, run_len=run_len, frames=frames, frame_len=frame_len, cout=cout, group=group,
                        waves=2, act=int(rng.choice(ACTS)))
    for w in plan.waves:
        if rng.random() < 0.6:
            w.bias = synth.f16_bits(rng.normal(0, 0.1, w.cout))
    if rng.random() < 0.5:
        plan.waves[1].has_residual, plan.waves[1].res_off = True, plan.waves[0].y_off
    notes = f"cout {cout}, group {group}, fan-in {fan_in}, run_len {run_len}, {frames} x {frame_len} tokens, tile {n_tile}"
    x = synth.random_input(plan, 700 + seed, dist="normal")
    npn = NativePlan.from_plan(plan, device=0)
    try:
        for i in range(npn.num_waves):
            info = npn.wave_info(i)
            assert info.path == PATH_UMMA and info.weights_in_tmem == 0 and info.n_tile == n_tile, (notes, info.path, info.weights_in_tmem, info.n_tile)
    finally:
        npn.close()
    try:
        check_per_wave(plan, run_gpu(plan, x, PATH_AUTO))
    except AssertionError as e:
        raise AssertionError(f"{notes}: {e}") from None
