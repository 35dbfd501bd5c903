"""Seeded synthetic connectome plans (host side, numpy).

Integer choices (run starts, pruning masks, sampled groups) come from a stateless 64-bit mixer so
that a host and a device generator can agree bit for bit; floating inputs of the small plans are
drawn once on the host with numpy and stored as FP16. The reference's own generator sorts each
index row and uses per-synapse indices (whitepaper/sparse_wmma_kernel/tests/benchmark_common.cuh:
81-111); the plans here instead draw *runs* of consecutive substrate rows per neuron group, which is
the connectivity the benchmark configurations describe.
"""
from __future__ import annotations

import numpy as np

from .plan import ACT_NONE, ACT_RELU, Plan, Wave, expand_runs

_M64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


def splitmix64(x: np.ndarray) -> np.ndarray:
    """Vectorised splitmix64 finaliser on uint64 arrays."""
    x = np.asarray(x, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = x + np.uint64(_GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def mix(seed: int, tag: int, counter: np.ndarray) -> np.ndarray:
    """h = splitmix64(seed ^ tag*GOLDEN ^ counter)."""
    base = np.uint64((int(seed) ^ ((int(tag) * _GOLDEN) & _M64)) & _M64)
    return splitmix64(np.asarray(counter, dtype=np.uint64) ^ base)


def uniform_int(seed: int, tag: int, counter: np.ndarray, n: int) -> np.ndarray:
    """Integers in [0, n): (h >> 11) mod n."""
    return (mix(seed, tag, counter) >> np.uint64(11)) % np.uint64(n)


def f16_bits(a: np.ndarray) -> np.ndarray:
    return np.asarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def run_starts(seed: int, wave: int, groups: int, runs: int, run_len: int, rows_available: int) -> np.ndarray:
    """Run start rows [groups, runs]: uniform over run_len-aligned rows of [0, rows_available),
    with replacement; a run never straddles the end."""
    slots = rows_available // run_len
    ctr = np.arange(groups * runs, dtype=np.uint64)
    s = uniform_int(seed, 1000 + wave, ctr, slots).astype(np.int64) * run_len
    return s.reshape(groups, runs)


def sparse_plan(*, seed: int, input_rows: int, waves: int, cout: int, runs: int, run_len: int,
                columns: int, group: int = 128, act: int = ACT_RELU, bias_scale: float = 0.01,
                weight_std: float | None = None, name: str = "synthetic") -> Plan:
    """Layered sparse plan: wave w gathers `runs` runs of `run_len` rows from the input rows and the
    rows of all earlier waves. Rows are laid out [input | wave0 | wave1 | ...]."""
    pitch = (columns + 63) // 64 * 64
    fan_in = runs * run_len
    assert fan_in % 32 == 0 and fan_in >= 64, "fan-in must already satisfy the padding rule"
    assert cout % group == 0 and cout % 16 == 0
    total_rows = input_rows + waves * cout
    rng = np.random.default_rng(seed)
    std = weight_std if weight_std is not None else (1.0 / fan_in) ** 0.5
    ws = []
    for w in range(waves):
        rows_avail = input_rows + w * cout
        starts = run_starts(seed, w, cout // group, runs, run_len, rows_avail)
        idx = expand_runs(starts, run_len, pitch)
        wt = f16_bits(rng.normal(0.0, std, size=(cout, fan_in)))
        bias = f16_bits(bias_scale * rng.normal(0.0, 1.0, size=cout)) if bias_scale else None
        ws.append(Wave(cout=cout, group=group, fan_in=fan_in, idx=idx, weights=wt, bias=bias,
                       y_off=rows_avail * pitch, act=act, cin=rows_avail, src_off=0,
                       name=f"wave{w}", w_out=columns))
    return Plan(canvas_elems=total_rows * pitch, pitch=pitch, columns=columns, input_off=0,
                input_c=input_rows, output_off=(input_rows + (waves - 1) * cout) * pitch,
                output_c=cout, waves=ws, name=name)


def scattered_rows_plan(*, seed: int, input_rows: int, waves: int, cout: int, fan_in: int, columns: int, group: int = 128,
                        act: int = ACT_RELU, bias_scale: float = 0.01, chained: bool = True) -> Plan:
    """The reference benchmark's kind of gather table (whitepaper/sparse_wmma_kernel/tests/benchmark_common.cuh:81-111): every
    neuron group draws `fan_in` single rows uniformly (with replacement) and sorts them — no runs. With `chained` a wave
    may also draw rows of the waves before it (so that the waves depend on each other); otherwise all waves read the input
    rows only, like the benchmark's independent waves over one substrate."""
    pitch = (columns + 63) // 64 * 64
    assert fan_in % 32 == 0 and fan_in >= 64 and cout % group == 0 and cout % 16 == 0
    rng = np.random.default_rng(seed)
    ws = []
    for w in range(waves):
        rows_avail = input_rows + (w * cout if chained else 0)
        groups = cout // group
        rows = uniform_int(seed, 3000 + w, np.arange(groups * fan_in, dtype=np.uint64), rows_avail).astype(np.int64).reshape(groups, fan_in)
        rows.sort(axis=1)
        wt = f16_bits(rng.normal(0.0, (1.0 / fan_in) ** 0.5, size=(cout, fan_in)))
        bias = f16_bits(bias_scale * rng.normal(0.0, 1.0, size=cout)) if bias_scale else None
        ws.append(Wave(cout=cout, group=group, fan_in=fan_in, idx=(rows * pitch).astype(np.uint32), weights=wt, bias=bias,
                       y_off=(input_rows + w * cout) * pitch, act=act, cin=rows_avail, src_off=0, name=f"scattered{w}", w_out=columns))
    total_rows = input_rows + waves * cout
    return Plan(canvas_elems=total_rows * pitch, pitch=pitch, columns=columns, input_off=0, input_c=input_rows,
                output_off=(input_rows + (waves - 1) * cout) * pitch, output_c=cout, waves=ws, name="scattered_rows")


def config0(seed: int = 1234, group: int = 128) -> Plan:
    """Tiny connectome: 4096 input rows, 2 waves x 1024 neurons, fan-in 256 = 16 runs of 16 rows,
    ReLU, 32 columns."""
    return sparse_plan(seed=seed, input_rows=4096, waves=2, cout=1024, runs=16, run_len=16,
                       columns=32, group=group, act=ACT_RELU, bias_scale=0.01, name="config0")


def config2_scaled(seed: int = 99, *, input_rows: int = 65536, cout: int = 2048, waves: int = 2,
                   columns: int = 64) -> Plan:
    """Same connectivity rule as the ultra-sparse plan (fan-in 4096 = 64 runs of 64 rows, group 128,
    ReLU, no bias) at a size the CPU oracle finishes in seconds."""
    return sparse_plan(seed=seed, input_rows=input_rows, waves=waves, cout=cout, runs=64, run_len=64,
                       columns=columns, group=128, act=ACT_RELU, bias_scale=0.0, name="config2_scaled")


def dense_chain(seed: int, dims: list[int], columns: int, act: int = ACT_NONE, group: int = 0,
                weight_std: float = 0.02, residual_from: dict[int, int] | None = None) -> Plan:
    """A chain of dense linears expressed as waves: every neuron gathers all rows of the previous
    tensor (one run covering the full input width). `dims` = [d_in, d1, d2, ...]."""
    from .plan import choose_group_size, round_up_cout, round_up_fan_in
    pitch = (columns + 63) // 64 * 64
    rng = np.random.default_rng(seed)
    row0 = [0]
    pads = [dims[0]]
    for d in dims[1:]:
        row0.append(row0[-1] + pads[-1])
        pads.append(round_up_cout(d))
    ws = []
    for li in range(1, len(dims)):
        d_in, d_out = dims[li - 1], dims[li]
        cout = pads[li]
        fan_in = round_up_fan_in(d_in)
        g = group or choose_group_size(cout, pitch // 64)
        offs = np.zeros(fan_in, dtype=np.uint32)
        offs[:d_in] = (row0[li - 1] + np.arange(d_in)) * pitch
        idx = np.tile(offs, (cout // g, 1))
        wt = np.zeros((cout, fan_in), dtype=np.float32)
        wt[:d_out, :d_in] = rng.normal(0.0, weight_std, size=(d_out, d_in))
        bias = np.zeros(cout, dtype=np.float32)
        bias[:d_out] = 0.01 * rng.normal(size=d_out)
        res = residual_from.get(li) if residual_from else None
        ws.append(Wave(cout=cout, group=g, fan_in=fan_in, idx=idx, weights=f16_bits(wt), bias=f16_bits(bias),
                       y_off=row0[li] * pitch, act=act, logical_cout=d_out, fan_in_raw=d_in, cin=d_in,
                       src_off=row0[li - 1] * pitch, has_residual=res is not None,
                       res_off=(row0[res] * pitch if res is not None else 0), name=f"linear{li}", w_out=columns))
    total_rows = row0[-1] + pads[-1]
    return Plan(canvas_elems=(total_rows * pitch + 127) // 128 * 128, pitch=pitch, columns=columns,
                input_off=0, input_c=dims[0], output_off=row0[-1] * pitch, output_c=dims[-1], waves=ws,
                name="dense_chain")


def token_shift_plan(seed: int, *, rows_in: int = 256, cout: int = 256, runs: int = 8, run_len: int = 16, frames: int = 2,
                     frame_len: int = 256, group: int = 128, act: int = ACT_NONE, waves: int = 2, max_shift: int = 7) -> Plan:
    """Receptive-field token-shift plan: `frames` sequences of `frame_len` tokens side by side in every row; every run of
    `run_len` rows is read 0..max_shift tokens earlier, with zero padding at the start of each frame."""
    rng = np.random.default_rng(seed)
    pitch = frames * frame_len
    fan_in = runs * run_len
    ws, total = [], rows_in
    for wi in range(waves):
        groups = cout // group
        starts = run_starts(seed, wi, groups, runs, run_len, total)
        idx = expand_runs(starts, run_len, pitch)
        sh_run = rng.integers(0, max_shift + 1, size=(groups, runs)).astype(np.uint8)
        shifts = np.repeat(sh_run, run_len, axis=1)
        wt = f16_bits(rng.normal(0, (1.0 / fan_in) ** 0.5, (cout, fan_in)))
        ws.append(Wave(cout=cout, group=group, fan_in=fan_in, idx=idx, weights=wt, bias=None, y_off=total * pitch, act=act,
                       shifts=shifts, frame_len=frame_len, name=f"shift{wi}"))
        total += cout
    return Plan(canvas_elems=total * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=rows_in,
                output_off=(total - cout) * pitch, output_c=cout, waves=ws, name="token_shift")


def random_input(plan: Plan, seed: int, dist: str = "uniform") -> np.ndarray:
    """FP16 bit patterns for the input rows, [input_c, pitch]; columns >= plan.columns are zero."""
    rng = np.random.default_rng(seed)
    x = np.zeros((plan.input_c, plan.pitch), dtype=np.float32)
    if dist == "uniform":
        x[:, :plan.columns] = rng.uniform(-1.0, 1.0, size=(plan.input_c, plan.columns))
    else:
        x[:, :plan.columns] = rng.normal(0.0, 1.0, size=(plan.input_c, plan.columns))
    return f16_bits(x)
