"""Catalogue of the golden cases: small seeded plans covering the epilogue variants and gather forms of the hot path.

The reference ships no golden vectors for this path (its licence also forbids running it), so the fixtures beside this
file are outputs of the CPU oracle, accepted only where the oracle's C++ implementation and its independent numpy
float64 restatement agree (see make_golden.py). They freeze the behaviour the CUDA path is compared with.
"""
import numpy as np

from snntome_b200 import synth
from snntome_b200.plan import (ACT_GELU, ACT_LEAKY_RELU, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, Plan, Wave, expand_runs)


def _shifted(seed, *, rows_in, cout, runs, run_len, frames, frame_len, group, act, waves):
    rng = np.random.default_rng(seed)
    pitch = frames * frame_len
    fan_in = runs * run_len
    ws, total = [], rows_in
    for wi in range(waves):
        groups = cout // group
        starts = synth.run_starts(seed, wi, groups, runs, run_len, total)
        idx = expand_runs(starts, run_len, pitch)
        shifts = np.repeat(rng.integers(0, 8, size=(groups, runs)).astype(np.uint8), run_len, axis=1)
        w = synth.f16_bits(rng.normal(0, (1.0 / fan_in) ** 0.5, (cout, fan_in)))
        ws.append(Wave(cout=cout, group=group, fan_in=fan_in, idx=idx, weights=w, bias=None, y_off=total * pitch, act=act,
                       shifts=shifts, frame_len=frame_len, name=f"shift{wi}"))
        total += cout
    return Plan(canvas_elems=total * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=rows_in,
                output_off=(total - cout) * pitch, output_c=cout, waves=ws)


def _residual_map():
    plan = synth.dense_chain(seed=41, dims=[128, 128, 128], columns=64, act=ACT_RELU, weight_std=0.1, residual_from={2: 1})
    plan.waves[1].cout_map = np.random.default_rng(5).permutation(plan.waves[1].cout).astype(np.uint16)
    return plan


def _residual_plain():
    return synth.dense_chain(seed=43, dims=[128, 128, 128], columns=64, act=ACT_SILU, weight_std=0.1, residual_from={2: 1})


# name -> (plan builder, input seed, input distribution)
CASES = {
    "sparse_runs16_relu": (lambda: synth.sparse_plan(seed=301, input_rows=512, waves=2, cout=128, runs=8, run_len=16, columns=64,
                                                     group=128, act=ACT_RELU), 1, "uniform"),
    "sparse_group16_none": (lambda: synth.sparse_plan(seed=302, input_rows=256, waves=1, cout=64, runs=4, run_len=16, columns=48,
                                                      group=16, act=ACT_NONE), 2, "normal"),
    "sparse_runs64_two_tiles": (lambda: synth.sparse_plan(seed=303, input_rows=1024, waves=1, cout=128, runs=2, run_len=64, columns=128,
                                                          group=128, act=ACT_LEAKY_RELU), 3, "normal"),
    "dense_sigmoid": (lambda: synth.dense_chain(seed=304, dims=[96, 80, 48], columns=64, act=ACT_SIGMOID, weight_std=0.1), 4, "uniform"),
    "dense_gelu": (lambda: synth.dense_chain(seed=305, dims=[192, 128, 64], columns=64, act=ACT_GELU, weight_std=0.08), 5, "normal"),
    "residual_with_row_map": (_residual_map, 6, "normal"),
    "residual_after_activation": (_residual_plain, 7, "normal"),
    "token_shift_two_frames": (lambda: _shifted(306, rows_in=128, cout=128, runs=4, run_len=16, frames=2, frame_len=64, group=128,
                                                act=ACT_GELU, waves=2), 8, "normal"),
}


def build(name):
    maker, seed, dist = CASES[name]
    plan = maker()
    return plan, synth.random_input(plan, seed, dist=dist)


def output_rows(plan, canvas):
    """The rows every wave wrote, concatenated in wave order (uint16 FP16 bit patterns)."""
    return np.concatenate([canvas[w.y_off: w.y_off + w.cout * plan.pitch] for w in plan.waves])
