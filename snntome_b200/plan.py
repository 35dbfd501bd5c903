"""Host-side plan description: the fields of the reference's wave plan that the hot path consumes.

A *plan* is a fixed list of *waves* over one FP16 arena (the "canvas" / activation substrate).
Field meaning follows the reference structs `K44ExecCmd` (wavec/k44_plan_types.hpp:603-650),
`K44WavePlan` (:663-693) and the 1-D branch of `K44ResDesc::init` (:498-516):

* the canvas is addressed in FP16 elements; a tensor with C channels occupies C rows of
  ``pitch`` elements (``channel_stride`` in the reference), ``pitch`` a multiple of 64;
* columns are cut into tiles of 64 (``tile_off_X[t] = tile_off_Y[t] = 64*t`` in 1-D layouts);
* a wave owns ``cout`` output rows starting at element ``y_off``; groups of ``group`` consecutive
  neurons (the reference's "cluster size" S) share one list of ``B`` gather offsets, every neuron
  has its own ``B`` weights and a bias.

Everything is plain numpy so that the same object feeds the CPU oracle, the `.tcff` writer and the
device packer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, ACT_LEAKY_RELU, ACT_GELU = range(6)
ACT_NAMES = ["NONE", "RELU", "SIGMOID", "SILU", "LEAKY_RELU", "GELU"]


def round_up_fan_in(b_raw: int) -> int:
    """Fan-in padding rule (wavec/k44_plan_types.hpp:162-165): multiple of 32, at least 64."""
    return max(64, (int(b_raw) + 31) // 32 * 32)


def round_up_cout(cout: int) -> int:
    """Output-row padding rule (wavec/k44_plan_types.hpp:157-160): multiple of 16, at least 16."""
    return max(16, (int(cout) + 15) // 16 * 16)


def choose_group_size(cout_pad: int, num_tiles: int, force: int = 0) -> int:
    """Neuron-group size selection (wavec/k44_plan_types.hpp:167-186)."""
    if force:
        g = force
        while g >= 16:
            if cout_pad % g == 0:
                return g
            g >>= 1
    if cout_pad % 128 == 0 and (cout_pad >= 640 or num_tiles <= 64):
        return 128
    for g in (64, 32):
        if cout_pad % g == 0:
            return g
    return 16


@dataclass
class Wave:
    """One `K44_WAVE` command."""

    cout: int                      # padded output rows (multiple of 16)
    group: int                     # neurons sharing one gather list
    fan_in: int                    # B, padded synapses per neuron
    idx: np.ndarray                # uint32 [cout // group, fan_in], FP16-element offsets
    weights: np.ndarray            # uint16 [cout, fan_in], FP16 bit patterns, row-major
    bias: Optional[np.ndarray]     # uint16 [cout] or None
    y_off: int                     # canvas element offset of output row 0
    act: int = ACT_NONE
    logical_cout: int = 0
    fan_in_raw: int = 0
    cin: int = 0
    src_off: int = 0               # informational (first input row), stored in the .tcff aux tag
    res_off: int = 0
    has_residual: bool = False
    x_base_off: int = 0            # added to every gather offset (index rebasing above 0x70000000)
    cout_map: Optional[np.ndarray] = None   # uint16 [cout] logical row -> stored row
    name: str = ""
    h_out: int = 1
    w_out: int = 1
    # Receptive-field token shift: synapse s of group g reads its row `shifts[g][s]` columns (tokens) earlier;
    # columns whose position inside their frame of `frame_len` columns is below the shift read zero.
    shifts: Optional[np.ndarray] = None     # uint8 [cout // group, fan_in]
    frame_len: int = 0                      # 0: the whole row is one frame

    def __post_init__(self):
        if not self.logical_cout:
            self.logical_cout = self.cout
        if not self.fan_in_raw:
            self.fan_in_raw = self.fan_in
        self.idx = np.ascontiguousarray(self.idx, dtype=np.uint32).reshape(self.cout // self.group, self.fan_in)
        self.weights = np.ascontiguousarray(self.weights).view(np.uint16).reshape(self.cout, self.fan_in)
        if self.bias is not None:
            self.bias = np.ascontiguousarray(self.bias).view(np.uint16).reshape(self.cout)
        if self.cout_map is not None:
            self.cout_map = np.ascontiguousarray(self.cout_map, dtype=np.uint16).reshape(self.cout)
        if self.shifts is not None:
            self.shifts = np.ascontiguousarray(self.shifts, dtype=np.uint8).reshape(self.cout // self.group, self.fan_in)

    @property
    def synapses(self) -> int:
        return self.logical_cout * self.fan_in_raw


@dataclass
class Plan:
    """A compiled wave plan over a 1-D token layout."""

    canvas_elems: int
    pitch: int                     # channel_stride: elements between consecutive rows
    columns: int                   # valid columns (tokens / batch entries); <= pitch
    input_off: int
    input_c: int
    output_off: int
    output_c: int
    waves: List[Wave] = field(default_factory=list)
    name: str = "K44Model"

    @property
    def num_tiles(self) -> int:
        return self.pitch // 64

    def tile_offsets(self) -> np.ndarray:
        return (np.arange(self.num_tiles, dtype=np.uint32) * 64).astype(np.uint32)

    def flops(self) -> float:
        """2 * synapses * columns, padding not counted."""
        return 2.0 * sum(w.synapses for w in self.waves) * self.columns


def expand_runs(starts: np.ndarray, run_len: int, pitch: int) -> np.ndarray:
    """Expand per-group run starts (row numbers) into per-synapse element offsets.

    ``starts`` is [groups, runs]; the result is [groups, runs*run_len] with entry
    ``(start + r) * pitch`` — consecutive substrate rows are ``pitch`` elements apart.
    """
    starts = np.asarray(starts, dtype=np.int64)
    r = np.arange(run_len, dtype=np.int64)
    rows = starts[:, :, None] + r[None, None, :]
    return (rows.reshape(starts.shape[0], -1) * int(pitch)).astype(np.uint32)
