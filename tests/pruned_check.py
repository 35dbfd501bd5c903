"""Shared by the one-GPU and the two-GPU test of the cluster-pruned 8B wave chain (BASELINE configs[4]) at its full size:
walks the chain wave by wave and, for sampled waves and neuron groups, lets the oracle recompute the group's rows from what the
device itself holds — the rows the group gathers (read back from the canvas right after the wave ran, while they are still
intact), the group's weights (unpacked from the device's packed copy) and the residual rows."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import oracle as O
from snntome_b200.plan import Plan, Wave

RTOL, ATOL = 2e-3, 1e-3


def sampled_waves(num_waves: int):
    """q, o (+residual), gate (SiLU), down (+residual) of the first layer, two waves from the middle, the last down, the lm_head."""
    layers = (num_waves - 1) // 7
    picks = {0, 3, 4, 6, 7 * (layers // 2) + 5, 7 * (layers // 2) + 1, 7 * (layers - 1) + 6, num_waves - 1}
    return sorted(p for p in picks if 0 <= p < num_waves)


def check_wave(plan, info, wi: int, canvas, groups_per_wave: int = 3, seed: int = 0):
    """Compare `groups_per_wave` sampled groups of this rank's rows of wave `wi` with the oracle. Returns the largest absolute error."""
    import torch
    pitch = info["pitch"]
    starts, run_len, row0, res_row0, act = info["tables"][wi]
    cv2 = canvas.view(-1, pitch)
    wrm = plan.weights_rowmajor(wi)                                      # device [rows of this rank, fan_in] int16
    fan_in = starts.shape[1] * run_len
    rng = np.random.default_rng(1000 + wi + seed)
    worst = 0.0
    for g in rng.choice(starts.shape[0], size=min(groups_per_wave, starts.shape[0]), replace=False):
        rows = (torch.from_numpy(starts[g].astype(np.int64))[:, None] + torch.arange(run_len)[None, :]).reshape(-1).cuda()
        x = cv2[rows].cpu().numpy().view(np.uint16)                      # [fan_in, pitch]: the gathered rows as the device saw them
        wg = wrm[g * 128:(g + 1) * 128].cpu().numpy().view(np.uint16)
        got = cv2[row0 + g * 128: row0 + (g + 1) * 128].cpu().numpy().view(np.uint16)
        # a one-wave plan over a private canvas: [gathered rows | residual rows | output rows]
        has_res = res_row0 is not None
        res = cv2[res_row0 + g * 128: res_row0 + (g + 1) * 128].cpu().numpy().view(np.uint16) if has_res else np.zeros((0, pitch), np.uint16)
        idx = (np.arange(fan_in, dtype=np.uint32) * pitch)[None, :]
        y_off = (fan_in + res.shape[0]) * pitch
        wave = Wave(cout=128, group=128, fan_in=fan_in, idx=idx, weights=wg, bias=None, y_off=y_off, act=act,
                    has_residual=has_res, res_off=fan_in * pitch if has_res else 0)
        small = Plan(canvas_elems=y_off + 128 * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=fan_in + res.shape[0],
                     output_off=y_off, output_c=128, waves=[wave])
        want = O.run_plan(small, np.concatenate([x, res], axis=0))[y_off:]
        ok, err, k = O.compare(got.reshape(-1), want, RTOL, ATOL)
        assert ok, f"wave {wi} group {int(g)}: max abs err {err} at row {k // pitch}, column {k % pitch}"
        worst = max(worst, float(err))
    return worst
