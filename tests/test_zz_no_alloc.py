"""The allocation-free wave entry point (k44b_wave_forward_static) against the regular plan path.

Some users of this library cannot let it allocate device memory — their HBM belongs to a framework arena or
a fixed budget, or they sit in a latency-critical loop where cudaMalloc's device-wide synchronisation is not
acceptable. They pass device pointers they own and the kernel's split-K scratch comes from a fixed array in
the library image. This test drives that entry point through the C ABI with buffers allocated by the test
(torch tensors standing in for the caller's arena), twice in a row, and compares both results with what the
regular plan-based entry point (k44b_execute_wave) writes for the same wave, within the parity tolerance
(the split-K sums meet through FP32 atomics, so runs agree to rounding, not bit for bit).

Collected last on purpose: a failure here cannot hide the result of any other test in a run that stops at
the first failure. It does not depend on state left by other tests and passes in a fresh process.
"""
import ctypes

import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import native, synth
from snntome_b200._lib import get_lib
from snntome_b200.native import PATH_UMMA, NativePlan
from snntome_b200.plan import ACT_SILU

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-3


def pack_tiled(w_bits: np.ndarray) -> np.ndarray:
    """Row-major [cout][fan_in] FP16 bits -> the packed order documented in include/k44b.h, on the host."""
    cout, fan_in = w_bits.shape
    mt, ks = (cout + 127) // 128, (fan_in + 63) // 64
    padded = np.zeros((mt * 128, ks * 64), dtype=np.uint16)
    padded[:cout, :fan_in] = w_bits
    v = padded.reshape(mt, 128, ks, 8, 8)                  # [m_tile][row][k_stage][chunk][8 halves]
    out = np.zeros((mt, ks, 128, 8, 8), dtype=np.uint16)   # [m_tile][k_stage][row][chunk position][8 halves]
    for r in range(128):
        for c in range(8):
            out[:, :, r, c ^ (r & 7), :] = v[:, r, :, c, :]
    return out.reshape(-1)


def call_static(lib, canvas, plan, wave, d_w, d_rows, rows_per_box, d_bias, group, k_splits):
    import torch
    err = ctypes.create_string_buffer(512)
    rc = lib.k44b_wave_forward_static(
        ctypes.c_void_p(canvas.data_ptr()), canvas.numel(), plan.pitch, ctypes.c_void_p(d_w.data_ptr()),
        ctypes.c_void_p(d_rows.data_ptr()), rows_per_box, ctypes.c_void_p(d_bias.data_ptr()) if d_bias is not None else None,
        wave.cout, group, wave.fan_in, int(wave.act), wave.y_off, k_splits,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, 512)
    return rc, err.value.decode()


def test_static_scratch_wave_matches_plan_path_twice():
    import torch
    lib = get_lib()
    plan = synth.dense_chain(seed=301, dims=[1024, 384], columns=128, act=ACT_SILU, weight_std=0.04)
    wave = plan.waves[0]
    x = synth.random_input(plan, 302)
    xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)

    # regular entry point
    npn = NativePlan.from_plan(plan, force_path=PATH_UMMA)
    ref_canvas = npn.canvas_tensor()
    ref_canvas[: xt.numel()] = xt
    npn.execute_wave(0)
    assert npn.status() == 0
    want = ref_canvas.cpu().numpy().view(np.uint16)
    a, b = wave.y_off, wave.y_off + wave.cout * plan.pitch
    ok, err, k = O.compare(want[a:b], O.run_plan(plan, x)[a:b], RTOL, ATOL)
    assert ok, ("plan path vs oracle", err, k)

    # the caller's own buffers
    rows_per_box, rows = native.analyze_gather(wave, plan.pitch, plan.canvas_elems)
    assert rows_per_box == 64
    d_rows = torch.from_numpy(rows.astype(np.int32)).cuda()
    d_w = torch.from_numpy(pack_tiled(wave.weights).view(np.int16)).cuda()
    d_bias = torch.from_numpy(wave.bias.view(np.int16)).cuda()
    canvas = torch.zeros(plan.canvas_elems, dtype=torch.float16, device="cuda")
    canvas[: xt.numel()] = xt
    for call in range(2):
        canvas[a:b] = 0
        rc, msg = call_static(lib, canvas, plan, wave, d_w, d_rows, rows_per_box, d_bias, wave.cout, k_splits=4)
        assert rc == 0, msg
        got = canvas.cpu().numpy().view(np.uint16)
        ok, err, k = O.compare(got[a:b], want[a:b], RTOL, ATOL)
        assert ok, (f"call {call}", err, k)
        assert np.array_equal(got[:a], want[:a])          # inputs untouched
    npn.close()


def test_static_scratch_rejects_oversize_wave():
    import torch
    lib = get_lib()
    dummy = torch.zeros(4096, dtype=torch.float16, device="cuda")
    err = ctypes.create_string_buffer(512)
    # 65 tiles of 128 neurons x 64 columns exceed the 64 the fixed array holds
    cout, pitch = 65 * 128, 64
    rc = lib.k44b_wave_forward_static(ctypes.c_void_p(dummy.data_ptr()), (cout + 64) * pitch, pitch, ctypes.c_void_p(dummy.data_ptr()),
                                      ctypes.c_void_p(dummy.data_ptr()), 64, None, cout, cout, 64, 0, 64 * pitch, 1, None, err, 512)
    assert rc == -1
    assert "K44B_STATIC_MAX_TILES" in err.value.decode() and "64" in err.value.decode()
