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


@pytest.mark.parametrize("case", ["direct_epilogue", "groups_of_128", "partial_last_tile_no_bias"])
def test_static_scratch_other_shapes_and_no_allocation(case):
    """More shapes through the allocation-free entry point, each against the oracle: one CTA per tile with the epilogue written
    straight from tensor memory (k_splits = 1), three groups of 128 neurons with their own run lists, and a wave whose last
    128-neuron tile is partly empty (208 rows) with no bias. The second call of each case also checks the property the entry
    point exists for: the device's free memory is the same before and after the call."""
    import torch
    lib = get_lib()
    if case == "direct_epilogue":
        plan = synth.dense_chain(seed=311, dims=[512, 256], columns=64, act=ACT_SILU, weight_std=0.05)
        k_splits, group = 1, None
    elif case == "groups_of_128":
        plan = synth.sparse_plan(seed=312, input_rows=2048, waves=1, cout=384, runs=8, run_len=32, columns=128, group=128)
        k_splits, group = 2, 128
    else:
        plan = synth.dense_chain(seed=313, dims=[320, 208], columns=64, weight_std=0.05)
        k_splits, group = 3, None
    wave = plan.waves[0]
    if case == "partial_last_tile_no_bias":
        wave.bias = None
    x = synth.random_input(plan, 314)
    want = O.run_plan(plan, x)
    rows_per_box, rows = native.analyze_gather(wave, plan.pitch, plan.canvas_elems)
    assert rows_per_box in (8, 16, 32, 64)
    xt = torch.from_numpy(x.view(np.int16).reshape(-1)).cuda().view(torch.float16)
    d_rows = torch.from_numpy(rows.astype(np.int32)).cuda()
    d_w = torch.from_numpy(pack_tiled(wave.weights).view(np.int16)).cuda()
    d_bias = torch.from_numpy(wave.bias.view(np.int16)).cuda() if wave.bias is not None else None
    canvas = torch.zeros(plan.canvas_elems, dtype=torch.float16, device="cuda")
    canvas[plan.input_off: plan.input_off + xt.numel()] = xt
    a, b = wave.y_off, wave.y_off + wave.cout * plan.pitch
    for call in range(2):
        canvas[a:b] = 0
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc, msg = call_static(lib, canvas, plan, wave, d_w, d_rows, rows_per_box, d_bias, group or wave.cout, k_splits=k_splits)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert rc == 0, msg
        if call == 1:       # (the first call on a device may load the kernels' module)
            assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes across the call"
        got = canvas.cpu().numpy().view(np.uint16)
        ok, err, k = O.compare(got[a:b], want[a:b], RTOL, ATOL)
        assert ok, (case, f"call {call}", err, k)


def test_static_scratch_refuses_a_capturing_stream():
    """Every call waits for the stream and reads a status word back, which cannot be recorded into a graph: a call made on a
    stream that is being captured is refused with a message and leaves the capture intact."""
    import torch
    lib = get_lib()
    dummy = torch.zeros(64 * 64 * 4, dtype=torch.float16, device="cuda")
    rows = torch.zeros(8, dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    err = ctypes.create_string_buffer(512)
    with torch.cuda.graph(g, stream=side):
        rc = lib.k44b_wave_forward_static(ctypes.c_void_p(dummy.data_ptr()), dummy.numel(), 64, ctypes.c_void_p(dummy.data_ptr()),
                                          ctypes.c_void_p(rows.data_ptr()), 64, None, 128, 128, 64, 0, 64 * 64, 1,
                                          ctypes.c_void_p(side.cuda_stream), err, 512)
        dummy.add_(0)       # something capturable, so the graph is not empty
    assert rc == -1 and "captur" in err.value.decode()


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
