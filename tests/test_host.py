"""CPU-only checks of the shipped library's host logic against the oracle: the C ABI surface, FP16 and
hash helpers, the graph -> wave compiler, the `.tcff` writer / loader and the gather analysis. No
compute call is made (there is no CPU path to call)."""
import ctypes
import json
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import native, synth
from snntome_b200._lib import PROTOTYPES, get_lib, last_error
from snntome_b200.plan import ACT_RELU, ACT_SILU, Plan, Wave
from snntome_b200.wavec import WaveError, WaveGraph

ROOT = Path(__file__).resolve().parents[1]

# The 26 entry points the reference's ctypes binding resolves at import time (wavec/wavec.py:28-132).
REFERENCE_BINDING_SYMBOLS = """wavec_create wavec_destroy wavec_gpu_release wavec_add_input wavec_add_flatten wavec_add_conv2d
wavec_add_linear_f32 wavec_add_linear_f16 wavec_add_maxpool wavec_add_upsample2x wavec_add_rmsnorm wavec_add_swiglu
wavec_add_rope_gqa_attn wavec_add_split wavec_add_slice wavec_add_concat wavec_set_output wavec_set_reuse_canvas
wavec_set_batch_size wavec_set_target_preset wavec_compile wavec_get_summary_json wavec_save_tcff wavec_load_tcff_weights
wavec_gpu_init_plan wavec_gpu_infer_f32""".split()


def test_library_exports_every_declared_symbol():
    lib = get_lib()
    declared = set()
    for hdr in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", hdr.read_text(), flags=re.S)
        declared |= set(re.findall(r"\b((?:wavec|k44b)_[a-z0-9_]+)\s*\(", text))
    assert len(declared) >= 50
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(PROTOTYPES), declared ^ set(PROTOTYPES)
    for name in REFERENCE_BINDING_SYMBOLS:
        assert hasattr(lib, name)
    assert len(REFERENCE_BINDING_SYMBOLS) == 26


def test_null_handles_fail_cleanly():
    lib = get_lib()
    assert lib.wavec_compile(None) == -1
    assert lib.wavec_gpu_init_plan(None) == -1
    assert lib.wavec_gpu_infer_f32(None, None, 0, None, 0, None) == -1
    assert lib.wavec_get_summary_json(None) == b"{}"
    assert lib.k44b_execute(None, None) == -1
    lib.wavec_destroy(None)


def test_f16_and_hash_helpers_match_oracle():
    lib = get_lib()
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.normal(0, 1, 50000), rng.normal(0, 1e-6, 50000), rng.uniform(-70000, 70000, 20000),
                        [0.0, -0.0, np.inf, -np.inf, 65504, 65520, 2.0 ** -24, 2.0 ** -25, 3e-8]]).astype(np.float32)
    h = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    x = np.concatenate([x, ((h[:-1] + h[1:]) / 2).astype(np.float32)])
    got = np.empty(x.size, dtype=np.uint16)
    lib.k44b_f32_to_f16(x.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), got.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), x.size)
    assert np.array_equal(got, O.f32_to_f16(x))
    data = rng.integers(0, 256, 5000, dtype=np.uint8)
    assert lib.k44b_fnv1a64(data.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)), data.size) == O.fnv1a64_py(data.tobytes())
    assert lib.k44b_fnv1a64(None, 0) == 0xCBF29CE484222325


@pytest.mark.parametrize("cout,B", [(16, 64), (48, 96), (256, 512)])
def test_container_weight_order_matches_oracle(cout, B):
    lib = get_lib()
    w = np.random.default_rng(cout).integers(0, 65536, (cout, B), dtype=np.uint16)
    enc = np.empty(cout * B, dtype=np.uint16)
    u16p = ctypes.POINTER(ctypes.c_uint16)
    lib.k44b_rowmajor_to_wmma(w.ctypes.data_as(u16p), enc.ctypes.data_as(u16p), cout, B)
    assert np.array_equal(enc, O.rowmajor_to_wmma(w))
    dec = np.empty((cout, B), dtype=np.uint16)
    lib.k44b_wmma_to_rowmajor(enc.ctypes.data_as(u16p), dec.ctypes.data_as(u16p), cout, B)
    assert np.array_equal(dec, w)


def _mlp_graph(dims, columns, acts, residual=None, seed=0, weights=True, default_S=0):
    rng = np.random.default_rng(seed)
    g = WaveGraph(batch_size=columns, default_S=default_S)
    g.add_input("x", dims[0], 1, 1, is_1d=True)
    prev, arrays = "x", []
    for i in range(1, len(dims)):
        w = rng.normal(0, 0.05, (dims[i], dims[i - 1])).astype(np.float32) if weights else np.zeros((dims[i], dims[i - 1]), np.float32)
        b = rng.normal(0, 0.1, dims[i]).astype(np.float32) if weights else None
        res = residual.get(i) if residual else None
        g.add_linear(f"fc{i}", prev, f"t{i}", dims[i - 1], dims[i], w, b, act=acts[i - 1], res_blob=res)
        arrays.append((w, b))
        prev = f"t{i}"
    g.set_output(prev)
    return g, arrays


def _plan_from_summary(summary, arrays, columns):
    """Rebuild the compiled plan independently in Python from the summary's offsets."""
    pitch = (columns + 63) // 64 * 64
    waves = []
    for cmd, (w, b) in zip(summary["cmds"], arrays):
        cout, B, cin, log = cmd["Cout"], cmd["B"], cmd["Cin"], cmd["logical_Cout"]
        wt = np.zeros((cout, B), np.float32)
        wt[:log, :cin] = w
        bias = np.zeros(cout, np.float32)
        if b is not None:
            bias[:log] = b
        offs = np.zeros(B, np.uint32)
        offs[:cin] = cmd["src_off"] + np.arange(cin) * pitch
        waves.append(Wave(cout=cout, group=cmd["S"], fan_in=B, idx=np.tile(offs, (cout // cmd["S"], 1)),
                          weights=O.f32_to_f16(wt), bias=O.f32_to_f16(bias), y_off=cmd["y_off"],
                          act={"NONE": 0, "RELU": 1, "SIGMOID": 2, "SILU": 3, "LEAKY_RELU": 4, "GELU": 5}[cmd["act"]],
                          logical_cout=log, fan_in_raw=cmd["B_raw"], cin=cin, src_off=cmd["src_off"],
                          has_residual=cmd["has_residual"], name=cmd["name"], h_out=cmd["h_out"], w_out=cmd["w_out"]))
    return Plan(canvas_elems=summary["canvas_elems"], pitch=pitch, columns=columns, input_off=0, input_c=summary["input_shape"][0],
                output_off=waves[-1].y_off, output_c=summary["output_shape"][0], waves=waves)


def test_graph_compile_rules():
    g, _ = _mlp_graph([100, 200, 40], 32, ["relu", None])
    s = g.compile().summary
    assert s["batch_size"] == 32 and s["num_waves"] == 2 and s["input_shape"] == [100, 1, 32] and s["output_shape"] == [40, 1, 32]
    c0, c1 = s["cmds"]
    # fan-in padded to a multiple of 32 (min 64), rows to a multiple of 16, group size by divisibility
    assert (c0["B"], c0["B_raw"], c0["Cout"], c0["logical_Cout"], c0["S"]) == (128, 100, 208, 200, 16)
    assert (c1["B"], c1["B_raw"], c1["Cout"], c1["logical_Cout"], c1["S"]) == (224, 200, 48, 40, 16)
    # rows are 64 elements apart (32 columns padded to one 64-wide tile); regions are placed back to back
    assert c0["src_off"] == 0 and c0["y_off"] == 100 * 64 and c1["src_off"] == c0["y_off"] and c1["y_off"] == (100 + 208) * 64
    assert s["canvas_elems"] == (100 + 208 + 48) * 64 and s["canvas_bytes"] == 2 * s["canvas_elems"]
    assert abs(s["total_gflops"] - 2 * (100 * 200 + 200 * 40) * 32 / 1e9) < 1e-12
    assert s["target_profile"] == "b200" and s["target_num_cus"] == 148


def test_group_size_selection():
    for cout, want in [(1024, 128), (128, 128), (192, 64), (96, 32), (80, 16)]:
        g, _ = _mlp_graph([64, cout], 8, [None])
        assert g.compile().summary["cmds"][0]["S"] == want
    g, _ = _mlp_graph([64, 1024], 8, [None], default_S=32)
    assert g.compile().summary["cmds"][0]["S"] == 32


def test_canvas_reuses_dead_tensors():
    g, _ = _mlp_graph([64, 128, 128, 128, 64], 64, [None] * 4)
    s = g.compile().summary
    offs = [c["y_off"] for c in s["cmds"]]
    # x stays live (allocation 0 is never retired); t1 dies after fc2, so fc3's output reuses its rows
    assert offs[0] == 64 * 64 and offs[1] == offs[0] + 128 * 64 and offs[2] == offs[0]
    assert s["canvas_elems"] < (64 + 128 * 3 + 64) * 64


def test_unsupported_nodes_are_refused():
    g = WaveGraph()
    with pytest.raises(WaveError, match="multiple of 4"):
        g.add_input("img", 3, 32, 30)                 # image widths come in whole 4-pixel quads
    g.add_input("x", 64, 1, 1, is_1d=True)
    with pytest.raises(WaveError, match="already has its input"):
        g.add_input("img", 3, 32, 32)
    with pytest.raises(WaveError, match="2-D image input"):
        g.add_maxpool("p", "x", "y")                  # image nodes need an image graph
    with pytest.raises(WaveError, match="head_dim"):
        g.add_rope_gqa_attn("a", "x", "x", "x", "y", 2, 1, 32)
    with pytest.raises(WaveError):
        g.add_conv2d("c", "x", "y", 64, 64, 3, 3, np.zeros((64, 64, 3, 3)), pad=1)
    with pytest.raises(WaveError):
        g.add_linear("fc", "nope", "y", 64, 64, np.zeros((64, 64), np.float32))
        g.compile()


def test_tcff_bytes_match_oracle_writer(tmp_path):
    g, arrays = _mlp_graph([96, 256, 64], 40, ["silu", "relu"], residual=None, seed=4)
    plan = g.compile()
    path = tmp_path / "m.tcff"
    assert plan.save_tcff(path, "Unit") == 2
    got = path.read_bytes()
    want = O.tcff_write(_plan_from_summary(plan.summary, arrays, 40), prefix="Unit")
    assert len(got) == len(want)
    assert got == want
    parsed = O.tcff_read(got)
    assert parsed["canvas_bytes"] == plan.canvas_bytes and parsed["flags"] == 1


def test_tcff_load_roundtrip_and_batch_rule(tmp_path):
    g, _ = _mlp_graph([64, 128, 32], 1, ["relu", None], seed=5)
    plan = g.compile()
    a = tmp_path / "a.tcff"
    plan.save_tcff(a)
    g2, _ = _mlp_graph([64, 128, 32], 1, ["relu", None], weights=False)
    plan2 = g2.compile()
    b0 = tmp_path / "b0.tcff"
    plan2.save_tcff(b0)
    assert b0.read_bytes() != a.read_bytes()
    plan2.load_tcff_weights(a)
    b1 = tmp_path / "b1.tcff"
    plan2.save_tcff(b1)
    assert b1.read_bytes() == a.read_bytes()


def test_tcff_corruption_is_reported(tmp_path):
    g, _ = _mlp_graph([64, 64], 1, [None], seed=6)
    plan = g.compile()
    good = tmp_path / "g.tcff"
    plan.save_tcff(good)
    blob = bytearray(good.read_bytes())
    cases = {"magic": (9, "magic"), "master": (21, "master header hash"), "payload": (300, "hash mismatch")}
    for name, (pos, msg) in cases.items():
        bad = bytearray(blob)
        bad[pos] ^= 0x40
        p = tmp_path / f"{name}.tcff"
        p.write_bytes(bytes(bad))
        with pytest.raises(WaveError, match=msg):
            plan.load_tcff_weights(p)
    p = tmp_path / "short.tcff"
    p.write_bytes(bytes(blob[:100]))
    with pytest.raises(WaveError, match="shorter"):
        plan.load_tcff_weights(p)
    bad = bytearray(blob)
    bad[4:8] = (len(blob) + 10).to_bytes(4, "little")
    p = tmp_path / "ifd.tcff"
    p.write_bytes(bytes(bad))
    with pytest.raises(WaveError, match="IFD"):
        plan.load_tcff_weights(p)
    with pytest.raises(WaveError, match="cannot open"):
        plan.load_tcff_weights(tmp_path / "missing.tcff")
    # the process is still alive and the plan still usable
    plan.load_tcff_weights(good)


def test_gather_analysis_finds_runs():
    plan = synth.config0()
    w = plan.waves[0]
    h, rows = native.analyze_gather(w, plan.pitch, plan.canvas_elems)
    assert h == 16
    starts = synth.run_starts(1234, 0, w.cout // w.group, 16, 16, 4096)
    assert np.array_equal(rows.reshape(starts.shape), starts.astype(np.uint32))
    # dense chain: one long run, fetched as 64-row boxes; fan-in 96 pads the last stage with null boxes
    dplan = synth.dense_chain(seed=1, dims=[96, 128], columns=64)
    h, rows = native.analyze_gather(dplan.waves[0], dplan.pitch, dplan.canvas_elems)
    assert h == 32 and list(rows) == [0, 32, 64, 0]
    # consecutive rows in different order are not a run
    w2 = dplan.waves[0]
    w2.idx[:, :8] = w2.idx[:, :8][:, ::-1].copy()
    h, rows = native.analyze_gather(w2, dplan.pitch, dplan.canvas_elems)
    # ... the table then holds one row per synapse (padded to whole 64-synapse stages with row 0)
    assert h == 1 and list(rows[:10]) == [7, 6, 5, 4, 3, 2, 1, 0, 8, 9] and rows.size == 128 and list(rows[96:]) == [0] * 32
    # element offsets that are not row aligned (token shift) select the general path
    w3 = synth.dense_chain(seed=1, dims=[128, 128], columns=64).waves[0]
    w3.idx += 3
    h, _ = native.analyze_gather(w3, 64, 1 << 20)
    assert h == 0 and "shift" in last_error()
    # groups of 16 neurons cannot share a 128-row tensor-core tile
    p16 = synth.config0(group=16)
    h, _ = native.analyze_gather(p16.waves[0], p16.pitch, p16.canvas_elems)
    assert h == 0 and "128" in last_error()


def test_gpu_calls_fail_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("device present")
    g, _ = _mlp_graph([64, 64], 1, [None])
    plan = g.compile()
    with pytest.raises(WaveError, match="no CUDA device"):
        plan.init_gpu()
    with pytest.raises(native.NativeError, match="no CUDA device"):
        native.NativePlan.create(1024, 64, 64)
