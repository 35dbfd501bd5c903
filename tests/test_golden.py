"""Golden fixtures (tests/golden): known answers of the published pieces (FNV-1a-64, IEEE binary16, the 16x16-tile
vector index), and frozen oracle outputs of small plans — checked against the oracle on the CPU and against the CUDA
path, through the C ABI, on the GPU."""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import pytest

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "golden"))

import cases  # noqa: E402
from oracle import oracle as O  # noqa: E402

KAT = json.loads((HERE / "golden" / "kat.json").read_text())
RTOL, ATOL = 2e-3, 1e-3


def fp16_key(u):
    u = u.astype(np.int32)
    return np.where(u & 0x8000, 0x8000 - (u & 0x7fff), 0x8000 + u)


def test_fnv1a64_known_answers():
    for text, want in KAT["fnv1a64"].items():
        assert f"{O.fnv1a64(text.encode()):016x}" == want
        assert f"{O.fnv1a64_py(text.encode()):016x}" == want


def test_binary16_known_answers():
    vals = np.array([float(k) for k in KAT["f32_to_f16"]], dtype=np.float32)
    want = np.array([int(v, 16) for v in KAT["f32_to_f16"].values()], dtype=np.uint16)
    assert np.array_equal(O.f32_to_f16(vals), want)
    with np.errstate(over="ignore"):
        assert np.array_equal(vals.astype(np.float16).view(np.uint16), want)


def test_tile_order_known_answers():
    for e in KAT["wmma_vec_index"]:
        B, cout = e["B"], 48
        w = np.arange(cout * B, dtype=np.uint16).reshape(cout, B)              # element value = row-major position
        tiled = O.rowmajor_to_wmma(w).reshape(-1, 8)
        assert tiled[e["index"], 0] == e["j"] * B + e["k8"] * 8


def test_library_helpers_match_known_answers():
    import ctypes
    from snntome_b200._lib import get_lib
    lib = get_lib()
    for text, want in KAT["fnv1a64"].items():
        b = (ctypes.c_uint8 * max(1, len(text)))(*text.encode())
        assert f"{lib.k44b_fnv1a64(b, len(text)):016x}" == want
    vals = np.array([float(k) for k in KAT["f32_to_f16"]], dtype=np.float32)
    out = np.zeros(vals.size, dtype=np.uint16)
    lib.k44b_f32_to_f16(vals.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), vals.size)
    assert [f"{v:04x}" for v in out] == list(KAT["f32_to_f16"].values())


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_oracle_reproduces_golden(name):
    plan, x = cases.build(name)
    meta = KAT["cases"][name]
    assert hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest() == meta["input_sha256"], "seeded input changed"
    assert hashlib.sha256(b"".join(np.ascontiguousarray(w.weights).tobytes() for w in plan.waves)).hexdigest() == meta["weights_sha256"]
    want = np.load(HERE / "golden" / f"{name}.npz")["out"]
    got = cases.output_rows(plan, O.run_plan(plan, x))
    exact = all(w.act in (0, 1, 4) for w in plan.waves)
    d = np.abs(fp16_key(got) - fp16_key(want)).max()
    assert d <= (0 if exact else 1), f"{name}: oracle differs from the fixture by {d} ulp"   # 1 ulp: libm's exp / erf may differ between hosts


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(cases.CASES))
@pytest.mark.parametrize("path", ["auto", "fma"])
def test_cuda_path_matches_golden(name, path):
    import torch
    from snntome_b200.native import PATH_AUTO, PATH_FMA, NativePlan
    plan, x = cases.build(name)
    want = np.load(HERE / "golden" / f"{name}.npz")["out"]
    npn = NativePlan.from_plan(plan, device=0, force_path=PATH_AUTO if path == "auto" else PATH_FMA)
    canvas = npn.canvas_tensor()
    xt = torch.from_numpy(np.ascontiguousarray(x).view(np.int16).reshape(-1)).cuda().view(torch.float16)
    canvas[plan.input_off: plan.input_off + xt.numel()] = xt
    npn.execute()
    assert npn.status() == 0
    got = cases.output_rows(plan, canvas.cpu().numpy().view(np.uint16))
    npn.close()
    ok, err, k = O.compare(got, want, RTOL, ATOL)
    assert ok, f"{name} ({path}): max abs err {err} at element {k}"
