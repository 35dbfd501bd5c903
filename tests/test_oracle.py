"""Pins the CPU oracle: known-answer vectors, numpy.float16, and a numpy float64 restatement."""
import numpy as np
import pytest

from oracle import oracle as O
from snntome_b200 import synth
from snntome_b200.plan import ACT_GELU, ACT_LEAKY_RELU, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, Plan, Wave

# Published FNV-1a 64-bit test vectors (Fowler/Noll/Vo reference test suite).
FNV_KAT = [
    (b"", 0xCBF29CE484222325),
    (b"a", 0xAF63DC4C8601EC8C),
    (b"b", 0xAF63DF4C8601F1A5),
    (b"foobar", 0x85944171F73967E8),
]


@pytest.mark.parametrize("data,want", FNV_KAT)
def test_fnv1a64_known_answers(data, want):
    assert O.fnv1a64(data) == want
    assert O.fnv1a64_py(data) == want


def test_fnv_c_matches_python_on_random_bytes():
    rng = np.random.default_rng(0)
    for n in (1, 7, 255, 256, 4097):
        b = rng.integers(0, 256, size=n, dtype=np.uint8).tobytes()
        assert O.fnv1a64(b) == O.fnv1a64_py(b)


def test_f16_to_f32_all_bit_patterns():
    bits = np.arange(65536, dtype=np.uint16)
    got = O.f16_to_f32(bits)
    want = bits.view(np.float16).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_f32_to_f16_matches_numpy_rte():
    rng = np.random.default_rng(1)
    pieces = [
        rng.normal(0, 1, 200000), rng.normal(0, 1e-5, 100000), rng.normal(0, 1e-7, 100000),
        rng.uniform(-70000, 70000, 100000), np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9,
        np.inf, -np.inf, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 2.0 ** -14, 2.0 ** -14 * 0.9999]),
    ]
    x = np.concatenate(pieces).astype(np.float32)
    # every half value and every midpoint between neighbouring halves (ties must go to even)
    h = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    mid = ((h[:-1] + h[1:]) / 2).astype(np.float32)
    x = np.concatenate([x, h.astype(np.float32), mid, -mid])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(O.f32_to_f16(x), want)


def test_f64_to_f16_rounds_once():
    """The wave oracle stores its double results with one rounding: equal to numpy's float64 -> float16 everywhere,
    including values a hair off a half-way point of the half grid, where rounding through float32 first goes wrong."""
    rng = np.random.default_rng(5)
    halves = np.arange(0, 0x7bff, dtype=np.uint16).view(np.float16).astype(np.float64)
    mid = (halves[:-1] + halves[1:]) / 2                               # exact half-way points (ties)
    eps = np.abs(mid) * 2.0 ** -40 + 2.0 ** -60                        # far below float32 resolution
    vals = np.concatenate([mid, mid + eps, mid - eps, -mid, -(mid + eps), rng.normal(0, 10, 20000), rng.normal(0, 1e-5, 20000),
                           rng.uniform(-7e4, 7e4, 20000), [0.0, -0.0, 65519.999, 65520.0, -65520.0, 1e300, -1e300, 2.0 ** -25, 2.0 ** -25 * 1.0000001]])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = O.f64_to_f16(vals)
    assert np.array_equal(got, want)
    twice = vals.astype(np.float32).astype(np.float16).view(np.uint16)
    assert (twice != want).any()                                        # the case this guards against exists in the set


def test_f32_to_f16_nan_stays_nan():
    x = np.array([np.nan, -np.nan], dtype=np.float32)
    got = O.f32_to_f16(x)
    assert np.all((got & 0x7C00) == 0x7C00) and np.all((got & 0x3FF) != 0)


@pytest.mark.parametrize("cout,B", [(16, 64), (32, 96), (128, 256), (48, 64)])
def test_wmma_order_roundtrip_and_twin(cout, B):
    rng = np.random.default_rng(cout * 1000 + B)
    w = rng.integers(0, 65536, size=(cout, B), dtype=np.uint16)
    enc = O.rowmajor_to_wmma(w)
    assert np.array_equal(enc, O.rowmajor_to_wmma_numpy(w))
    assert np.array_equal(O.wmma_to_rowmajor(enc, cout, B), w)
    # spot-check the formula: vector (tile, lane) <- neuron (lane & 15), k-half (lane >> 4)
    v = enc.reshape(-1, 8)
    assert np.array_equal(v[0], w[0, 0:8]) and np.array_equal(v[16], w[0, 8:16]) and np.array_equal(v[1], w[1, 0:8])


def _small_plan(act, group, with_res=False, with_map=False, bias=True, seed=5):
    rng = np.random.default_rng(seed)
    pitch, rows_in, cout, B = 64, 96, 32, 64
    idx = (rng.integers(0, rows_in, size=(cout // group, B)) * pitch).astype(np.uint32)
    w = synth.f16_bits(rng.normal(0, 0.2, size=(cout, B)))
    b = synth.f16_bits(rng.normal(0, 0.1, size=cout)) if bias else None
    cmap = rng.permutation(cout).astype(np.uint16) if with_map else None
    y_off = (rows_in + cout) * pitch
    wave = Wave(cout=cout, group=group, fan_in=B, idx=idx, weights=w, bias=b, y_off=y_off, act=act,
                has_residual=with_res, res_off=rows_in * pitch, cout_map=cmap)
    plan = Plan(canvas_elems=(rows_in + 2 * cout) * pitch, pitch=pitch, columns=40, input_off=0,
                input_c=rows_in + cout, output_off=y_off, output_c=cout, waves=[wave])
    return plan


@pytest.mark.parametrize("act", [ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, ACT_LEAKY_RELU, ACT_GELU])
@pytest.mark.parametrize("group", [16, 32])
def test_wave_cpp_matches_numpy_float64(act, group):
    plan = _small_plan(act, group)
    x = synth.random_input(plan, 3)
    a = O.run_plan(plan, x)
    b = O.run_plan(plan, x, use_numpy=True)
    # both round an (almost) exact double sum to FP16: allow 1 ulp for sums that sit on a tie
    ok, err, k = O.compare(a, b, rtol=1e-3, atol=1e-6)
    assert ok, (err, k)
    assert np.mean(a != b) < 1e-3


@pytest.mark.parametrize("with_map", [False, True])
def test_wave_residual_order_rule(with_map):
    """Residual goes in before the activation when a row map is present, after it otherwise."""
    plan = _small_plan(ACT_RELU, 16, with_res=True, with_map=with_map)
    x = synth.random_input(plan, 4, dist="normal")
    a = O.run_plan(plan, x)
    b = O.run_plan(plan, x, use_numpy=True)
    ok, err, k = O.compare(a, b, rtol=1e-3, atol=1e-6)
    assert ok, (err, k)
    out = a[plan.output_off:].view(np.float16)
    if with_map:
        assert out.min() >= 0          # relu applied last
    else:
        assert out.min() < 0           # residual added after relu can be negative


def test_dense_wave_equals_matmul():
    plan = synth.dense_chain(seed=2, dims=[64, 48], columns=64, act=ACT_NONE)
    x = synth.random_input(plan, 9)
    canvas = O.run_plan(plan, x)
    w = plan.waves[0]
    W = w.weights.view(np.float16).astype(np.float64)[:48, :64]
    b = w.bias.view(np.float16).astype(np.float64)[:48]
    X = x.view(np.float16).astype(np.float64)
    want = (W @ X + b[:, None]).astype(np.float32).astype(np.float16)
    got = canvas[plan.output_off: plan.output_off + 48 * 64].view(np.float16).reshape(48, 64)
    assert np.mean(got != want) < 1e-3
    assert np.allclose(got.astype(np.float64), want.astype(np.float64), rtol=1e-3, atol=1e-6)


def test_padding_rows_get_activation_of_zero():
    """Padded output rows carry zero weights and bias but are still written (sigmoid -> 0.5),
    wavec/k44_plan_types.hpp:339 and wavec/k44_wave_compiler.hpp:755-779."""
    plan = synth.dense_chain(seed=2, dims=[64, 40], columns=64, act=ACT_SIGMOID)
    canvas = O.run_plan(plan, synth.random_input(plan, 1))
    w = plan.waves[0]
    assert w.cout == 48 and w.logical_cout == 40
    pad = canvas[w.y_off + 40 * 64: w.y_off + 48 * 64].view(np.float16)
    assert np.all(pad == np.float16(0.5))


def test_out_of_range_index_is_rejected():
    plan = _small_plan(ACT_NONE, 16)
    plan.waves[0].idx[0, 0] = plan.canvas_elems
    with pytest.raises(IndexError):
        O.run_plan(plan, synth.random_input(plan, 1))


def test_stage3_error_band():
    """Sanity band, not parity: FP32 accumulation in 16-synapse chunks + FP16 store differs from the
    exact sum by ~3e-3 mean at B=1024, U(-1,1) data (white_paper_readme.md:115-123)."""
    rng = np.random.default_rng(7)
    B = 1024
    errs = []
    for _ in range(300):
        w = synth.f16_bits(rng.uniform(-1, 1, B))
        x = synth.f16_bits(rng.uniform(-1, 1, B))
        out = np.zeros(1, dtype=np.float32)
        O.lib().k44o_dot_stage3(O._p(w, O.u16p), O._p(x, O.u16p), B, 0.0, O._p(out, O.f32p))
        exact = float(w.view(np.float16).astype(np.float64) @ x.view(np.float16).astype(np.float64))
        errs.append(abs(out[0] - exact))
    assert 5e-4 < np.mean(errs) < 1e-2


def test_tcff_python_roundtrip_and_corruption():
    plan = synth.config0(group=128)
    blob = O.tcff_write(plan)
    assert len(blob) % 256 == 0 and blob[:2] == b"II" and blob[8:16] == b"TCFFv1.0"
    parsed = O.tcff_read(blob)
    assert len(parsed["waves"]) == 2
    for w, pw in zip(plan.waves, parsed["waves"]):
        assert pw["params"][:5] == [w.cin, w.cout, w.fan_in, w.group, 16]
        assert np.array_equal(O.wmma_to_rowmajor(pw["weights_wmma"], w.cout, w.fan_in), w.weights)
        assert np.array_equal(pw["idx"].reshape(w.idx.shape), w.idx)
        assert np.array_equal(pw["bias"], w.bias)
    bad = bytearray(blob)
    bad[300] ^= 1
    with pytest.raises(ValueError):
        O.tcff_read(bytes(bad))
    bad = bytearray(blob)
    bad[20] ^= 1
    with pytest.raises(ValueError):
        O.tcff_read(bytes(bad))


def test_token_shift_oracle_twins_agree_and_pad_causally():
    rng = np.random.default_rng(11)
    pitch, frame, rows_in, cout, B = 128, 64, 40, 16, 64
    idx = (rng.integers(0, rows_in, size=(1, B)) * pitch).astype(np.uint32)
    shifts = rng.integers(0, 8, size=(1, B)).astype(np.uint8)
    w = synth.f16_bits(rng.normal(0, 0.2, size=(cout, B)))
    wave = Wave(cout=cout, group=16, fan_in=B, idx=idx, weights=w, bias=None, y_off=rows_in * pitch, act=ACT_GELU,
                shifts=shifts, frame_len=frame)
    plan = Plan(canvas_elems=(rows_in + cout) * pitch, pitch=pitch, columns=pitch, input_off=0, input_c=rows_in,
                output_off=rows_in * pitch, output_c=cout, waves=[wave])
    x = synth.random_input(plan, 5, dist="normal")
    a = O.run_plan(plan, x)
    b = O.run_plan(plan, x, use_numpy=True)
    ok, err, k = O.compare(a, b, rtol=1e-3, atol=1e-6)
    assert ok, (err, k)
    # direct statement for one output element: column 64 is token 0 of the second frame -> only shift-0 taps contribute
    X = x.view(np.float16).astype(np.float64).reshape(rows_in, pitch)
    W = w.view(np.float16).astype(np.float64)
    rows = idx[0] // pitch
    for col in (64, 66, 3, 127):
        acc = sum(W[5, s] * X[rows[s], col - shifts[0, s]] for s in range(B) if (col % frame) >= shifts[0, s])
        want = np.float16(0.5 * acc * (1 + __import__("math").erf(acc * 0.7071067811865476)))
        got = a[wave.y_off + 5 * pitch + col: wave.y_off + 5 * pitch + col + 1].view(np.float16)[0]
        assert abs(float(got) - float(want)) <= 1e-3 + 2e-3 * abs(float(want))


# ---- element-wise / attention oracle (oracle/valu.py) against independent loops ---------------------------------------
def _f16(a):
    return np.asarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def test_valu_oracle_rmsnorm_swiglu_against_direct_formulas():
    from oracle import valu as V
    rng = np.random.default_rng(1)
    dim, pitch = 48, 16
    canvas = np.zeros(4 * dim * pitch, dtype=np.uint16)
    canvas[: 2 * dim * pitch] = _f16(rng.normal(0, 1, 2 * dim * pitch))
    gamma = _f16(1 + 0.2 * rng.normal(size=dim))
    x = canvas[: dim * pitch].view(np.float16).astype(np.float64).reshape(dim, pitch)
    u = canvas[dim * pitch: 2 * dim * pitch].view(np.float16).astype(np.float64).reshape(dim, pitch)
    V.rmsnorm(canvas, 0, 2 * dim * pitch, dim, pitch, 1e-5, gamma)
    V.swiglu(canvas, 0, dim * pitch, 3 * dim * pitch, dim, pitch)
    g = gamma.view(np.float16).astype(np.float64)
    want_n = np.empty((dim, pitch))
    for t in range(pitch):
        ms = sum(x[c, t] ** 2 for c in range(dim)) / dim
        for c in range(dim):
            want_n[c, t] = x[c, t] / np.sqrt(ms + 1e-5) * g[c]
    got_n = canvas[2 * dim * pitch: 3 * dim * pitch].view(np.float16).astype(np.float64).reshape(dim, pitch)
    assert np.allclose(got_n, want_n, rtol=1e-3, atol=1e-4)
    got_s = canvas[3 * dim * pitch:].view(np.float16).astype(np.float64).reshape(dim, pitch)
    assert np.allclose(got_s, x * u, rtol=1e-3, atol=1e-4)


def test_valu_oracle_rope_and_attention_against_direct_loops():
    from oracle import valu as V
    rng = np.random.default_rng(2)
    h_q, h_kv, hd, seq, frames = 4, 2, 8, 6, 2
    pitch = seq * frames
    rq, rk = h_q * hd, h_kv * hd
    canvas = np.zeros((2 * rq + 2 * rk) * pitch, dtype=np.uint16)
    canvas[: (rq + 2 * rk) * pitch] = _f16(rng.normal(0, 1, (rq + 2 * rk) * pitch))
    q_off, k_off, v_off, o_off = 0, rq * pitch, (rq + rk) * pitch, (rq + 2 * rk) * pitch
    q0 = canvas[q_off:k_off].view(np.float16).astype(np.float64).reshape(rq, pitch)
    V.rope(canvas, q_off, h_q, hd, pitch, seq, 10000.0, False)
    V.rope(canvas, k_off, h_kv, hd, pitch, seq, 10000.0, False)
    q = canvas[q_off:k_off].view(np.float16).astype(np.float64).reshape(rq, pitch)
    k = canvas[k_off:v_off].view(np.float16).astype(np.float64).reshape(rk, pitch)
    v = canvas[v_off:o_off].view(np.float16).astype(np.float64).reshape(rk, pitch)
    # rotary: pair (p, p + hd/2), angle = position * theta^(-2p/hd), position restarts in every sequence
    for h in range(h_q):
        for p in range(hd // 2):
            for t in range(pitch):
                ang = (t % seq) * 10000.0 ** (-2.0 * p / hd)
                a, b = q0[h * hd + p, t], q0[h * hd + p + hd // 2, t]
                assert abs(q[h * hd + p, t] - (a * np.cos(ang) - b * np.sin(ang))) < 2e-3
                assert abs(q[h * hd + p + hd // 2, t] - (a * np.sin(ang) + b * np.cos(ang))) < 2e-3
    V.causal_attention(canvas, q_off, k_off, v_off, o_off, h_q, h_kv, hd, pitch, seq)
    out = canvas[o_off:].view(np.float16).astype(np.float64).reshape(rq, pitch)
    for h in range(h_q):
        kv = h // (h_q // h_kv)
        for t in range(pitch):
            s0 = (t // seq) * seq
            sc = np.array([q[h * hd:(h + 1) * hd, t] @ k[kv * hd:(kv + 1) * hd, u] / np.sqrt(hd) for u in range(s0, t + 1)])
            p = np.exp(sc - sc.max()); p /= p.sum()
            want = sum(p[i] * v[kv * hd:(kv + 1) * hd, s0 + i] for i in range(len(p)))
            assert np.allclose(out[h * hd:(h + 1) * hd, t], want, rtol=2e-3, atol=1e-3)


def test_valu_oracle_decode_attention_equals_causal_attention_on_the_last_token():
    """Appending tokens one by one through the cache must reproduce, for the newest token, what causal attention over
    the whole sequence computes (same rotary positions)."""
    from oracle import valu as V
    rng = np.random.default_rng(3)
    h_q, h_kv, hd, T, pitch = 4, 2, 8, 5, 8
    rq, rk = h_q * hd, h_kv * hd
    toks = _f16(rng.normal(0, 1, (T, rq + 2 * rk, pitch)))           # per step: q, k, v rows for `pitch` sequences
    # decode path
    sizes = [rq, rk, rk, rq, rk * T, rk * T]
    offs = [int(x) for x in np.cumsum([0] + sizes) * pitch]
    dec = np.zeros(offs[-1], dtype=np.uint16)
    for pos in range(T):
        dec[: offs[3]] = toks[pos].reshape(-1)
        V.decode_attention(dec, offs[0], offs[1], offs[2], offs[3], offs[4], offs[5], h_q, h_kv, hd, pitch, T, pos)
    got = dec[offs[3]: offs[4]].view(np.float16).astype(np.float64).reshape(rq, pitch)
    # the same history as one sequence per column: prefill layout [channels][T] for every column separately
    for b in range(pitch):
        pre = np.zeros((2 * rq + 2 * rk) * T, dtype=np.uint16)
        pre[: (rq + 2 * rk) * T] = np.ascontiguousarray(toks[:, :, b].T).reshape(-1)
        V.rope(pre, 0, h_q, hd, T, T)
        V.rope(pre, rq * T, h_kv, hd, T, T)
        V.causal_attention(pre, 0, rq * T, (rq + rk) * T, (rq + 2 * rk) * T, h_q, h_kv, hd, T, T)
        want = pre[(rq + 2 * rk) * T:].view(np.float16).astype(np.float64).reshape(rq, T)[:, T - 1]
        assert np.allclose(got[:, b], want, rtol=3e-3, atol=2e-3)
