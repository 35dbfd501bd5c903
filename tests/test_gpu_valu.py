"""GPU parity of the element-wise / attention commands (RMSNorm, SwiGLU product, rotary + causal attention, decode
attention against a key / value cache), called through the C ABI, against the numpy float64 oracle (oracle/valu.py).
Tolerance rtol 2e-3 / atol 1e-3 as for the waves (FP16 storage, FP32 arithmetic on the device)."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import valu as V
from snntome_b200.native import NativePlan

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-3


def f16(a):
    return np.asarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def run(plan_builder, canvas_bits, pitch, columns=None):
    import torch
    npn = NativePlan.create(canvas_bits.size, pitch, columns or pitch, device=0)
    plan_builder(npn)
    c = npn.canvas_tensor()
    c.copy_(torch.from_numpy(canvas_bits.view(np.int16)).cuda().view(torch.float16))
    return npn, c


def close(got, want, what):
    ok, err, k = O.compare(got, want, RTOL, ATOL)
    assert ok, f"{what}: max abs err {err} at element {k}"


@pytest.mark.parametrize("dim,pitch,with_gamma", [(256, 64, True), (2048, 64, False), (520, 192, True)])
def test_rmsnorm(dim, pitch, with_gamma):
    rng = np.random.default_rng(dim)
    canvas = np.zeros(2 * dim * pitch, dtype=np.uint16)
    canvas[: dim * pitch] = f16(rng.normal(0, 1.5, dim * pitch))
    gamma = f16(1.0 + 0.1 * rng.normal(size=dim)) if with_gamma else None
    npn, c = run(lambda p: p.add_rmsnorm(0, dim * pitch, dim, 1e-5, gamma), canvas, pitch)
    npn.execute()
    assert npn.status() == 0
    V.rmsnorm(canvas, 0, dim * pitch, dim, pitch, 1e-5, gamma)
    close(c.cpu().numpy().view(np.uint16)[dim * pitch:], canvas[dim * pitch:], "rmsnorm")
    npn.close()


def test_swiglu_product():
    rows, pitch = 768, 128
    rng = np.random.default_rng(3)
    canvas = np.zeros(3 * rows * pitch, dtype=np.uint16)
    canvas[: 2 * rows * pitch] = f16(rng.normal(0, 1, 2 * rows * pitch))
    npn, c = run(lambda p: p.add_swiglu(0, rows * pitch, 2 * rows * pitch, rows), canvas, pitch)
    npn.execute()
    V.swiglu(canvas, 0, rows * pitch, 2 * rows * pitch, rows, pitch)
    close(c.cpu().numpy().view(np.uint16)[2 * rows * pitch:], canvas[2 * rows * pitch:], "swiglu")
    npn.close()


@pytest.mark.parametrize("h_q,h_kv,hd,seq,frames,llama3", [(4, 2, 64, 64, 1, False), (8, 2, 64, 96, 2, True), (4, 4, 128, 64, 2, False)])
def test_rope_and_causal_attention(h_q, h_kv, hd, seq, frames, llama3):
    pitch = seq * frames
    pitch_pad = (pitch + 63) // 64 * 64
    rng = np.random.default_rng(h_q * 100 + hd)
    rq, rk = h_q * hd, h_kv * hd
    offs = np.cumsum([0, rq, rk, rk, rq]) * pitch_pad
    canvas = np.zeros(int(offs[-1]), dtype=np.uint16)
    body = rng.normal(0, 1, (rq + 2 * rk, pitch_pad)).astype(np.float32)
    body[:, pitch:] = 0
    canvas[: (rq + 2 * rk) * pitch_pad] = f16(body).reshape(-1)
    q_off, k_off, v_off, o_off = (int(x) for x in offs[:4])
    npn, c = run(lambda p: p.add_rope_attn(q_off, k_off, v_off, o_off, h_q, h_kv, hd, seq, 10000.0, llama3), canvas, pitch_pad, pitch)
    npn.execute()
    assert npn.status() == 0
    V.rope(canvas, q_off, h_q, hd, pitch_pad, seq, 10000.0, llama3)
    V.rope(canvas, k_off, h_kv, hd, pitch_pad, seq, 10000.0, llama3)
    V.causal_attention(canvas, q_off, k_off, v_off, o_off, h_q, h_kv, hd, pitch_pad, seq, columns=pitch)
    got = c.cpu().numpy().view(np.uint16)
    close(got[q_off:v_off].reshape(-1, pitch_pad)[:, :pitch].reshape(-1), canvas[q_off:v_off].reshape(-1, pitch_pad)[:, :pitch].reshape(-1), "rotated q, k")
    close(got[o_off:].reshape(-1, pitch_pad)[:, :pitch].reshape(-1), canvas[o_off:].reshape(-1, pitch_pad)[:, :pitch].reshape(-1), "attention output")
    npn.close()


@pytest.mark.parametrize("h_q,h_kv,max_seq,steps", [(8, 2, 128, [0, 1, 63, 64, 100]), (4, 4, 64, [5])])
def test_decode_attention_with_cache(h_q, h_kv, max_seq, steps):
    import torch
    hd, pitch = 64, 64
    rng = np.random.default_rng(h_q + max_seq)
    rq, rk = h_q * hd, h_kv * hd
    sizes = [rq, rk, rk, rq, rk * max_seq, rk * max_seq]
    offs = [int(x) for x in np.cumsum([0] + sizes) * pitch]
    q_off, k_off, v_off, o_off, kc_off, vc_off = offs[:6]
    canvas = np.zeros(offs[-1], dtype=np.uint16)
    canvas[kc_off:] = f16(rng.normal(0, 1, offs[-1] - kc_off))       # a cache that already holds earlier positions
    npn, c = run(lambda p: p.add_decode_attn(q_off, k_off, v_off, o_off, kc_off, vc_off, h_q, h_kv, hd, max_seq), canvas, pitch)
    for pos in steps:
        new = f16(rng.normal(0, 1, (rq + 2 * rk) * pitch))
        canvas[: v_off + rk * pitch] = new
        c[: v_off + rk * pitch] = torch.from_numpy(new.view(np.int16)).cuda().view(torch.float16)
        npn.set_decode_pos(pos)
        npn.execute_graph()                      # the same graph for every position
        assert npn.status() == 0
        V.decode_attention(canvas, q_off, k_off, v_off, o_off, kc_off, vc_off, h_q, h_kv, hd, pitch, max_seq, pos)
        got = c.cpu().numpy().view(np.uint16)
        close(got[o_off:kc_off], canvas[o_off:kc_off], f"decode attention at position {pos}")
        close(got[kc_off:], canvas[kc_off:], f"caches after position {pos}")
    npn.close()


def test_embedding_gather_and_argmax_are_exact():
    import torch
    vocab, dim, pitch, cols, rows = 1000, 256, 64, 50, 3000
    rng = np.random.default_rng(21)
    table = f16(rng.normal(0, 1, (vocab, dim)))
    tokens = rng.integers(0, vocab, size=cols).astype(np.int32)
    logits = (rng.integers(-40, 40, size=(rows, pitch)) / 8.0).astype(np.float16)          # coarse values: plenty of ties
    logits[rows - 1, 7] = np.float16(np.nan)
    canvas = np.zeros((dim + rows) * pitch, dtype=np.uint16)
    canvas[dim * pitch:] = logits.view(np.uint16).reshape(-1)
    d_table = torch.from_numpy(table.view(np.int16)).cuda()
    npn, c = run(lambda p: (p.add_embedding(d_table.data_ptr(), vocab, dim, 0), p.add_argmax(dim * pitch, rows)), canvas, pitch, cols)
    npn.set_tokens(tokens)
    npn.execute_graph()
    assert npn.status() == 0
    got = c.cpu().numpy().view(np.uint16)[: dim * pitch].reshape(dim, pitch)
    assert np.array_equal(got[:, :cols], table[tokens].T)
    assert not got[:, cols:].any()
    want = np.argmax(np.where(np.isnan(logits), -np.inf, logits.astype(np.float32)), axis=0)   # first maximum wins
    assert np.array_equal(npn.next_tokens(pitch), want.astype(np.int32))
    npn.close()


def test_greedy_loop_feeds_tokens_back_on_the_device():
    """embedding -> dense wave (logits) -> arg-max with feedback, replayed as one graph: every step's token must be a
    maximiser of the logits the oracle computes from the previous token (within the wave tolerance), and the decode
    position advances and saturates."""
    import torch
    from snntome_b200 import synth
    from snntome_b200.plan import Plan, Wave
    vocab, dim, pitch, cols = 512, 128, 64, 64
    rng = np.random.default_rng(22)
    table = f16(rng.normal(0, 1, (vocab, dim)))
    w = f16(rng.normal(0, 0.3, (vocab, dim)))
    offs = (np.arange(dim, dtype=np.uint32) * pitch)[None, :].repeat(vocab // 128, axis=0)
    wave = Wave(cout=vocab, group=128, fan_in=dim, idx=offs, weights=w, bias=None, y_off=dim * pitch, act=0, name="lm_head")
    plan = Plan(canvas_elems=(dim + vocab) * pitch, pitch=pitch, columns=cols, input_off=0, input_c=dim, output_off=dim * pitch, output_c=vocab, waves=[wave])
    d_table = torch.from_numpy(table.view(np.int16)).cuda()
    npn = NativePlan.create(plan.canvas_elems, pitch, cols, device=0)
    npn.add_embedding(d_table.data_ptr(), vocab, dim, 0)
    npn.add_wave(wave)
    npn.add_argmax(dim * pitch, vocab, advance=True, max_seq=3)
    tokens = rng.integers(0, vocab, size=cols).astype(np.int32)
    npn.set_tokens(tokens)
    npn.set_decode_pos(0)
    for step in range(4):
        npn.execute_graph()
        nxt = npn.next_tokens(cols)
        assert npn.status() == 0
        canvas = np.zeros(plan.canvas_elems, dtype=np.uint16)
        canvas[: dim * pitch].reshape(dim, pitch)[:, :cols] = table[tokens].T
        O.wave_forward(canvas, wave, plan)
        logits = canvas[dim * pitch:].view(np.float16).reshape(vocab, pitch)[:, :cols].astype(np.float32)
        chosen = logits[nxt, np.arange(cols)]
        assert np.all(chosen >= logits.max(axis=0) - (ATOL + RTOL * np.abs(logits.max(axis=0)))), f"step {step}"
        tokens = nxt                                      # what the device fed back
    npn.close()
