"""A whole decoder layer through the reference-facing builder API (`WaveGraph`: RMSNorm, q/k/v/o linears, rotary +
causal GQA attention, gated MLP with SwiGLU, residuals), the way the reference's own example drives it
(wavec/examples/example_llm.py:66-140), against a numpy float64 model. Tolerances are the example's: max-abs error
below 2e-2 and cosine similarity above 0.9999 (example_llm.py:139)."""
import json
import os

import numpy as np
import pytest

from snntome_b200.wavec import WaveGraph

D, H_Q, H_KV, HD, D_FFN, SEQ = 256, 4, 2, 64, 512, 64


def weights(seed=7):
    rng = np.random.default_rng(seed)
    r = lambda *s, k=0.08: (rng.standard_normal(s) * k).astype(np.float16).astype(np.float32)
    w = dict(x=r(D, 1, SEQ, k=0.25), g1=(1 + rng.standard_normal(D) * 0.1).astype(np.float16).astype(np.float32),
             g2=(1 + rng.standard_normal(D) * 0.1).astype(np.float16).astype(np.float32), wq=r(D, D), wk=r(H_KV * HD, D), wv=r(H_KV * HD, D),
             wo=r(D, D), wg=r(D_FFN, D), wu=r(D_FFN, D), wd=r(D, D_FFN))
    return w


def build(w, fold=True):
    g = WaveGraph(max_B_per_wave=512, default_S=64, fold_rmsnorm_gamma=fold, reuse_canvas=True)
    g.add_input("tokens_in", c=D, h=1, w=SEQ, is_1d=True)
    g.add_rmsnorm("attn_norm", "tokens_in", "x_norm1", D, w["g1"], eps=1e-5)
    g.add_linear("q_proj", "x_norm1", "q", D, D, w["wq"], act="none")
    g.add_linear("k_proj", "x_norm1", "k", D, H_KV * HD, w["wk"], act="none")
    g.add_linear("v_proj", "x_norm1", "v", D, H_KV * HD, w["wv"], act="none")
    g.add_rope_gqa_attn("rope_gqa", "q", "k", "v", "attn_out", H_Q, H_KV, HD, rope_theta=10000.0)
    g.add_linear("o_proj", "attn_out", "h_mid", D, D, w["wo"], act="none", res_blob="tokens_in")
    g.add_rmsnorm("ffn_norm", "h_mid", "x_norm2", D, w["g2"], eps=1e-5)
    g.add_linear("gate_proj", "x_norm2", "gate", D, D_FFN, w["wg"], act="silu")
    g.add_linear("up_proj", "x_norm2", "up", D, D_FFN, w["wu"], act="none")
    g.add_swiglu("swiglu", "gate", "up", "ffn_act", D_FFN)
    g.add_linear("down_proj", "ffn_act", "tokens_out", D_FFN, D, w["wd"], act="none", res_blob="h_mid")
    g.set_output("tokens_out")
    return g


def reference(w):
    def rms(x, g):
        return x / np.sqrt(np.mean(x * x, axis=0, keepdims=True) + 1e-5) * g[:, None]

    def rope(t, heads):
        out = t.copy()
        half = HD // 2
        inv = np.exp(2.0 * np.arange(half) * (-np.log(10000.0) / HD))
        ang = np.arange(t.shape[1])[None, :] * inv[:, None]
        c, s = np.cos(ang), np.sin(ang)
        for h in range(heads):
            a, b = t[h * HD: h * HD + half], t[h * HD + half: (h + 1) * HD]
            out[h * HD: h * HD + half], out[h * HD + half: (h + 1) * HD] = a * c - b * s, a * s + b * c
        return out

    x = w["x"][:, 0, :].astype(np.float64)
    n1 = rms(x, w["g1"])
    q, k, v = rope(w["wq"] @ n1, H_Q), rope(w["wk"] @ n1, H_KV), w["wv"] @ n1
    att = np.zeros_like(q)
    mask = np.triu(np.full((SEQ, SEQ), -1e9), k=1)
    for h in range(H_Q):
        kv = h // (H_Q // H_KV)
        sc = q[h * HD:(h + 1) * HD].T @ k[kv * HD:(kv + 1) * HD] / np.sqrt(HD) + mask
        p = np.exp(sc - sc.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        att[h * HD:(h + 1) * HD] = (p @ v[kv * HD:(kv + 1) * HD].T).T
    h_mid = w["wo"] @ att + x
    n2 = rms(h_mid, w["g2"])
    gate = w["wg"] @ n2
    return (w["wd"] @ (gate / (1 + np.exp(-gate)) * (w["wu"] @ n2)) + h_mid)[:, None, :]


def test_layer_compiles_with_folded_scales():
    plan = build(weights()).compile()
    s = plan.summary
    assert s["num_folded_rmsnorms"] == 2 and s["num_waves"] == 7 and s["num_cmds"] == 11
    types = [c["type"] for c in s["cmds"]]
    assert types == ["RMSNORM", "K44_WAVE", "K44_WAVE", "K44_WAVE", "ROPE_GQA_ATTN", "K44_WAVE", "RMSNORM", "K44_WAVE", "K44_WAVE", "SWIGLU", "K44_WAVE"]
    assert s["output_shape"] == [D, 1, SEQ]


@pytest.mark.gpu
@pytest.mark.parametrize("fold", [True, False])
def test_decoder_layer_matches_float64_model(fold, tmp_path):
    w = weights()
    plan = build(w, fold=fold).compile()
    assert plan.summary["num_folded_rmsnorms"] == (2 if fold else 0)
    path = os.path.join(tmp_path, "layer.tcff")
    plan.save_tcff(path, model_prefix="LLM_Block")           # seven wave pages; the other commands carry no tensors
    plan.load_tcff_weights(path)
    y, gpu_ms = plan.infer_f32(w["x"])
    want = reference(w)
    err = float(np.max(np.abs(y - want)))
    cos = float(np.dot(y.ravel(), want.ravel()) / (np.linalg.norm(y) * np.linalg.norm(want)))
    assert err < 2e-2 and cos > 0.9999, (err, cos)


@pytest.mark.gpu
def test_mini_decoder_step_with_cache_matches_oracle():
    """The decode-full benchmark plan at a small size (2 layers, hidden 256, 4/2 heads x 64, FFN 512, vocabulary 1024, a
    cache of 64 positions): embedding gather, RMSNorm, q/k/v waves, rotary + attention against the cache, o wave with
    residual, RMSNorm, gated MLP with SwiGLU product, final norm, lm_head, arg-max — one CUDA graph, replayed at two
    positions — against the oracle replaying the same command list on a copy of the device's canvas, weights and table."""
    import sys
    from pathlib import Path
    import torch
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import bench
    from oracle import oracle as O
    from oracle import valu as V
    from snntome_b200.plan import Plan, Wave
    cfg = dict(hidden=256, layers=2, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024, columns=64)
    ctx, pitch = 64, 64
    plan, params, rows = bench.build_decoder_plan(cfg, 0, full=True, ctx=ctx)
    H, F, Vv, KV = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["kv_heads"] * cfg["head_dim"]
    off = lambda n: rows[n] * pitch
    canvas_t = plan.canvas_tensor()
    n_cmd = plan.num_waves
    wave_ids = [i for i in range(n_cmd) if plan.wave_info(i).path != 2]
    assert len(wave_ids) == 7 * cfg["layers"] + 1
    weights = [plan.weights_rowmajor(i).cpu().numpy().view(np.uint16) for i in wave_ids]
    table = plan.embedding_table.cpu().numpy().view(np.uint16).reshape(Vv, H)
    rng = np.random.default_rng(12)
    for pos in (ctx - 1, 17):
        tokens = rng.integers(0, Vv, size=64).astype(np.int32)
        ref = canvas_t.cpu().numpy().view(np.uint16).copy()            # caches and leftovers exactly as the device has them
        plan.set_tokens(tokens)
        plan.set_decode_pos(pos)
        plan.execute_graph()
        got_tokens = plan.next_tokens(64)
        assert plan.status() == 0
        got = canvas_t.cpu().numpy().view(np.uint16)

        def wave(k, src, dst, cin, cout, act=0, res=None):
            idx = ((rows[src] + np.arange(cin, dtype=np.uint32)) * pitch)[None, :].repeat(cout // 128, axis=0)
            w = Wave(cout=cout, group=128, fan_in=cin, idx=idx, weights=weights[k], bias=None, y_off=off(dst), act=act,
                     has_residual=res is not None, res_off=off(res) if res else 0)
            O.wave_forward(ref, w, Plan(canvas_elems=ref.size, pitch=pitch, columns=64, input_off=0, input_c=1, output_off=0, output_c=1, waves=[w]))

        ref[off("x0"): off("x0") + H * pitch].reshape(H, pitch)[:] = table[tokens].T
        x_in, x_out, k = "x0", "x1", 0
        for layer in range(cfg["layers"]):
            V.rmsnorm(ref, off(x_in), off("n"), H, pitch, 1e-5)
            wave(k, "n", "q", H, H); wave(k + 1, "n", "k", H, KV); wave(k + 2, "n", "v", H, KV)
            V.decode_attention(ref, off("q"), off("k"), off("v"), off("att"), off(f"kcache{layer}"), off(f"vcache{layer}"), cfg["heads"], cfg["kv_heads"],
                               cfg["head_dim"], pitch, ctx, pos, 500000.0, True)
            wave(k + 3, "att", "h", H, H, res=x_in)
            V.rmsnorm(ref, off("h"), off("n"), H, pitch, 1e-5)
            wave(k + 4, "n", "g", H, F, act=3); wave(k + 5, "n", "u", H, F)
            V.swiglu(ref, off("g"), off("u"), off("f"), F, pitch)
            wave(k + 6, "f", x_out, F, H, res="h")
            x_in, x_out, k = x_out, x_in, k + 7
        V.rmsnorm(ref, off(x_in), off("n"), H, pitch, 1e-5)
        wave(k, "n", "logits", H, Vv)
        a, b = off("logits"), off("logits") + Vv * pitch
        # two layers of FP16 intermediates: compare the logits with a tolerance scaled to their spread, then the tokens
        lg, lw = got[a:b].view(np.float16).astype(np.float32), ref[a:b].view(np.float16).astype(np.float32)
        assert np.max(np.abs(lg - lw)) < 5e-3 * max(1.0, float(np.abs(lw).max())), float(np.max(np.abs(lg - lw)))
        lw2 = lw.reshape(Vv, pitch)
        chosen = lw2[got_tokens, np.arange(64)]
        assert np.all(chosen >= lw2.max(axis=0) - 1e-2 * np.maximum(1.0, np.abs(lw2.max(axis=0))))
        for layer in range(cfg["layers"]):                        # the caches received the same new rows
            ok, err, kk = O.compare(got[off(f"kcache{layer}"): off(f"kcache{layer}") + 2 * KV * ctx * pitch],
                                    ref[off(f"kcache{layer}"): off(f"kcache{layer}") + 2 * KV * ctx * pitch], 4e-3, 2e-3)
            assert ok, (layer, err, kk)
    plan.close()
