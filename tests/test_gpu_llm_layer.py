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
