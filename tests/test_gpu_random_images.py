"""GPU parity on seeded random image graphs through the reference-facing builder API: input size and channels, the sequence
of operations (3x3 / 1x1 convolutions with stride 1 or 2, activations, residuals, 2x2 and 5x5 max-pools, nearest upsampling,
2x2 transposed convolutions, slices and concats), canvas reuse and the number of frames per inference are drawn per case. The
model each result is compared with is plain numpy in float64 that rounds every stored tensor to FP16, as the canvas does."""
import numpy as np
import pytest

from oracle import image as I
from snntome_b200.wavec import WaveError, WaveGraph

pytestmark = pytest.mark.gpu
ACTS = ["none", "relu", "sigmoid", "silu", "leaky_relu", "gelu"]


def _act(z, name):
    from math import erf
    if name == "relu":
        return np.maximum(z, 0)
    if name == "sigmoid":
        return 1 / (1 + np.exp(-z))
    if name == "silu":
        return z / (1 + np.exp(-z))
    if name == "leaky_relu":
        return np.maximum(z, 0.1 * z)
    if name == "gelu":
        return 0.5 * z * (1 + np.vectorize(erf)(z / np.sqrt(2.0)))
    return z


def _f16(a):
    return a.astype(np.float16).astype(np.float64)


def _pool5(x):
    xp = np.pad(x, ((0, 0), (2, 2), (2, 2)), constant_values=-65504.0)
    out = np.full_like(x, -65504.0)
    for dy in range(5):
        for dx in range(5):
            out = np.maximum(out, xp[:, dy: dy + x.shape[1], dx: dx + x.shape[2]])
    return out


def draw_graph(seed: int):
    """Returns (graph, frames, input shape, model), model(x[C, H, W]) -> output of one frame."""
    rng = np.random.default_rng(4000 + seed)
    frames = int(rng.choice([1, 1, 2, 3]))
    C = int(rng.choice([3, 4, 8, 16]))
    H = int(rng.choice([8, 12, 16, 24, 32, 48]))
    W = int(rng.choice([16, 24, 32, 40, 64, 96, 128]))
    g = WaveGraph(reuse_canvas=bool(rng.integers(0, 2)), batch_size=frames)
    g.add_input("t0", C, H, W)
    r16 = lambda *s, k: (rng.standard_normal(s) * k).astype(np.float16).astype(np.float32)
    shapes = {"t0": (C, H, W)}
    contiguous = {"t0"}                          # tensors stored as consecutive planes (what pools, upsampling and residuals need)
    steps = []                                   # (kind, out, ins, params) in execution order, for the numpy model
    cur, n, notes = "t0", 0, [f"{frames} frame(s)", f"input {C}x{H}x{W}"]
    n_ops = int(rng.integers(3, 8))
    for k in range(n_ops):
        c, h, w = shapes[cur]
        last = k == n_ops - 1
        kinds = ["conv3", "conv1"]
        if not last:
            if h % 2 == 0 and w % 8 == 0 and h >= 4 and w >= 16:
                kinds += ["conv3s2"] + (["pool2"] if cur in contiguous else [])
            if cur in contiguous:
                kinds += ["pool5"]
                if h * 2 <= 96 and w * 2 <= 192:
                    kinds += ["up", "upconv"]
            if c >= 16 and c % 2 == 0:
                kinds += ["slice"]
            if any(s[1:] == (h, w) and t != cur for t, s in shapes.items()):
                kinds += ["concat"]
        kind = str(rng.choice(kinds))
        n += 1
        out = f"t{n}"
        if kind in ("conv3", "conv1", "conv3s2"):
            ksz = 1 if kind == "conv1" else 3
            stride = 2 if kind == "conv3s2" else 1
            cout = int(rng.choice([8, 16, 24, 32, 48]))
            wt, b = r16(cout, c, ksz, ksz, k=(1.0 / (c * ksz * ksz)) ** 0.5), r16(cout, k=0.05)
            act = str(rng.choice(ACTS))
            ho, wo = (h // 2, w // 2) if stride == 2 else (h, w)
            res = None
            cands = [t for t, s in shapes.items() if s == (cout, ho, wo) and t in contiguous]
            if cands and rng.random() < 0.5:
                res = str(rng.choice(cands))
            g.add_conv2d(f"op{n}", cur, out, c, cout, ksz, ksz, wt, b, stride=stride, pad=ksz // 2, act=act, res_blob=res)
            shapes[out] = (cout, ho, wo)
            contiguous.add(out)
            steps.append(("conv", out, [cur], dict(w=wt, b=b, stride=stride, pad=ksz // 2, act=act, res=res)))
            notes.append(f"{kind}->{cout}{'+res' if res else ''} {act}")
        elif kind == "pool2":
            g.add_maxpool(f"op{n}", cur, out, kernel_size=2, stride=2, pad=0)
            shapes[out] = (c, h // 2, w // 2); contiguous.add(out)
            steps.append(("pool2", out, [cur], {})); notes.append("pool2")
        elif kind == "pool5":
            g.add_maxpool(f"op{n}", cur, out, kernel_size=5, stride=1, pad=2)
            shapes[out] = (c, h, w); contiguous.add(out)
            steps.append(("pool5", out, [cur], {})); notes.append("pool5")
        elif kind == "up":
            g.add_upsample2x(f"op{n}", cur, out)
            shapes[out] = (c, 2 * h, 2 * w); contiguous.add(out)
            steps.append(("up", out, [cur], {})); notes.append("up")
        elif kind == "upconv":
            cout = int(rng.choice([8, 16, 24]))
            wt, b = r16(cout, c, 4, k=(1.0 / c) ** 0.5), r16(cout, k=0.05)
            g.add_upconv2x2(f"op{n}", cur, out, c, cout, wt, b)
            shapes[out] = (cout, 2 * h, 2 * w); contiguous.add(out)
            steps.append(("upconv", out, [cur], dict(w=wt, b=b))); notes.append(f"upconv->{cout}")
        elif kind == "slice":
            other = f"t{n}x"
            g.add_slice(f"op{n}", cur, [out, other], [c // 2, c // 2])
            shapes[out] = shapes[other] = (c // 2, h, w)
            if cur in contiguous:
                contiguous.update([out, other])
            steps.append(("slice", out, [cur], dict(lo=0, hi=c // 2)))
            steps.append(("slice", other, [cur], dict(lo=c // 2, hi=c)))
            if rng.random() < 0.5:
                out = other
            notes.append("slice")
        else:
            other = str(rng.choice([t for t, s in shapes.items() if s[1:] == (h, w) and t != cur]))
            g.add_concat(f"op{n}", [cur, other], out)
            shapes[out] = (c + shapes[other][0], h, w)
            steps.append(("concat", out, [cur, other], {})); notes.append(f"concat {other}")
        cur = out
    g.set_output(cur)

    def model(x):
        t = {"t0": _f16(x)}
        for kind, out, ins, p in steps:
            a = t[ins[0]]
            if kind == "conv":
                z = _act(I.conv2d_direct(a, p["w"], p["b"], p["stride"], p["pad"]), p["act"])
                if p["res"]:
                    z = z + t[p["res"]]
                t[out] = _f16(z)
            elif kind == "pool2":
                c, h, w = a.shape
                t[out] = a.reshape(c, h // 2, 2, w // 2, 2).max(axis=(2, 4))
            elif kind == "pool5":
                t[out] = _pool5(a)
            elif kind == "up":
                t[out] = np.repeat(np.repeat(a, 2, axis=1), 2, axis=2)
            elif kind == "upconv":
                c, h, w = a.shape
                u = np.zeros((p["w"].shape[0], 2 * h, 2 * w))
                for py in range(2):
                    for px in range(2):
                        u[:, py::2, px::2] = np.einsum("oi,iyx->oyx", p["w"][:, :, 2 * py + px].astype(np.float64), a) + p["b"].astype(np.float64)[:, None, None]
                t[out] = _f16(u)
            elif kind == "slice":
                t[out] = a[p["lo"]: p["hi"]]
            else:
                t[out] = np.concatenate([a, t[ins[1]]])
        return t[cur]

    return g, frames, (C, H, W), model, ", ".join(notes)


@pytest.mark.parametrize("seed", range(40))
def test_random_image_graph_matches_the_numpy_model(seed):
    g, frames, shape, model, notes = draw_graph(seed)
    try:
        plan = g.compile()
    except WaveError as e:                       # the generator only draws what the compiler documents; a refusal is a failure
        raise AssertionError(f"{notes}: compile refused: {e}") from None
    rng = np.random.default_rng(5000 + seed)
    xs = (rng.standard_normal((frames,) + shape) * 0.7).astype(np.float16).astype(np.float32)
    got, _ = plan.infer_f32(xs if frames > 1 else xs[0])
    got = got.reshape((frames,) + got.shape[-3:])
    for f in range(frames):
        want = model(xs[f])
        g64 = got[f].astype(np.float64)
        assert g64.shape == want.shape, notes
        err = np.abs(g64 - want)
        tol = 4e-3 + 6e-3 * np.abs(want)          # a one-ulp FP16 difference in a stored tensor may pass through later layers
        bad = err > tol
        assert bad.mean() < 2e-4 and err.max() < 3e-2, f"{notes}: frame {f}: max err {err.max()}, {bad.sum()} of {bad.size} outside tolerance"
        if np.linalg.norm(want) > 0:
            cos = float((g64 * want).sum() / (np.linalg.norm(g64) * np.linalg.norm(want) + 1e-30))
            assert cos > 0.9999, f"{notes}: frame {f}: cosine {cos}"
