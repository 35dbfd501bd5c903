"""The 2-D image path on the GPU: waves over haloed planes (both layouts: rows of whole 64-pixel tiles, and arbitrary widths with
masked tiles) and the weight-free glue commands through the C ABI against the oracle's restatement, and the building-block graph
of the reference's image example through the reference-facing builder API against a direct numpy model within the example's
own tolerance (max-abs error below 1e-2, cosine above 0.9999: wavec/examples/example_yolov8.py:136)."""
import numpy as np
import pytest

from oracle import image as I
from oracle import oracle as O
from snntome_b200.native import PATH_AUTO, PATH_FMA, PATH_MMA, NativePlan
from test_image_oracle import _yolo_block, yolo_block_reference

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 1e-3


def _run_waves(canvas0, waves, force_path):
    import torch
    npn = NativePlan.create(canvas0.size, 64, 64, device=0, force_path=force_path)
    for w in waves:
        npn.add_image_wave(cout=w.cout, group=w.group, fan_in=w.fan_in, idx=w.idx, weights=w.weights, bias=w.bias, y_off=w.y_off, act=w.act,
                           plane_stride=w.lay.plane, tile_off_x=w.lay.tile_off_x, tile_off_y=w.lay.tile_off_y, tile_mask=w.lay.masked,
                           has_residual=w.has_residual, res_off=w.res_off, name=w.name)
    cv = npn.canvas_tensor()
    cv.copy_(torch.from_numpy(canvas0.view(np.int16)).cuda().view(torch.float16))
    npn.execute()
    assert npn.status() == 0
    paths = [npn.wave_info(i).path for i in range(npn.num_waves)]
    out = cv.cpu().numpy().view(np.uint16)
    npn.close()
    return out, paths


@pytest.mark.parametrize("path", [PATH_AUTO, PATH_FMA])
@pytest.mark.parametrize("H,W,group", [(8, 64, 16), (6, 40, 32), (5, 128, 64), (7, 12, 16), (24, 100, 16)])
def test_convolution_waves_over_planes(H, W, group, path):
    """A 3x3 convolution followed by a 1x1 one with a residual, over a plane layout with whole 64-pixel tiles (W % 64 == 0) or with
    masked tiles; every element of the output planes — pixels and halos — must equal the oracle's."""
    rng = np.random.default_rng(H * 1000 + W)
    lay = I.Layout2D(H, W)
    cin, c1, c2 = 5, 64, 24
    x = (rng.standard_normal((cin, H, W)) * 0.5).astype(np.float16)
    w1 = (rng.standard_normal((c1, cin, 3, 3)) * 0.2).astype(np.float16)
    b1 = (rng.standard_normal(c1) * 0.1).astype(np.float16)
    w2 = (rng.standard_normal((c2, c1, 1, 1)) * 0.1).astype(np.float16)
    x_at, y1_at = 0, 8 * lay.plane
    y2_at = y1_at + 64 * lay.plane
    canvas = np.zeros(y2_at + 64 * lay.plane + 256, dtype=np.uint16)
    canvas[: cin * lay.plane] = I.to_planes(x.view(np.uint16), lay).reshape(-1)
    waves = [I.conv_wave(lay, [x_at + c * lay.plane for c in range(cin)], w1.view(np.uint16), b1.view(np.uint16), y1_at, act=3, group=group, name="conv3x3"),
             I.conv_wave(lay, [y1_at + c * lay.plane for c in range(c1)], w2.view(np.uint16), None, y2_at, act=1, kh=1, kw=1, group=group if 64 % group == 0 and group <= 32 else 16,
                         residual_off=y1_at, name="conv1x1_res")]
    want = canvas.copy()
    for w in waves:
        I.wave_forward_2d(want, w)
    got, paths = _run_waves(canvas, waves, path)
    assert all(p == (PATH_FMA if path == PATH_FMA else PATH_MMA) for p in paths)
    for w in waves:
        a, b = w.y_off, w.y_off + w.cout * lay.plane
        ok, err, k = O.compare(got[a:b], want[a:b], RTOL, ATOL)
        assert ok, (w.name, err, k)
    assert np.array_equal(got[: cin * lay.plane], canvas[: cin * lay.plane])            # the input planes are untouched
    # and against a direct convolution of the image (no planes, no taps)
    z = I.conv2d_direct(x, w1, b1, 1, 1)
    y1 = I.from_planes(got[y1_at: y1_at + c1 * lay.plane].reshape(c1, -1), lay).view(np.float16).astype(np.float64)
    assert np.abs(y1 - z / (1 + np.exp(-z))).max() < 6e-3


def test_glue_commands_on_planes():
    """max-pool 2x2 and 5x5, nearest upsampling, space-to-depth, the transposed-convolution scatter and the halo clear, each
    against the oracle's numpy restatement, bit for bit (values are moved or compared, never rounded)."""
    import torch
    rng = np.random.default_rng(9)
    lin, lout = I.Layout2D(12, 40), I.Layout2D(6, 20)
    C = 6
    x = rng.standard_normal((C, 12, 40)).astype(np.float16)
    at = {"x": 0, "p2": C * lin.plane}
    at["p5"] = at["p2"] + C * lout.plane
    at["s2d"] = at["p5"] + C * lin.plane
    at["up"] = at["s2d"] + 4 * C * lout.plane
    at["sc"] = at["up"] + C * lin.plane
    at["dirty"] = at["sc"] + C * lin.plane
    total = at["dirty"] + C * lin.plane + 64
    canvas = np.zeros(total, dtype=np.uint16)
    canvas[: C * lin.plane] = I.to_planes(x.view(np.uint16), lin).reshape(-1)
    canvas[at["dirty"]: at["dirty"] + C * lin.plane] = rng.integers(1, 30000, C * lin.plane).astype(np.uint16)   # a recycled region
    gi, go = (lin.H, lin.W, lin.W_pad, lin.plane), (lout.H, lout.W, lout.W_pad, lout.plane)
    want = canvas.copy()
    I.maxpool2(want, at["x"], at["p2"], C, lin, lout)
    I.maxpool5(want, at["x"], at["p5"], C, lin)
    I.space_to_depth(want, at["x"], at["s2d"], C, lin, lout)
    I.upsample2(want, at["p2"], at["up"], C, lout, lin)
    I.upconv_scatter(want, at["s2d"], at["sc"], C, lout, lin)
    I.halo_clear(want, at["dirty"], C, lin)
    npn = NativePlan.create(total, 64, 64, device=0)
    npn.add_image_op("maxpool2", at["x"], at["p2"], C, gi, go)
    npn.add_image_op("maxpool5", at["x"], at["p5"], C, gi, gi)
    npn.add_image_op("space_to_depth", at["x"], at["s2d"], C, gi, go)
    npn.add_image_op("upsample2", at["p2"], at["up"], C, go, gi)
    npn.add_image_op("upconv_scatter", at["s2d"], at["sc"], C, go, gi)
    npn.add_image_op("halo_clear", 0, at["dirty"], C, None, gi)
    cv = npn.canvas_tensor()
    cv.copy_(torch.from_numpy(canvas.view(np.int16)).cuda().view(torch.float16))
    npn.execute()
    assert npn.status() == 0
    got = cv.cpu().numpy().view(np.uint16)
    npn.close()
    for name in at:
        a = at[name]
        b = min([v for v in at.values() if v > a] + [total])
        assert np.array_equal(got[a:b], want[a:b]), name


@pytest.mark.parametrize("reuse", [True, False])
@pytest.mark.parametrize("H,W", [(64, 64), (48, 40)])
def test_image_example_block_through_the_builder_api(H, W, reuse):
    """Stem 3x3, C2f (1x1, slice, two 3x3 with a residual, concat, 1x1) and SPPF (1x1, three 5x5 max-pools, concat, 1x1) built with the
    reference's graph-builder calls, executed through wavec_gpu_infer_f32 with dense FP32 images in and out — twice, so that a
    recycled canvas has to clear its halos — against the numpy model."""
    g, P = _yolo_block(np.random.default_rng(42), H, W, reuse)
    plan = g.compile()
    want = yolo_block_reference(P)
    for _ in range(2):
        got, ms = plan.infer_f32(P["x"])
        got = got.astype(np.float64)
        err = np.abs(got - want).max()
        cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
        assert err < 1e-2 and cos > 0.9999, (err, cos)


def test_strided_convolution_pooling_upsampling_and_transposed_convolution_through_the_builder_api():
    """A small encoder / decoder: 3x3 stride-2 convolution (space-to-depth + wave), 2x2 max-pool, nearest upsampling, 2x2 transposed
    convolution (phase wave + scatter), a skip concat, against a direct numpy model."""
    from snntome_b200.wavec import WaveGraph
    rng = np.random.default_rng(5)
    r = lambda *s, k=0.15: (rng.standard_normal(s) * k).astype(np.float16).astype(np.float32)
    H, W = 32, 48
    x = r(4, H, W, k=0.5)
    w_d, b_d = r(16, 4, 3, 3), r(16, k=0.05)          # stride 2: 32x48 -> 16x24
    w_u, b_u = r(8, 16, 4), r(8, k=0.05)              # transposed 2x2: 16x24 -> 32x48
    w_o, b_o = r(8, 12, 3, 3), r(8, k=0.05)           # on concat(up, x)
    w_p, b_p = r(8, 16, 1, 1), r(8, k=0.05)           # on pool(down) upsampled
    g = WaveGraph(reuse_canvas=False)
    g.add_input("x", 4, H, W)
    g.add_conv2d("down", "x", "d", 4, 16, 3, 3, w_d, b_d, stride=2, pad=1, act="relu")
    g.add_upconv2x2("up", "d", "u", 16, 8, w_u, b_u)
    g.add_concat("cat", ["u", "x"], "ux")
    g.add_conv2d("mix", "ux", "m", 12, 8, 3, 3, w_o, b_o, stride=1, pad=1, act="silu")
    g.add_maxpool("pool", "d", "dp", kernel_size=2, stride=2, pad=0)      # 16x24 -> 8x12
    g.add_upsample2x("up1", "dp", "dq")                                    # -> 16x24
    g.add_upsample2x("up2", "dq", "dr")                                    # -> 32x48
    g.add_conv2d("proj", "dr", "out", 16, 8, 1, 1, w_p, b_p, stride=1, pad=0, act="none", res_blob="m")
    g.set_output("out")
    plan = g.compile()
    got, _ = plan.infer_f32(x)
    # numpy model
    d = np.maximum(I.conv2d_direct(x, w_d, b_d, 2, 1), 0)
    u = np.zeros((8, H, W))
    for py in range(2):
        for px in range(2):
            u[:, py::2, px::2] = np.einsum("oi,iyx->oyx", w_u[:, :, 2 * py + px].astype(np.float64), d) + b_u[:, None, None]
    z = I.conv2d_direct(np.concatenate([u, x]), w_o, b_o, 1, 1)
    m = z / (1 + np.exp(-z))
    dp = d.reshape(16, 8, 2, 12, 2).max(axis=(2, 4))
    dr = np.repeat(np.repeat(dp, 4, axis=1), 4, axis=2)
    want = I.conv2d_direct(dr, w_p, b_p, 1, 0) + m
    err = np.abs(got.astype(np.float64) - want).max()
    cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    assert err < 1.5e-2 and cos > 0.9999, (err, cos)


@pytest.mark.parametrize("H,W,frames", [(64, 64, 3), (48, 40, 2)])
def test_several_frames_per_wave(H, W, frames):
    """wavec_set_batch_size on an image graph: the frames of a channel lie side by side in the canvas, every wave and glue
    command covers all of them, and wavec_gpu_infer_f32 takes and returns dense [frame][channel][y][x]. Each frame must equal
    the numpy model of that frame alone (stem + C2f + SPPF block; whole-tile and masked layouts; recycled regions)."""
    from snntome_b200.wavec import WaveGraph
    g, P = _yolo_block(np.random.default_rng(42), H, W, True)
    g._lib.wavec_set_batch_size(g._handle, frames)
    plan = g.compile()
    assert plan.summary["batch_size"] == frames
    rng = np.random.default_rng(77)
    xs = (rng.standard_normal((frames,) + P["x"].shape) * 0.25).astype(np.float16).astype(np.float32)
    got, _ = plan.infer_f32(xs)
    assert got.shape[0] == frames
    for f in range(frames):
        Pf = dict(P, x=xs[f])
        want = yolo_block_reference(Pf)
        g64 = got[f].astype(np.float64)
        err = np.abs(g64 - want).max()
        cos = float((g64 * want).sum() / (np.linalg.norm(g64) * np.linalg.norm(want)))
        assert err < 1e-2 and cos > 0.9999, (f, err, cos)
    assert np.abs(got[0] - got[1]).max() > 1e-3           # the frames really differ


def test_several_frames_through_strided_and_transposed_convolutions():
    """The encoder / decoder graph (space-to-depth, 2x2 pooling, upsampling, transposed-convolution scatter) with two frames."""
    from snntome_b200.wavec import WaveGraph
    rng = np.random.default_rng(5)
    r = lambda *s, k=0.15: (rng.standard_normal(s) * k).astype(np.float16).astype(np.float32)
    H, W, F = 32, 48, 2
    xs = r(F, 4, H, W, k=0.5)
    w_d, b_d = r(16, 4, 3, 3), r(16, k=0.05)
    w_u, b_u = r(8, 16, 4), r(8, k=0.05)
    w_o, b_o = r(8, 12, 3, 3), r(8, k=0.05)
    w_p, b_p = r(8, 16, 1, 1), r(8, k=0.05)
    g = WaveGraph(reuse_canvas=True, batch_size=F)
    g.add_input("x", 4, H, W)
    g.add_conv2d("down", "x", "d", 4, 16, 3, 3, w_d, b_d, stride=2, pad=1, act="relu")
    g.add_upconv2x2("up", "d", "u", 16, 8, w_u, b_u)
    g.add_concat("cat", ["u", "x"], "ux")
    g.add_conv2d("mix", "ux", "m", 12, 8, 3, 3, w_o, b_o, stride=1, pad=1, act="silu")
    g.add_maxpool("pool", "d", "dp", kernel_size=2, stride=2, pad=0)
    g.add_upsample2x("up1", "dp", "dq")
    g.add_upsample2x("up2", "dq", "dr")
    g.add_conv2d("proj", "dr", "out", 16, 8, 1, 1, w_p, b_p, stride=1, pad=0, act="none", res_blob="m")
    g.set_output("out")
    plan = g.compile()
    got, _ = plan.infer_f32(xs)
    for f in range(F):
        x = xs[f]
        d = np.maximum(I.conv2d_direct(x, w_d, b_d, 2, 1), 0)
        u = np.zeros((8, H, W))
        for py in range(2):
            for px in range(2):
                u[:, py::2, px::2] = np.einsum("oi,iyx->oyx", w_u[:, :, 2 * py + px].astype(np.float64), d) + b_u[:, None, None]
        z = I.conv2d_direct(np.concatenate([u, x]), w_o, b_o, 1, 1)
        m = z / (1 + np.exp(-z))
        dp = d.reshape(16, 8, 2, 12, 2).max(axis=(2, 4))
        dr = np.repeat(np.repeat(dp, 4, axis=1), 4, axis=2)
        want = I.conv2d_direct(dr, w_p, b_p, 1, 0) + m
        g64 = got[f].astype(np.float64)
        err = np.abs(g64 - want).max()
        cos = float((g64 * want).sum() / (np.linalg.norm(g64) * np.linalg.norm(want)))
        assert err < 1.5e-2 and cos > 0.9999, (f, err, cos)


def test_detector_network_frames_equal_single_image_runs():
    """The benchmark's detector backbone + neck at 384 x 384 (plane widths 384 .. 12: whole-tile and masked layouts, five
    stride-2 convolutions, SPPF, two upsample + concat stages): a plan built for three frames must return, frame by frame,
    exactly the bits the one-frame plan returns for the same image — same weights, same arithmetic, only the layout differs."""
    import bench
    size = 384
    g1, rng = bench.build_image_graph(size, seed=11, frames=1)
    p1 = g1.compile()
    g3, _ = bench.build_image_graph(size, seed=11, frames=3)
    p3 = g3.compile()
    xs = np.random.default_rng(12).standard_normal((3, 3, size, size)).astype(np.float32)
    got3, _ = p3.infer_f32(xs)
    assert got3.shape == (3, 64, size // 8, size // 8) and np.isfinite(got3).all()
    for f in range(3):
        one, _ = p1.infer_f32(xs[f])
        assert np.array_equal(one, got3[f]), f"frame {f}: max abs difference {np.abs(one - got3[f]).max()}"
    assert np.abs(got3[0] - got3[1]).max() > 1e-3
