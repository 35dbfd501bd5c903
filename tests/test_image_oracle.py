"""The 2-D image path on the CPU: the plane layouts and the oracle's wave over planes against direct numpy references that do
not share the layout code, the graph compiler's image path (commands, shapes, .tcff round trip), and the library's own layout
tables (through the compiled plan's summary) against the oracle's restatement."""
import json

import numpy as np
import pytest

from oracle import image as I
from oracle import oracle as O
from snntome_b200.wavec import WaveError, WaveGraph


@pytest.mark.parametrize("H,W", [(8, 64), (6, 40), (5, 128), (7, 12), (16, 100)])
def test_plane_layout_tiles_cover_every_pixel_exactly_once(H, W):
    lay = I.Layout2D(H, W)
    hits = np.zeros(lay.plane + 64, dtype=np.int32)
    for t in range(lay.num_tiles):
        e = int(lay.tile_off_y[t])
        base, mask = ((e & 0xFFFF) << 2, e >> 16) if lay.masked else (e, 0xFFFF)
        for q in range(16):
            if (mask >> q) & 1:
                hits[base + 4 * q: base + 4 * q + 4] += 1
    pix = np.zeros_like(hits)
    for y in range(H):
        pix[lay.pixel(y, 0): lay.pixel(y, 0) + W] = 1
    assert np.array_equal(hits, pix)                       # stored elements == pixels, halos never written
    # the gather anchor sits one row up and one element left of the tile's first stored element
    first = ((lay.tile_off_y & 0xFFFF) << 2) if lay.masked else lay.tile_off_y
    assert np.array_equal(lay.tile_off_x.astype(np.int64), first.astype(np.int64) - lay.W_pad - 1)


@pytest.mark.parametrize("H,W,k", [(8, 64, 3), (6, 40, 3), (9, 20, 1), (4, 128, 3)])
def test_wave_over_planes_equals_a_direct_convolution(H, W, k):
    rng = np.random.default_rng(H * W + k)
    lay = I.Layout2D(H, W)
    cin, cout = 6, 24
    x = (rng.standard_normal((cin, H, W)) * 0.5).astype(np.float16)
    w = (rng.standard_normal((cout, cin, k, k)) * 0.2).astype(np.float16)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float16)
    r = (rng.standard_normal((32, H, W)) * 0.3).astype(np.float16)
    x_at, r_at, y_at = 0, cin * lay.plane, (cin + 32) * lay.plane
    canvas = np.zeros(y_at + 32 * lay.plane + 256, dtype=np.uint16)
    canvas[x_at: r_at] = I.to_planes(x.view(np.uint16), lay).reshape(-1)
    canvas[r_at: y_at] = I.to_planes(r.view(np.uint16), lay).reshape(-1)
    wave = I.conv_wave(lay, [x_at + c * lay.plane for c in range(cin)], w.view(np.uint16), b.view(np.uint16), y_at, act=3, kh=k, kw=k, group=16,
                       residual_off=r_at)
    I.wave_forward_2d(canvas, wave)
    got = I.from_planes(canvas[y_at: y_at + cout * lay.plane].reshape(cout, lay.plane), lay).view(np.float16).astype(np.float64)
    z = I.conv2d_direct(x, w, b, 1, k // 2)
    want = z / (1 + np.exp(-z)) + r[:cout].astype(np.float64)
    assert np.abs(got - want).max() < 4e-3
    # nothing but pixels was written
    out_planes = canvas[y_at: y_at + 32 * lay.plane].copy()
    cleared = out_planes.copy()
    I.halo_clear(cleared, 0, 32, lay)
    assert np.array_equal(out_planes, cleared)


def test_glue_commands_against_plain_numpy():
    rng = np.random.default_rng(3)
    lin, lout = I.Layout2D(8, 24), I.Layout2D(4, 12)
    x = rng.standard_normal((3, 8, 24)).astype(np.float16)
    canvas = np.zeros(3 * lin.plane + 12 * lout.plane + 3 * lin.plane + 64, dtype=np.uint16)
    canvas[: 3 * lin.plane] = I.to_planes(x.view(np.uint16), lin).reshape(-1)
    d = 3 * lin.plane
    I.maxpool2(canvas, 0, d, 3, lin, lout)
    got = I.from_planes(canvas[d: d + 3 * lout.plane].reshape(3, -1), lout).view(np.float16)
    assert np.array_equal(got, x.reshape(3, 4, 2, 12, 2).max(axis=(2, 4)))
    I.space_to_depth(canvas, 0, d, 3, lin, lout)
    s2d = I.from_planes(canvas[d: d + 12 * lout.plane].reshape(12, -1), lout).view(np.float16)
    for c in range(3):
        for py in range(2):
            for px in range(2):
                assert np.array_equal(s2d[4 * c + 2 * py + px], x[c, py::2, px::2])
    u = d + 12 * lout.plane
    I.upsample2(canvas, d, u, 3, lout, lin)                 # (the first three half-resolution planes)
    up = I.from_planes(canvas[u: u + 3 * lin.plane].reshape(3, -1), lin).view(np.float16)
    assert np.array_equal(up[:, ::2, ::2], s2d[:3]) and np.array_equal(up[:, 1::2, 1::2], s2d[:3])
    I.upconv_scatter(canvas, d, u, 3, lout, lin)            # phase planes q * 3 + c -> pixel parity q
    sc = I.from_planes(canvas[u: u + 3 * lin.plane].reshape(3, -1), lin).view(np.float16)
    for q in range(4):
        assert np.array_equal(sc[:, q // 2::2, q % 2::2], s2d[3 * q: 3 * q + 3])


def _yolo_block(rng, H=64, W=64, reuse=True):
    """The building-block graph of the reference's image example (wavec/examples/example_yolov8.py:52-137): stem 3x3, a C2f
    block (1x1, slice, two 3x3 with a residual, concat, 1x1) and an SPPF block (1x1, three 5x5 max-pools, concat, 1x1)."""
    r = lambda *s, k=0.1: (rng.standard_normal(s) * k).astype(np.float16).astype(np.float32)
    P = dict(x=r(16, H, W, k=0.25), w_stem=r(32, 16, 3, 3), b_stem=r(32, k=0.05), w_cv1=r(32, 32, 1, 1), b_cv1=r(32, k=0.05),
             w_bn1=r(16, 16, 3, 3), b_bn1=r(16, k=0.05), w_bn2=r(16, 16, 3, 3), b_bn2=r(16, k=0.05), w_cv2=r(32, 48, 1, 1), b_cv2=r(32, k=0.05),
             w_sp1=r(16, 32, 1, 1), b_sp1=r(16, k=0.05), w_sp2=r(32, 64, 1, 1), b_sp2=r(32, k=0.05))
    g = WaveGraph(max_B_per_wave=288, reuse_canvas=reuse)
    g.add_input("images", c=16, h=H, w=W, is_1d=False)
    g.add_conv2d("stem", "images", "stem_out", 16, 32, 3, 3, P["w_stem"], P["b_stem"], stride=1, pad=1, act="silu")
    g.add_conv2d("c2f_cv1", "stem_out", "c2f_cv1_out", 32, 32, 1, 1, P["w_cv1"], P["b_cv1"], stride=1, pad=0, act="silu")
    g.add_slice("c2f_split", "c2f_cv1_out", ["c2f_a", "c2f_b"], [16, 16])
    g.add_conv2d("c2f_bn1", "c2f_b", "c2f_bn1_out", 16, 16, 3, 3, P["w_bn1"], P["b_bn1"], stride=1, pad=1, act="silu")
    g.add_conv2d("c2f_bn2", "c2f_bn1_out", "c2f_bn2_out", 16, 16, 3, 3, P["w_bn2"], P["b_bn2"], stride=1, pad=1, act="none", res_blob="c2f_b")
    g.add_concat("c2f_cat", ["c2f_a", "c2f_b", "c2f_bn2_out"], "c2f_cat_out")
    g.add_conv2d("c2f_cv2", "c2f_cat_out", "c2f_out", 48, 32, 1, 1, P["w_cv2"], P["b_cv2"], stride=1, pad=0, act="silu")
    g.add_conv2d("sppf_cv1", "c2f_out", "sp1", 32, 16, 1, 1, P["w_sp1"], P["b_sp1"], stride=1, pad=0, act="silu")
    g.add_maxpool("sppf_m1", "sp1", "m1", kernel_size=5, stride=1, pad=2)
    g.add_maxpool("sppf_m2", "m1", "m2", kernel_size=5, stride=1, pad=2)
    g.add_maxpool("sppf_m3", "m2", "m3", kernel_size=5, stride=1, pad=2)
    g.add_concat("sppf_cat", ["sp1", "m1", "m2", "m3"], "sp_cat")
    g.add_conv2d("sppf_cv2", "sp_cat", "out", 64, 32, 1, 1, P["w_sp2"], P["b_sp2"], stride=1, pad=0, act="silu")
    g.set_output("out")
    return g, P


def yolo_block_reference(P):
    silu = lambda v: v / (1 + np.exp(-v))
    conv = lambda x, w, b, pad: I.conv2d_direct(x, w, b, 1, pad)

    def pool5(x):
        xp = np.pad(x, ((0, 0), (2, 2), (2, 2)), constant_values=-65504.0)
        out = np.full_like(x, -65504.0)
        for dy in range(5):
            for dx in range(5):
                out = np.maximum(out, xp[:, dy: dy + x.shape[1], dx: dx + x.shape[2]])
        return out

    s = silu(conv(P["x"], P["w_stem"], P["b_stem"], 1))
    c1 = silu(conv(s, P["w_cv1"], P["b_cv1"], 0))
    ca, cb = c1[:16], c1[16:]
    bn1 = silu(conv(cb, P["w_bn1"], P["b_bn1"], 1))
    bn2 = conv(bn1, P["w_bn2"], P["b_bn2"], 1) + cb
    c2 = silu(conv(np.concatenate([ca, cb, bn2]), P["w_cv2"], P["b_cv2"], 0))
    sp1 = silu(conv(c2, P["w_sp1"], P["b_sp1"], 0))
    m1 = pool5(sp1); m2 = pool5(m1); m3 = pool5(m2)
    return silu(conv(np.concatenate([sp1, m1, m2, m3]), P["w_sp2"], P["b_sp2"], 0))


@pytest.mark.parametrize("reuse", [True, False])
def test_image_graph_compiles_to_waves_pools_and_halo_clears(reuse, tmp_path):
    g, _ = _yolo_block(np.random.default_rng(42), reuse=reuse)
    plan = g.compile()
    s = plan.summary
    assert s["input_shape"] == [16, 64, 64] and s["output_shape"] == [32, 64, 64]
    assert s["num_waves"] == 7 and s["num_eliminated_concats"] == 2 and s["num_eliminated_splits"] == 1
    types = [c["type"] for c in s["cmds"] if c["type"] != "HALO_CLEAR"]
    assert types == ["K44_WAVE"] * 6 + ["MAXPOOL_5X5"] * 3 + ["K44_WAVE"]
    assert ("HALO_CLEAR" in [c["type"] for c in s["cmds"]]) == reuse        # recycled regions need their halos cleared, fresh ones never do
    stem = s["cmds"][[c["name"] for c in s["cmds"]].index("stem")]
    assert stem["B_raw"] == 16 * 9 and stem["B"] == 160 and stem["Cout"] == 32 and stem["h_out"] == 64 and stem["w_out"] == 64
    # the container round trip of an image plan
    path = tmp_path / "block.tcff"
    assert plan.save_tcff(path) == 7
    plan.load_tcff_weights(path)
    if not reuse:
        lay = I.Layout2D(64, 64)
        assert s["canvas_elems"] >= 240 * lay.plane       # 16 + 32 + 32 + 16 + 16 + 32 + 16 + 3 * 16 + 32 planes, none shared


def test_image_graph_rejects_what_it_cannot_lay_out():
    g = WaveGraph()
    g.add_input("img", 3, 32, 32)
    with pytest.raises(WaveError, match="1x1 .* and 3x3"):
        g.add_conv2d("c", "img", "y", 3, 8, 5, 5, np.zeros((8, 3, 5, 5), np.float32), pad=2)
    with pytest.raises(WaveError, match="2x2 / stride 2"):
        g.add_maxpool("p", "img", "y", kernel_size=3, stride=1, pad=1)
    g.add_conv2d("c", "img", "y", 3, 8, 3, 3, np.zeros((8, 3, 3, 3), np.float32), pad=1, act="relu")
    g.add_maxpool("p", "y", "z", kernel_size=2, stride=2, pad=0)
    g.add_conv2d("bad", "z", "q", 8, 8, 1, 1, np.zeros((8, 8, 1, 1), np.float32), pad=0, res_blob="y")   # residual at another resolution
    with pytest.raises(WaveError, match="wrong shape"):
        g.compile()


def test_several_frames_per_wave_scale_the_plan():
    """wavec_set_batch_size on an image graph: channel stride = frames x frame stride, every tile table lists all frames'
    tiles, arithmetic and canvas scale with the frame count; masked layouts refuse frame counts whose planes leave the
    16-bit quad offset of their tile table."""
    g1, _ = _yolo_block(np.random.default_rng(42), 48, 40, False)
    s1 = g1.compile().summary
    g3, _ = _yolo_block(np.random.default_rng(42), 48, 40, False)
    g3._lib.wavec_set_batch_size(g3._handle, 3)
    s3 = g3.compile().summary
    assert s3["batch_size"] == 3 and s1["batch_size"] == 1
    assert abs(s3["total_gflops"] - 3 * s1["total_gflops"]) < 1e-6 * s3["total_gflops"] + 1e-4
    assert 2.9 * s1["canvas_elems"] < s3["canvas_elems"] < 3.1 * s1["canvas_elems"]
    assert s3["input_shape"] == s1["input_shape"] and s3["output_shape"] == s1["output_shape"]
    big, _ = _yolo_block(np.random.default_rng(42), 48, 40, False)
    big._lib.wavec_set_batch_size(big._handle, 200)          # 200 x 2304 elements per masked plane > 2^18
    with pytest.raises(WaveError, match="no plane layout"):
        big.compile()
