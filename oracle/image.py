"""CPU restatement of the 2-D image path — TEST INFRASTRUCTURE ONLY (see oracle.py for the rules).

Plane layouts (wavec/k44_plan_types.hpp:517-600), the convolution tap rule (wavec/k44_wave_compiler.hpp:692-807) and the
weight-free glue commands (kernels/common/kernel44_valu_pack.cuh:30-103), each written from the semantics in numpy. A plane
is an image with a zero halo: pixel (y, x) sits at (y + 1) * W_pad + 4 + x.

PARITY UNPINNED for output values, like the 1-D oracle: the reference ships no image fixtures. The pieces here are pinned
against each other: the wave oracle over planes against a direct numpy convolution of the unpadded image
(tests/test_image_oracle.py), which does not share the layout code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import oracle as O


@dataclass
class Layout2D:
    H: int
    W: int
    H_pad: int = 0
    W_pad: int = 0
    masked: bool = False
    plane: int = 0                     # elements per channel plane
    tile_off_x: np.ndarray = field(default=None, repr=False)
    tile_off_y: np.ndarray = field(default=None, repr=False)

    def __post_init__(self):
        H, W = self.H, self.W
        assert W % 4 == 0 and H > 0
        self.H_pad = H + 2
        if W % 64 == 0:
            self.masked = False
            self.W_pad = W + 8
            self.plane = self.H_pad * self.W_pad
            ty, tx = np.meshgrid(np.arange(H), np.arange(W // 64), indexing="ij")
            self.tile_off_x = (ty * self.W_pad + 4 + tx * 64 - 1).reshape(-1).astype(np.uint32)
            self.tile_off_y = ((ty + 1) * self.W_pad + 4 + tx * 64).reshape(-1).astype(np.uint32)
        else:
            self.masked = True
            self.W_pad = W + 4
            tiles = (H * self.W_pad + 63) // 64
            self.plane = (2 * self.W_pad + tiles * 64 + 63) // 64 * 64
            t = np.arange(tiles)
            first = self.W_pad + 4 + 64 * t                    # plane offset of the tile's first element
            self.tile_off_x = (first - self.W_pad - 1).astype(np.uint32)
            rel = (64 * t)[:, None] + 4 * np.arange(16)[None, :]
            pixel = (rel // self.W_pad < H) & (rel % self.W_pad < W)
            mask = (pixel.astype(np.uint32) << np.arange(16, dtype=np.uint32)[None, :]).sum(axis=1).astype(np.uint32)
            self.tile_off_y = (((first >> 2) & 0xFFFF).astype(np.uint32) | (mask << np.uint32(16))).astype(np.uint32)

    @property
    def num_tiles(self) -> int:
        return int(self.tile_off_x.size)

    def pixel(self, y, x):
        return (y + 1) * self.W_pad + 4 + x

    def tap(self, plane_off: int, dy: int, dx: int) -> int:
        return plane_off + (1 + dy) * self.W_pad + (1 + dx)


def to_planes(img_f16_bits: np.ndarray, lay: Layout2D) -> np.ndarray:
    """[C, H, W] FP16 bits -> [C, plane] with zero halo."""
    C = img_f16_bits.shape[0]
    out = np.zeros((C, lay.plane), dtype=np.uint16)
    rows = (np.arange(lay.H)[:, None] + 1) * lay.W_pad + 4 + np.arange(lay.W)[None, :]
    out[:, rows.reshape(-1)] = img_f16_bits.reshape(C, -1)
    return out


def from_planes(planes: np.ndarray, lay: Layout2D) -> np.ndarray:
    rows = (np.arange(lay.H)[:, None] + 1) * lay.W_pad + 4 + np.arange(lay.W)[None, :]
    return planes[:, rows.reshape(-1)].reshape(planes.shape[0], lay.H, lay.W)


@dataclass
class ImageWave:
    """A wave over image planes: weights [cout, fan_in] FP16 bits, idx [cout // group, fan_in] element offsets (tap rule)."""
    cout: int
    group: int
    fan_in: int
    idx: np.ndarray
    weights: np.ndarray
    bias: np.ndarray | None
    y_off: int
    act: int
    lay: Layout2D
    has_residual: bool = False
    res_off: int = 0
    x_base_off: int = 0
    name: str = "conv"


def conv_wave(lay: Layout2D, in_planes: list[int], w_f16_bits: np.ndarray, bias_bits, y_off: int, act: int, kh: int = 3, kw: int = 3,
              group: int = 16, residual_off: int | None = None, name: str = "conv") -> ImageWave:
    """Stride-1 'same' convolution as a wave: synapse ch * taps + ky * kw + kx reads plane(ch) at tap (ky - kh//2, kx - kw//2)."""
    cout, cin = w_f16_bits.shape[0], w_f16_bits.shape[1]
    taps = kh * kw
    cout_pad = max(16, (cout + 15) // 16 * 16)
    raw = cin * taps
    fan_in = max(64, (raw + 31) // 32 * 32)
    assert cout_pad % group == 0
    offs = np.zeros(fan_in, dtype=np.uint32)
    for ch in range(cin):
        for ky in range(kh):
            for kx in range(kw):
                offs[ch * taps + ky * kw + kx] = lay.tap(in_planes[ch], ky - kh // 2, kx - kw // 2)
    w = np.zeros((cout_pad, fan_in), dtype=np.uint16)
    w[:cout, :raw] = w_f16_bits.reshape(cout, raw)
    b = np.zeros(cout_pad, dtype=np.uint16)
    if bias_bits is not None:
        b[:cout] = bias_bits
    return ImageWave(cout=cout_pad, group=group, fan_in=fan_in, idx=np.tile(offs, (cout_pad // group, 1)), weights=w, bias=b, y_off=y_off, act=act,
                     lay=lay, has_residual=residual_off is not None, res_off=residual_off or 0, name=name)


def wave_forward_2d(canvas: np.ndarray, w: ImageWave) -> None:
    """Run one image wave in place on the canvas (uint16 FP16 bits) with the C++ oracle."""
    L = O.lib()
    idx = np.ascontiguousarray(w.idx, dtype=np.uint32)
    wt = np.ascontiguousarray(w.weights, dtype=np.uint16)
    rc = L.k44o_wave_forward_2d(
        O._p(canvas, O.u16p), canvas.size, O._p(wt, O.u16p), O._p(idx, O.u32p), O._p(w.bias, O.u16p) if w.bias is not None else None,
        w.cout, w.group, w.fan_in, int(w.act), 1 if w.has_residual else 0, int(w.y_off), int(w.res_off), int(w.x_base_off), int(w.lay.plane),
        O._p(w.lay.tile_off_x, O.u32p), O._p(w.lay.tile_off_y, O.u32p), w.lay.num_tiles, 1 if w.lay.masked else 0)
    if rc != 0:
        raise IndexError("oracle: an image wave leaves the canvas")


# ---- weight-free glue on planes (FP16 values are only moved or compared, never rounded) ---------------------------
def _img(canvas, off, planes, lay):
    return from_planes(canvas[off: off + planes * lay.plane].reshape(planes, lay.plane), lay)


def _put(canvas, off, img_bits, lay):
    """Write the pixels of [C, H, W] into the planes at `off`, leaving halos as they are."""
    C = img_bits.shape[0]
    view = canvas[off: off + C * lay.plane].reshape(C, lay.plane)
    rows = (np.arange(lay.H)[:, None] + 1) * lay.W_pad + 4 + np.arange(lay.W)[None, :]
    view[:, rows.reshape(-1)] = img_bits.reshape(C, -1)


def maxpool2(canvas, src, dst, planes, lin: Layout2D, lout: Layout2D):
    x = _img(canvas, src, planes, lin).view(np.float16)
    m = np.maximum(np.maximum(x[:, 0::2, 0::2], x[:, 0::2, 1::2]), np.maximum(x[:, 1::2, 0::2], x[:, 1::2, 1::2]))
    _put(canvas, dst, np.ascontiguousarray(m).view(np.uint16), lout)


def maxpool5(canvas, src, dst, planes, lay: Layout2D):
    x = _img(canvas, src, planes, lay).view(np.float16).astype(np.float32)
    xp = np.pad(x, ((0, 0), (2, 2), (2, 2)), constant_values=-65504.0)
    m = np.full_like(x, -65504.0)
    for dy in range(5):
        for dx in range(5):
            m = np.maximum(m, xp[:, dy: dy + lay.H, dx: dx + lay.W])
    _put(canvas, dst, m.astype(np.float16).view(np.uint16), lay)


def upsample2(canvas, src, dst, planes, lin: Layout2D, lout: Layout2D):
    x = _img(canvas, src, planes, lin)
    _put(canvas, dst, np.repeat(np.repeat(x, 2, axis=1), 2, axis=2), lout)


def space_to_depth(canvas, src, dst, cin, lin: Layout2D, lout: Layout2D):
    x = _img(canvas, src, cin, lin)
    out = np.zeros((4 * cin, lout.H, lout.W), dtype=np.uint16)
    for py in range(2):
        for px in range(2):
            out[2 * py + px:: 4] = x[:, py::2, px::2]
    _put(canvas, dst, out, lout)


def upconv_scatter(canvas, src, dst, cout, lin: Layout2D, lout: Layout2D):
    q = _img(canvas, src, 4 * cout, lin)
    out = np.zeros((cout, lout.H, lout.W), dtype=np.uint16)
    for py in range(2):
        for px in range(2):
            out[:, py::2, px::2] = q[(2 * py + px) * cout: (2 * py + px + 1) * cout]
    _put(canvas, dst, out, lout)


def halo_clear(canvas, dst, planes, lay: Layout2D):
    view = canvas[dst: dst + planes * lay.plane].reshape(planes, lay.plane)
    keep = np.zeros(lay.plane, dtype=bool)
    rows = (np.arange(lay.H)[:, None] + 1) * lay.W_pad + 4 + np.arange(lay.W)[None, :]
    keep[rows.reshape(-1)] = True
    view[:, ~keep] = 0


# ---- direct numpy references (no planes, no taps): what the image tests compare against ------------------------------
def conv2d_direct(x: np.ndarray, w: np.ndarray, b: np.ndarray | None, stride: int = 1, pad: int = 0) -> np.ndarray:
    """float64 convolution of [C, H, W] with [O, C, kh, kw] (cross-correlation, as every framework defines it)."""
    x = x.astype(np.float64); w = w.astype(np.float64)
    kh, kw = w.shape[2], w.shape[3]
    xp = np.pad(x, ((0, 0), (pad, pad), (pad, pad)))
    ho = (x.shape[1] + 2 * pad - kh) // stride + 1
    wo = (x.shape[2] + 2 * pad - kw) // stride + 1
    out = np.zeros((w.shape[0], ho, wo))
    for dy in range(kh):
        for dx in range(kw):
            out += np.einsum("oi,iyx->oyx", w[:, :, dy, dx], xp[:, dy: dy + ho * stride: stride, dx: dx + wo * stride: stride])
    if b is not None:
        out += b.astype(np.float64)[:, None, None]
    return out
