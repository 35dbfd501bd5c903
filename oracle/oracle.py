"""CPU oracle for the wave-executor path — TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module. It is used by `tests/`, by the smoke check
and by the CPU-baseline leg of the benchmark, always as the checker and never as the thing measured
against a target or shipped.

PARITY UNPINNED for output values: the reference has no golden vectors, fixtures or CPU executor
for this path and may not be compiled or run. The oracle is pinned instead by published FNV-1a
known-answer vectors, by numpy.float16 for the FP16 conversions and by a numpy float64 restatement
of the wave arithmetic (`wave_forward_numpy`), see tests/test_oracle.py.

Two layers:
  * `libk44oracle.so` (oracle/k44_oracle.cpp): OpenMP C++ used for anything sizeable;
  * pure numpy / Python twins of the same functions for cross-checking the C++ and for the
    `.tcff` container (reader and writer written against the byte layout of
    wavec/k44_tcff_io.hpp:100-300, 319-428).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import struct
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None

u8p = ctypes.POINTER(ctypes.c_uint8)
u16p = ctypes.POINTER(ctypes.c_uint16)
u32p = ctypes.POINTER(ctypes.c_uint32)
f32p = ctypes.POINTER(ctypes.c_float)


def _cpu_tag() -> str:
    """The oracle is built with -march=native; key the binary on the host's CPU flags so that a
    binary built on one machine is never loaded on a different micro-architecture."""
    flags = ""
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                flags = line
                break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


def build(force: bool = False) -> Path:
    out = _HERE / "_build" / f"libk44oracle-{_cpu_tag()}.so"
    src = _HERE / "k44_oracle.cpp"
    if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        out.parent.mkdir(exist_ok=True)
        cmd = ["g++", "-O3", "-march=native", "-fopenmp", "-fPIC", "-std=c++17", "-shared",
               "-o", str(out), str(src)]
        subprocess.run(cmd, check=True)
    return out


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(str(build()))
        L.k44o_fnv1a64.argtypes = [u8p, ctypes.c_uint64]
        L.k44o_fnv1a64.restype = ctypes.c_uint64
        L.k44o_f32_to_f16.argtypes = [f32p, u16p, ctypes.c_uint64]
        L.k44o_f16_to_f32.argtypes = [u16p, f32p, ctypes.c_uint64]
        L.k44o_f64_to_f16.argtypes = [ctypes.POINTER(ctypes.c_double), u16p, ctypes.c_uint64]
        L.k44o_rowmajor_to_wmma.argtypes = [u16p, u16p, ctypes.c_uint32, ctypes.c_uint32]
        L.k44o_wmma_to_rowmajor.argtypes = [u16p, u16p, ctypes.c_uint32, ctypes.c_uint32]
        L.k44o_wave_forward.argtypes = [
            u16p, ctypes.c_uint64, u16p, u32p, u16p, u16p,
            ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_int,
            ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32,
            u32p, u32p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, u8p, ctypes.c_uint32]
        L.k44o_wave_forward.restype = ctypes.c_int
        L.k44o_wave_forward_2d.argtypes = [
            u16p, ctypes.c_uint64, u16p, u32p, u16p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_int,
            ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32, u32p, u32p, ctypes.c_uint32, ctypes.c_int]
        L.k44o_wave_forward_2d.restype = ctypes.c_int
        L.k44o_dot_stage3.argtypes = [u16p, u16p, ctypes.c_uint32, ctypes.c_float, f32p]
        L.k44o_num_threads.restype = ctypes.c_int
        L.k44o_set_num_threads.argtypes = [ctypes.c_int]
        _LIB = L
    return _LIB


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


# ----------------------------------------------------------------------------------------------
# scalar helpers
# ----------------------------------------------------------------------------------------------
def fnv1a64(data: bytes) -> int:
    buf = np.frombuffer(data, dtype=np.uint8)
    if buf.size == 0:
        return lib().k44o_fnv1a64(None, 0)
    return lib().k44o_fnv1a64(_p(buf, u8p), buf.size)


def fnv1a64_py(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def f32_to_f16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().k44o_f32_to_f16(_p(a, f32p), _p(out, u16p), a.size)
    return out


def f64_to_f16(a: np.ndarray) -> np.ndarray:
    """Double -> FP16 bits with a single rounding (what the wave oracle stores)."""
    a = np.ascontiguousarray(a, dtype=np.float64)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().k44o_f64_to_f16(_p(a, ctypes.POINTER(ctypes.c_double)), _p(out, u16p), a.size)
    return out


def f16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().k44o_f16_to_f32(_p(a, u16p), _p(out, f32p), a.size)
    return out


def rowmajor_to_wmma(w: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint16)
    cout, B = w.shape
    out = np.empty(cout * B, dtype=np.uint16)
    lib().k44o_rowmajor_to_wmma(_p(w, u16p), _p(out, u16p), cout, B)
    return out


def wmma_to_rowmajor(wm: np.ndarray, cout: int, B: int) -> np.ndarray:
    wm = np.ascontiguousarray(wm, dtype=np.uint16).reshape(-1)
    out = np.empty((cout, B), dtype=np.uint16)
    lib().k44o_wmma_to_rowmajor(_p(wm, u16p), _p(out, u16p), cout, B)
    return out


def rowmajor_to_wmma_numpy(w: np.ndarray) -> np.ndarray:
    """Index-arithmetic twin of the C++ tile walk (wavec/k44_plan_types.hpp:363-375): destination
    vector g = (tile, lane) takes source vector (n_blk*16 + (lane & 15)) * B/8 + 2*k_blk + (lane >> 4)."""
    cout, B = w.shape
    v = np.ascontiguousarray(w, dtype=np.uint16).reshape(cout * B // 8, 8)
    bv8, bv16 = B // 8, B // 16
    g = np.arange(cout // 16 * bv16 * 32)
    tile, lane = g // 32, g % 32
    src = ((tile // bv16) * 16 + (lane & 15)) * bv8 + 2 * (tile % bv16) + (lane >> 4)
    return v[src].reshape(-1)


# ----------------------------------------------------------------------------------------------
# wave arithmetic
# ----------------------------------------------------------------------------------------------
def wave_forward(canvas: np.ndarray, wave, plan, rows: tuple[int, int] | None = None) -> None:
    """Run one wave in place on `canvas` (uint16 FP16 bits, 1-D) with the C++ oracle."""
    assert canvas.dtype == np.uint16 and canvas.flags.c_contiguous
    toff = plan.tile_offsets()
    r0, r1 = rows if rows is not None else (0, wave.cout)
    shifts = getattr(wave, "shifts", None)
    if shifts is not None:
        shifts = np.ascontiguousarray(shifts, dtype=np.uint8)
        assert shifts.shape == wave.idx.shape
    rc = lib().k44o_wave_forward(
        _p(canvas, u16p), canvas.size, _p(wave.weights, u16p), _p(wave.idx, u32p),
        _p(wave.bias, u16p) if wave.bias is not None else None,
        _p(wave.cout_map, u16p) if wave.cout_map is not None else None,
        wave.cout, wave.group, wave.fan_in, int(wave.act), 1 if wave.has_residual else 0,
        wave.y_off, wave.res_off, wave.x_base_off, plan.pitch,
        _p(toff, u32p), _p(toff, u32p), toff.size, r0, r1,
        _p(shifts, u8p) if shifts is not None else None, int(getattr(wave, "frame_len", 0) or 0))
    if rc != 0:
        raise IndexError("oracle: gather or store offset outside the canvas")


_SQRT1_2 = 0.70710678118654752440


def _act_numpy(v: np.ndarray, act: int) -> np.ndarray:
    if act == 1:
        return np.maximum(v, 0.0)
    if act == 2:
        return 1.0 / (1.0 + np.exp(-v))
    if act == 3:
        return v / (1.0 + np.exp(-v))
    if act == 4:
        return np.maximum(v, 0.1 * v)
    if act == 5:
        from math import erf
        return 0.5 * v * (1.0 + np.vectorize(erf)(v * _SQRT1_2))
    return v


def wave_forward_numpy(canvas: np.ndarray, wave, plan) -> None:
    """float64 numpy restatement of the same formula (small sizes only); independent of the C++."""
    cv = canvas.view(np.float16)
    out_rows = []
    ncols = plan.pitch
    col = np.arange(ncols, dtype=np.int64)
    shifts = getattr(wave, "shifts", None)
    flen = int(getattr(wave, "frame_len", 0) or 0) or ncols
    for j in range(wave.cout):
        irow = wave.idx[j // wave.group].astype(np.int64) + wave.x_base_off
        if shifts is None:
            x = cv[irow[:, None] + col[None, :]].astype(np.float64)          # [B, pitch]
        else:
            sh = shifts[j // wave.group].astype(np.int64)
            x = cv[np.maximum(irow[:, None] + col[None, :] - sh[:, None], 0)].astype(np.float64)
            x = np.where((col[None, :] % flen) >= sh[:, None], x, 0.0)
        w = wave.weights[j].view(np.float16).astype(np.float64)
        acc = w @ x
        if wave.bias is not None:
            acc = acc + float(wave.bias[j:j + 1].view(np.float16)[0])
        oj = int(wave.cout_map[j]) if wave.cout_map is not None else j
        if wave.has_residual:
            r = cv[wave.res_off + oj * plan.pitch + col].astype(np.float64)
            acc = _act_numpy(acc + r, wave.act) if wave.cout_map is not None else _act_numpy(acc, wave.act) + r
        else:
            acc = _act_numpy(acc, wave.act)
        out_rows.append((oj, acc.astype(np.float16)))       # one rounding, from double
    for oj, row in out_rows:
        cv[wave.y_off + oj * plan.pitch: wave.y_off + (oj + 1) * plan.pitch] = row


def make_canvas(plan, x_bits: np.ndarray) -> np.ndarray:
    """Zero canvas with the input rows written at `input_off` (input is [input_c, pitch] FP16 bits)."""
    canvas = np.zeros(plan.canvas_elems, dtype=np.uint16)
    x = np.ascontiguousarray(x_bits, dtype=np.uint16).reshape(plan.input_c, plan.pitch)
    canvas[plan.input_off: plan.input_off + x.size] = x.reshape(-1)
    return canvas


def run_plan(plan, x_bits: np.ndarray, use_numpy: bool = False) -> np.ndarray:
    """Execute every wave in order; returns the final canvas (FP16 bits)."""
    canvas = make_canvas(plan, x_bits)
    for w in plan.waves:
        (wave_forward_numpy if use_numpy else wave_forward)(canvas, w, plan)
    return canvas


def compare(got_bits: np.ndarray, want_bits: np.ndarray, rtol: float = 2e-3, atol: float = 1e-3):
    """Tolerance check used by every output-parity test: |got - want| <= atol + rtol*|want|.
    Returns (ok, max_abs_err, worst_index)."""
    g = np.asarray(got_bits).view(np.float16).astype(np.float64).reshape(-1)
    w = np.asarray(want_bits).view(np.float16).astype(np.float64).reshape(-1)
    if g.shape != w.shape:
        return False, float("inf"), -1
    err = np.abs(g - w)
    bad = ~(err <= atol + rtol * np.abs(w))
    bad |= np.isnan(g) != np.isnan(w)
    k = int(np.argmax(np.where(np.isnan(err), np.inf, err))) if err.size else -1
    return (not bool(bad.any())), (float(err[k]) if err.size else 0.0), k


# ----------------------------------------------------------------------------------------------
# .tcff container, pure Python (byte layout: wavec/k44_tcff_io.hpp:100-300; reader rules :319-428)
# ----------------------------------------------------------------------------------------------
TAG_MAGIC, TAG_PARAMS, TAG_AUX, TAG_HASH, TAG_GEOM = 0x8440, 0x8441, 0x8442, 0x8443, 0x8444
MAGIC_WAVE = 0x45564157
_ACT = ["NONE", "RELU", "SIGMOID", "SILU", "LEAKY_RELU"]


def _pad256(b: bytearray) -> None:
    b.extend(b"\0" * (-len(b) % 256))


def tcff_write(plan, prefix: str = "K44Model", include_geometry: bool = True) -> bytes:
    """Serialise a plan. Header 0..255, then per wave: weights (16x16-tile order) | idx | bias, each
    padded to 256, hashed with FNV-1a-64 including the padding, followed by a 21/22-entry IFD and
    its 2-byte-aligned external values, padded to 256. Canvas pages are never written."""
    out = bytearray()
    out += b"II" + struct.pack("<HI", 42, 0) + b"TCFFv1.0"
    canvas_bytes = (plan.canvas_elems * 2) & 0xFFFFFFFF
    out += struct.pack("<IIII", 256, len(plan.waves), canvas_bytes, 1)
    out += struct.pack("<Q", fnv1a64_py(bytes(out[8:32])))
    _pad256(out)
    prev_ptr = 4
    n = len(plan.waves)
    for wi, w in enumerate(plan.waves):
        start = len(out)
        w_off = len(out)
        wbytes = rowmajor_to_wmma_numpy(w.weights).tobytes()
        out += wbytes
        _pad256(out)
        idx_off = len(out)
        ibytes = w.idx.astype("<u4").tobytes()
        out += ibytes
        _pad256(out)
        b_off = len(out)
        bias = w.bias if w.bias is not None else np.zeros(w.cout, dtype=np.uint16)
        bbytes = bias.astype("<u2").tobytes()
        out += bbytes
        _pad256(out)
        end = len(out)
        h = fnv1a64(bytes(out[start:end]))
        ifd_off = len(out)
        out[prev_ptr:prev_ptr + 4] = struct.pack("<I", ifd_off)
        ntags = 21 + (1 if include_geometry else 0)
        ext_base = ifd_off + 2 + ntags * 12 + 4
        ext = bytearray()

        def add(data: bytes) -> int:
            if len(ext) & 1:
                ext.append(0)
            off = ext_base + len(ext)
            ext.extend(data)
            return off

        act_name = _ACT[w.act] if w.act < len(_ACT) else "NONE"
        page = f"{prefix}_Wave_{wi:03d}_{w.fan_in}x{w.cout}_S{w.group}".encode()[:127] + b"\0"
        desc = (f"TCFF {prefix} Wave {wi}/{n} | Cin={w.cin} Cout={w.cout}(log={w.logical_cout}) B={w.fan_in} "
                f"S={w.group} Act={act_name} Res={int(w.has_residual)} | W=0x{w_off:x} Idx=0x{idx_off:x} "
                f"Bias=0x{b_off:x} | FNV1a64=0x{h:016x}").encode()[:319] + b"\0"
        desc_off = add(desc)
        page_off = add(page)
        rat_off = add(struct.pack("<II", 1, 1))
        params = [w.cin, w.cout, w.fan_in, w.group, 16, 3, w.act, int(w.has_residual), w.h_out, w.w_out]
        wp_off = add(struct.pack(f"<{len(params)}I", *params))
        aux = [w_off, len(wbytes), idx_off, len(ibytes), b_off, len(bbytes), w.src_off & 0xFFFFFFFF,
               w.y_off & 0xFFFFFFFF, start, end, w.res_off & 0xFFFFFFFF]
        aux_off = add(struct.pack(f"<{len(aux)}I", *aux))
        hash_off = add(struct.pack("<II", h & 0xFFFFFFFF, h >> 32))
        entries = [(254, 4, 1, 2), (256, 4, 1, w.fan_in), (257, 4, 1, w.cout), (258, 3, 1, 16), (259, 3, 1, 1),
                   (262, 3, 1, 1), (266, 3, 1, 1), (270, 2, len(desc), desc_off), (273, 4, 1, w_off),
                   (277, 3, 1, 1), (278, 4, 1, w.cout), (279, 4, 1, len(wbytes)), (282, 5, 1, rat_off),
                   (283, 5, 1, rat_off), (285, 2, len(page), page_off), (297, 3, 2, wi | (n << 16)),
                   (339, 3, 1, 3), (TAG_MAGIC, 4, 1, MAGIC_WAVE), (TAG_PARAMS, 4, len(params), wp_off),
                   (TAG_AUX, 4, len(aux), aux_off), (TAG_HASH, 4, 2, hash_off)]
        if include_geometry:
            tokens = max(1, w.w_out)
            geom = [2 if tokens > 1 else 1, tokens, w.logical_cout, 1, 1, 1, plan.pitch, 1, 1, 0]
            geom_off = add(struct.pack(f"<{len(geom)}I", *geom))
            entries.append((TAG_GEOM, 4, len(geom), geom_off))
        out += struct.pack("<H", len(entries))
        for tag, typ, cnt, val in entries:
            out += struct.pack("<HHII", tag, typ, cnt, val & 0xFFFFFFFF)
        prev_ptr = len(out)
        out += struct.pack("<I", 0)
        out += ext
        _pad256(out)
    return bytes(out)


def tcff_read(data: bytes) -> dict:
    """Parse a container; verifies the master hash and every wave hash. Returns
    {'canvas_bytes', 'flags', 'waves': [{'params', 'aux', 'weights_wmma', 'idx', 'bias', 'hash', 'geom'}]}"""
    if len(data) < 256 or data[:2] != b"II" or struct.unpack_from("<H", data, 2)[0] != 42:
        raise ValueError("not a little-endian TIFF container")
    if data[8:16] != b"TCFFv1.0":
        raise ValueError("missing TCFFv1.0 magic")
    if struct.unpack_from("<Q", data, 32)[0] != fnv1a64_py(data[8:32]):
        raise ValueError("master header hash mismatch")
    align, nw, canvas_bytes, flags = struct.unpack_from("<IIII", data, 16)
    waves = []
    ifd = struct.unpack_from("<I", data, 4)[0]
    while ifd:
        if ifd + 2 > len(data):
            raise ValueError("IFD offset past end of file")
        ntags = struct.unpack_from("<H", data, ifd)[0]
        tags = {}
        for i in range(ntags):
            tag, typ, cnt, val = struct.unpack_from("<HHII", data, ifd + 2 + 12 * i)
            tags[tag] = (typ, cnt, val)
        nxt = struct.unpack_from("<I", data, ifd + 2 + 12 * ntags)[0]
        if tags.get(TAG_MAGIC, (0, 0, 0))[2] == MAGIC_WAVE:
            _, acnt, aoff = tags[TAG_AUX]
            if acnt < 10:
                raise ValueError("aux tag too short")
            aux = list(struct.unpack_from(f"<{acnt}I", data, aoff))
            h = struct.unpack_from("<Q", data, tags[TAG_HASH][2])[0]
            if aux[9] > len(data) or fnv1a64(data[aux[8]:aux[9]]) != h:
                raise ValueError(f"wave {len(waves)} hash mismatch")
            _, pcnt, poff = tags[TAG_PARAMS]
            params = list(struct.unpack_from(f"<{pcnt}I", data, poff))
            geom = None
            if TAG_GEOM in tags:
                _, gcnt, goff = tags[TAG_GEOM]
                geom = list(struct.unpack_from(f"<{gcnt}I", data, goff))
            waves.append({
                "params": params, "aux": aux, "hash": h, "geom": geom,
                "weights_wmma": np.frombuffer(data, dtype="<u2", count=aux[1] // 2, offset=aux[0]).copy(),
                "idx": np.frombuffer(data, dtype="<u4", count=aux[3] // 4, offset=aux[2]).copy(),
                "bias": np.frombuffer(data, dtype="<u2", count=aux[5] // 2, offset=aux[4]).copy(),
            })
        ifd = nxt
    if len(waves) != nw:
        raise ValueError("wave count does not match the header")
    return {"canvas_bytes": canvas_bytes, "flags": flags, "alignment": align, "waves": waves}
