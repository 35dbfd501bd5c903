"""Native plan API (include/k44b.h): device-resident canvas, caller-supplied stream, plans built from
arrays or a `.tcff` file. PyTorch is used only to view device memory and to name streams."""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from ._lib import PlaneGeom, WaveDesc, WaveInfo, get_lib, last_error
from .plan import Plan, Wave

PATH_AUTO, PATH_FMA, PATH_UMMA = -1, 0, 1
PATH_AUX, PATH_MMA = 2, 3        # reported by wave_info: element-wise command | general wave kernel on mma.sync


class NativeError(RuntimeError):
    pass


class _CudaView:
    """Minimal __cuda_array_interface__ carrier so that torch can wrap a raw device pointer."""

    def __init__(self, ptr: int, n: int, typestr: str, keepalive):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3}
        self._keepalive = keepalive


def _ptr(a: Optional[np.ndarray]):
    return a.ctypes.data if a is not None else None


def wave_desc(w: Wave, *, device_weights_ptr: int = 0, run_rows: Optional[np.ndarray] = None, run_len: int = 0,
              run_shifts: Optional[np.ndarray] = None):
    """Fill a k44b_wave_desc from a `Wave`. Returns (desc, keepalive list)."""
    d = WaveDesc()
    d.cout, d.logical_cout, d.cin, d.group = w.cout, w.logical_cout, w.cin, w.group
    d.fan_in, d.fan_in_raw, d.act, d.has_residual = w.fan_in, w.fan_in_raw, int(w.act), int(bool(w.has_residual))
    d.y_off, d.src_off, d.res_off, d.x_base_off = int(w.y_off), int(w.src_off), int(w.res_off), int(w.x_base_off)
    keep = [w]
    if run_rows is not None:
        rr = np.ascontiguousarray(run_rows, dtype=np.uint32)
        keep.append(rr)
        d.run_rows, d.run_len, d.idx = rr.ctypes.data, int(run_len), None
        if run_shifts is not None:
            rs = np.ascontiguousarray(run_shifts, dtype=np.uint8)
            keep.append(rs)
            d.shifts = rs.ctypes.data
    else:
        d.idx = _ptr(w.idx)
        if w.shifts is not None:
            d.shifts = _ptr(w.shifts)
    d.frame_len = int(w.frame_len or 0)
    if device_weights_ptr:
        d.weights, d.weights_on_device = device_weights_ptr, 1
    else:
        d.weights, d.weights_on_device = _ptr(w.weights), 0
    d.bias = _ptr(w.bias)
    d.cout_map = _ptr(w.cout_map)
    name = (w.name or "wave").encode()
    keep.append(name)
    d.name = name
    return d, keep


class NativePlan:
    def __init__(self, ptr: int, owned: bool = True, keepalive=None):
        self._lib = get_lib()
        self._ptr = ptr
        self._owned = owned
        self._keepalive = keepalive

    # -- construction ------------------------------------------------------------------------------
    @classmethod
    def create(cls, canvas_elems: int, pitch: int, columns: int, device: int = 0, force_path: int = PATH_AUTO) -> "NativePlan":
        lib = get_lib()
        p = lib.k44b_plan_create(int(device), int(canvas_elems), int(pitch), int(columns), int(force_path))
        if not p:
            raise NativeError(f"plan_create: {last_error()}")
        return cls(p)

    @classmethod
    def from_plan(cls, plan: Plan, device: int = 0, force_path: int = PATH_AUTO) -> "NativePlan":
        np_ = cls.create(plan.canvas_elems, plan.pitch, plan.columns, device, force_path)
        for w in plan.waves:
            np_.add_wave(w)
        np_.set_io(plan.input_off, plan.input_c, plan.output_off, plan.output_c, plan.columns)
        return np_

    @classmethod
    def from_tcff(cls, path, pitch_hint: int = 0, device: int = 0, force_path: int = PATH_AUTO) -> "NativePlan":
        lib = get_lib()
        p = lib.k44b_plan_from_tcff(str(path).encode(), int(pitch_hint), int(device), int(force_path))
        if not p:
            raise NativeError(f"plan_from_tcff: {last_error()}")
        return cls(p)

    def add_wave(self, w: Wave, **kw) -> None:
        d, keep = wave_desc(w, **kw)
        rc = self._lib.k44b_plan_add_wave(self._ptr, ctypes.byref(d))
        del keep
        if rc != 0:
            raise NativeError(f"add_wave: {last_error()}")

    def add_wave_desc(self, d: WaveDesc) -> None:
        if self._lib.k44b_plan_add_wave(self._ptr, ctypes.byref(d)) != 0:
            raise NativeError(f"add_wave: {last_error()}")

    def set_io(self, input_off: int, input_c: int, output_off: int, output_c: int, width: int) -> None:
        if self._lib.k44b_plan_set_io(self._ptr, int(input_off), int(input_c), int(output_off), int(output_c), int(width)) != 0:
            raise NativeError(f"set_io: {last_error()}")

    def close(self) -> None:
        if self._ptr and self._owned:
            self._lib.k44b_plan_destroy(self._ptr)
        self._ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- inspection ----------------------------------------------------------------------------------
    @property
    def num_waves(self) -> int:
        return self._lib.k44b_num_waves(self._ptr)

    @property
    def canvas_elems(self) -> int:
        return int(self._lib.k44b_canvas_elems(self._ptr))

    def wave_info(self, i: int) -> WaveInfo:
        info = WaveInfo()
        if self._lib.k44b_wave_info(self._ptr, i, ctypes.byref(info)) != 0:
            raise NativeError(f"wave_info: {last_error()}")
        return info

    @property
    def launch_count(self) -> int:
        return int(self._lib.k44b_launch_count(self._ptr))

    def canvas_tensor(self):
        """The canvas as a torch.float16 CUDA tensor (zero-copy view)."""
        import torch
        view = _CudaView(self._lib.k44b_canvas_ptr(self._ptr), self.canvas_elems, "<f2", self)
        return torch.as_tensor(view, device="cuda")

    # -- execution -----------------------------------------------------------------------------------
    def execute(self, stream=None) -> None:
        """Queue all waves. `stream`: a torch.cuda.Stream, a raw cudaStream_t integer, or None for torch's
        current stream."""
        if stream is None:
            import torch
            sp = torch.cuda.current_stream().cuda_stream
        elif hasattr(stream, "cuda_stream"):
            sp = stream.cuda_stream
        else:
            sp = int(stream)
        if self._lib.k44b_execute(self._ptr, ctypes.c_void_p(sp)) != 0:
            raise NativeError(f"execute: {last_error()}")

    def _stream_ptr(self, stream) -> int:
        if stream is None:
            import torch
            return torch.cuda.current_stream().cuda_stream
        return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)

    def execute_graph(self, stream=None) -> None:
        """Replay all waves as one CUDA graph (built on first use)."""
        if self._lib.k44b_execute_graph(self._ptr, ctypes.c_void_p(self._stream_ptr(stream))) != 0:
            raise NativeError(f"execute_graph: {last_error()}")

    def execute_wave(self, wave: int, stream=None) -> None:
        if self._lib.k44b_execute_wave(self._ptr, int(wave), ctypes.c_void_p(self._stream_ptr(stream))) != 0:
            raise NativeError(f"execute_wave: {last_error()}")

    def infer_f16(self, h_in_ptr: int, h_out_ptr: int, stream=None) -> float:
        """Host FP16 buffers (raw addresses, canvas layout, ideally pinned) -> device waves -> host."""
        ms = ctypes.c_float(0.0)
        rc = self._lib.k44b_infer_f16(self._ptr, ctypes.c_void_p(h_in_ptr), ctypes.c_void_p(h_out_ptr), ctypes.byref(ms),
                                      ctypes.c_void_p(self._stream_ptr(stream)))
        if rc != 0:
            raise NativeError(f"infer_f16: {last_error()}")
        return float(ms.value)

    def infer_f16_begin(self, h_in_ptr: int) -> None:
        """Start uploading an inference's input (host FP16 rows, pinned) into the staging buffer; returns at once."""
        if self._lib.k44b_infer_f16_begin(self._ptr, ctypes.c_void_p(h_in_ptr)) != 0:
            raise NativeError(f"infer_f16_begin: {last_error()}")

    def infer_f16_next(self, h_in_next_ptr: int, h_out_ptr: int, stream=None) -> float:
        """Complete the staged inference (blocking) and, if `h_in_next_ptr` is not 0, start the next upload under its waves."""
        ms = ctypes.c_float(0.0)
        rc = self._lib.k44b_infer_f16_next(self._ptr, ctypes.c_void_p(h_in_next_ptr or None), ctypes.c_void_p(h_out_ptr or None), ctypes.byref(ms),
                                           ctypes.c_void_p(self._stream_ptr(stream)))
        if rc != 0:
            raise NativeError(f"infer_f16_next: {last_error()}")
        return float(ms.value)

    # -- element-wise / attention commands between waves ----------------------------------------------------------
    def add_rmsnorm(self, src_off: int, dst_off: int, dim: int, eps: float = 1e-5, gamma_bits=None, name: str = "rmsnorm") -> None:
        g = None
        if gamma_bits is not None:
            g = np.ascontiguousarray(gamma_bits, dtype=np.uint16)
            g = g.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))
        if self._lib.k44b_plan_add_rmsnorm(self._ptr, name.encode(), int(src_off), int(dst_off), int(dim), float(eps), g) != 0:
            raise NativeError(f"add_rmsnorm: {last_error()}")

    def add_swiglu(self, gate_off: int, up_off: int, dst_off: int, rows: int, name: str = "swiglu") -> None:
        if self._lib.k44b_plan_add_swiglu(self._ptr, name.encode(), int(gate_off), int(up_off), int(dst_off), int(rows)) != 0:
            raise NativeError(f"add_swiglu: {last_error()}")

    def add_rope_attn(self, q_off, k_off, v_off, out_off, h_q, h_kv, head_dim, seq_len, theta=10000.0, llama3=False, name="rope_attn") -> None:
        if self._lib.k44b_plan_add_rope_attn(self._ptr, name.encode(), int(q_off), int(k_off), int(v_off), int(out_off), int(h_q), int(h_kv),
                                             int(head_dim), float(theta), int(bool(llama3)), int(seq_len)) != 0:
            raise NativeError(f"add_rope_attn: {last_error()}")

    def add_decode_attn(self, q_off, k_off, v_off, out_off, kcache_off, vcache_off, h_q, h_kv, head_dim, max_seq, theta=10000.0, llama3=False,
                        name="decode_attn") -> None:
        if self._lib.k44b_plan_add_decode_attn(self._ptr, name.encode(), int(q_off), int(k_off), int(v_off), int(out_off), int(kcache_off),
                                               int(vcache_off), int(h_q), int(h_kv), int(head_dim), int(max_seq), float(theta), int(bool(llama3))) != 0:
            raise NativeError(f"add_decode_attn: {last_error()}")

    def add_embedding(self, table_dev_ptr: int, vocab: int, dim: int, dst_off: int, name: str = "embedding") -> None:
        """`table_dev_ptr`: FP16 [vocab][dim] row-major in device memory; the caller keeps it alive."""
        if self._lib.k44b_plan_add_embedding(self._ptr, name.encode(), ctypes.c_void_p(int(table_dev_ptr)), int(vocab), int(dim), int(dst_off)) != 0:
            raise NativeError(f"add_embedding: {last_error()}")

    def add_argmax(self, src_off: int, rows: int, advance: bool = False, max_seq: int = 0, name: str = "argmax") -> None:
        if self._lib.k44b_plan_add_argmax(self._ptr, name.encode(), int(src_off), int(rows), int(bool(advance)), int(max_seq)) != 0:
            raise NativeError(f"add_argmax: {last_error()}")

    # -- 2-D image planes -------------------------------------------------------------------------------------------------
    IMAGE_OPS = {"maxpool2": 7, "maxpool5": 8, "upsample2": 9, "space_to_depth": 10, "upconv_scatter": 11, "halo_clear": 12}

    def add_image_wave(self, *, cout, group, fan_in, idx, weights, bias, y_off, act, plane_stride, tile_off_x, tile_off_y, tile_mask,
                       has_residual=False, res_off=0, x_base_off=0, fan_in_raw=0, logical_cout=0, name="conv") -> None:
        """A wave over haloed image planes: `idx` [cout // group, fan_in] tap offsets, `weights` [cout, fan_in] FP16 bits (host),
        tile tables as described in include/k44b.h."""
        keep = [np.ascontiguousarray(idx, dtype=np.uint32), np.ascontiguousarray(weights, dtype=np.uint16),
                np.ascontiguousarray(tile_off_x, dtype=np.uint32), np.ascontiguousarray(tile_off_y, dtype=np.uint32),
                np.ascontiguousarray(bias, dtype=np.uint16) if bias is not None else None, name.encode()]
        d = WaveDesc()
        d.cout, d.logical_cout, d.group, d.fan_in, d.fan_in_raw = int(cout), int(logical_cout or cout), int(group), int(fan_in), int(fan_in_raw or fan_in)
        d.act, d.has_residual, d.y_off, d.res_off, d.x_base_off = int(act), int(bool(has_residual)), int(y_off), int(res_off), int(x_base_off)
        d.idx, d.weights, d.weights_on_device = keep[0].ctypes.data, keep[1].ctypes.data, 0
        d.tile_off_x, d.tile_off_y, d.num_tiles = keep[2].ctypes.data, keep[3].ctypes.data, int(keep[2].size)
        d.tile_mask, d.plane_stride = int(bool(tile_mask)), int(plane_stride)
        d.bias = keep[4].ctypes.data if keep[4] is not None else None
        d.name = keep[5]
        rc = self._lib.k44b_plan_add_wave(self._ptr, ctypes.byref(d))
        del keep
        if rc != 0:
            raise NativeError(f"add_image_wave: {last_error()}")

    def add_image_op(self, op: str, src_off: int, dst_off: int, planes: int, geom_in, geom_out, name: str = "") -> None:
        """`op` in IMAGE_OPS; geometries are (h, w, w_pad, plane_stride) tuples (geom_in may be None for halo_clear)."""
        gi = PlaneGeom(*[int(v) for v in geom_in]) if geom_in is not None else None
        go = PlaneGeom(*[int(v) for v in geom_out])
        rc = self._lib.k44b_plan_add_image_op(self._ptr, self.IMAGE_OPS[op], (name or op).encode(), int(src_off), int(dst_off), int(planes),
                                              ctypes.byref(gi) if gi is not None else None, ctypes.byref(go))
        if rc != 0:
            raise NativeError(f"add_image_op: {last_error()}")

    def set_tokens(self, tokens, stream=None) -> None:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        if self._lib.k44b_plan_set_tokens(self._ptr, t.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(t.size), ctypes.c_void_p(self._stream_ptr(stream))) != 0:
            raise NativeError(f"set_tokens: {last_error()}")

    def next_tokens(self, n: int, stream=None) -> np.ndarray:
        out = np.empty(int(n), dtype=np.int32)
        if self._lib.k44b_plan_get_next_tokens(self._ptr, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(n), ctypes.c_void_p(self._stream_ptr(stream))) != 0:
            raise NativeError(f"next_tokens: {last_error()}")
        return out

    def set_decode_pos(self, pos: int, stream=None) -> None:
        if self._lib.k44b_plan_set_decode_pos(self._ptr, int(pos), ctypes.c_void_p(self._stream_ptr(stream))) != 0:
            raise NativeError(f"set_decode_pos: {last_error()}")

    # -- neuron sharding over several GPUs: rows go straight into the peers' canvases ------------------------------
    def ipc_handles(self):
        """(canvas handle, sync-block handle): two 64-byte CUDA IPC handles for the other ranks' processes."""
        hc, hs = ctypes.create_string_buffer(64), ctypes.create_string_buffer(64)
        if self._lib.k44b_plan_ipc_handles(self._ptr, hc, hs) != 0:
            raise NativeError(f"ipc_handles: {last_error()}")
        return hc.raw, hs.raw

    def set_peers_ipc(self, rank: int, world: int, canvas_handles, sync_handles) -> None:
        """`canvas_handles` / `sync_handles`: one 64-byte handle per rank, indexed by rank (own entries ignored)."""
        hc, hs = b"".join(canvas_handles), b"".join(sync_handles)
        if len(hc) != 64 * world or len(hs) != 64 * world:
            raise NativeError("set_peers_ipc: one 64-byte handle per rank is required")
        if self._lib.k44b_plan_set_peers_ipc(self._ptr, int(rank), int(world), hc, hs) != 0:
            raise NativeError(f"set_peers_ipc: {last_error()}")

    def set_peers_raw(self, rank: int, world: int, canvas_ptrs, sync_ptrs) -> None:
        """Device pointers that are already valid on this GPU (plans of the same process), indexed by rank."""
        arr = ctypes.c_void_p * world
        if self._lib.k44b_plan_set_peers_raw(self._ptr, int(rank), int(world), arr(*canvas_ptrs), arr(*sync_ptrs)) != 0:
            raise NativeError(f"set_peers_raw: {last_error()}")

    def peer_latency(self, peer_rank: int, initiator: bool, iters: int = 1000, payload_bytes: int = 0, stream=None) -> float:
        """Nanoseconds per signalling round trip with `peer_rank` (see k44b_plan_peer_latency); both ranks must call it."""
        ns = ctypes.c_float(0.0)
        if self._lib.k44b_plan_peer_latency(self._ptr, int(peer_rank), int(bool(initiator)), int(iters), int(payload_bytes), ctypes.byref(ns),
                                            ctypes.c_void_p(self._stream_ptr(stream))) != 0:
            raise NativeError(f"peer_latency: {last_error()}")
        return float(ns.value)

    def launch_hulls(self) -> np.ndarray:
        """uint64 [launches, 4]: per launch of a step, the canvas intervals {read_lo, read_hi, write_lo, write_hi} it may touch."""
        n = self._lib.k44b_plan_num_launches(self._ptr)
        if n < 0:
            raise NativeError(f"num_launches: {last_error()}")
        out = np.zeros((n, 4), dtype=np.uint64)
        if n and self._lib.k44b_plan_launch_hulls(self._ptr, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), n) != 0:
            raise NativeError(f"launch_hulls: {last_error()}")
        return out

    def set_peer_hulls(self, hulls: np.ndarray) -> None:
        """`hulls`: uint64 [world, launches, 4], the `launch_hulls()` tables of all ranks, indexed by rank."""
        h = np.ascontiguousarray(hulls, dtype=np.uint64)
        if h.ndim != 3 or h.shape[2] != 4:
            raise NativeError("set_peer_hulls: expected an array of shape [world, launches, 4]")
        if self._lib.k44b_plan_set_peer_hulls(self._ptr, int(h.shape[0]), h.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), int(h.shape[1])) != 0:
            raise NativeError(f"set_peer_hulls: {last_error()}")

    @property
    def canvas_ptr(self) -> int:
        return int(self._lib.k44b_canvas_ptr(self._ptr))

    @property
    def sync_ptr(self) -> int:
        p = self._lib.k44b_plan_sync_ptr(self._ptr)
        if not p:
            raise NativeError(f"sync_ptr: {last_error()}")
        return int(p)

    def status(self) -> int:
        st = ctypes.c_uint32(0)
        rc = self._lib.k44b_status(self._ptr, ctypes.byref(st))
        if rc != 0:
            raise NativeError(f"status {st.value:#x}: {last_error()}")
        return st.value

    def status_code(self) -> int:
        """Like `status`, but a non-zero kernel status is returned instead of raised (the word is cleared either way)."""
        st = ctypes.c_uint32(0)
        self._lib.k44b_status(self._ptr, ctypes.byref(st))
        return st.value

    def infer_f32(self, x: np.ndarray, out_elems: int):
        x32 = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(out_elems, dtype=np.float32)
        ms = ctypes.c_float(0.0)
        f32p = ctypes.POINTER(ctypes.c_float)
        rc = self._lib.k44b_infer_f32(self._ptr, x32.ctypes.data_as(f32p), int(x32.size), out.ctypes.data_as(f32p), int(out.size), ctypes.byref(ms))
        if rc != 0:
            raise NativeError(f"infer_f32: {last_error()}")
        return out, float(ms.value)

    def weights_rowmajor(self, wave: int):
        """Unpack wave `wave`'s packed device weights to a [cout, fan_in] uint16 torch tensor."""
        import torch
        info = self.wave_info(wave)
        t = torch.empty((info.cout, info.fan_in), dtype=torch.int16, device="cuda")
        if self._lib.k44b_wave_weights_rowmajor(self._ptr, wave, ctypes.c_void_p(t.data_ptr())) != 0:
            raise NativeError(f"weights_rowmajor: {last_error()}")
        return t


def compute_peer_slack(hulls: np.ndarray) -> np.ndarray:
    """Host-only: per launch, how many of the launches just before it a sharded rank need not wait for (see k44b.h)."""
    h = np.ascontiguousarray(hulls, dtype=np.uint64)
    out = np.zeros(h.shape[1], dtype=np.uint32)
    get_lib().k44b_compute_peer_slack(h.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), int(h.shape[0]), int(h.shape[1]),
                                      out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)))
    return out


def fill_normal_f16(tensor, seed: int, scale: float) -> None:
    """Fill a CUDA float16 tensor with scale*N(0,1) from a stateless hash (library kernel)."""
    import torch
    lib = get_lib()
    rc = lib.k44b_fill_normal_f16(ctypes.c_void_p(tensor.data_ptr()), tensor.numel(), int(seed), float(scale),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise NativeError(f"fill_normal_f16: {last_error()}")


def analyze_gather(w: Wave, pitch: int, canvas_elems: int):
    """Host-only: returns (rows per box or 0, run table as uint32 array)."""
    lib = get_lib()
    d, keep = wave_desc(w)
    cap = (w.cout // w.group) * ((w.fan_in + 63) // 64 * 64)       # at most one entry per synapse (scattered rows)
    out = np.zeros(cap, dtype=np.uint32)
    cnt = ctypes.c_uint64(0)
    h = lib.k44b_analyze_gather(ctypes.byref(d), int(pitch), int(canvas_elems), out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)),
                                cap, ctypes.byref(cnt))
    del keep
    if h < 0:
        raise NativeError(f"analyze_gather: {last_error()}")
    return h, out[: cnt.value].copy()
