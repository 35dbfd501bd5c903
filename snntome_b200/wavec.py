"""Python front end with the class and method names of the reference binding (wavec/wavec.py:147-344):
`WaveGraph.add_* / set_output / compile() -> WavePlan`, `WavePlan.save_tcff / load_tcff_weights /
init_gpu / infer_f32`. Unlike the reference binding, failures of the builder calls are raised instead
of being ignored, and a plan can hand out its device canvas (`WavePlan.native`)."""
from __future__ import annotations

import ctypes
import json
from pathlib import Path
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np

from ._lib import get_lib, last_error

ACT_MAP = {
    None: 0, "none": 0, "identity": 0, "linear": 0,
    "relu": 1, "sigmoid": 2, "silu": 3, "swish": 3, "leaky_relu": 4, "gelu": 5,
}

_f32p = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)


class WaveError(RuntimeError):
    pass


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise WaveError(f"{what}: {last_error()}")


class WavePlan:
    """Compiled plan: `.tcff` I/O and GPU execution (reference: wavec/wavec.py:147-208)."""

    def __init__(self, handle, lib, summary: dict, owner):
        self._handle, self._lib, self.summary = handle, lib, summary
        self._owner = owner            # keeps the WaveGraph (and its handle) alive
        self._gpu_initialized = False

    @property
    def total_gflops(self) -> float:
        return float(self.summary.get("total_gflops", 0.0))

    @property
    def canvas_bytes(self) -> int:
        return int(self.summary.get("canvas_bytes", 0))

    @property
    def num_wave_dispatches(self) -> int:
        return int(self.summary.get("num_waves", 0))

    def save_tcff(self, tcff_path: Union[str, Path], model_prefix: str = "K44Model") -> int:
        _check(self._lib.wavec_save_tcff(self._handle, str(tcff_path).encode(), model_prefix.encode()), "save_tcff")
        return self.num_wave_dispatches

    def load_tcff_weights(self, tcff_path: Union[str, Path]) -> None:
        _check(self._lib.wavec_load_tcff_weights(self._handle, str(tcff_path).encode()), "load_tcff_weights")
        self._gpu_initialized = False

    def init_gpu(self, device: int = 0, force_path: int = -1) -> None:
        if not self._gpu_initialized:
            self._lib.k44b_set_device(self._handle, int(device))
            self._lib.k44b_set_force_path(self._handle, int(force_path))
            _check(self._lib.wavec_gpu_init_plan(self._handle), "init_gpu")
            self._gpu_initialized = True

    def release_gpu(self) -> None:
        self._lib.wavec_gpu_release(self._handle)
        self._gpu_initialized = False

    def infer_f32(self, x: np.ndarray) -> Tuple[np.ndarray, float]:
        """x: dense FP32 [C, 1, W] (or [C, W]) for token graphs, [C, H, W] for image graphs ([B, C, H, W] when the graph was built
        with batch_size B > 1); returns (output in the same arrangement, device milliseconds of the waves)."""
        self.init_gpu()
        x32 = np.ascontiguousarray(x, dtype=np.float32)
        c, h, w = tuple(self.summary["output_shape"])
        b = int(self.summary.get("batch_size", 1))
        out = np.empty((b, c, h, w) if (h > 1 and b > 1) else (c, h, w), dtype=np.float32)
        ms = ctypes.c_float(0.0)
        rc = self._lib.wavec_gpu_infer_f32(self._handle, x32.ctypes.data_as(_f32p), int(x32.size),
                                           out.ctypes.data_as(_f32p), int(out.size), ctypes.byref(ms))
        _check(rc, "infer_f32")
        return out, float(ms.value)

    @property
    def native(self):
        """The executor's plan as a `snntome_b200.native.NativePlan` view (after init_gpu)."""
        from .native import NativePlan
        self.init_gpu()
        ptr = self._lib.k44b_handle_plan(self._handle)
        if not ptr:
            raise WaveError("plan has no GPU state")
        return NativePlan(ptr, owned=False, keepalive=self)


class WaveGraph:
    """Graph builder (reference: wavec/wavec.py:211-344). 1-D token plans and 2-D image plans (convolutions 1x1 / 3x3 with stride
    1 or 2, max-pools 2x2 / 5x5, nearest upsampling, 2x2 transposed convolution) compile."""

    def __init__(self, max_B_per_wave: int = 288, default_S: int = 0, kv_cache_max_seq: int = 2048,
                 fold_rmsnorm_gamma: bool = True, reuse_canvas: bool = False, batch_size: int = 1, target: str = "auto"):
        self._lib = get_lib()
        self._handle = self._lib.wavec_create(int(max_B_per_wave), int(default_S), int(kv_cache_max_seq),
                                              1 if fold_rmsnorm_gamma else 0)
        if not self._handle:
            raise WaveError("wavec_create failed")
        self._lib.wavec_set_reuse_canvas(self._handle, 1 if reuse_canvas else 0)
        self._lib.wavec_set_batch_size(self._handle, int(batch_size))
        self._lib.wavec_set_target_preset(self._handle, target.encode())

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.wavec_destroy(self._handle)
            self._handle = None

    def add_input(self, name: str, c: int, h: int = 1, w: int = 1, is_1d: bool = False) -> str:
        _check(self._lib.wavec_add_input(self._handle, name.encode(), int(c), int(h), int(w), 1 if is_1d else 0), "add_input")
        return name

    def add_linear(self, name: str, in_blob: str, out_blob: str, cin: int, cout: int, weights: np.ndarray,
                   bias: Optional[np.ndarray] = None, act: Optional[str] = None, res_blob: Optional[str] = None) -> str:
        b32 = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
        bp = b32.ctypes.data_as(_f32p) if b32 is not None else None
        res = res_blob.encode() if res_blob else None
        a = ACT_MAP[act] if act in ACT_MAP else int(act)
        if weights.dtype in (np.float16, np.uint16):
            w16 = np.ascontiguousarray(weights).view(np.uint16)
            rc = self._lib.wavec_add_linear_f16(self._handle, name.encode(), in_blob.encode(), out_blob.encode(), int(cin),
                                                int(cout), a, w16.ctypes.data_as(_u16p), bp, res)
        else:
            w32 = np.ascontiguousarray(weights, dtype=np.float32)
            rc = self._lib.wavec_add_linear_f32(self._handle, name.encode(), in_blob.encode(), out_blob.encode(), int(cin),
                                                int(cout), a, w32.ctypes.data_as(_f32p), bp, res)
        _check(rc, "add_linear")
        return out_blob

    def add_conv2d(self, name: str, in_blob: str, out_blob: str, cin: int, cout: int, kh: int, kw: int,
                   weights: np.ndarray, bias: Optional[np.ndarray] = None, stride: int = 1, pad: int = 0,
                   act: Optional[str] = "silu", res_blob: Optional[str] = None) -> str:
        w32 = np.ascontiguousarray(weights, dtype=np.float32)
        b32 = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
        rc = self._lib.wavec_add_conv2d(self._handle, name.encode(), in_blob.encode(), out_blob.encode(), int(cin), int(cout),
                                        int(kh), int(kw), int(stride), int(pad), ACT_MAP.get(act, 0), w32.ctypes.data_as(_f32p),
                                        b32.ctypes.data_as(_f32p) if b32 is not None else None,
                                        res_blob.encode() if res_blob else None)
        _check(rc, "add_conv2d")
        return out_blob

    def _names(self, blobs: Sequence[str]):
        return (ctypes.c_char_p * len(blobs))(*[b.encode() for b in blobs])

    def add_split(self, name: str, in_blob: str, out_blobs: Sequence[str]) -> List[str]:
        _check(self._lib.wavec_add_split(self._handle, name.encode(), in_blob.encode(), len(out_blobs), self._names(out_blobs)), "add_split")
        return list(out_blobs)

    def add_slice(self, name: str, in_blob: str, out_blobs: Sequence[str], slice_sizes: Sequence[int]) -> List[str]:
        sz = (ctypes.c_int * len(slice_sizes))(*[int(s) for s in slice_sizes]) if slice_sizes else None
        _check(self._lib.wavec_add_slice(self._handle, name.encode(), in_blob.encode(), len(out_blobs), self._names(out_blobs), sz), "add_slice")
        return list(out_blobs)

    def add_concat(self, name: str, in_blobs: Sequence[str], out_blob: str) -> str:
        _check(self._lib.wavec_add_concat(self._handle, name.encode(), len(in_blobs), self._names(in_blobs), out_blob.encode()), "add_concat")
        return out_blob

    # Weight-free nodes between waves.
    def add_rmsnorm(self, name, in_blob, out_blob, dim, gamma, eps=1e-5, pre_folded=False):
        g = np.ascontiguousarray(gamma, dtype=np.float32)
        _check(self._lib.wavec_add_rmsnorm(self._handle, name.encode(), in_blob.encode(), out_blob.encode(), int(dim),
                                           ctypes.c_float(eps), g.ctypes.data_as(_f32p), 1 if pre_folded else 0), "add_rmsnorm")

    def add_swiglu(self, name, gate_blob, up_blob, out_blob, dim=0):
        _check(self._lib.wavec_add_swiglu(self._handle, name.encode(), gate_blob.encode(), up_blob.encode(), out_blob.encode()), "add_swiglu")

    def add_rope_gqa_attn(self, name, q_blob, k_blob, v_blob, out_blob, h_q, h_kv, head_dim, rope_theta=10000.0, llama3_scaling=False):
        _check(self._lib.wavec_add_rope_gqa_attn(self._handle, name.encode(), q_blob.encode(), k_blob.encode(), v_blob.encode(),
                                                 out_blob.encode(), int(h_q), int(h_kv), int(head_dim), ctypes.c_float(rope_theta),
                                                 1 if llama3_scaling else 0), "add_rope_gqa_attn")

    def add_maxpool(self, name, in_blob, out_blob, kernel_size=5, stride=1, pad=2):
        _check(self._lib.wavec_add_maxpool(self._handle, name.encode(), in_blob.encode(), out_blob.encode(), int(kernel_size),
                                           int(stride), int(pad)), "add_maxpool")

    def add_upsample2x(self, name, in_blob, out_blob):
        _check(self._lib.wavec_add_upsample2x(self._handle, name.encode(), in_blob.encode(), out_blob.encode()), "add_upsample2x")

    def add_upconv2x2(self, name, in_blob, out_blob, cin, cout, weights, bias=None):
        """2x2 / stride-2 transposed convolution; `weights` [cout, cin, 4] with phase q = 2 * (y & 1) + (x & 1) innermost
        (the C entry point exists in the reference, wavec/k44_wave_executor.cu:761; its Python wrapper has no method for it)."""
        w32 = np.ascontiguousarray(weights, dtype=np.float32)
        b32 = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
        _check(self._lib.wavec_add_upconv2x2(self._handle, name.encode(), in_blob.encode(), out_blob.encode(), int(cin), int(cout),
                                             w32.ctypes.data_as(_f32p), b32.ctypes.data_as(_f32p) if b32 is not None else None), "add_upconv2x2")
        return out_blob

    def set_output(self, out_blob: str) -> None:
        _check(self._lib.wavec_set_output(self._handle, out_blob.encode()), "set_output")

    def compile(self) -> WavePlan:
        _check(self._lib.wavec_compile(self._handle), "compile")
        raw = self._lib.wavec_get_summary_json(self._handle)
        return WavePlan(self._handle, self._lib, json.loads(raw.decode()) if raw else {}, owner=self)
