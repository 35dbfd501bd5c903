"""Loader for libk44wavec.so (ctypes). The library is the product: there is no Python or CPU
fallback, and a missing library is an error, not a reason to degrade."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_uint8, c_uint16, c_uint32, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libk44wavec.so"
_LIB = None


class WaveDesc(ctypes.Structure):
    """k44b_wave_desc (include/k44b.h)."""
    _fields_ = [
        ("cout", c_uint32), ("logical_cout", c_uint32), ("cin", c_uint32), ("group", c_uint32),
        ("fan_in", c_uint32), ("fan_in_raw", c_uint32), ("act", c_int32), ("has_residual", c_uint32),
        ("y_off", c_uint64), ("src_off", c_uint64), ("res_off", c_uint64), ("x_base_off", c_uint64),
        ("idx", c_void_p), ("run_rows", c_void_p), ("run_len", c_uint32), ("weights_on_device", c_uint32),
        ("weights", c_void_p), ("bias", c_void_p), ("cout_map", c_void_p), ("name", c_char_p),
        ("shifts", c_void_p), ("frame_len", c_uint32),
        ("tile_off_x", c_void_p), ("tile_off_y", c_void_p), ("num_tiles", c_uint32), ("tile_mask", c_uint32), ("plane_stride", c_uint32),
    ]


class PlaneGeom(ctypes.Structure):
    """k44b_plane_geom (include/k44b.h)."""
    _fields_ = [("h", c_uint32), ("w", c_uint32), ("w_pad", c_uint32), ("plane_stride", c_uint32)]


class WaveInfo(ctypes.Structure):
    """k44b_wave_info_t (include/k44b.h)."""
    _fields_ = [
        ("cout", c_uint32), ("group", c_uint32), ("fan_in", c_uint32), ("box_rows", c_uint32),
        ("path", c_int32), ("n_tile", c_uint32), ("k_splits", c_uint32), ("synapses", c_uint64), ("weight_bytes", c_uint64),
        ("m_blocks", c_uint32), ("cta_pairs", c_uint32), ("weights_in_tmem", c_uint32), ("reserved0", c_uint32),
    ]


# name -> (restype, argtypes); the wavec_* block has the prototypes the reference's binding declares
# (wavec/wavec.py:28-132) plus the four C-only entry points.
_f32p, _u16p, _strs = POINTER(c_float), POINTER(c_uint16), POINTER(c_char_p)
PROTOTYPES = {
    "wavec_create": (c_void_p, [c_int, c_int, c_int, c_int]),
    "wavec_destroy": (None, [c_void_p]),
    "wavec_gpu_release": (c_int, [c_void_p]),
    "wavec_add_input": (c_int, [c_void_p, c_char_p, c_int, c_int, c_int, c_int]),
    "wavec_add_flatten": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p]),
    "wavec_add_conv2d": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _f32p, _f32p, c_char_p]),
    "wavec_add_conv2d_f16": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _u16p, _f32p, c_char_p]),
    "wavec_add_linear_f32": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_int, _f32p, _f32p, c_char_p]),
    "wavec_add_linear_f16": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_int, _u16p, _f32p, c_char_p]),
    "wavec_add_linear_bf16": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_int, _u16p, _f32p, c_char_p]),
    "wavec_add_upconv2x2": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, _f32p, _f32p]),
    "wavec_add_maxpool": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_int]),
    "wavec_add_upsample2x": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p]),
    "wavec_add_rmsnorm": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_float, _f32p, c_int]),
    "wavec_add_swiglu": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_char_p]),
    "wavec_add_rope_gqa_attn": (c_int, [c_void_p, c_char_p, c_char_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_int, c_float, c_int]),
    "wavec_add_split": (c_int, [c_void_p, c_char_p, c_char_p, c_int, _strs]),
    "wavec_add_slice": (c_int, [c_void_p, c_char_p, c_char_p, c_int, _strs, POINTER(c_int)]),
    "wavec_add_concat": (c_int, [c_void_p, c_char_p, c_int, _strs, c_char_p]),
    "wavec_set_output": (c_int, [c_void_p, c_char_p]),
    "wavec_set_reuse_canvas": (c_int, [c_void_p, c_int]),
    "wavec_set_batch_size": (c_int, [c_void_p, c_int]),
    "wavec_set_target_preset": (c_int, [c_void_p, c_char_p]),
    "wavec_compile": (c_int, [c_void_p]),
    "wavec_get_summary_json": (c_char_p, [c_void_p]),
    "wavec_save_tcff_ex": (c_int, [c_void_p, c_char_p, c_char_p, c_int, c_int]),
    "wavec_save_tcff": (c_int, [c_void_p, c_char_p, c_char_p]),
    "wavec_load_tcff_weights": (c_int, [c_void_p, c_char_p]),
    "wavec_gpu_init_plan": (c_int, [c_void_p]),
    "wavec_gpu_infer_f32": (c_int, [c_void_p, _f32p, c_int, _f32p, c_int, _f32p]),
    # native additions (include/k44b.h)
    "k44b_plan_create": (c_void_p, [c_int, c_uint64, c_uint32, c_uint32, c_int]),
    "k44b_plan_add_wave": (c_int, [c_void_p, POINTER(WaveDesc)]),
    "k44b_plan_set_io": (c_int, [c_void_p, c_uint64, c_uint32, c_uint64, c_uint32, c_uint32]),
    "k44b_plan_from_tcff": (c_void_p, [c_char_p, c_uint32, c_int, c_int]),
    "k44b_plan_destroy": (None, [c_void_p]),
    "k44b_canvas_ptr": (c_void_p, [c_void_p]),
    "k44b_canvas_elems": (c_uint64, [c_void_p]),
    "k44b_num_waves": (c_int, [c_void_p]),
    "k44b_wave_info": (c_int, [c_void_p, c_int, POINTER(WaveInfo)]),
    "k44b_execute": (c_int, [c_void_p, c_void_p]),
    "k44b_execute_graph": (c_int, [c_void_p, c_void_p]),
    "k44b_execute_wave": (c_int, [c_void_p, c_int, c_void_p]),
    "k44b_infer_f16": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(c_float), c_void_p]),
    "k44b_infer_f16_begin": (c_int, [c_void_p, c_void_p]),
    "k44b_infer_f16_next": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(c_float), c_void_p]),
    "k44b_status": (c_int, [c_void_p, POINTER(c_uint32)]),
    "k44b_infer_f32": (c_int, [c_void_p, _f32p, c_int, _f32p, c_int, _f32p]),
    "k44b_plan_add_rmsnorm": (c_int, [c_void_p, c_char_p, c_uint64, c_uint64, c_uint32, c_float, _u16p]),
    "k44b_plan_add_swiglu": (c_int, [c_void_p, c_char_p, c_uint64, c_uint64, c_uint64, c_uint32]),
    "k44b_plan_add_rope_attn": (c_int, [c_void_p, c_char_p, c_uint64, c_uint64, c_uint64, c_uint64, c_uint32, c_uint32, c_uint32, c_float, c_int, c_uint32]),
    "k44b_plan_add_decode_attn": (c_int, [c_void_p, c_char_p, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_uint32, c_uint32, c_uint32,
                                           c_uint32, c_float, c_int]),
    "k44b_plan_set_decode_pos": (c_int, [c_void_p, c_int, c_void_p]),
    "k44b_plan_add_image_op": (c_int, [c_void_p, c_int, c_char_p, c_uint64, c_uint64, c_uint32, POINTER(PlaneGeom), POINTER(PlaneGeom)]),
    "k44b_plan_add_embedding": (c_int, [c_void_p, c_char_p, c_void_p, c_uint32, c_uint32, c_uint64]),
    "k44b_plan_add_argmax": (c_int, [c_void_p, c_char_p, c_uint64, c_uint32, c_int, c_uint32]),
    "k44b_plan_set_tokens": (c_int, [c_void_p, POINTER(ctypes.c_int32), c_uint32, c_void_p]),
    "k44b_plan_get_next_tokens": (c_int, [c_void_p, POINTER(ctypes.c_int32), c_uint32, c_void_p]),
    "k44b_plan_ipc_handles": (c_int, [c_void_p, c_void_p, c_void_p]),
    "k44b_plan_set_peers_ipc": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "k44b_plan_set_peers_raw": (c_int, [c_void_p, c_int, c_int, POINTER(c_void_p), POINTER(c_void_p)]),
    "k44b_plan_sync_ptr": (c_void_p, [c_void_p]),
    "k44b_plan_peer_latency": (c_int, [c_void_p, c_int, c_int, c_uint32, c_uint32, POINTER(c_float), c_void_p]),
    "k44b_plan_num_launches": (c_int, [c_void_p]),
    "k44b_plan_launch_hulls": (c_int, [c_void_p, POINTER(c_uint64), c_uint64]),
    "k44b_plan_set_peer_hulls": (c_int, [c_void_p, c_int, POINTER(c_uint64), c_uint64]),
    "k44b_compute_peer_slack": (None, [POINTER(c_uint64), c_int, c_uint64, POINTER(c_uint32)]),
    "k44b_launch_count": (c_uint64, [c_void_p]),
    "k44b_wave_weights_rowmajor": (c_int, [c_void_p, c_int, c_void_p]),
    "k44b_wave_forward_static": (c_int, [c_void_p, c_uint64, c_uint32, c_void_p, c_void_p, c_uint32, c_void_p, c_uint32, c_uint32, c_uint32,
                                         c_int, c_uint64, c_uint32, c_void_p, c_char_p, c_uint32]),
    "k44b_set_device": (c_int, [c_void_p, c_int]),
    "k44b_set_force_path": (c_int, [c_void_p, c_int]),
    "k44b_handle_plan": (c_void_p, [c_void_p]),
    "k44b_last_error": (c_char_p, []),
    "k44b_version": (c_char_p, []),
    "k44b_fill_normal_f16": (c_int, [c_void_p, c_uint64, c_uint64, c_float, c_void_p]),
    "k44b_fnv1a64": (c_uint64, [POINTER(c_uint8), c_uint64]),
    "k44b_f32_to_f16": (None, [_f32p, _u16p, c_uint64]),
    "k44b_rowmajor_to_wmma": (None, [_u16p, _u16p, c_uint32, c_uint32]),
    "k44b_wmma_to_rowmajor": (None, [_u16p, _u16p, c_uint32, c_uint32]),
    "k44b_analyze_gather": (c_int, [POINTER(WaveDesc), c_uint32, c_uint64, POINTER(c_uint32), c_uint64, POINTER(c_uint64)]),
}


def get_lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m snntome_b200.build` (needs nvcc). "
                "There is no CPU implementation to fall back to.")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)          # raises AttributeError if a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB


def last_error() -> str:
    return (get_lib().k44b_last_error() or b"").decode("utf-8", "replace")
