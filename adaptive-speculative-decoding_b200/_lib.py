"""ctypes binding of libasd_b200.so (the C ABI declared in include/asd_b200.h).

There is no CPU fallback: if the shared library is missing this raises, and the CUDA entry
points raise ``AsdError`` when the device or the kernel launch fails."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class AsdError(RuntimeError):
    pass


class ModelConfigC(ctypes.Structure):
    """mirror of ``asd_model_config`` (include/asd_b200.h)"""
    _fields_ = [("hidden", ctypes.c_int), ("n_layers", ctypes.c_int), ("n_heads", ctypes.c_int),
                ("n_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int), ("ffn", ctypes.c_int),
                ("vocab", ctypes.c_int), ("rms_eps", ctypes.c_float), ("max_tokens", ctypes.c_int),
                ("page_size", ctypes.c_int), ("tp_rank", ctypes.c_int), ("tp_size", ctypes.c_int)]


class MezilixLayerC(ctypes.Structure):
    """mirror of ``asd_mezilix_layer_config``"""
    _fields_ = [("heads", ctypes.c_int), ("dim", ctypes.c_int), ("rot_dim", ctypes.c_int), ("vdim", ctypes.c_int),
                ("kv_rank", ctypes.c_int), ("rot_dims", ctypes.c_int), ("window", ctypes.c_int),
                ("rot_base", ctypes.c_float), ("scale", ctypes.c_float), ("experts", ctypes.c_int),
                ("top", ctypes.c_int), ("ff", ctypes.c_int)]


class MezilixConfigC(ctypes.Structure):
    """mirror of ``asd_mezilix_config``"""
    _fields_ = [("width", ctypes.c_int), ("vocab", ctypes.c_int), ("n_layers", ctypes.c_int), ("eps", ctypes.c_float),
                ("buckets", ctypes.c_int), ("mul_prev", ctypes.c_int), ("mul_cur", ctypes.c_int),
                ("max_tokens", ctypes.c_int), ("page_size", ctypes.c_int), ("ring", ctypes.c_int),
                ("dtype", ctypes.c_int)]


class RivetarLayerC(ctypes.Structure):
    """mirror of ``asd_rivetar_layer_config``"""
    _fields_ = [("type", ctypes.c_int), ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("dim", ctypes.c_int),
                ("vdim", ctypes.c_int), ("rot_dim", ctypes.c_int), ("kv_rank", ctypes.c_int), ("q_rank", ctypes.c_int),
                ("decay_rank", ctypes.c_int), ("rot_dims", ctypes.c_int), ("rot_interleaved", ctypes.c_int),
                ("window", ctypes.c_int), ("keep_first", ctypes.c_int), ("rot_base", ctypes.c_float),
                ("scale", ctypes.c_float), ("tau", ctypes.c_float), ("ff", ctypes.c_int)]


class RivetarConfigC(ctypes.Structure):
    """mirror of ``asd_rivetar_config``"""
    _fields_ = [("width", ctypes.c_int), ("vocab", ctypes.c_int), ("n_layers", ctypes.c_int), ("eps", ctypes.c_float),
                ("embed_scale", ctypes.c_float), ("logit_softcap", ctypes.c_float), ("loop_start", ctypes.c_int),
                ("loop_stop", ctypes.c_int), ("loop_times", ctypes.c_int), ("max_tokens", ctypes.c_int),
                ("page_size", ctypes.c_int), ("ring", ctypes.c_int), ("dtype", ctypes.c_int)]


class MavipelLayerC(ctypes.Structure):
    """mirror of ``asd_mavipel_layer_config``"""
    _fields_ = [(n, ctypes.c_int) for n in (
        "type", "heads", "kv_heads", "dim", "vdim", "conv", "decay_rank", "gate_rank", "a_heads", "a_kv_heads", "a_dim",
        "a_vdim", "rot_dims", "window", "r_heads", "r_dim", "r_decay_rank", "ff_kind", "ff", "experts", "top", "expert_ff",
        "shared_ff")] + [(n, ctypes.c_float) for n in ("rot_base", "scale", "softcap", "left_scale", "right_scale")]


class MavipelConfigC(ctypes.Structure):
    """mirror of ``asd_mavipel_config``"""
    _fields_ = [("width", ctypes.c_int), ("vocab", ctypes.c_int), ("n_layers", ctypes.c_int), ("eps", ctypes.c_float),
                ("norm_groups", ctypes.c_int), ("loop_start", ctypes.c_int), ("loop_stop", ctypes.c_int),
                ("loop_times", ctypes.c_int), ("max_tokens", ctypes.c_int), ("page_size", ctypes.c_int),
                ("ring", ctypes.c_int), ("dtype", ctypes.c_int)]


class LukopelLayerC(ctypes.Structure):
    """mirror of ``asd_lukopel_layer_config``"""
    _fields_ = [(n, ctypes.c_int) for n in (
        "heads", "kv_heads", "dim", "vdim", "norm_whole", "v_unit", "gated", "chunk", "far", "temp_every", "ff_kind",
        "ff")] + [(n, ctypes.c_float) for n in ("scale", "temp_coef")]


class LukopelConfigC(ctypes.Structure):
    """mirror of ``asd_lukopel_config``"""
    _fields_ = [("width", ctypes.c_int), ("vocab", ctypes.c_int), ("n_layers", ctypes.c_int), ("eps", ctypes.c_float),
                ("embed_scale", ctypes.c_float), ("streams", ctypes.c_int), ("max_positions", ctypes.c_int),
                ("loop_start", ctypes.c_int), ("loop_stop", ctypes.c_int), ("loop_times", ctypes.c_int),
                ("max_tokens", ctypes.c_int), ("page_size", ctypes.c_int), ("ring", ctypes.c_int),
                ("dtype", ctypes.c_int)]


def library_path() -> str:
    return os.path.join(_HERE, "libasd_b200.so")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise AsdError(f"{path} not found: run `python -c 'import __graft_entry__ as g; g.build()'` "
                       "(there is no CPU fallback for the CUDA path)")
    L = ctypes.CDLL(path)
    c = ctypes
    vp, i32, f32, f64, sz = c.c_void_p, c.c_int, c.c_float, c.c_double, c.c_size_t
    sigs = {
        "asd_abi_version": (i32, []),
        "asd_last_error": (c.c_char_p, []),
        "asd_launch_count": (c.c_longlong, []),
        "asd_reset_launch_count": (None, []),
        "asd_reject_sample_workspace_bytes": (sz, [i32, i32]),
        "asd_reject_sample_set_impl": (None, [i32]),
        "asd_reject_sample": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, f32, vp, vp, vp, vp, vp, vp, vp]),
        "asd_reject_sample_host": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, f32, vp, vp, vp, vp, vp]),
        "asd_stop_rule": (i32, [vp, vp, i32, i32, f64, i32, f64, f64, vp, vp, vp]),
        "asd_stop_rule_host": (i32, [vp, vp, i32, f64, i32, f64, f64, vp]),
        "asd_stop_rule_rows": (i32, [vp, vp, vp, i32, i32, i32, f64, f64, vp, vp, vp]),
        "asd_stop_rule_rows_host": (i32, [vp, vp, vp, i32, i32, i32, f64, f64, vp, vp]),
        "asd_cascade_decide": (i32, [vp, vp, i32, i32, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, f64, i32, f64, f64,
                                     f64, vp, vp, vp, vp]),
        "asd_engine_persist_trace": (i32, [vp, vp]),
        "asd_engine_peer_connect": (i32, [vp, i32]),
        "asd_bayesian_adjustment_host": (f64, [f64, f64, f64, f64]),
        "asd_linear_bf16": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp]),
        "asd_linear_bf16_tc": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp]),
        "asd_linear_plan": (i32, [i32, i32, i32, i32, vp, vp, vp]),
        "asd_engine_create": (vp, [vp]),
        "asd_engine_destroy": (None, [vp]),
        "asd_engine_set_layer": (i32, [vp, i32, vp, vp, vp, vp, vp, vp, vp]),
        "asd_engine_set_globals": (i32, [vp, vp, vp, vp, vp]),
        "asd_engine_kv_pool_bytes": (sz, [vp, i32]),
        "asd_engine_set_kv": (i32, [vp, vp, i32, vp, i32, i32]),
        "asd_engine_set_allreduce": (i32, [vp, vp, vp]),
        "asd_engine_set_option": (i32, [vp, c.c_char_p, i32]),
        "asd_engine_ipc_export": (i32, [vp, vp]),
        "asd_engine_ipc_import": (i32, [vp, vp]),
        "asd_engine_tp_error": (i32, [vp]),
        "asd_engine_profile_read": (i32, [vp, vp, vp, i32]),
        "asd_debug_gemm_trace": (i32, [vp, i32]),
        "asd_debug_attn_trace": (i32, [vp, i32]),
        "asd_engine_forward": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, vp, i32, vp, c.c_longlong, vp]),
        "asd_mezilix_create": (vp, [vp, vp]),
        "asd_mezilix_destroy": (None, [vp]),
        "asd_mezilix_set_globals": (i32, [vp, vp, vp, vp, vp]),
        "asd_mezilix_set_layer": (i32, [vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
        "asd_mezilix_cache_bytes": (sz, [vp, i32]),
        "asd_mezilix_set_cache": (i32, [vp, vp, i32, vp, i32, i32, vp, vp]),
        "asd_mezilix_set_option": (i32, [vp, c.c_char_p, i32]),
        "asd_mezilix_forward": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, vp, i32, vp, c.c_longlong, vp, vp]),
        "asd_linear_simt": (i32, [vp, i32, vp, i32, vp, i32, i32, i32, i32, vp]),
        "asd_linear_tc": (i32, [vp, i32, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, vp]),
        "asd_mezilix_device_error": (i32, [vp]),
        "asd_mezilix_profile_read": (i32, [vp, vp, vp, i32]),
        "asd_rivetar_create": (vp, [vp, vp]),
        "asd_rivetar_destroy": (None, [vp]),
        "asd_rivetar_set_tensor": (i32, [vp, i32, c.c_char_p, vp]),
        "asd_rivetar_cache_bytes": (sz, [vp, i32]),
        "asd_rivetar_state_bytes": (sz, [vp, i32]),
        "asd_rivetar_set_cache": (i32, [vp, vp, i32, vp, i32, i32, vp]),
        "asd_rivetar_set_option": (i32, [vp, c.c_char_p, i32]),
        "asd_rivetar_forward": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, vp, i32, vp, c.c_longlong, vp, vp]),
        "asd_rivetar_profile_read": (i32, [vp, vp, vp, i32]),
        "asd_rivetar_device_error": (i32, [vp]),
        "asd_mavipel_create": (vp, [vp, vp]),
        "asd_mavipel_destroy": (None, [vp]),
        "asd_mavipel_set_tensor": (i32, [vp, i32, c.c_char_p, vp]),
        "asd_mavipel_cache_bytes": (sz, [vp, i32]),
        "asd_mavipel_state_bytes": (sz, [vp, i32]),
        "asd_mavipel_set_cache": (i32, [vp, vp, i32, vp, i32, i32, vp]),
        "asd_mavipel_set_option": (i32, [vp, c.c_char_p, i32]),
        "asd_mavipel_forward": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, vp, i32, vp, c.c_longlong, vp, vp]),
        "asd_mavipel_profile_read": (i32, [vp, vp, vp, i32]),
        "asd_mavipel_device_error": (i32, [vp]),
        "asd_lukopel_create": (vp, [vp, vp]),
        "asd_lukopel_destroy": (None, [vp]),
        "asd_lukopel_set_tensor": (i32, [vp, i32, c.c_char_p, vp]),
        "asd_lukopel_cache_bytes": (sz, [vp, i32]),
        "asd_lukopel_state_bytes": (sz, [vp, i32]),
        "asd_lukopel_set_cache": (i32, [vp, vp, i32, vp, i32, i32, vp]),
        "asd_lukopel_set_option": (i32, [vp, c.c_char_p, i32]),
        "asd_lukopel_forward": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, vp, i32, vp, c.c_longlong, vp, vp]),
        "asd_lukopel_profile_read": (i32, [vp, vp, vp, i32]),
        "asd_lukopel_device_error": (i32, [vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(L, name, None)
        if fn is None:       # a library built with only some components (build.py) lacks the others' entry points
            continue
        fn.restype = res
        fn.argtypes = args
    _LIB = L
    return L


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().asd_last_error().decode("utf-8", "replace")
        raise AsdError(f"{what}: {msg}" if what else msg)


def declared_symbols() -> list[str]:
    """every asd_* function declared in include/asd_b200.h (used by the ABI test)"""
    import re
    hdr = os.path.join(os.path.dirname(_HERE), "include", "asd_b200.h")
    with open(hdr) as f:
        text = f.read()
    return sorted(set(re.findall(r"ASD_API[^;(]*?\b(asd_[a-z0-9_]+)\s*\(", text)))
