"""ctypes bindings of the C ABI in ``include/lm_b200.h`` (``csrc/liblm_b200.so``).

Like ``_lib.py`` there is no fallback: a missing library is built with nvcc on first use, and a failing call raises.
"""

from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

from . import build as _build

MIXER_SINK_ATTENTION, MIXER_TALK_ATTENTION, MIXER_HGRN2, MIXER_CHANNEL_DELTA, MIXER_LATENT_ATTENTION, MIXER_MLSTM = 1, 2, 3, 4, 5, 6
MIXER_GATED_DELTA, MIXER_RETENTION = 7, 8
FF_NONE, FF_ROUTED_EXPERTS, FF_DENSE = 0, 1, 2
NORM_DYT, NORM_LAYER, NORM_RMS = 0, 1, 2
FORM_SEQUENTIAL, FORM_PARALLEL, FORM_STREAMS = 0, 1, 2
ACT_SILU_GLU, ACT_XIELU, ACT_CLAMPED_GLU, ACT_RELU2 = 0, 1, 2, 3
ROUTER_SIGMOID_INPUT, ROUTER_SOFTMAX_TOP, ROUTER_SOFTMAX_GROUPED = 0, 1, 2
GATE_SIGMOID, GATE_NONE, GATE_SILU = 0, 1, 2
ROT_INTERLEAVED, ROT_HALF = 0, 1
ABI_VERSION = 4
PRECISION_FP32, PRECISION_BF16 = 0, 1
E_OK, E_INVAL, E_CUDA, E_NOMEM, E_UNSUPPORTED = 0, -1, -2, -3, -5

_vp, _i, _f = C.c_void_p, C.c_int32, C.c_float


class Norm(C.Structure):
    _fields_ = [("w", _vp), ("b", _vp), ("alpha", _f), ("kind", _i)]


class Layer(C.Structure):
    _fields_ = [("mixer", _i), ("heads", _i), ("kv_heads", _i), ("dim", _i), ("window", _i), ("keep_first", _i),
                ("scale", _f), ("softcap", _f), ("ff", _i), ("experts", _i), ("top", _i), ("expert_ff", _i),
                ("shared_ff", _i), ("norm_mix_in", Norm), ("norm_mix_out", Norm), ("norm_ff_in", Norm), ("norm_ff_out", Norm),
                ("tap_mix", _vp), ("tap_ff", _vp), ("w_qk", _vp), ("q_norm", _vp), ("k_norm", _vp), ("temp", _vp),
                ("slopes", _vp), ("sink", _vp), ("w_o", _vp), ("w_router", _vp), ("w_gate_up", _vp), ("w_down", _vp),
                ("ws_gate_up", _vp), ("ws_down", _vp), ("k_pages", _vp), ("v_pages", _vp), ("tail_mix", _vp), ("tail_ff", _vp),
                # the parallel form
                ("form", _i), ("vdim", _i), ("rot_dims", _i), ("conv_taps", _i), ("rank_a", _i), ("rank_g", _i), ("dense_ff", _i),
                ("act", _i), ("act_p", _f), ("act_q", _f), ("unit_eps", _f), ("n_in", _i), ("k_out", _i), ("w_in", _vp),
                ("in_bias", _vp), ("w_out", _vp), ("w_pre", _vp), ("rot_freq", _vp), ("talk", _vp), ("head_norm", _vp),
                ("lower", _vp), ("conv_w", _vp), ("a_log", _vp), ("dt_bias", _vp), ("w_a2", _vp), ("w_g2", _vp),
                ("rec_state", _vp), ("conv_tail", _vp),
                # the stream form
                ("streams", _i), ("hc_in", _vp * 2), ("hc_out", _vp * 2), ("hc_mix", _vp * 2), ("q_rank", _i), ("kv_rank", _i),
                ("q_lat_norm", _vp), ("kv_lat_norm", _vp), ("w_uq", _vp), ("w_uk_t", _vp), ("w_uv", _vp), ("latent_pages", _vp),
                ("gate_cap", _f), ("rec_aux", _vp), ("router", _i), ("router_bias", _vp), ("act_limit", _f), ("shared_limit", _f),
                # further mechanisms of the stream form
                ("parallel", _i), ("mixer_gate", _i), ("rot_layout", _i), ("rot_dim", _i), ("head_decay", _vp),
                ("identity_experts", _i), ("group_count", _i), ("group_keep", _i), ("route_scale", _f), ("route_correction", _vp),
                ("shared_gate", _i)]


class Model(C.Structure):
    _fields_ = [("n_layer", _i), ("width", _i), ("vocab", _i), ("taps", _i), ("page_size", _i), ("max_pages", _i),
                ("n_slots", _i), ("max_rows", _i), ("eps", _f), ("precision", _i), ("embed", _vp), ("head", _vp),
                ("final_norm", Norm), ("page_table", _vp), ("step_graphs", _i), ("logit_scale", _f), ("embed_scale", _f),
                ("embed_norm", _vp)]


_ci = C.c_int
_SIGNATURES = {
    "lm_b200_abi_version": (_ci, []),
    "lm_b200_last_cuda_error": (C.c_char_p, []),
    "lm_b200_launch_count": (C.c_int64, []),
    "lm_b200_engine_create": (_ci, [C.POINTER(Model), C.POINTER(Layer), _ci, C.POINTER(_vp)]),
    "lm_b200_engine_destroy": (_ci, [_vp]),
    "lm_b200_engine_workspace_bytes": (C.c_size_t, [_vp]),
    "lm_b200_forward": (_ci, [_vp, _vp, _ci, _ci, _ci, _vp, _vp, _vp]),
    "lm_b200_op_norm_tapmix": (_ci, [_vp, _ci, _ci, _vp, _vp, _ci, _ci, _vp, _vp]),
    "lm_b200_op_mixer": (_ci, [_vp, _ci, _vp, _vp, _ci, _ci, _vp, _vp]),
    "lm_b200_op_attention": (_ci, [_vp, _ci, _vp, _vp, _ci, _ci, _vp, _vp]),
    "lm_b200_op_mixer_kernels": (_ci, [_vp, _ci, _vp, _vp, _ci, _ci, _vp, _vp]),
    "lm_b200_op_ff": (_ci, [_vp, _ci, _vp, _ci, _vp, _vp]),
    "lm_b200_op_linear": (_ci, [_vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "lm_b200_op_linear_tc": (_ci, [_vp, _vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "lm_b200_argmax_rows": (_ci, [_vp, _ci, _ci, _vp, _vp]),
}

_lib = None


def header_symbols() -> list[str]:
    text = (Path(_build.INCLUDE) / "lm_b200.h").read_text()
    return sorted(set(re.findall(r"\b(lm_b200_[a-z0-9_]+)\s*\(", text)))


def load(build_if_missing: bool = True) -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LM_LIB
    if build_if_missing and _build.is_stale("lm"):
        try:
            _build.build(target="lm")
        except Exception as e:
            if not path.exists():
                raise RuntimeError(f"liblm_b200.so is missing and could not be built: {e}") from e
    if not path.exists():
        raise RuntimeError(f"{path} not found: run `python -m dia_tts_prune_b200.build lm` (there is no CPU fallback)")
    lib = C.CDLL(str(path))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if lib.lm_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("liblm_b200.so ABI version mismatch")
    _lib = lib
    return lib


def check(rc: int, what: str = "") -> None:
    if rc == 0:
        return
    msg = {E_INVAL: "invalid argument", E_CUDA: "CUDA error", E_NOMEM: "out of memory",
           E_UNSUPPORTED: "not supported on this path"}.get(rc, f"error {rc}")
    if rc == E_CUDA:
        msg += f" [{load().lm_b200_last_cuda_error().decode()}]"
    if rc == E_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}")
    if rc == E_INVAL:
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg}")
