"""ctypes binding of libanygpu_b200.so (the C ABI declared in include/b200_mamba2.h).

The library is the product; this module only loads it and declares argument types. There is no fallback:
if the library is missing or a call returns a non-zero status, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libanygpu_b200.so")

F16, F32 = 0, 1
W_KN, W_NK = 0, 1

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_f32 = ctypes.c_float
_sz = ctypes.c_size_t


class B200Error(RuntimeError):
    def __init__(self, fn, status, text, cuda_err):
        super().__init__(f"{fn} failed: status {status} ({text}), last CUDA error {cuda_err}")
        self.status = status


class Mamba2Config(ctypes.Structure):
    _fields_ = [("d_model", _i64), ("d_inner", _i64), ("nheads", _i64), ("headdim", _i64), ("d_state", _i64),
                ("ngroups", _i64), ("d_conv", _i64), ("chunk", _i64), ("norm_group_size", _i64), ("eps", _f32)]


class Mamba2Weights(ctypes.Structure):
    _fields_ = [("in_proj_weight", _vp), ("conv1d_weight", _vp), ("conv1d_bias", _vp), ("dt_bias", _vp), ("A_log", _vp),
                ("D", _vp), ("norm_weight", _vp), ("out_proj_weight", _vp), ("in_proj_layout", _int), ("out_proj_layout", _int)]


# name -> (restype, argtypes); mirrors include/b200_mamba2.h one to one
SIGNATURES = {
    "b200_status_string": (ctypes.c_char_p, [_int]),
    "b200_last_cuda_error": (_int, []),
    "b200_abi_version": (_int, []),
    "b200_last_device_error": (_int, [_vp, ctypes.POINTER(ctypes.c_uint32)]),
    "b200_launch_count": (ctypes.c_longlong, [_int]),
    "b200_linear_kernel_name": (ctypes.c_char_p, [_int, _i64, _i64, _i64]),
    "b200_debug_linear_starved_producer": (_int, [_vp, _i64, _vp, _int, _vp, _i64, _i64, _i64, _i64, ctypes.c_uint32, _vp]),
    "b200_linear": (_int, [_int, _vp, _i64, _vp, _int, _vp, _i64, _i64, _i64, _i64, _vp]),
    "b200_causal_conv1d": (_int, [_int, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_causal_conv1d_tokens": (_int, [_int, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_causal_conv1d_update": (_int, [_int, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "b200_gated_rmsnorm": (_int, [_int, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _vp]),
    "b200_mamba_chunk_scan_combined_workspace_bytes": (_sz, [_i64] * 7),
    "b200_mamba_chunk_scan_combined": (_int, [_int, _vp, _i64, _vp, _i64, _vp, _int, _vp, _i64, _vp, _i64, _vp, _vp, _vp,
                                              _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "b200_mamba_chunk_scan_combined_static_capacity": (_sz, []),
    "b200_mamba_chunk_scan_combined_static": (_int, [_int, _vp, _i64, _vp, _i64, _vp, _int, _vp, _i64, _vp, _i64, _vp, _vp, _vp,
                                                     _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_selective_state_update": (_int, [_int, _vp, _vp, _i64, _vp, _i64, _vp, _int, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64,
                                           _i64, _i64, _i64, _i64, _i64, _int, _vp]),
    "b200_mamba2_mixer_prefill_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64, _i64]),
    "b200_mamba2_mixer_prefill": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp, _i64, _i64,
                                         _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200_mamba2_mixer_prefill_host_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64, _i64]),
    "b200_mamba2_mixer_prefill_host": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp, _i64,
                                              _i64, _vp, _sz, _vp]),
    "b200_mamba2_mixer_prefill_host_ex": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp, _i64,
                                              _i64, _vp, _sz, _vp, _int]),
    "b200_mamba2_mixer_prefill_tp_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64, _i64]),
    "b200_mamba2_mixer_prefill_tp_partial": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp, _vp,
                                                    _i64, _i64, _vp, _vp, _vp, _sz, _vp]),
    "b200_mamba2_mixer_tp_finish": (_int, [_int, _vp, _vp, _i64, _i64, _i64, _f32, _vp]),
    "b200_mamba2_mixer_decode_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64]),
    "b200_mamba2_mixer_decode": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp, _vp, _vp, _i64,
                                        _vp, _sz, _vp]),
    "b200_mamba2_mixer_prefill_continue_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64, _i64]),
    "b200_mamba2_mixer_prefill_continue": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp, _i64,
                                                  _i64, _vp, _vp, _vp, _sz, _vp]),
    "b200_mamba2_mixer_prefill_varlen_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64]),
    "b200_mamba2_mixer_prefill_varlen": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp,
                                                ctypes.POINTER(ctypes.c_int64), _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200_mamba2_mixer_prefill_sp_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64, _i64]),
    "b200_mamba2_mixer_prefill_sp_begin": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _vp, _i64, _i64,
                                                  _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200_ssm_segment_prefix": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp]),
    "b200_mamba2_mixer_prefill_sp_finish": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _i64, _i64,
                                                   _vp, _vp, _vp, _sz, _vp]),
    "b200_rms_norm": (_int, [_int, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _int, _vp]),
    "b200_mamba2_decoder_prefill_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64, _i64]),
    "b200_mamba2_decoder_prefill": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _f32, _vp, _vp,
                                           _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200_mamba2_decoder_decode_workspace_bytes": (_sz, [ctypes.POINTER(Mamba2Config), _int, _i64]),
    "b200_mamba2_decoder_decode": (_int, [_int, ctypes.POINTER(Mamba2Config), ctypes.POINTER(Mamba2Weights), _vp, _f32, _vp, _vp,
                                          _vp, _vp, _i64, _vp, _sz, _vp]),
    "b200_stage_timing_enable": (_int, [_int]),
    "b200_stage_timing_collect": (_int, [ctypes.POINTER(_f32), ctypes.POINTER(_int)]),
}

_lib = None


def load():
    """Loads the shared library (raises if it has not been built: run `python -m anygpu_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} not built; run `python -m anygpu_b200.build`")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(fn_name, status):
    if status != 0:
        lib = load()
        raise B200Error(fn_name, status, lib.b200_status_string(status).decode(), lib.b200_last_cuda_error())


def call(fn_name, *args):
    """Calls an int-status entry point and raises B200Error on a non-zero status."""
    check(fn_name, getattr(load(), fn_name)(*args))
