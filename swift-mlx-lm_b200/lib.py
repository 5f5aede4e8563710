"""ctypes binding of libswlm_cuda.so (include/swlm.h). No fallback: a missing library raises."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libswlm_cuda.so")

NAME_MAX = 96


class SwlmError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"swlm status {status}: {message}")
        self.status = status


class Step(C.Structure):
    """Mirror of `swlm_step` (include/swlm_plan.h)."""

    _fields_ = [
        ("kind", C.c_int32),
        ("layer", C.c_int32),
        ("in_buf", C.c_int32),
        ("in2_buf", C.c_int32),
        ("in3_buf", C.c_int32),
        ("out_buf", C.c_int32),
        ("n", C.c_int32),
        ("k", C.c_int32),
        ("heads", C.c_int32),
        ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("rope_dim", C.c_int32),
        ("conv_kernel", C.c_int32),
        ("eps", C.c_float),
        ("weight_bias", C.c_float),
        ("scale", C.c_float),
        ("rope_base", C.c_float),
        ("weight", C.c_char * NAME_MAX),
        ("weight2", C.c_char * NAME_MAX),
        ("window_left", C.c_int32),
        ("in4_buf", C.c_int32),
        ("groups", C.c_int32),
        ("key_dim", C.c_int32),
        ("value_dim", C.c_int32),
        ("weight3", C.c_char * NAME_MAX),
        ("weight4", C.c_char * NAME_MAX),
    ]


class BuffersDesc(C.Structure):
    """Mirror of `swlm_buffers_desc` (include/swlm_plan.h)."""

    _fields_ = [
        ("hidden", C.c_int32),
        ("slot_dim", C.c_int32),
        ("vocab", C.c_int32),
        ("max_seq", C.c_int32),
        ("max_batch", C.c_int32),
        ("kv_layers", C.c_int32),
        ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("conv_layers", C.c_int32),
        ("conv_dim", C.c_int32),
        ("conv_kernel", C.c_int32),
        ("ssm_layers", C.c_int32),
        ("ssm_heads", C.c_int32),
        ("ssm_groups", C.c_int32),
        ("ssm_key_dim", C.c_int32),
        ("ssm_value_dim", C.c_int32),
        ("ssm_conv_kernel", C.c_int32),
        ("kv_scheme", C.c_int32),
        ("kv_qjl_dim", C.c_int32),
    ]


# name -> (restype, argtypes); every symbol include/swlm.h declares
_P = C.c_void_p
_I = C.c_int
SIGNATURES = {
    "swlm_version": (C.c_char_p, []),
    "swlm_device_count": (_I, []),
    "swlm_last_error": (C.c_char_p, []),
    "swlm_ctx_create": (_I, [_I, _I, _I, C.POINTER(_P)]),
    "swlm_ctx_destroy": (None, [_P]),
    "swlm_weights_add_q4g64_mlx": (_I, [_P, C.c_char_p, _I, _I, _P, _P, _P, _I]),
    "swlm_weights_add_q4g64_staf": (_I, [_P, C.c_char_p, _I, _I, _P, _I]),
    "swlm_weights_add_q4g128_mlx": (_I, [_P, C.c_char_p, _I, _I, _P, _P, _P, _I]),
    "swlm_weights_add_q4g128_staf": (_I, [_P, C.c_char_p, _I, _I, _P, _I]),
    "swlm_weights_add_dense_bf16": (_I, [_P, C.c_char_p, C.c_int64, C.c_int64, _P, _I]),
    "swlm_weights_add_dense_f32": (_I, [_P, C.c_char_p, C.c_int64, _P]),
    "swlm_weights_bytes": (C.c_int64, [_P]),
    "swlm_plan_build": (_I, [_P, C.POINTER(Step), _I, C.POINTER(BuffersDesc), C.POINTER(_P)]),
    "swlm_plan_destroy": (None, [_P]),
    "swlm_plan_launch_count": (_I, [_P]),
    "swlm_plan_describe": (_I, [_P, C.c_char_p, _I]),
    "swlm_state_create": (_I, [_P, C.POINTER(_P)]),
    "swlm_state_destroy": (None, [_P]),
    "swlm_state_set_stream": (_I, [_P, _P]),
    "swlm_state_set_prefill_chunk": (_I, [_P, _I]),
    "swlm_state_reset": (_I, [_P]),
    "swlm_state_snapshot": (_I, [_P, C.POINTER(_P)]),
    "swlm_state_restore": (_I, [_P, _P]),
    "swlm_snap_destroy": (None, [_P]),
    "swlm_position": (_I, [_P]),
    "swlm_prefill": (_I, [_P, _P, _I, _P]),
    "swlm_decode": (_I, [_P, _P, _P]),
    "swlm_decode_n": (_I, [_P, _P, _I, _P]),
    "swlm_decode_n_async": (_I, [_P, _P, _I]),
    "swlm_read_tokens": (_I, [_P, _I, _P]),
    "swlm_sync": (_I, [_P]),
    "swlm_read_logits": (_I, [_P, _P, C.c_size_t]),
    "swlm_read_buffer": (_I, [_P, _I, _P, _I]),
    "swlm_write_buffer": (_I, [_P, _I, _P, _I]),
    "swlm_read_kv": (_I, [_P, _I, _I, _I, _I, _I, _P]),
    "swlm_write_kv": (_I, [_P, _I, _I, _I, _I, _I, _P]),
    "swlm_kv_scheme_supported": (_I, [_I]),
    "swlm_state_get_rotors": (_I, [_P, _P, C.c_size_t]),
    "swlm_state_set_rotors": (_I, [_P, _P, C.c_size_t]),
    "swlm_read_qjl": (_I, [_P, _I, _I, _I, _I, _P]),
    "swlm_read_conv": (_I, [_P, _I, _I, _P]),
    "swlm_read_ssm_state": (_I, [_P, _I, _I, _P]),
    "swlm_set_position": (_I, [_P, _I]),
    "swlm_set_positions": (_I, [_P, _P]),
    "swlm_get_positions": (_I, [_P, _P]),
    "swlm_prefill_seq": (_I, [_P, _I, _P, _I, _P]),
    "swlm_state_reset_seq": (_I, [_P, _I]),
    "swlm_run_step": (_I, [_P, C.POINTER(Step), _P, _P]),
    "swlm_launches": (C.c_int64, [_P]),
    "swlm_profile_kind": (_I, [_P, _I, _I]),
    "swlm_tp_export": (_I, [_P, _P]),
    "swlm_tp_attach": (_I, [_P, _P]),
    "swlm_tp_status": (_I, [_P]),
    "swlm_tp_check_heads": (_I, [_I, _I, _I]),
    "swlm_shard_range": (_I, [_I, _I, _I, _I, _I, C.POINTER(_I)]),
    "swlm_op_qgemm": (_I, [_P, C.c_char_p, _I, _P, _P]),
    "swlm_op_qgemm_dev": (_I, [_P, C.c_char_p, _I, _P, _P, _P]),
    "swlm_op_dequant_bf16": (_I, [_P, C.c_char_p, _P]),
    "swlm_op_flash_decode_scratch_bytes": (C.c_size_t, [_I, _I, _I, _I, _I]),
    "swlm_op_flash_decode_dev": (_I, [_P, _I, _I, _I, _I, _I, _I, C.c_float, _P, _P, _P, _P, _P, _P]),
    "swlm_op_flash_decode_noalloc_capacity": (C.c_size_t, []),
    "swlm_op_flash_decode_noalloc_dev": (_I, [_P, _I, _I, _I, _I, _I, _I, C.c_float, _P, _P, _P, _P, _P]),
}


class Library:
    """The loaded shared object with typed entry points."""

    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
                "(there is no CPU or PyTorch fallback for this path)"
            )
        self.path = path
        self.dll = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.dll, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn)

    def check(self, status: int) -> None:
        if status != 0:
            raise SwlmError(status, self.swlm_last_error().decode("utf-8", "replace"))


_LIB = None


def load_library() -> Library:
    global _LIB
    if _LIB is None:
        _LIB = Library()
    return _LIB
