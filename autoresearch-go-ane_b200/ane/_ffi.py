"""ctypes binding of libane_b200.so.  There is no CPU fallback: if the CUDA library is
missing or cannot be loaded, importing this module raises."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int32, c_int64, c_uint8, c_uint16, c_uint32, c_uint64, c_void_p

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("ANE_B200_LIB", os.path.join(_PKG, "lib", "libane_b200.so"))

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"libane_b200.so not found at {LIB_PATH}; build it with `make -C {_PKG}` "
        "(or __graft_entry__.build()). There is no CPU fallback."
    )
lib = ctypes.CDLL(LIB_PATH)

DTYPE_BF16, DTYPE_F32, DTYPE_BF16X3 = 0, 1, 2
ARCH_REFERENCE, ARCH_LLAMA = 0, 1


class Options(ctypes.Structure):
    _fields_ = [
        ("struct_size", c_uint32),
        ("dim", c_int32), ("hidden", c_int32), ("n_layers", c_int32), ("n_heads", c_int32), ("n_kv_heads", c_int32),
        ("vocab", c_int32), ("seq", c_int32), ("batch", c_int32), ("arch", c_int32), ("quirks", c_int32),
        ("compute_dtype", c_int32), ("rope_theta", c_float), ("accum_steps", c_int32), ("lr", c_float),
        ("seed", c_int64),
        ("adam_beta1", c_float), ("adam_beta2", c_float), ("adam_eps", c_float), ("weight_decay", c_float),
        ("grad_clip", c_float), ("loss_scale", c_float),
        ("embed_lr_mult", c_float), ("scalar_lr_mult", c_float), ("lambda_lr_mult", c_float),
        ("lambda_beta1", c_float), ("lambda_beta2", c_float),
        ("use_ane", c_int32), ("hybrid_backward", c_int32), ("device", c_int32), ("rank", c_int32),
        ("world_size", c_int32), ("debug_taps", c_int32), ("ce_chunk_rows", c_int32), ("ce_chunk_cols", c_int32),
        ("reserved", c_int32 * 5),
    ]


class StepResult(ctypes.Structure):
    _fields_ = [
        ("struct_size", c_uint32), ("loss", c_float),
        ("step_ns", c_int64), ("compile_ns", c_int64), ("startup_compile_ns", c_int64), ("device_eval_ns", c_int64),
        ("cpu_work_ns", c_int64), ("weight_refresh_ns", c_int64), ("final_head_ns", c_int64),
        ("embed_grad_ns", c_int64), ("rms_dw_ns", c_int64), ("dw_gemm_ns", c_int64), ("dw_wait_ns", c_int64),
        ("adam_ns", c_int64), ("flushed", c_int32), ("device_status", c_int32),
    ]


class State(ctypes.Structure):
    _fields_ = [
        ("struct_size", c_uint32), ("cum_steps", c_uint32), ("cum_batches", c_uint32), ("adam_t", c_uint32),
        ("pending_steps", c_uint32), ("token_pos", c_uint64), ("last_loss", c_float), ("pad_", c_float),
        ("cum_train_ms", c_double), ("cum_wall_ms", c_double),
    ]


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("struct_size", c_uint32), ("dtype", c_int32), ("d_a", c_void_p), ("d_b", c_void_p), ("d_c", c_void_p),
        ("m", c_int32), ("n", c_int32), ("k", c_int32), ("lda", c_int32), ("ldb", c_int32), ("ldc", c_int32),
        ("a_mn", c_int32), ("b_mn", c_int32), ("out_mode", c_int32), ("alpha", c_float),
        ("d_res1", c_void_p), ("d_s1", c_void_p), ("d_res2", c_void_p), ("d_s2", c_void_p), ("ldres", c_int32),
        ("split_k", c_int32), ("d_aux", c_void_p), ("ldaux", c_int32), ("pad_", c_int32),
    ]


# Every symbol include/ane_b200.h declares, with its ctypes signature.
SIGNATURES = {
    "ane_device_count": (c_int32, []),
    "ane_dev_set": (c_int32, [c_int32]),
    "ane_dev_malloc": (c_void_p, [c_uint64]),
    "ane_dev_free": (c_int32, [c_void_p]),
    "ane_host_malloc": (c_void_p, [c_uint64]),
    "ane_host_free": (c_int32, [c_void_p]),
    "ane_dev_h2d": (c_int32, [c_void_p, c_void_p, c_uint64]),
    "ane_dev_d2h": (c_int32, [c_void_p, c_void_p, c_uint64]),
    "ane_dev_memset": (c_int32, [c_void_p, c_int32, c_uint64]),
    "ane_dev_sync": (c_int32, []),
    "ane_timer_begin": (c_int32, []),
    "ane_timer_end": (c_int32, [POINTER(c_float)]),
    "ane_ops_last_error": (c_char_p, []),
    "ane_ops_device_status": (c_int32, [POINTER(c_int32)]),
    "ane_op_cast_f32_to_bf16": (c_int32, [c_void_p, c_void_p, c_uint64]),
    "ane_op_cast_bf16_to_f32": (c_int32, [c_void_p, c_void_p, c_uint64]),
    "ane_op_gemm": (c_int32, [POINTER(GemmArgs)]),
    "ane_op_sample_rows": (c_int32, [c_void_p, c_void_p, c_float, c_void_p, c_int32, c_int32]),
    "ane_op_sumsq": (c_int32, [c_void_p, c_uint64, c_float, c_void_p]),
    "ane_op_sumsq_noalloc": (c_int32, [c_void_p, c_uint64, c_float, c_void_p]),
    "ane_op_sumsq_noalloc_last_error": (c_char_p, []),
    "ane_dp_unique_id": (c_int32, [POINTER(c_uint8)]),
    "ane_open": (c_int32, [POINTER(Options), POINTER(c_uint16), c_uint64, POINTER(c_uint8), POINTER(c_void_p)]),
    "ane_close": (c_int32, [c_void_p]),
    "ane_last_error": (c_char_p, [c_void_p]),
    "ane_version": (c_uint32, []),
    "ane_sampler_seed": (c_uint64, [c_int64]),
    "ane_sample_windows": (c_int32, [POINTER(c_uint64), c_uint64, c_uint32, c_uint32, c_uint32, c_uint32, POINTER(c_uint64)]),
    "ane_step": (c_int32, [c_void_p, POINTER(StepResult)]),
    "ane_step_tokens": (c_int32, [c_void_p, POINTER(c_uint16), POINTER(c_uint16), c_uint32, POINTER(StepResult)]),
    "ane_flush": (c_int32, [c_void_p, POINTER(c_double)]),
    "ane_eval_logits": (c_int32, [c_void_p, POINTER(c_uint16), c_uint32, POINTER(c_float), c_uint64, c_uint32]),
    "ane_eval_loss": (c_int32, [c_void_p, POINTER(c_uint16), c_uint32, POINTER(c_double), POINTER(c_uint64)]),
    "ane_decode_greedy": (c_int32, [c_void_p, POINTER(c_uint16), c_uint32, c_uint32, c_uint32, POINTER(c_uint16)]),
    "ane_decode_sample": (c_int32, [c_void_p, POINTER(c_uint16), c_uint32, c_uint32, c_uint32, c_float, POINTER(c_double),
                                    POINTER(c_uint16)]),
    "ane_set_lr": (c_int32, [c_void_p, c_float]),
    "ane_get_lr": (c_float, [c_void_p]),
    "ane_get_state": (c_int32, [c_void_p, POINTER(State)]),
    "ane_set_state": (c_int32, [c_void_p, POINTER(State)]),
    "ane_reseed": (c_int32, [c_void_p, c_int64]),
    "ane_tensor_size": (c_int64, [c_void_p, c_uint32, c_uint32]),
    "ane_import_tensor": (c_int32, [c_void_p, c_uint32, c_uint32, c_uint32, POINTER(c_float), c_uint64]),
    "ane_export_tensor": (c_int32, [c_void_p, c_uint32, c_uint32, c_uint32, POINTER(c_float), c_uint64]),
    "ane_get_tap": (c_int64, [c_void_p, c_uint32, c_uint32, POINTER(c_float), c_uint64]),
    "ane_launch_count": (c_uint64, [c_void_p]),
    "ane_engine_timer_begin": (c_int32, [c_void_p]),
    "ane_engine_timer_end": (c_int32, [c_void_p, POINTER(c_float)]),
    "ane_profile_gemm": (c_int32, [c_void_p, c_int32]),
    "ane_profile_read": (c_int32, [c_void_p, POINTER(c_double), POINTER(c_double), POINTER(c_uint64)]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _f = getattr(lib, _name)  # AttributeError here means the library is stale: fail loudly
    _f.restype = _res
    _f.argtypes = _args
