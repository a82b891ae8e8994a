"""ctypes binding of ``libforge_b200.so`` (declarations follow include/forge_b200.h).

The library is required: importing this module raises if the shared object is missing, and
every compute entry point returns an error status when no CUDA device is present.  There is no
CPU fallback anywhere in the package.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libforge_b200.so")


class ForgeModelConfig(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int32), ("intermediate_size", C.c_int32), ("num_layers", C.c_int32),
        ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("vocab_size", C.c_int32), ("max_seq_len", C.c_int32),
        ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float),
        ("quant", C.c_int32), ("qkv_bias", C.c_int32), ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("sliding_window", C.c_int32),
        ("proj_quant", C.c_int32 * 8),
    ]


STATUS = {0: "OK", 1: "INVALID_ARG", 2: "SHAPE", 3: "KV_FULL", 4: "CUDA", 5: "TIMEOUT", 6: "UNSUPPORTED", 7: "COMM"}


class ForgeError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"forge_b200 status {code} ({STATUS.get(code, '?')}): {text}")
        self.code = code


vp, i32, f32, sz, u32 = C.c_void_p, C.c_int32, C.c_float, C.c_size_t, C.c_uint32


class ForgeSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("repeat_penalty", C.c_float),
                ("seed", C.c_uint64)]


# name -> (restype, argtypes); every symbol the public header declares
SIGNATURES = {
    "forge_last_error": (C.c_char_p, []),
    "forge_device_count": (i32, []),
    "forge_matmul_mat_q8_0": (i32, [vp, i32, vp, vp, i32, i32, vp]),
    "forge_matmul_mat_q4_0": (i32, [vp, i32, vp, vp, i32, i32, vp]),
    "forge_matmul_vec_q4_k": (i32, [vp, i32, vp, vp, i32, i32, vp]),
    "forge_matmul_vec_q6_k": (i32, [vp, i32, vp, vp, i32, i32, vp]),
    "forge_packed_create": (i32, [i32, vp, i32, i32, vp, C.POINTER(vp)]),
    "forge_packed_destroy": (None, [vp]),
    "forge_matmul_mat_packed": (i32, [vp, i32, vp, vp, vp]),
    "forge_matmul_decode_batch": (i32, [vp, i32, vp, vp, vp]),
    "forge_packed_check": (i32, [vp, vp]),
    "forge_rms_norm": (i32, [vp, vp, vp, i32, i32, f32, vp]),
    "forge_rope_table": (i32, [vp, i32, i32, f32]),
    "forge_rope": (i32, [vp, i32, i32, i32, i32, vp, vp]),
    "forge_silu_mul": (i32, [vp, vp, vp, sz, vp]),
    "forge_residual_add": (i32, [vp, vp, sz, vp]),
    "forge_kv_append_f16": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "forge_attention_flash": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "forge_attention_flash_static": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "forge_attention_flash_batch": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]),
    "forge_argmax": (i32, [vp, vp, i32, vp]),
    "forge_attention_sliding": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]),
    "forge_attention_sliding_batch": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]),
    "forge_quantize_q8_0_host": (i32, [vp, sz, vp]),
    "forge_quantize_q4_0_host": (i32, [vp, sz, vp, i32]),
    "forge_quantize_q4_k_host": (i32, [vp, sz, vp]),
    "forge_quantize_q6_k_host": (i32, [vp, sz, vp]),
    "forge_gguf_open": (i32, [vp, sz, C.POINTER(vp)]),
    "forge_gguf_close": (None, [vp]),
    "forge_gguf_version": (i32, [vp]),
    "forge_gguf_tensor_count": (C.c_int64, [vp]),
    "forge_gguf_data_offset": (C.c_uint64, [vp]),
    "forge_gguf_tensor_info": (i32, [vp, C.c_int64, C.POINTER(C.c_char_p), C.POINTER(i32), C.POINTER(i32), C.POINTER(C.c_uint64),
                                    C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "forge_gguf_model_config": (i32, [vp, C.POINTER(ForgeModelConfig)]),
    "forge_gguf_tensor_to_f32": (i32, [vp, C.c_int64, vp, sz]),
    "forge_gguf_weights_bin_size": (sz, [vp]),
    "forge_gguf_export_weights_bin": (i32, [vp, vp, sz]),
    "forge_weights_bin_size": (sz, [C.POINTER(ForgeModelConfig)]),
    "forge_model_create": (i32, [C.POINTER(ForgeModelConfig), vp, sz, i32, C.POINTER(vp)]),
    "forge_model_destroy": (None, [vp]),
    "forge_model_stream": (vp, [vp]),
    "forge_model_vocab_size": (sz, [vp]),
    "forge_score_chunk": (i32, [vp, vp, vp, sz, vp]),
    "forge_apply_repeat_penalty": (i32, [vp, i32, vp, sz, f32]),
    "forge_sample": (i32, [vp, i32, f32, i32, f32, C.POINTER(C.c_uint64), C.POINTER(u32)]),
    "forge_generate": (i32, [vp, vp, vp, sz, i32, C.POINTER(ForgeSampling), vp, sz, vp, C.POINTER(i32)]),
    "forge_tp_unique_id": (i32, [vp]),
    "forge_model_tp_init": (i32, [vp, vp]),
    "forge_model_tp_exchange_export": (i32, [vp, vp]),
    "forge_model_tp_exchange_attach": (i32, [vp, vp]),
    "forge_model_set_gemm_passes": (i32, [vp, i32]),
    "forge_model_set_prefill_mode": (i32, [vp, i32]),
    "forge_model_set_wait_limit": (i32, [vp, u32]),
    "forge_kv_create": (i32, [vp, i32, i32, C.POINTER(vp)]),
    "forge_kv_reset": (i32, [vp]),
    "forge_kv_len": (i32, [vp, i32]),
    "forge_kv_destroy": (None, [vp]),
    "forge_kv_read": (i32, [vp, i32, i32, i32, vp]),
    "forge_kv_save_size": (sz, [vp, i32]),
    "forge_kv_save": (i32, [vp, i32, vp, sz]),
    "forge_kv_load": (i32, [vp, i32, vp, sz]),
    "forge_forward": (i32, [vp, vp, u32, vp]),
    "forge_forward_prefill": (i32, [vp, vp, vp, sz, vp]),
    "forge_forward_seq": (i32, [vp, vp, i32, u32, vp]),
    "forge_forward_prefill_seq": (i32, [vp, vp, i32, vp, sz, vp]),
    "forge_forward_batch": (i32, [vp, vp, i32, vp, vp]),
    "forge_generate_greedy": (i32, [vp, vp, vp, sz, i32, vp]),
    "forge_decode_greedy_batch": (i32, [vp, vp, i32, vp, i32, vp]),
    "forge_hidden_trace_enable": (i32, [vp, i32]),
    "forge_hidden_trace_read": (i32, [vp, vp, sz, C.POINTER(i32)]),
    "forge_last_timing": (i32, [vp, C.POINTER(f32), C.POINTER(f32), C.POINTER(C.c_int64)]),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m forge_llm_b200.build` (nvcc, sm_100a). "
        "forge_llm_b200 has no CPU or PyTorch fallback.")

lib = C.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def check(status: int) -> None:
    if status != 0:
        raise ForgeError(status, (lib.forge_last_error() or b"").decode())
