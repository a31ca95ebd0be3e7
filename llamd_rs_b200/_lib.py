"""ctypes loader for libllamd_cuda.so.

There is no CPU fallback: if the library is missing or cannot be loaded the
import of any op raises, and every op raises when no CUDA device is present.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libllamd_cuda.so")

_lib = None

vp, i32, f32, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); every symbol include/llamd_cuda.h declares.
SIGNATURES = {
    "llamd_cuda_device_count": (i32, []),
    "llamd_cuda_device_info": (i32, [i32, C.c_char_p, i32, C.c_char_p, i32, C.POINTER(sz), C.POINTER(i32), C.POINTER(i32)]),
    "llamd_cuda_free_mem": (sz, []),
    "llamd_cuda_set_device": (i32, [i32]),
    "llamd_cuda_last_error_string": (C.c_char_p, []),
    "llamd_cuda_upload": (vp, [vp, sz]),
    "llamd_cuda_release": (None, [vp]),
    "llamd_fwd_alloc": (vp, [sz]),
    "llamd_fwd_free": (None, [vp]),
    "llamd_fwd_upload": (i32, [vp, vp, sz]),
    "llamd_fwd_download": (i32, [vp, vp, sz]),
    "llamd_fwd_memset": (i32, [vp, i32, sz]),
    "llamd_fwd_sync": (i32, []),
    "llamd_fwd_free_mem": (sz, []),
    "llamd_fwd_last_error": (i32, []),
    "llamd_fwd_stream_init": (i32, []),
    "llamd_fwd_stream": (vp, []),
    "llamd_fwd_launch_count": (C.c_ulonglong, []),
    "llamd_fwd_set_pdl": (None, [i32]),
    "llamd_fwd_set_batch_group": (None, [i32]),
    "llamd_fwd_rms_norm_rows": (None, [vp, vp, i32, i32, f32]),
    "llamd_fwd_softmax_rows": (None, [vp, vp, i32, i32]),
    "llamd_fwd_silu": (None, [vp, vp, sz]),
    "llamd_fwd_expf": (None, [vp, vp, sz]),
    "llamd_cuda_exp_exceptions": (C.c_longlong, []),
    "llamd_cuda_exp_window_on": (i32, []),
    "llamd_fwd_mul": (None, [vp, vp, vp, sz]),
    "llamd_fwd_scale": (None, [vp, f32, vp, sz]),
    "llamd_fwd_matmul_f32": (None, [vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_rope_rows": (None, [vp, vp, i32, i32, i32, vp]),
    "llamd_fwd_get_rows_f32": (None, [vp, vp, vp, i32, i32]),
    "llamd_fwd_repack_q6k_at": (None, [vp, vp, sz, sz]),
    "llamd_fwd_timer_start": (i32, []),
    "llamd_fwd_timer_stop": (i32, [C.POINTER(f32)]),
    "llamd_fwd_begin_capture": (i32, []),
    "llamd_fwd_end_capture": (i32, []),
    "llamd_fwd_graph_launch": (i32, []),
    "llamd_fwd_has_graph": (i32, []),
    "llamd_fwd_graph_destroy": (None, []),
    "llamd_cuda_q6k_tiled_bytes": (sz, [sz]),
    "llamd_fwd_repack_q6k": (None, [vp, vp, sz]),
    "llamd_cuda_upload_q6k": (vp, [vp, sz]),
    "llamd_fwd_unpack_q6k": (None, [vp, vp, sz]),
    "llamd_fwd_dequantize_q6k": (None, [vp, sz, sz, vp]),
    "llamd_cuda_q8_0_tiled_bytes": (sz, [sz, sz]),
    "llamd_fwd_repack_q8_0": (None, [vp, vp, sz, sz]),
    "llamd_cuda_upload_q8_0": (vp, [vp, sz, sz]),
    "llamd_fwd_dequantize_q8_0": (None, [vp, sz, sz, vp]),
    "llamd_cuda_matvec_q6k_resident": (i32, [vp, vp, vp, vp, i32, i32]),
    "llamd_cuda_matvec_grouped": (i32, [vp, vp, vp, vp, vp, i32, i32, i32]),
    "llamd_cuda_matvec_bench": (i32, [vp, vp, vp, i32, i32, i32, C.POINTER(f32)]),
    "llamd_cuda_matvec_grouped_bench": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, C.POINTER(f32)]),
    "llamd_cuda_quantize_q8k": (i32, [vp, i32, vp, vp, vp]),
    "llamd_cuda_matvec_q6k_f32": (i32, [vp, vp, vp, i32, i32, i32]),
    "llamd_cuda_matvec_q8_0_f32": (i32, [vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_quantize": (None, [vp, vp, vp, i32]),
    "llamd_fwd_quantize_bsums": (None, [vp, vp, vp, vp, i32]),
    "llamd_fwd_matvec": (None, [vp, vp, vp, vp, i32, i32]),
    "llamd_fwd_matvec_batch": (None, [vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_matvec_x3": (None, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_matvec_x3_batch": (None, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
    "llamd_fwd_matvec_grouped": (None, [vp, vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_matvec_grouped_x2": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_matvec_grouped_pa": (None, [vp, vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_matvec_grouped_x2_batch": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_matvec_grouped_pa_batch": (None, [vp, vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_matvec_f32act": (None, [vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_matvec_grouped_pa_silu": (None, [vp, vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_transpose_f32": (None, [vp, vp, i32, i32]),
    "llamd_fwd_matvec_f32": (None, [vp, vp, vp, i32, i32]),
    "llamd_fwd_matvec_f32_batch": (None, [vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_matvec_q8_0": (None, [vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_embed": (None, [vp, i32, vp, i32]),
    "llamd_fwd_embed_meta": (None, [vp, vp, vp, i32, i32]),
    "llamd_fwd_rms_norm_mul": (None, [vp, vp, vp, i32, f32, i32]),
    "llamd_fwd_head_rms_norm_mul": (None, [vp, vp, vp, i32, i32, f32]),
    "llamd_fwd_rms_norm_quant": (None, [vp, vp, vp, vp, vp, i32, f32, i32]),
    "llamd_fwd_add_rms_norm_quant": (None, [vp, vp, vp, vp, vp, vp, vp, i32, f32, i32]),
    "llamd_fwd_combine_rms_norm_quant": (None, [vp, vp, vp, i32, vp, vp, vp, vp, vp, i32, f32, i32]),
    "llamd_fwd_qk_norm_rope_store": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32, i32]),
    "llamd_fwd_qk_norm_rope_store_kv16": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32, i32]),
    "llamd_fwd_qk_norm_rope_store_tile_kv16": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32]),
    "llamd_fwd_attention_meta_kv16": (None, [vp, vp, vp, vp, vp, i32, i32, i32, vp, i32, i32]),
    "llamd_fwd_kv16_expand": (None, [vp, vp, vp, vp, i32, i32]),
    "llamd_fwd_attention_rope_meta": (None, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32, i32]),
    "llamd_fwd_attention_rope_meta_kv16": (None, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32, i32]),
    "llamd_cuda_rope_table": (i32, [vp, i32, i32, f32]),
    "llamd_fwd_rope": (None, [vp, i32, i32, i32, vp]),
    "llamd_fwd_norm_rope": (None, [vp, vp, i32, i32, vp, vp, f32, i32]),
    "llamd_fwd_k_norm_rope_store": (None, [vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32, i32]),
    "llamd_fwd_kv_store": (None, [vp, vp, vp, vp, i32, i32]),
    "llamd_fwd_attention": (None, [vp, vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_attention_meta": (None, [vp, vp, vp, vp, vp, i32, i32, i32, vp, i32, i32]),
    "llamd_fwd_attention_noalloc": (i32, [vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_add": (None, [vp, vp, vp, i32]),
    "llamd_fwd_silu_mul": (None, [vp, vp, vp, i32]),
    "llamd_fwd_silu_mul_quant": (None, [vp, vp, vp, vp, vp, i32]),
    "llamd_fwd_router": (None, [vp, i32, i32, vp, vp, vp, i32]),
    "llamd_fwd_router_matvec": (None, [vp, vp, i32, i32, i32, vp, vp, vp, vp, vp, i32]),
    "llamd_fwd_norm_router": (None, [vp, vp, vp, vp, vp, vp, vp, vp, i32, f32, i32, i32, vp, vp, vp, vp, vp, i32]),
    "llamd_fwd_moe_combine": (None, [vp, vp, vp, i32, i32]),
    "llamd_fwd_moe_combine_add": (None, [vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_argmax": (None, [vp, i32, vp, vp, vp, i32, i32]),
    "llamd_fwd_matvec_tokens": (None, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
    "llamd_fwd_expert_major": (None, [vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_q8k_residue_major": (None, [vp, vp, sz]),
    "llamd_fwd_gemm_tokens": (None, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
    "llamd_fwd_expert_gemm": (None, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_qk_norm_rope_store_tile": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32]),
    "llamd_fwd_attention_tile": (None, [vp, vp, vp, vp, vp, i32, i32, i32, vp, i32, i32]),
    "llamd_fwd_matvec_grouped_x2_owned": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32]),
    "llamd_fwd_matvec_grouped_pa_owned": (None, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
    "llamd_fwd_ep_dispatch": (None, [vp, vp, vp, vp, vp, vp, i32, i32]),
    "llamd_fwd_ep_combine": (None, [vp, vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_matvec_grouped_x2_silu_quant": (None, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_attention_meta_quant": (None, [vp, vp, vp, vp, vp, i32, i32, i32, vp, i32, i32, vp, vp, vp]),
    "llamd_model_ep_p2p_export": (i32, [vp, vp]),
    "llamd_model_ep_p2p_attach": (i32, [vp, vp, i32]),
    "llamd_cuda_ep_ipc_export": (i32, [vp, vp]),
    "llamd_cuda_ep_ipc_open": (vp, [vp]),
    "llamd_cuda_ep_ipc_close": (None, [vp]),
    "llamd_fwd_act_f16_rm": (None, [vp, vp, vp, C.c_size_t]),
    "llamd_fwd_gemm_tokens_tc": (None, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
    "llamd_fwd_expert_gemm_tc": (None, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]),
    "llamd_fwd_gemm_tc_status": (i32, []),
    "llamd_fwd_matvec_q8_0_status": (i32, []),
    "llamd_fwd_matmul_f32_tokens": (None, [vp, vp, vp, i32, i32, i32]),
    "llamd_fwd_attention_prefill": (None, [vp, vp, vp, vp, vp, i32, i32, i32, vp, i32, i32, i32]),
    "llamd_fwd_moe_group": (None, [vp, i32, i32, i32, vp, vp, vp, vp]),
    "llamd_fwd_moe_group_work": (None, [vp, i32, i32, i32, vp, vp, vp, vp, vp, vp]),
}


class LibraryMissing(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load the CUDA library (once). Raises LibraryMissing when it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO):
            raise LibraryMissing(
                f"{SO} is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU fallback)")
        L = C.CDLL(SO)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
