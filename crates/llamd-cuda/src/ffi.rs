//! The raw boundary of the CUDA library: one declaration per function of include/llamd_cuda.h,
//! include/llamd_cuda_model.h and include/llamd_gguf.h. WRITTEN BY gen_ffi.py -- edit the headers, then rerun it.
//! Nothing here checks anything; the safe wrappers of this crate validate lengths and ids before they call in.
#![allow(non_camel_case_types, dead_code, clippy::too_many_arguments)]

use std::os::raw::{c_char, c_int, c_longlong, c_uint, c_ulonglong, c_void};

/// Opaque handles of the library.
#[repr(C)]
pub struct llamd_model {
    _private: [u8; 0],
}
#[repr(C)]
pub struct llamd_gguf {
    _private: [u8; 0],
}

/// `llamd_hparams` of include/llamd_cuda_model.h, field for field.
#[repr(C)]
#[derive(Debug, Clone, Copy, Default, PartialEq)]
pub struct llamd_hparams {
    pub n_layer: i32,
    pub n_embd: i32,
    pub n_head: i32,
    pub n_head_kv: i32,
    pub head_dim: i32,
    pub n_expert: i32,
    pub n_expert_used: i32,
    pub n_ff_expert: i32,
    pub n_vocab: i32,
    pub rope_freq_base: f32,
    pub rms_eps: f32,
}

// ---- include/llamd_cuda.h
unsafe extern "C" {
    pub fn llamd_cuda_device_count() -> c_int;
    pub fn llamd_cuda_device_info(dev: c_int, name: *mut c_char, name_len: c_int, arch: *mut c_char, arch_len: c_int, total_mem: *mut usize, sm_count: *mut c_int, warp_size: *mut c_int) -> c_int;
    pub fn llamd_cuda_free_mem() -> usize;
    pub fn llamd_cuda_set_device(dev: c_int) -> c_int;
    pub fn llamd_cuda_last_error_string() -> *const c_char;
    pub fn llamd_cuda_upload(host: *const c_void, bytes: usize) -> *mut c_void;
    pub fn llamd_cuda_release(dev: *mut c_void);
    pub fn llamd_fwd_alloc(bytes: usize) -> *mut c_void;
    pub fn llamd_fwd_free(p: *mut c_void);
    pub fn llamd_fwd_upload(dst: *mut c_void, src: *const c_void, bytes: usize) -> c_int;
    pub fn llamd_fwd_download(dst: *mut c_void, src: *const c_void, bytes: usize) -> c_int;
    pub fn llamd_fwd_memset(p: *mut c_void, value: c_int, bytes: usize) -> c_int;
    pub fn llamd_fwd_sync() -> c_int;
    pub fn llamd_fwd_free_mem() -> usize;
    pub fn llamd_fwd_last_error() -> c_int;
    pub fn llamd_fwd_stream_init() -> c_int;
    pub fn llamd_fwd_launch_count() -> c_ulonglong;
    pub fn llamd_fwd_set_pdl(on: c_int);
    pub fn llamd_fwd_set_batch_group(g: c_int);
    pub fn llamd_fwd_stream() -> *mut c_void;
    pub fn llamd_fwd_timer_start() -> c_int;
    pub fn llamd_fwd_timer_stop(ms_out: *mut f32) -> c_int;
    pub fn llamd_fwd_begin_capture() -> c_int;
    pub fn llamd_fwd_end_capture() -> c_int;
    pub fn llamd_fwd_graph_launch() -> c_int;
    pub fn llamd_fwd_has_graph() -> c_int;
    pub fn llamd_fwd_graph_destroy();
    pub fn llamd_cuda_q6k_tiled_bytes(n_blocks: usize) -> usize;
    pub fn llamd_fwd_repack_q6k(d_src: *const c_void, d_dst: *mut c_void, n_blocks: usize);
    pub fn llamd_fwd_repack_q6k_at(d_src: *const c_void, d_dst: *mut c_void, n_blocks: usize, dst_first: usize);
    pub fn llamd_cuda_upload_q6k(host_blocks: *const c_void, n_blocks: usize) -> *mut c_void;
    pub fn llamd_fwd_unpack_q6k(d_tiled: *const c_void, d_dst: *mut c_void, n_blocks: usize);
    pub fn llamd_fwd_dequantize_q6k(d_tiled: *const c_void, first_block: usize, n_blocks: usize, d_out: *mut f32);
    pub fn llamd_cuda_q8_0_tiled_bytes(rows: usize, blocks_per_row: usize) -> usize;
    pub fn llamd_fwd_repack_q8_0(d_src: *const c_void, d_dst: *mut c_void, rows: usize, blocks_per_row: usize);
    pub fn llamd_cuda_upload_q8_0(host_blocks: *const c_void, rows: usize, blocks_per_row: usize) -> *mut c_void;
    pub fn llamd_fwd_dequantize_q8_0(d_tiled: *const c_void, rows: usize, blocks_per_row: usize, d_out: *mut f32);
    pub fn llamd_cuda_matvec_q6k_resident(d_w: *const c_void, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int) -> c_int;
    pub fn llamd_cuda_matvec_grouped(d_w: *const c_void, eid: *const i32, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int, n_used: c_int) -> c_int;
    pub fn llamd_cuda_matvec_bench(d_w: *const c_void, aq: *const i8, ad: *const f32, blocks: c_int, rows: c_int, iters: c_int, ms_out: *mut f32) -> c_int;
    pub fn llamd_cuda_matvec_grouped_bench(d_w: *const c_void, eid: *const i32, aq: *const i8, ad: *const f32, blocks: c_int, rows: c_int, n_used: c_int, iters: c_int, ms_out: *mut f32) -> c_int;
    pub fn llamd_cuda_quantize_q8k(x: *const f32, nblocks: c_int, qs: *mut i8, d: *mut f32, bsums: *mut i16) -> c_int;
    pub fn llamd_cuda_matvec_q6k_f32(d_w: *const c_void, x: *const f32, out: *mut f32, blocks: c_int, rows: c_int, nseq: c_int) -> c_int;
    pub fn llamd_cuda_matvec_q8_0_f32(d_w: *const c_void, x: *const f32, out: *mut f32, blocks32: c_int, rows: c_int, nseq: c_int) -> c_int;
    pub fn llamd_fwd_quantize(x: *const f32, qs: *mut i8, d: *mut f32, nblocks: c_int);
    pub fn llamd_fwd_quantize_bsums(x: *const f32, qs: *mut i8, d: *mut f32, bsums: *mut i16, nblocks: c_int);
    pub fn llamd_fwd_matvec(w: *const c_void, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int);
    pub fn llamd_fwd_matvec_batch(w: *const c_void, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_x3(w0: *const c_void, w1: *const c_void, w2: *const c_void, aq: *const i8, ad: *const f32, o0: *mut f32, o1: *mut f32, o2: *mut f32, blocks: c_int, rows0: c_int, rows1: c_int, rows2: c_int);
    pub fn llamd_fwd_matvec_x3_batch(w0: *const c_void, w1: *const c_void, w2: *const c_void, aq: *const i8, ad: *const f32, o0: *mut f32, o1: *mut f32, o2: *mut f32, blocks: c_int, rows0: c_int, rows1: c_int, rows2: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_grouped(w: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int, n_used: c_int);
    pub fn llamd_fwd_matvec_grouped_x2(wa: *const c_void, wb: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, oa: *mut f32, ob: *mut f32, blocks: c_int, rows: c_int, n_used: c_int);
    pub fn llamd_fwd_matvec_grouped_pa(w: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int, n_used: c_int);
    pub fn llamd_fwd_matvec_grouped_x2_batch(wa: *const c_void, wb: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, oa: *mut f32, ob: *mut f32, blocks: c_int, rows: c_int, n_used: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_grouped_pa_batch(w: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int, n_used: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_f32act(w: *const c_void, x: *const f32, out: *mut f32, blocks: c_int, rows: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_grouped_pa_silu(w: *const c_void, ids: *const i32, gate: *const f32, up: *const f32, out: *mut f32, blocks: c_int, rows: c_int, n_used: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_f32(w: *const f32, x: *const f32, out: *mut f32, k: c_int, rows: c_int);
    pub fn llamd_fwd_matvec_f32_batch(w: *const f32, x: *const f32, out: *mut f32, k: c_int, rows: c_int, nseq: c_int);
    pub fn llamd_fwd_transpose_f32(w: *const f32, wt: *mut f32, rows: c_int, k: c_int);
    pub fn llamd_fwd_matvec_q8_0(w: *const c_void, x: *const f32, out: *mut f32, blocks32: c_int, rows: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_q8_0_status() -> c_int;
    pub fn llamd_fwd_embed(table: *const c_void, token: c_int, out: *mut f32, blocks: c_int);
    pub fn llamd_fwd_embed_meta(table: *const c_void, meta: *const i32, out: *mut f32, blocks: c_int, nseq: c_int);
    pub fn llamd_fwd_rms_norm_mul(x: *const f32, w: *const f32, out: *mut f32, n: c_int, eps: f32, nseq: c_int);
    pub fn llamd_fwd_head_rms_norm_mul(x: *const f32, w: *const f32, out: *mut f32, n_head: c_int, hd: c_int, eps: f32);
    pub fn llamd_fwd_rms_norm_quant(x: *const f32, w: *const f32, out: *mut f32, qs: *mut i8, d: *mut f32, n: c_int, eps: f32, nseq: c_int);
    pub fn llamd_fwd_add_rms_norm_quant(x: *const f32, residual: *const f32, sum_out: *mut f32, w: *const f32, out: *mut f32, qs: *mut i8, d: *mut f32, n: c_int, eps: f32, nseq: c_int);
    pub fn llamd_fwd_combine_rms_norm_quant(x: *const f32, down: *const f32, weights: *const f32, n_used: c_int, sum_out: *mut f32, w: *const f32, out: *mut f32, qs: *mut i8, d: *mut f32, n: c_int, eps: f32, nseq: c_int);
    pub fn llamd_cuda_rope_table(host_out: *mut f32, max_pos: c_int, hd: c_int, freq_base: f32) -> c_int;
    pub fn llamd_fwd_rope(x: *mut f32, pos: c_int, n_head: c_int, hd: c_int, rope_tab: *const f32);
    pub fn llamd_fwd_norm_rope(x: *mut f32, w: *const f32, n_head: c_int, hd: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, nseq: c_int);
    pub fn llamd_fwd_k_norm_rope_store(k: *mut f32, w: *const f32, v: *const f32, kc: *mut f32, vc: *mut f32, n_head_kv: c_int, hd: c_int, kv_dim: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, nseq: c_int, max_kv: c_int);
    pub fn llamd_fwd_qk_norm_rope_store(q: *mut f32, wq: *const f32, k: *mut f32, wk: *const f32, v: *const f32, kc: *mut f32, vc: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, nseq: c_int, max_kv: c_int);
    pub fn llamd_fwd_kv_store(kc: *mut f32, vc: *mut f32, k: *const f32, v: *const f32, pos: c_int, kv_dim: c_int);
    pub fn llamd_fwd_attention(q: *const f32, kc: *const f32, vc: *const f32, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, n_kv: c_int);
    pub fn llamd_fwd_attention_meta(q: *const f32, kc: *const f32, vc: *const f32, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, max_kv: c_int, nseq: c_int);
    pub fn llamd_fwd_attention_noalloc(q: *const f32, kc: *const f32, vc: *const f32, out: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, n_kv: c_int) -> c_int;
    pub fn llamd_fwd_add(a: *const f32, b: *const f32, out: *mut f32, n: c_int);
    pub fn llamd_fwd_silu_mul(gate: *const f32, up: *const f32, out: *mut f32, n: c_int);
    pub fn llamd_fwd_silu_mul_quant(gate: *const f32, up: *const f32, out: *mut f32, qs: *mut i8, d: *mut f32, n: c_int);
    pub fn llamd_fwd_router(logits: *const f32, n_expert: c_int, n_used: c_int, ids: *mut i32, weights: *mut f32, probs: *mut f32, nseq: c_int);
    pub fn llamd_fwd_router_matvec(w: *const f32, x: *const f32, k: c_int, n_expert: c_int, n_used: c_int, logits: *mut f32, ids: *mut i32, weights: *mut f32, probs: *mut f32, counter: *mut c_uint, nseq: c_int);
    pub fn llamd_fwd_norm_router(w: *const f32, x: *const f32, residual: *const f32, x_out: *mut f32, w_norm: *const f32, xn_out: *mut f32, qs: *mut i8, d: *mut f32, k: c_int, eps: f32, n_expert: c_int, n_used: c_int, logits: *mut f32, ids: *mut i32, weights: *mut f32, probs: *mut f32, counter: *mut c_uint, nseq: c_int);
    pub fn llamd_fwd_moe_combine(down: *const f32, weights: *const f32, out: *mut f32, n_used: c_int, n_embd: c_int);
    pub fn llamd_fwd_moe_combine_add(down: *const f32, weights: *const f32, residual: *const f32, out: *mut f32, n_used: c_int, n_embd: c_int, nseq: c_int);
    pub fn llamd_fwd_argmax(x: *const f32, n: c_int, scratch_v: *mut f32, scratch_i: *mut i32, out: *mut i32, nblocks: c_int, nseq: c_int);
    pub fn llamd_fwd_moe_group(ids: *const i32, n_expert: c_int, n_used: c_int, nseq: c_int, gstart: *mut i32, gcount: *mut i32, ptoken: *mut i32, pslot: *mut i32);
    pub fn llamd_fwd_moe_group_work(ids: *const i32, n_expert: c_int, n_used: c_int, nseq: c_int, gstart: *mut i32, gcount: *mut i32, ptoken: *mut i32, pslot: *mut i32, work: *mut i32, n_work: *mut i32);
    pub fn llamd_fwd_matvec_tokens(w0: *const c_void, w1: *const c_void, w2: *const c_void, aq: *const i8, ad: *const f32, o0: *mut f32, o1: *mut f32, o2: *mut f32, blocks: c_int, rows0: c_int, rows1: c_int, rows2: c_int, ntok: c_int);
    pub fn llamd_fwd_expert_major(wa: *const c_void, wb: *const c_void, work: *const i32, n_work: *const i32, max_items: c_int, act_map: *const i32, pslot: *const i32, aq: *const i8, ad: *const f32, oa: *mut f32, ob: *mut f32, blocks: c_int, rows: c_int, n_expert: c_int);
    pub fn llamd_fwd_q8k_residue_major(aq: *const i8, aq_rm: *mut c_void, nblocks: usize);
    pub fn llamd_fwd_gemm_tokens(w0: *const c_void, w1: *const c_void, w2: *const c_void, aq_rm: *const c_void, ad: *const f32, o0: *mut f32, o1: *mut f32, o2: *mut f32, blocks: c_int, rows0: c_int, rows1: c_int, rows2: c_int, ntok: c_int);
    pub fn llamd_fwd_expert_gemm(wa: *const c_void, wb: *const c_void, gstart: *const i32, gcount: *const i32, act_map: *const i32, pslot: *const i32, aq_rm: *const c_void, ad: *const f32, oa: *mut f32, ob: *mut f32, blocks: c_int, rows: c_int, n_expert: c_int);
    pub fn llamd_fwd_qk_norm_rope_store_tile(q: *mut f32, wq: *const f32, k: *mut f32, wk: *const f32, v: *const f32, kc: *mut f32, vc: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, ntok: c_int);
    pub fn llamd_fwd_attention_tile(q: *const f32, kc: *const f32, vc: *const f32, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, max_kv: c_int, ntok: c_int);
    pub fn llamd_fwd_qk_norm_rope_store_kv16(q: *mut f32, wq: *const f32, k: *mut f32, wk: *const f32, v: *const f32, kc: *mut c_void, vc: *mut c_void, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, nseq: c_int, max_kv: c_int);
    pub fn llamd_fwd_qk_norm_rope_store_tile_kv16(q: *mut f32, wq: *const f32, k: *mut f32, wk: *const f32, v: *const f32, kc: *mut c_void, vc: *mut c_void, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, ntok: c_int);
    pub fn llamd_fwd_attention_meta_kv16(q: *const f32, kc: *const c_void, vc: *const c_void, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, max_kv: c_int, nseq: c_int);
    pub fn llamd_fwd_kv16_expand(kc16: *const c_void, vc16: *const c_void, kc32: *mut f32, vc32: *mut f32, n_pos: c_int, kv_dim: c_int);
    pub fn llamd_fwd_attention_rope_meta(q: *const f32, wq: *const f32, k: *const f32, wk: *const f32, v: *const f32, kc: *mut f32, vc: *mut f32, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, max_kv: c_int, nseq: c_int);
    pub fn llamd_fwd_attention_rope_meta_kv16(q: *const f32, wq: *const f32, k: *const f32, wk: *const f32, v: *const f32, kc: *mut c_void, vc: *mut c_void, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, rope_tab: *const f32, eps: f32, max_kv: c_int, nseq: c_int);
    pub fn llamd_fwd_matvec_grouped_x2_silu_quant(wa: *const c_void, wb: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, oa: *mut f32, ob: *mut f32, counter: *mut c_uint, qs: *mut i8, d: *mut f32, blocks: c_int, rows: c_int, n_used: c_int, nseq: c_int);
    pub fn llamd_fwd_attention_meta_quant(q: *const f32, kc: *const f32, vc: *const f32, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, max_kv: c_int, nseq: c_int, counter: *mut c_uint, qs: *mut i8, d: *mut f32);
    pub fn llamd_fwd_act_f16_rm(aq: *const i8, ad: *const f32, act16: *mut c_void, nblocks: usize);
    pub fn llamd_fwd_gemm_tokens_tc(w0: *const c_void, w1: *const c_void, w2: *const c_void, act16: *const c_void, o0: *mut f32, o1: *mut f32, o2: *mut f32, blocks: c_int, rows0: c_int, rows1: c_int, rows2: c_int, ntok: c_int);
    pub fn llamd_fwd_expert_gemm_tc(wa: *const c_void, wb: *const c_void, gstart: *const i32, gcount: *const i32, act_map: *const i32, pslot: *const i32, act16: *const c_void, oa: *mut f32, ob: *mut f32, blocks: c_int, rows: c_int, n_expert: c_int, max_count: c_int);
    pub fn llamd_fwd_gemm_tc_status() -> c_int;
    pub fn llamd_fwd_matvec_grouped_x2_owned(wa: *const c_void, wb: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, oa: *mut f32, ob: *mut f32, blocks: c_int, rows: c_int, n_used: c_int, n_slots: c_int, own_lo: c_int, own_hi: c_int);
    pub fn llamd_fwd_matvec_grouped_pa_owned(w: *const c_void, ids: *const i32, aq: *const i8, ad: *const f32, out: *mut f32, blocks: c_int, rows: c_int, n_slots: c_int, own_lo: c_int, own_hi: c_int);
    pub fn llamd_fwd_ep_dispatch(ids: *const i32, ad: *const f32, aq: *const i8, ids_all: *mut i32, ad_all: *mut f32, aq_all: *mut i8, n_used: c_int, blocks: c_int);
    pub fn llamd_fwd_ep_combine(send: *const f32, recv: *mut f32, ids: *const i32, down: *mut f32, n_used: c_int, n_embd: c_int, n_expert: c_int);
    pub fn llamd_fwd_rms_norm_rows(x: *const f32, out: *mut f32, n: c_int, rows: c_int, eps: f32);
    pub fn llamd_fwd_softmax_rows(x: *const f32, out: *mut f32, n: c_int, rows: c_int);
    pub fn llamd_fwd_silu(x: *const f32, out: *mut f32, n: usize);
    pub fn llamd_fwd_expf(x: *const f32, out: *mut f32, n: usize);
    pub fn llamd_cuda_exp_exceptions() -> c_longlong;
    pub fn llamd_cuda_exp_window_on() -> c_int;
    pub fn llamd_fwd_mul(a: *const f32, b: *const f32, out: *mut f32, n: usize);
    pub fn llamd_fwd_scale(x: *const f32, by: f32, out: *mut f32, n: usize);
    pub fn llamd_fwd_matmul_f32(w: *const f32, x: *const f32, out: *mut f32, k: c_int, m: c_int, n: c_int);
    pub fn llamd_fwd_rope_rows(x: *const f32, out: *mut f32, row_len: c_int, rows: c_int, head_dim: c_int, sincos: *const f32);
    pub fn llamd_fwd_get_rows_f32(table: *const f32, ids: *const u32, out: *mut f32, row_len: c_int, n_ids: c_int);
    pub fn llamd_fwd_matmul_f32_tokens(w: *const f32, x: *const f32, out: *mut f32, k: c_int, rows: c_int, ntok: c_int);
    pub fn llamd_fwd_attention_prefill(q: *const f32, kc: *const f32, vc: *const f32, out: *mut f32, scores: *mut f32, n_head: c_int, n_head_kv: c_int, hd: c_int, meta: *const i32, max_kv: c_int, ntok: c_int, n_kv_max: c_int);
}

// ---- include/llamd_cuda_model.h
unsafe extern "C" {
    pub fn llamd_cuda_ep_unique_id(out128: *mut c_void) -> c_int;
    pub fn llamd_cuda_ep_init(rank: c_int, world: c_int, id128: *const c_void) -> c_int;
    pub fn llamd_cuda_ep_finalize();
    pub fn llamd_cuda_ep_rank() -> c_int;
    pub fn llamd_model_ep_p2p_export(m: *mut llamd_model, out_record: *mut c_void) -> c_int;
    pub fn llamd_model_ep_p2p_attach(m: *mut llamd_model, all: *const c_void, world: c_int) -> c_int;
    pub fn llamd_cuda_ep_ipc_export(dev: *const c_void, handle64: *mut c_void) -> c_int;
    pub fn llamd_cuda_ep_ipc_open(handle64: *const c_void) -> *mut c_void;
    pub fn llamd_cuda_ep_ipc_close(mapped: *mut c_void);
    pub fn llamd_cuda_ep_world() -> c_int;
    pub fn llamd_cuda_ep_set_timeout_ms(ms: c_int);
    pub fn llamd_model_ep_status(m: *mut llamd_model) -> c_int;
    pub fn llamd_cuda_ep_init_local(rank: c_int, world: c_int) -> c_int;
    pub fn llamd_model_ep_p2p_buffers(m: *mut llamd_model, out: *mut *mut c_void) -> c_int;
    pub fn llamd_model_ep_tile_cap(m: *mut llamd_model) -> c_int;
    pub fn llamd_model_ep_p2p_attach_ptrs(m: *mut llamd_model, ptrs: *const *mut c_void, world: c_int) -> c_int;
    pub fn llamd_model_create(hp: *const llamd_hparams, max_kv: c_int, max_seq: c_int) -> *mut llamd_model;
    pub fn llamd_model_free(m: *mut llamd_model);
    pub fn llamd_model_error(m: *mut llamd_model) -> *const c_char;
    pub fn llamd_model_set_tensor(m: *mut llamd_model, layer: c_int, which: c_int, first_block: usize, host: *const c_void, count: usize) -> c_int;
    pub fn llamd_model_weight_bytes(m: *mut llamd_model) -> usize;
    pub fn llamd_model_set_option(m: *mut llamd_model, name: *const c_char, value: c_int) -> c_int;
    pub fn llamd_model_resident_profile(m: *mut llamd_model, out32: *mut c_ulonglong) -> c_int;
    pub fn llamd_model_forward(m: *mut llamd_model, token: i32, pos: i32, out_token: *mut i32) -> c_int;
    pub fn llamd_model_forward_batch(m: *mut llamd_model, tokens: *const i32, positions: *const i32, nseq: c_int, out_tokens: *mut i32) -> c_int;
    pub fn llamd_model_prefill(m: *mut llamd_model, tokens: *const i32, n_tokens: c_int, base_pos: c_int, out_token: *mut i32) -> c_int;
    pub fn llamd_model_verify(m: *mut llamd_model, tokens: *const i32, n_tokens: c_int, base_pos: c_int, out_tokens: *mut i32) -> c_int;
    pub fn llamd_model_decode(m: *mut llamd_model, first_token: i32, start_pos: i32, n: c_int, out_tokens: *mut i32, ms_out: *mut f32) -> c_int;
    pub fn llamd_model_bench_matvecs(m: *mut llamd_model, iters: c_int, nseq: c_int, ms_out: *mut f32, launches_out: *mut c_int) -> c_int;
    pub fn llamd_model_launches_per_pass(m: *mut llamd_model) -> c_ulonglong;
    pub fn llamd_model_profile_pass(m: *mut llamd_model, token: i32, pos: i32, ms_out: *mut f32) -> c_int;
    pub fn llamd_model_logits(m: *mut llamd_model, host_out: *mut f32, nseq: c_int) -> c_int;
    pub fn llamd_model_read_trace(m: *mut llamd_model, x_out: *mut f32, ids_out: *mut i32) -> c_int;
    pub fn llamd_model_read_kv(m: *mut llamd_model, layer: c_int, seq: c_int, n_pos: c_int, k_out: *mut f32, v_out: *mut f32) -> c_int;
}

// ---- include/llamd_gguf.h
unsafe extern "C" {
    pub fn llamd_gguf_open(path: *const c_char, kind: *mut c_int, err: *mut c_char, err_len: usize) -> *mut llamd_gguf;
    pub fn llamd_gguf_parse(bytes: *const c_void, len: usize, kind: *mut c_int, err: *mut c_char, err_len: usize) -> *mut llamd_gguf;
    pub fn llamd_gguf_close(g: *mut llamd_gguf);
    pub fn llamd_gguf_version(g: *const llamd_gguf) -> u32;
    pub fn llamd_gguf_alignment(g: *const llamd_gguf) -> u64;
    pub fn llamd_gguf_data_offset(g: *const llamd_gguf) -> u64;
    pub fn llamd_gguf_file_size(g: *const llamd_gguf) -> u64;
    pub fn llamd_gguf_n_metadata(g: *const llamd_gguf) -> u64;
    pub fn llamd_gguf_n_tensors(g: *const llamd_gguf) -> u64;
    pub fn llamd_gguf_get_u64(g: *const llamd_gguf, key: *const c_char, out: *mut u64) -> c_int;
    pub fn llamd_gguf_get_f32(g: *const llamd_gguf, key: *const c_char, out: *mut f32) -> c_int;
    pub fn llamd_gguf_get_str(g: *const llamd_gguf, key: *const c_char, out: *mut c_char, len: usize, full_len: *mut usize) -> c_int;
    pub fn llamd_gguf_get_array_len(g: *const llamd_gguf, key: *const c_char, out: *mut u64) -> c_int;
    pub fn llamd_gguf_metadata_key(g: *const llamd_gguf, i: u64) -> *const c_char;
    pub fn llamd_gguf_find_tensor(g: *const llamd_gguf, name: *const c_char) -> i64;
    pub fn llamd_gguf_tensor_name(g: *const llamd_gguf, index: u64) -> *const c_char;
    pub fn llamd_gguf_tensor_info(g: *const llamd_gguf, index: u64, ggml_type: *mut u32, n_dims: *mut c_int, dims: *mut u64, offset: *mut u64) -> c_int;
    pub fn llamd_gguf_tensor_data(g: *const llamd_gguf, index: u64, data: *mut *const c_void, n_bytes: *mut usize, err: *mut c_char, err_len: usize) -> c_int;
    pub fn llamd_gguf_hparams(g: *const llamd_gguf, hp: *mut llamd_hparams, is_moe: *mut c_int, n_ff: *mut i32, n_ctx_train: *mut i32, err: *mut c_char, err_len: usize) -> c_int;
    pub fn llamd_gguf_verify_present(g: *const llamd_gguf, err: *mut c_char, err_len: usize) -> c_int;
    pub fn llamd_model_load_gguf(g: *const llamd_gguf, max_kv: c_int, max_seq: c_int, kind: *mut c_int, err: *mut c_char, err_len: usize) -> *mut llamd_model;
}
