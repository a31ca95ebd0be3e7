//! The `nseq` forms: up to [`max_seq`] independent sequences share every weight read. The counterpart of
//! `llamd-rocm/src/batch.rs` (`bop::*`). Buffers carry a leading sequence dimension: activations `[nseq][k]`, outputs
//! `[nseq][rows]`, `meta` = `[tok0, pos0, tok1, pos1, ...]`, KV caches `[nseq][max_kv][kv_dim]`.
//!
//! A weight block is unpacked once per CTA and applied to every sequence's activation; per sequence the arithmetic is
//! exactly the single-sequence op's, so a batch of N equals N single passes bit for bit.

use llamd_core::{Error, Result};

#[cfg(cuda)]
use crate::ffi;
use crate::forward::{launch, q6k_tiled_bytes, DevBuf};

/// `LLAMD_MAX_SEQ` of the C header.
pub const fn max_seq() -> usize {
    8
}

const QK: usize = llamd_quant::QK_K;

fn seqs(nseq: usize) -> Result<()> {
    if nseq == 0 || nseq > max_seq() {
        return Err(Error::malformed("batched op", format!("{nseq} sequences outside 1..={}", max_seq())));
    }
    Ok(())
}

pub mod bop {
    use super::*;

    fn f(p: &DevBuf) -> *mut f32 {
        p.ptr() as *mut f32
    }
    fn i(p: &DevBuf) -> *mut i32 {
        p.ptr() as *mut i32
    }
    fn q(p: &DevBuf) -> *mut i8 {
        p.ptr() as *mut i8
    }

    pub fn embed(table: &DevBuf, meta: &DevBuf, out: &DevBuf, blocks: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::embed", [(meta, nseq * 8), (out, nseq * blocks * QK * 4)], ffi::llamd_fwd_embed_meta(table.ptr(), i(meta), f(out), blocks as i32, nseq as i32))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn rms_norm_quant(x: &DevBuf, w: &DevBuf, out: &DevBuf, qs: &DevBuf, d: &DevBuf, n: usize, eps: f32, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        if n % QK != 0 {
            return Err(Error::malformed("bop::rms_norm_quant", format!("{n} is not a whole number of Q8_K blocks")));
        }
        launch!("bop::rms_norm_quant", [(x, nseq * n * 4), (w, n * 4), (out, nseq * n * 4), (qs, nseq * n), (d, nseq * n / QK * 4)],
                ffi::llamd_fwd_rms_norm_quant(f(x), f(w), f(out), q(qs), f(d), n as i32, eps, nseq as i32))
    }
    pub fn rms_norm_mul(x: &DevBuf, w: &DevBuf, out: &DevBuf, n: usize, eps: f32, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::rms_norm_mul", [(x, nseq * n * 4), (w, n * 4), (out, nseq * n * 4)], ffi::llamd_fwd_rms_norm_mul(f(x), f(w), f(out), n as i32, eps, nseq as i32))
    }
    /// `nblocks_total` = blocks per sequence x nseq: sequences are contiguous.
    pub fn quantize(x: &DevBuf, qs: &DevBuf, d: &DevBuf, nblocks_total: usize) -> Result<()> {
        launch!("bop::quantize", [(x, nblocks_total * QK * 4), (qs, nblocks_total * QK), (d, nblocks_total * 4)],
                ffi::llamd_fwd_quantize(f(x), q(qs), f(d), nblocks_total as i32))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn matvec(w: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::matvec", [(w, q6k_tiled_bytes(rows * blocks)), (aq, nseq * blocks * QK), (ad, nseq * blocks * 4), (out, nseq * rows * 4)],
                ffi::llamd_fwd_matvec_batch(w.ptr(), q(aq), f(ad), f(out), blocks as i32, rows as i32, nseq as i32))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn matvec_x3(w0: &DevBuf, w1: &DevBuf, w2: &DevBuf, aq: &DevBuf, ad: &DevBuf, o0: &DevBuf, o1: &DevBuf, o2: &DevBuf, blocks: usize, rows0: usize, rows1: usize, rows2: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::matvec_x3", [(w0, q6k_tiled_bytes(rows0 * blocks)), (w1, q6k_tiled_bytes(rows1 * blocks)), (w2, q6k_tiled_bytes(rows2 * blocks)), (aq, nseq * blocks * QK), (ad, nseq * blocks * 4), (o0, nseq * rows0 * 4), (o1, nseq * rows1 * 4), (o2, nseq * rows2 * 4)],
                ffi::llamd_fwd_matvec_x3_batch(w0.ptr(), w1.ptr(), w2.ptr(), q(aq), f(ad), f(o0), f(o1), f(o2), blocks as i32, rows0 as i32, rows1 as i32, rows2 as i32, nseq as i32))
    }
    /// gate and up of every sequence's routed experts: `ids` is `[nseq][n_used]`, outputs `[nseq * n_used][rows]`.
    #[allow(clippy::too_many_arguments)]
    pub fn grouped_x2(wa: &DevBuf, wb: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, oa: &DevBuf, ob: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        let wbytes = q6k_tiled_bytes(n_expert * rows * blocks);
        let slots = nseq * n_used;
        launch!("bop::grouped_x2", [(wa, wbytes), (wb, wbytes), (ids, slots * 4), (aq, nseq * blocks * QK), (ad, nseq * blocks * 4), (oa, slots * rows * 4), (ob, slots * rows * 4)],
                ffi::llamd_fwd_matvec_grouped_x2_batch(wa.ptr(), wb.ptr(), i(ids), q(aq), f(ad), f(oa), f(ob), blocks as i32, rows as i32, n_used as i32, nseq as i32))
    }
    /// The down projections: slot s (of nseq * n_used) reads its own activation.
    #[allow(clippy::too_many_arguments)]
    pub fn grouped_pa(w: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        let slots = nseq * n_used;
        launch!("bop::grouped_pa", [(w, q6k_tiled_bytes(n_expert * rows * blocks)), (ids, slots * 4), (aq, slots * blocks * QK), (ad, slots * blocks * 4), (out, slots * rows * 4)],
                ffi::llamd_fwd_matvec_grouped_pa_batch(w.ptr(), i(ids), q(aq), f(ad), f(out), blocks as i32, rows as i32, n_used as i32, nseq as i32))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn norm_rope(x: &DevBuf, w: &DevBuf, n_head: usize, hd: usize, meta: &DevBuf, rope_tab: &DevBuf, eps: f32, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::norm_rope", [(x, nseq * n_head * hd * 4), (w, hd * 4), (meta, nseq * 8)], ffi::llamd_fwd_norm_rope(f(x), f(w), n_head as i32, hd as i32, i(meta), f(rope_tab), eps, nseq as i32))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn k_norm_rope_store(k: &DevBuf, w: &DevBuf, v: &DevBuf, kc: &DevBuf, vc: &DevBuf, n_head_kv: usize, hd: usize, meta: &DevBuf, rope_tab: &DevBuf, eps: f32, nseq: usize, max_kv: usize) -> Result<()> {
        seqs(nseq)?;
        let kvd = n_head_kv * hd;
        launch!("bop::k_norm_rope_store", [(k, nseq * kvd * 4), (w, hd * 4), (v, nseq * kvd * 4), (kc, nseq * max_kv * kvd * 4), (vc, nseq * max_kv * kvd * 4), (meta, nseq * 8)],
                ffi::llamd_fwd_k_norm_rope_store(f(k), f(w), f(v), f(kc), f(vc), n_head_kv as i32, hd as i32, kvd as i32, i(meta), f(rope_tab), eps, nseq as i32, max_kv as i32))
    }
    /// Every sequence attends its own cache up to its own position. `scores`: `[nseq][n_head][max_kv]`.
    #[allow(clippy::too_many_arguments)]
    pub fn attention(qv: &DevBuf, kc: &DevBuf, vc: &DevBuf, out: &DevBuf, scores: &DevBuf, n_head: usize, n_head_kv: usize, hd: usize, meta: &DevBuf, max_kv: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        if n_head_kv == 0 || n_head % n_head_kv != 0 {
            return Err(Error::malformed("bop::attention", "head grouping"));
        }
        let kvd = n_head_kv * hd;
        launch!("bop::attention", [(qv, nseq * n_head * hd * 4), (kc, nseq * max_kv * kvd * 4), (vc, nseq * max_kv * kvd * 4), (out, nseq * n_head * hd * 4), (scores, nseq * n_head * max_kv * 4), (meta, nseq * 8)],
                ffi::llamd_fwd_attention_meta(f(qv), f(kc), f(vc), f(out), f(scores), n_head as i32, n_head_kv as i32, hd as i32, i(meta), max_kv as i32, nseq as i32))
    }
    pub fn add(a: &DevBuf, b: &DevBuf, o: &DevBuf, n: usize) -> Result<()> {
        launch!("bop::add", [(a, n * 4), (b, n * 4), (o, n * 4)], ffi::llamd_fwd_add(f(a), f(b), f(o), n as i32))
    }
    pub fn silu_mul(g: &DevBuf, u: &DevBuf, o: &DevBuf, n: usize) -> Result<()> {
        launch!("bop::silu_mul", [(g, n * 4), (u, n * 4), (o, n * 4)], ffi::llamd_fwd_silu_mul(f(g), f(u), f(o), n as i32))
    }
    pub fn matvec_f32(w: &DevBuf, x: &DevBuf, out: &DevBuf, k: usize, rows: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::matvec_f32", [(w, rows * k * 4), (x, nseq * k * 4), (out, nseq * rows * 4)], ffi::llamd_fwd_matvec_f32_batch(f(w), f(x), f(out), k as i32, rows as i32, nseq as i32))
    }
    pub fn router(logits: &DevBuf, n_expert: usize, n_used: usize, ids: &DevBuf, weights: &DevBuf, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        if n_used == 0 || n_used > n_expert || n_expert > 1024 || n_used > 64 {
            return Err(Error::malformed("moe routing", format!("{n_used} experts requested of {n_expert}")));
        }
        launch!("bop::router", [(logits, nseq * n_expert * 4), (ids, nseq * n_used * 4), (weights, nseq * n_used * 4)],
                ffi::llamd_fwd_router(f(logits), n_expert as i32, n_used as i32, i(ids), f(weights), std::ptr::null_mut(), nseq as i32))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn moe_combine_add(down: &DevBuf, weights: &DevBuf, residual: &DevBuf, out: &DevBuf, n_used: usize, n_embd: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::moe_combine_add", [(down, nseq * n_used * n_embd * 4), (weights, nseq * n_used * 4), (residual, nseq * n_embd * 4), (out, nseq * n_embd * 4)],
                ffi::llamd_fwd_moe_combine_add(f(down), f(weights), f(residual), f(out), n_used as i32, n_embd as i32, nseq as i32))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn argmax(x: &DevBuf, n: usize, scratch_v: &DevBuf, scratch_i: &DevBuf, out: &DevBuf, nblocks: usize, nseq: usize) -> Result<()> {
        seqs(nseq)?;
        launch!("bop::argmax", [(x, nseq * n * 4), (scratch_v, nseq * nblocks * 4), (scratch_i, nseq * nblocks * 4), (out, nseq * 4)],
                ffi::llamd_fwd_argmax(f(x), n as i32, f(scratch_v), i(scratch_i), i(out), nblocks as i32, nseq as i32))
    }
}
