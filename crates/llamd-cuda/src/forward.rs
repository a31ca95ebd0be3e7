//! Device buffers, the library stream, the captured graph and the per-op launches: the counterpart of
//! `llamd-rocm/src/forward.rs`, same names and argument order wherever an op exists on both sides.
//!
//! Every `op::*` function enqueues on the ONE stream the library owns and returns at once; nothing here
//! synchronises except [`sync`], [`DevBuf::download_f32`] and friends. Failures inside a launch are sticky in the
//! library and surface at the next [`sync`], once per token, as on the ROCm side. Before any launch the wrapper
//! checks that every buffer is large enough for the extents it passes: that check is what makes the call safe.
//!
//! Differences from the ROCm surface, all additive: RoPE takes a sin/cos table built on the host with the host's own
//! libm ([`rope_table`]) instead of `freq_base`, which is how the kernels reproduce the CPU path's `powf/sin/cos`
//! bit for bit; the `planar_*` names exist and run the tiled-layout kernels (this backend's one weight layout);
//! fused forms the ROCm crate does not have (`add_rms_norm_quant`, `combine_rms_norm_quant`, `qk_norm_rope_store`,
//! `router_matvec`, `silu_mul_quant`) sit beside the ones it has.

use std::ffi::c_void;

use llamd_core::{Error, Result};

#[cfg(cuda)]
use crate::ffi;
use crate::not_built;

/// A device allocation. Not `Clone`; freed on `Drop`.
pub struct DevBuf {
    #[cfg(cuda)]
    ptr: *mut c_void,
    bytes: usize,
}

// SAFETY: an opaque device pointer, only dereferenced by library calls on the library's single stream; freed once.
#[allow(unsafe_code)]
unsafe impl Send for DevBuf {}
#[allow(unsafe_code)]
unsafe impl Sync for DevBuf {}

impl DevBuf {
    pub fn new(bytes: usize) -> Result<Self> {
        #[cfg(not(cuda))]
        {
            let _ = bytes;
            not_built()
        }
        #[cfg(cuda)]
        {
            if !crate::available() {
                return Err(Error::unsupported("cuda", "no device present"));
            }
            // SAFETY: a size in, a pointer or null out.
            #[allow(unsafe_code)]
            let ptr = unsafe { ffi::llamd_fwd_alloc(bytes.max(1)) };
            if ptr.is_null() {
                return Err(Error::other(format!("cudaMalloc of {bytes} bytes failed: {}", crate::last_error_text())));
            }
            Ok(DevBuf { ptr, bytes })
        }
    }

    pub fn from_bytes(host: &[u8]) -> Result<Self> {
        let b = DevBuf::new(host.len())?;
        b.upload_bytes(host)?;
        Ok(b)
    }

    pub fn from_f32(host: &[f32]) -> Result<Self> {
        let b = DevBuf::new(host.len() * 4)?;
        b.upload_raw(host.as_ptr() as *const c_void, host.len() * 4)?;
        Ok(b)
    }

    pub fn zeroed(bytes: usize) -> Result<Self> {
        let b = DevBuf::new(bytes)?;
        b.zero()?;
        Ok(b)
    }

    pub fn bytes(&self) -> usize {
        self.bytes
    }

    /// The raw device address. Only meaningful to this crate's own launches.
    pub fn ptr(&self) -> *mut c_void {
        #[cfg(cuda)]
        {
            self.ptr
        }
        #[cfg(not(cuda))]
        std::ptr::null_mut()
    }

    fn upload_raw(&self, src: *const c_void, bytes: usize) -> Result<()> {
        if bytes > self.bytes {
            return Err(Error::malformed("device upload", format!("{bytes} bytes into a buffer of {}", self.bytes)));
        }
        #[cfg(not(cuda))]
        {
            let _ = src;
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: `bytes` fits the destination (checked) and every caller passes a source of at least that size.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_fwd_upload(self.ptr, src, bytes) };
            if rc != 0 {
                return Err(Error::other(format!("host to device copy failed: {}", crate::last_error_text())));
            }
            Ok(())
        }
    }

    fn download_raw(&self, dst: *mut c_void, bytes: usize) -> Result<()> {
        if bytes > self.bytes {
            return Err(Error::malformed("device download", format!("{bytes} bytes from a buffer of {}", self.bytes)));
        }
        #[cfg(not(cuda))]
        {
            let _ = dst;
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: `bytes` fits the source (checked) and every caller passes a destination of at least that size.
            // The call orders itself after the stream's queued work.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_fwd_download(dst, self.ptr, bytes) };
            if rc != 0 {
                return Err(Error::other(format!("device to host copy failed: {}", crate::last_error_text())));
            }
            Ok(())
        }
    }

    pub fn upload_bytes(&self, host: &[u8]) -> Result<()> {
        self.upload_raw(host.as_ptr() as *const c_void, host.len())
    }
    pub fn upload_f32(&self, host: &[f32]) -> Result<()> {
        self.upload_raw(host.as_ptr() as *const c_void, host.len() * 4)
    }
    pub fn upload_i32(&self, host: &[i32]) -> Result<()> {
        self.upload_raw(host.as_ptr() as *const c_void, host.len() * 4)
    }
    pub fn download_bytes(&self, out: &mut [u8]) -> Result<()> {
        self.download_raw(out.as_mut_ptr() as *mut c_void, out.len())
    }
    pub fn download_f32(&self, out: &mut [f32]) -> Result<()> {
        self.download_raw(out.as_mut_ptr() as *mut c_void, out.len() * 4)
    }
    pub fn download_i32(&self, out: &mut [i32]) -> Result<()> {
        self.download_raw(out.as_mut_ptr() as *mut c_void, out.len() * 4)
    }

    pub fn zero(&self) -> Result<()> {
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: the whole allocation, whose size this handle records.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_fwd_memset(self.ptr, 0, self.bytes) };
            if rc != 0 {
                return Err(Error::other(format!("cudaMemset failed: {}", crate::last_error_text())));
            }
            Ok(())
        }
    }
}

impl Drop for DevBuf {
    fn drop(&mut self) {
        #[cfg(cuda)]
        {
            // SAFETY: allocated by `llamd_fwd_alloc`, freed once. The library synchronises its stream before freeing,
            // so no queued launch still reads the buffer.
            #[allow(unsafe_code)]
            unsafe {
                ffi::llamd_fwd_free(self.ptr)
            };
        }
    }
}

pub fn free_memory() -> usize {
    #[cfg(cuda)]
    {
        // SAFETY: no arguments; 0 on failure.
        #[allow(unsafe_code)]
        unsafe {
            ffi::llamd_fwd_free_mem()
        }
    }
    #[cfg(not(cuda))]
    0
}

/// Create the library stream (and, once per process, the table that makes the device's `exp` identical to the host
/// libm's `expf`: about a second). Idempotent.
pub fn stream_init() -> Result<()> {
    #[cfg(not(cuda))]
    {
        not_built()
    }
    #[cfg(cuda)]
    {
        // SAFETY: no arguments.
        #[allow(unsafe_code)]
        let rc = unsafe { ffi::llamd_fwd_stream_init() };
        if rc != 0 {
            return Err(Error::other(format!("stream creation failed: {}", crate::last_error_text())));
        }
        Ok(())
    }
}

/// Wait for everything queued, then report the first failure any launch recorded since the last call.
pub fn sync() -> Result<()> {
    #[cfg(not(cuda))]
    {
        not_built()
    }
    #[cfg(cuda)]
    {
        let text = crate::last_error_text(); // read before the call below clears the state
        // SAFETY: no arguments. Returns -1 if the synchronise failed or a sticky error was pending, and clears it.
        #[allow(unsafe_code)]
        let rc = unsafe { ffi::llamd_fwd_sync() };
        if rc != 0 {
            let after = crate::last_error_text();
            return Err(Error::other(format!("CUDA stream failed: {}", if after.is_empty() { text } else { after })));
        }
        Ok(())
    }
}

/// sin/cos of every (position, pair) angle, computed on the host exactly as `CpuBackend::rope` computes them
/// (`powf`, `sin`, `cos` of the host libm), uploaded once per model: [max_pos][head_dim / 2][sin, cos].
pub fn rope_table(max_pos: usize, head_dim: usize, freq_base: f32) -> Result<DevBuf> {
    if max_pos == 0 || head_dim == 0 || head_dim % 2 != 0 {
        return Err(Error::malformed("rope table", format!("{max_pos} positions of head_dim {head_dim}")));
    }
    #[cfg(not(cuda))]
    {
        let _ = freq_base;
        not_built()
    }
    #[cfg(cuda)]
    {
        let mut tab = vec![0f32; max_pos * head_dim];
        // SAFETY: the table holds max_pos * head_dim floats, what the callee writes. Host-only: no device involved.
        #[allow(unsafe_code)]
        let rc = unsafe { ffi::llamd_cuda_rope_table(tab.as_mut_ptr(), max_pos as i32, head_dim as i32, freq_base) };
        if rc != 0 {
            return Err(Error::other("rope table refused"));
        }
        DevBuf::from_f32(&tab)
    }
}

/// One captured pass, replayed per token. Process-global in the library; the runtime type tags it with its owner.
pub mod graph {
    use super::*;

    fn status(rc: i32, what: &str) -> Result<()> {
        if rc == 0 {
            Ok(())
        } else {
            #[cfg(cuda)]
            let detail = crate::last_error_text();
            #[cfg(not(cuda))]
            let detail = String::new();
            Err(Error::other(format!("{what} failed: {detail}")))
        }
    }

    pub fn begin() -> Result<()> {
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: no arguments.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_fwd_begin_capture() };
            status(rc, "graph capture begin")
        }
    }
    pub fn end() -> Result<()> {
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: no arguments. A poisoned capture is discarded by the library.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_fwd_end_capture() };
            status(rc, "graph capture end")
        }
    }
    pub fn replay() -> Result<()> {
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: no arguments; fails if no graph exists.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_fwd_graph_launch() };
            status(rc, "graph launch")
        }
    }
    pub fn exists() -> bool {
        #[cfg(cuda)]
        {
            // SAFETY: no arguments.
            #[allow(unsafe_code)]
            unsafe {
                ffi::llamd_fwd_has_graph() != 0
            }
        }
        #[cfg(not(cuda))]
        false
    }
    pub fn destroy() {
        #[cfg(cuda)]
        {
            // SAFETY: no arguments; a no-op without a graph.
            #[allow(unsafe_code)]
            unsafe {
                ffi::llamd_fwd_graph_destroy()
            };
        }
    }
}

pub(crate) fn need(buf: &DevBuf, bytes: usize, what: &'static str) -> Result<()> {
    if buf.bytes() < bytes {
        return Err(Error::malformed(what, format!("buffer holds {} bytes, the launch touches {bytes}", buf.bytes())));
    }
    Ok(())
}

/// Check the listed (buffer, bytes) pairs, then make the FFI call. In a stub build the call is compiled out.
macro_rules! launch {
    ($what:literal, [$(($buf:expr, $bytes:expr)),* $(,)?], $call:expr) => {{
        $( $crate::forward::need($buf, $bytes, $what)?; )*
        #[cfg(not(cuda))]
        {
            $crate::not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: every pointer comes from a live DevBuf whose size was just checked against the extent the
            // kernel touches; scalars are passed by value. The launch is queued, nothing is dereferenced here.
            #[allow(unsafe_code)]
            unsafe {
                $call
            };
            Ok(())
        }
    }};
}
pub(crate) use launch;

const QK: usize = llamd_quant::QK_K;
const Q6K: usize = llamd_quant::Q6K_BLOCK_BYTES;

/// Bytes of `n_blocks` Q6_K blocks in the library's tiled layout (whole 32-block tiles of 6720 bytes).
pub fn q6k_tiled_bytes(n_blocks: usize) -> usize {
    n_blocks.div_ceil(32) * 32 * Q6K
}

pub mod op {
    //! One function per launch. `nseq` forms live in `bop`; the single-sequence forms here are what the ROCm
    //! runtime calls `op::*`.
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

    /// Repack `n_blocks` reference-layout blocks (already on the device) into the tiled layout.
    pub fn repack_q6k(src: &DevBuf, dst: &DevBuf, n_blocks: usize) -> Result<()> {
        launch!("repack_q6k", [(src, n_blocks * Q6K), (dst, q6k_tiled_bytes(n_blocks))], ffi::llamd_fwd_repack_q6k(src.ptr(), dst.ptr(), n_blocks))
    }
    pub fn unpack_q6k(tiled: &DevBuf, dst: &DevBuf, n_blocks: usize) -> Result<()> {
        launch!("unpack_q6k", [(tiled, q6k_tiled_bytes(n_blocks)), (dst, n_blocks * Q6K)], ffi::llamd_fwd_unpack_q6k(tiled.ptr(), dst.ptr(), n_blocks))
    }
    pub fn dequantize_q6k(tiled: &DevBuf, first_block: usize, n_blocks: usize, out: &DevBuf) -> Result<()> {
        launch!("dequantize_q6k", [(tiled, q6k_tiled_bytes(first_block + n_blocks)), (out, n_blocks * QK * 4)],
                ffi::llamd_fwd_dequantize_q6k(tiled.ptr(), first_block, n_blocks, f(out)))
    }

    pub fn embed(table: &DevBuf, token: u32, out: &DevBuf, blocks: usize) -> Result<()> {
        launch!("embed", [(table, q6k_tiled_bytes((token as usize + 1) * blocks)), (out, blocks * QK * 4)],
                ffi::llamd_fwd_embed(table.ptr(), token as i32, f(out), blocks as i32))
    }
    /// `meta` = [token, pos] on the device, so that a captured graph serves every token.
    pub fn embed_meta(table: &DevBuf, meta: &DevBuf, out: &DevBuf, blocks: usize) -> Result<()> {
        launch!("embed_meta", [(meta, 8), (out, blocks * QK * 4)], ffi::llamd_fwd_embed_meta(table.ptr(), i(meta), f(out), blocks as i32, 1))
    }
    pub fn rms_norm_mul(x: &DevBuf, w: &DevBuf, out: &DevBuf, n: usize, eps: f32) -> Result<()> {
        launch!("rms_norm_mul", [(x, n * 4), (w, n * 4), (out, n * 4)], ffi::llamd_fwd_rms_norm_mul(f(x), f(w), f(out), n as i32, eps, 1))
    }
    pub fn head_rms_norm_mul(x: &DevBuf, w: &DevBuf, out: &DevBuf, n_head: usize, hd: usize, eps: f32) -> Result<()> {
        launch!("head_rms_norm_mul", [(x, n_head * hd * 4), (w, hd * 4), (out, n_head * hd * 4)],
                ffi::llamd_fwd_head_rms_norm_mul(f(x), f(w), f(out), n_head as i32, hd as i32, eps))
    }
    /// norm * w as f32 (`out`, may alias nothing) and as Q8_K planes, one launch.
    pub fn rms_norm_quant(x: &DevBuf, w: &DevBuf, out: &DevBuf, qs: &DevBuf, d: &DevBuf, n: usize, eps: f32) -> Result<()> {
        if n % QK != 0 {
            return Err(Error::malformed("rms_norm_quant", format!("{n} is not a whole number of Q8_K blocks")));
        }
        launch!("rms_norm_quant", [(x, n * 4), (w, n * 4), (out, n * 4), (qs, n), (d, n / QK * 4)],
                ffi::llamd_fwd_rms_norm_quant(f(x), f(w), f(out), q(qs), f(d), n as i32, eps, 1))
    }
    /// x + residual -> sum_out, then as `rms_norm_quant`: the attention residual fused into the FFN norm.
    #[allow(clippy::too_many_arguments)]
    pub fn add_rms_norm_quant(x: &DevBuf, residual: &DevBuf, sum_out: &DevBuf, w: &DevBuf, out: &DevBuf, qs: &DevBuf, d: &DevBuf, n: usize, eps: f32) -> Result<()> {
        if n % QK != 0 {
            return Err(Error::malformed("add_rms_norm_quant", format!("{n} is not a whole number of Q8_K blocks")));
        }
        launch!("add_rms_norm_quant", [(x, n * 4), (residual, n * 4), (sum_out, n * 4), (w, n * 4), (out, n * 4), (qs, n), (d, n / QK * 4)],
                ffi::llamd_fwd_add_rms_norm_quant(f(x), f(residual), f(sum_out), f(w), f(out), q(qs), f(d), n as i32, eps, 1))
    }
    /// x + sum_e weights[e] * down[e] (routing order) -> sum_out, then as `rms_norm_quant`: the MoE combine of one layer
    /// fused into the attention norm of the next.
    #[allow(clippy::too_many_arguments)]
    pub fn combine_rms_norm_quant(x: &DevBuf, down: &DevBuf, weights: &DevBuf, n_used: usize, sum_out: &DevBuf, w: &DevBuf, out: &DevBuf, qs: &DevBuf, d: &DevBuf, n: usize, eps: f32) -> Result<()> {
        if n % QK != 0 {
            return Err(Error::malformed("combine_rms_norm_quant", format!("{n} is not a whole number of Q8_K blocks")));
        }
        launch!("combine_rms_norm_quant", [(x, n * 4), (down, n_used * n * 4), (weights, n_used * 4), (sum_out, n * 4), (w, n * 4), (out, n * 4), (qs, n), (d, n / QK * 4)],
                ffi::llamd_fwd_combine_rms_norm_quant(f(x), f(down), f(weights), n_used as i32, f(sum_out), f(w), f(out), q(qs), f(d), n as i32, eps, 1))
    }
    /// NeoX RoPE in place at `pos`, angles from [`rope_table`].
    pub fn rope(x: &DevBuf, pos: u32, n_head: usize, hd: usize, rope_tab: &DevBuf) -> Result<()> {
        launch!("rope", [(x, n_head * hd * 4), (rope_tab, (pos as usize + 1) * hd * 4)], ffi::llamd_fwd_rope(f(x), pos as i32, n_head as i32, hd as i32, f(rope_tab)))
    }
    /// Per-head norm then RoPE, position from `meta`.
    pub fn norm_rope(x: &DevBuf, w: &DevBuf, n_head: usize, hd: usize, meta: &DevBuf, rope_tab: &DevBuf, eps: f32) -> Result<()> {
        launch!("norm_rope", [(x, n_head * hd * 4), (w, hd * 4), (meta, 8)], ffi::llamd_fwd_norm_rope(f(x), f(w), n_head as i32, hd as i32, i(meta), f(rope_tab), eps, 1))
    }
    /// K: per-head norm, RoPE, then K and V into the cache at `meta`'s position.
    #[allow(clippy::too_many_arguments)]
    pub fn k_norm_rope_store(k: &DevBuf, w: &DevBuf, v: &DevBuf, kc: &DevBuf, vc: &DevBuf, n_head_kv: usize, hd: usize, meta: &DevBuf, rope_tab: &DevBuf, eps: f32, max_kv: usize) -> Result<()> {
        let kvd = n_head_kv * hd;
        launch!("k_norm_rope_store", [(k, kvd * 4), (w, hd * 4), (v, kvd * 4), (kc, max_kv * kvd * 4), (vc, max_kv * kvd * 4), (meta, 8)],
                ffi::llamd_fwd_k_norm_rope_store(f(k), f(w), f(v), f(kc), f(vc), n_head_kv as i32, hd as i32, kvd as i32, i(meta), f(rope_tab), eps, 1, max_kv as i32))
    }
    /// Q and K heads in one launch: QK-norm, RoPE, KV store.
    #[allow(clippy::too_many_arguments)]
    pub fn qk_norm_rope_store(qv: &DevBuf, wq: &DevBuf, k: &DevBuf, wk: &DevBuf, v: &DevBuf, kc: &DevBuf, vc: &DevBuf, n_head: usize, n_head_kv: usize, hd: usize, meta: &DevBuf, rope_tab: &DevBuf, eps: f32, max_kv: usize) -> Result<()> {
        let kvd = n_head_kv * hd;
        launch!("qk_norm_rope_store", [(qv, n_head * hd * 4), (wq, hd * 4), (k, kvd * 4), (wk, hd * 4), (v, kvd * 4), (kc, max_kv * kvd * 4), (vc, max_kv * kvd * 4), (meta, 8)],
                ffi::llamd_fwd_qk_norm_rope_store(f(qv), f(wq), f(k), f(wk), f(v), f(kc), f(vc), n_head as i32, n_head_kv as i32, hd as i32, i(meta), f(rope_tab), eps, 1, max_kv as i32))
    }
    pub fn kv_store(kc: &DevBuf, vc: &DevBuf, k: &DevBuf, v: &DevBuf, pos: u32, kv_dim: usize) -> Result<()> {
        let end = (pos as usize + 1) * kv_dim * 4;
        launch!("kv_store", [(kc, end), (vc, end), (k, kv_dim * 4), (v, kv_dim * 4)], ffi::llamd_fwd_kv_store(f(kc), f(vc), f(k), f(v), pos as i32, kv_dim as i32))
    }
    /// GQA attention of one query over `n_kv` cached positions. `scores`: [n_head][n_kv] floats of scratch.
    #[allow(clippy::too_many_arguments)]
    pub fn attention(qv: &DevBuf, kc: &DevBuf, vc: &DevBuf, out: &DevBuf, scores: &DevBuf, n_head: usize, n_head_kv: usize, hd: usize, n_kv: usize) -> Result<()> {
        if n_head_kv == 0 || n_head % n_head_kv != 0 || n_kv == 0 {
            return Err(Error::malformed("attention", "head grouping or an empty cache"));
        }
        let kvd = n_head_kv * hd;
        launch!("attention", [(qv, n_head * hd * 4), (kc, n_kv * kvd * 4), (vc, n_kv * kvd * 4), (out, n_head * hd * 4), (scores, n_head * n_kv * 4)],
                ffi::llamd_fwd_attention(f(qv), f(kc), f(vc), f(out), f(scores), n_head as i32, n_head_kv as i32, hd as i32, n_kv as i32))
    }
    /// The same with n_kv = meta's position + 1. `scores`: [n_head][max_kv].
    #[allow(clippy::too_many_arguments)]
    pub fn attention_meta(qv: &DevBuf, kc: &DevBuf, vc: &DevBuf, out: &DevBuf, scores: &DevBuf, n_head: usize, n_head_kv: usize, hd: usize, meta: &DevBuf, max_kv: usize) -> Result<()> {
        if n_head_kv == 0 || n_head % n_head_kv != 0 {
            return Err(Error::malformed("attention", "head grouping"));
        }
        let kvd = n_head_kv * hd;
        launch!("attention_meta", [(qv, n_head * hd * 4), (kc, max_kv * kvd * 4), (vc, max_kv * kvd * 4), (out, n_head * hd * 4), (scores, n_head * max_kv * 4), (meta, 8)],
                ffi::llamd_fwd_attention_meta(f(qv), f(kc), f(vc), f(out), f(scores), n_head as i32, n_head_kv as i32, hd as i32, i(meta), max_kv as i32, 1))
    }
    /// `attention` for hosts that may not allocate device memory when they call (their own pool owns the GPU): the score
    /// scratch is an array built into the library. n_head * n_kv <= 262144; make the first call at start-up.
    #[allow(clippy::too_many_arguments)]
    pub fn attention_noalloc(qv: &DevBuf, kc: &DevBuf, vc: &DevBuf, out: &DevBuf, n_head: usize, n_head_kv: usize, hd: usize, n_kv: usize) -> Result<()> {
        if n_head_kv == 0 || n_head % n_head_kv != 0 || n_kv == 0 {
            return Err(Error::malformed("attention", "head grouping or an empty cache"));
        }
        if n_head * n_kv > 262_144 {
            return Err(Error::malformed("attention_noalloc", format!("{n_head} heads x {n_kv} positions exceeds the built-in scratch of 262144 floats")));
        }
        let kvd = n_head_kv * hd;
        need(qv, n_head * hd * 4, "attention_noalloc")?;
        need(kc, n_kv * kvd * 4, "attention_noalloc")?;
        need(vc, n_kv * kvd * 4, "attention_noalloc")?;
        need(out, n_head * hd * 4, "attention_noalloc")?;
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: extents checked above.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_fwd_attention_noalloc(f(qv), f(kc), f(vc), f(out), n_head as i32, n_head_kv as i32, hd as i32, n_kv as i32) };
            if rc != 0 {
                return Err(Error::other(format!("attention_noalloc refused: {}", crate::last_error_text())));
            }
            Ok(())
        }
    }
    pub fn add(a: &DevBuf, b: &DevBuf, out: &DevBuf, n: usize) -> Result<()> {
        launch!("add", [(a, n * 4), (b, n * 4), (out, n * 4)], ffi::llamd_fwd_add(f(a), f(b), f(out), n as i32))
    }
    pub fn silu_mul(gate: &DevBuf, up: &DevBuf, out: &DevBuf, n: usize) -> Result<()> {
        launch!("silu_mul", [(gate, n * 4), (up, n * 4), (out, n * 4)], ffi::llamd_fwd_silu_mul(f(gate), f(up), f(out), n as i32))
    }
    /// silu(gate) * up and its Q8_K planes in one launch.
    pub fn silu_mul_quant(gate: &DevBuf, up: &DevBuf, qs: &DevBuf, d: &DevBuf, n: usize) -> Result<()> {
        if n % QK != 0 {
            return Err(Error::malformed("silu_mul_quant", format!("{n} is not a whole number of Q8_K blocks")));
        }
        launch!("silu_mul_quant", [(gate, n * 4), (up, n * 4), (qs, n), (d, n / QK * 4)],
                ffi::llamd_fwd_silu_mul_quant(f(gate), f(up), std::ptr::null_mut(), q(qs), f(d), n as i32))
    }
    /// Softmax over all experts, `n_used` best by (probability descending, index ascending), renormalised with the
    /// 2^-14 floor. `probs` may be omitted.
    pub fn router(logits: &DevBuf, n_expert: usize, n_used: usize, ids: &DevBuf, weights: &DevBuf, probs: Option<&DevBuf>) -> Result<()> {
        if n_used == 0 || n_used > n_expert || n_expert > 1024 || n_used > 64 {
            return Err(Error::malformed("moe routing", format!("{n_used} experts requested of {n_expert}")));
        }
        if let Some(p) = probs {
            need(p, n_expert * 4, "router")?;
        }
        let pp = probs.map(|p| p.ptr() as *mut f32).unwrap_or(std::ptr::null_mut());
        launch!("router", [(logits, n_expert * 4), (ids, n_used * 4), (weights, n_used * 4)],
                ffi::llamd_fwd_router(f(logits), n_expert as i32, n_used as i32, i(ids), f(weights), pp, 1))
    }
    /// The router's f32 matvec and the routing in one launch. `counter`: one zero-initialised word the launch leaves at zero.
    #[allow(clippy::too_many_arguments)]
    pub fn router_matvec(w: &DevBuf, x: &DevBuf, k: usize, n_expert: usize, n_used: usize, logits: &DevBuf, ids: &DevBuf, weights: &DevBuf, counter: &DevBuf) -> Result<()> {
        if n_used == 0 || n_used > n_expert || n_expert > 1024 || n_used > 64 || k % 4 != 0 {
            return Err(Error::malformed("moe routing", format!("{n_used} experts requested of {n_expert}, k {k}")));
        }
        launch!("router_matvec", [(w, n_expert * k * 4), (x, k * 4), (logits, n_expert * 4), (ids, n_used * 4), (weights, n_used * 4), (counter, 4)],
                ffi::llamd_fwd_router_matvec(f(w), f(x), k as i32, n_expert as i32, n_used as i32, f(logits), i(ids), f(weights), std::ptr::null_mut(), counter.ptr() as *mut u32, 1))
    }
    pub fn moe_combine(down: &DevBuf, weights: &DevBuf, out: &DevBuf, n_used: usize, n_embd: usize) -> Result<()> {
        launch!("moe_combine", [(down, n_used * n_embd * 4), (weights, n_used * 4), (out, n_embd * 4)],
                ffi::llamd_fwd_moe_combine(f(down), f(weights), f(out), n_used as i32, n_embd as i32))
    }
    pub fn moe_combine_add(down: &DevBuf, weights: &DevBuf, residual: &DevBuf, out: &DevBuf, n_used: usize, n_embd: usize) -> Result<()> {
        launch!("moe_combine_add", [(down, n_used * n_embd * 4), (weights, n_used * 4), (residual, n_embd * 4), (out, n_embd * 4)],
                ffi::llamd_fwd_moe_combine_add(f(down), f(weights), f(residual), f(out), n_used as i32, n_embd as i32, 1))
    }
    /// Greedy pick, lowest index on an exact tie. `scratch_v` / `scratch_i`: `nblocks` words each.
    pub fn argmax(x: &DevBuf, n: usize, scratch_v: &DevBuf, scratch_i: &DevBuf, out: &DevBuf, nblocks: usize) -> Result<()> {
        launch!("argmax", [(x, n * 4), (scratch_v, nblocks * 4), (scratch_i, nblocks * 4), (out, 4)],
                ffi::llamd_fwd_argmax(f(x), n as i32, f(scratch_v), i(scratch_i), i(out), nblocks as i32, 1))
    }
    /// y[row] = sum over t ascending of w[row][t] * x[t], from -0.0: the router's f32 matvec.
    pub fn matvec_f32(w: &DevBuf, x: &DevBuf, out: &DevBuf, k: usize, rows: usize) -> Result<()> {
        launch!("matvec_f32", [(w, rows * k * 4), (x, k * 4), (out, rows * 4)], ffi::llamd_fwd_matvec_f32(f(w), f(x), f(out), k as i32, rows as i32))
    }
    pub fn quantize(x: &DevBuf, qs: &DevBuf, d: &DevBuf, nblocks: usize) -> Result<()> {
        launch!("quantize", [(x, nblocks * QK * 4), (qs, nblocks * QK), (d, nblocks * 4)], ffi::llamd_fwd_quantize(f(x), q(qs), f(d), nblocks as i32))
    }

    // ---- the Q6_K matvec family. Weights are tiled-layout buffers (DeviceWeights or `repack_q6k`). ----
    pub fn matvec(w: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize) -> Result<()> {
        launch!("matvec", [(w, q6k_tiled_bytes(rows * blocks)), (aq, blocks * QK), (ad, blocks * 4), (out, rows * 4)],
                ffi::llamd_fwd_matvec(w.ptr(), q(aq), f(ad), f(out), blocks as i32, rows as i32))
    }
    /// Q, K and V against one activation, one launch.
    #[allow(clippy::too_many_arguments)]
    pub fn matvec_x3(w0: &DevBuf, w1: &DevBuf, w2: &DevBuf, aq: &DevBuf, ad: &DevBuf, o0: &DevBuf, o1: &DevBuf, o2: &DevBuf, blocks: usize, rows0: usize, rows1: usize, rows2: usize) -> Result<()> {
        launch!("matvec_x3", [(w0, q6k_tiled_bytes(rows0 * blocks)), (w1, q6k_tiled_bytes(rows1 * blocks)), (w2, q6k_tiled_bytes(rows2 * blocks)), (aq, blocks * QK), (ad, blocks * 4), (o0, rows0 * 4), (o1, rows1 * 4), (o2, rows2 * 4)],
                ffi::llamd_fwd_matvec_x3(w0.ptr(), w1.ptr(), w2.ptr(), q(aq), f(ad), f(o0), f(o1), f(o2), blocks as i32, rows0 as i32, rows1 as i32, rows2 as i32))
    }
    /// The expert gather: `ids` (device, n_used of them) pick experts of `rows` rows out of `w`, which holds `n_expert`.
    #[allow(clippy::too_many_arguments)]
    pub fn matvec_grouped(w: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize) -> Result<()> {
        launch!("matvec_grouped", [(w, q6k_tiled_bytes(n_expert * rows * blocks)), (ids, n_used * 4), (aq, blocks * QK), (ad, blocks * 4), (out, n_used * rows * 4)],
                ffi::llamd_fwd_matvec_grouped(w.ptr(), i(ids), q(aq), f(ad), f(out), blocks as i32, rows as i32, n_used as i32))
    }
    /// gate and up of the routed experts, one launch.
    #[allow(clippy::too_many_arguments)]
    pub fn matvec_grouped_x2(wa: &DevBuf, wb: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, oa: &DevBuf, ob: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize) -> Result<()> {
        let wbytes = q6k_tiled_bytes(n_expert * rows * blocks);
        launch!("matvec_grouped_x2", [(wa, wbytes), (wb, wbytes), (ids, n_used * 4), (aq, blocks * QK), (ad, blocks * 4), (oa, n_used * rows * 4), (ob, n_used * rows * 4)],
                ffi::llamd_fwd_matvec_grouped_x2(wa.ptr(), wb.ptr(), i(ids), q(aq), f(ad), f(oa), f(ob), blocks as i32, rows as i32, n_used as i32))
    }
    /// The down projection: slot s reads ITS OWN activation aq[s].
    #[allow(clippy::too_many_arguments)]
    pub fn matvec_grouped_per_act(w: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize) -> Result<()> {
        launch!("matvec_grouped_per_act", [(w, q6k_tiled_bytes(n_expert * rows * blocks)), (ids, n_used * 4), (aq, n_used * blocks * QK), (ad, n_used * blocks * 4), (out, n_used * rows * 4)],
                ffi::llamd_fwd_matvec_grouped_pa(w.ptr(), i(ids), q(aq), f(ad), f(out), blocks as i32, rows as i32, n_used as i32))
    }
    // The names `llamd-runtime`'s device path calls. This backend has one weight layout, so they are the calls above.
    pub fn planar_matvec(w: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize) -> Result<()> {
        matvec(w, aq, ad, out, blocks, rows)
    }
    #[allow(clippy::too_many_arguments)]
    pub fn planar_x3(w0: &DevBuf, w1: &DevBuf, w2: &DevBuf, aq: &DevBuf, ad: &DevBuf, o0: &DevBuf, o1: &DevBuf, o2: &DevBuf, blocks: usize, rows0: usize, rows1: usize, rows2: usize) -> Result<()> {
        matvec_x3(w0, w1, w2, aq, ad, o0, o1, o2, blocks, rows0, rows1, rows2)
    }
    #[allow(clippy::too_many_arguments)]
    pub fn planar_grouped(w: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize) -> Result<()> {
        matvec_grouped(w, ids, aq, ad, out, blocks, rows, n_used, n_expert)
    }
    #[allow(clippy::too_many_arguments)]
    pub fn planar_grouped_x2(wa: &DevBuf, wb: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, oa: &DevBuf, ob: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize) -> Result<()> {
        matvec_grouped_x2(wa, wb, ids, aq, ad, oa, ob, blocks, rows, n_used, n_expert)
    }
    #[allow(clippy::too_many_arguments)]
    pub fn planar_grouped_per_act(w: &DevBuf, ids: &DevBuf, aq: &DevBuf, ad: &DevBuf, out: &DevBuf, blocks: usize, rows: usize, n_used: usize, n_expert: usize) -> Result<()> {
        matvec_grouped_per_act(w, ids, aq, ad, out, blocks, rows, n_used, n_expert)
    }

    /// Q8_0 weights (tiled by `Q80Weights`-style upload) against f32 activations: dequantize, then the in-order f32 dot.
    pub fn matvec_q8_0(w: &DevBuf, x: &DevBuf, out: &DevBuf, blocks32: usize, rows: usize) -> Result<()> {
        launch!("matvec_q8_0", [(x, blocks32 * 32 * 4), (out, rows * 4)], ffi::llamd_fwd_matvec_q8_0(w.ptr(), f(x), f(out), blocks32 as i32, rows as i32, 1))
    }

    // ---- prefill: many tokens against shared weights ----
    /// The expert scatter plan: (token, slot) pairs counting-sorted by expert.
    #[allow(clippy::too_many_arguments)]
    pub fn moe_group(ids: &DevBuf, n_expert: usize, n_used: usize, ntok: usize, gstart: &DevBuf, gcount: &DevBuf, ptoken: &DevBuf, pslot: &DevBuf) -> Result<()> {
        let np = ntok * n_used;
        if n_expert == 0 || n_expert > 1024 || np > 40960 {
            return Err(Error::malformed("moe_group", format!("{n_expert} experts, {np} pairs (at most 1024 and 40960)")));
        }
        launch!("moe_group", [(ids, np * 4), (gstart, n_expert * 4), (gcount, n_expert * 4), (ptoken, np * 4), (pslot, np * 4)],
                ffi::llamd_fwd_moe_group(i(ids), n_expert as i32, n_used as i32, ntok as i32, i(gstart), i(gcount), i(ptoken), i(pslot)))
    }
    /// Q8_K quants [nblocks][256] -> the residue-major words the integer GEMM reads.
    pub fn q8k_residue_major(aq: &DevBuf, aq_rm: &DevBuf, nblocks: usize) -> Result<()> {
        launch!("q8k_residue_major", [(aq, nblocks * QK), (aq_rm, nblocks * QK)], ffi::llamd_fwd_q8k_residue_major(q(aq), aq_rm.ptr(), nblocks))
    }
    /// Up to three matrices against `ntok` activations on the integer tensor path; bit-identical to per-token `matvec`.
    #[allow(clippy::too_many_arguments)]
    pub fn gemm_tokens(w: [Option<&DevBuf>; 3], aq_rm: &DevBuf, ad: &DevBuf, out: [Option<&DevBuf>; 3], blocks: usize, rows: [usize; 3], ntok: usize) -> Result<()> {
        if w[0].is_none() || ntok == 0 {
            return Err(Error::malformed("gemm_tokens", "no matrix or no tokens"));
        }
        for j in 0..3 {
            match (w[j], out[j]) {
                (Some(wj), Some(oj)) => {
                    need(wj, q6k_tiled_bytes(rows[j] * blocks), "gemm_tokens")?;
                    need(oj, ntok * rows[j] * 4, "gemm_tokens")?;
                }
                (None, None) => {}
                _ => return Err(Error::malformed("gemm_tokens", "a matrix without an output, or the reverse")),
            }
        }
        let wp = |j: usize| w[j].map(|b| b.ptr() as *const c_void).unwrap_or(std::ptr::null());
        let op = |j: usize| out[j].map(|b| b.ptr() as *mut f32).unwrap_or(std::ptr::null_mut());
        let r = |j: usize| if w[j].is_some() { rows[j] as i32 } else { 0 };
        launch!("gemm_tokens", [(aq_rm, ntok * blocks * QK), (ad, ntok * blocks * 4)],
                ffi::llamd_fwd_gemm_tokens(wp(0), wp(1), wp(2), aq_rm.ptr(), f(ad), op(0), op(1), op(2), blocks as i32, r(0), r(1), r(2), ntok as i32))
    }
    /// The grouped expert GEMM over the scatter plan: pair p reads activation `act_map[p]` and writes row block `pslot[p]`.
    #[allow(clippy::too_many_arguments)]
    pub fn expert_gemm(wa: &DevBuf, wb: Option<&DevBuf>, gstart: &DevBuf, gcount: &DevBuf, act_map: &DevBuf, pslot: &DevBuf, aq_rm: &DevBuf, ad: &DevBuf, n_act: usize, oa: &DevBuf, ob: Option<&DevBuf>, blocks: usize, rows: usize, n_expert: usize, n_pairs: usize) -> Result<()> {
        let wbytes = q6k_tiled_bytes(n_expert * rows * blocks);
        if wb.is_some() != ob.is_some() {
            return Err(Error::malformed("expert_gemm", "a second matrix without a second output, or the reverse"));
        }
        if let (Some(b), Some(o)) = (wb, ob) {
            need(b, wbytes, "expert_gemm")?;
            need(o, n_pairs * rows * 4, "expert_gemm")?;
        }
        let wbp = wb.map(|b| b.ptr() as *const c_void).unwrap_or(std::ptr::null());
        let obp = ob.map(|b| b.ptr() as *mut f32).unwrap_or(std::ptr::null_mut());
        launch!("expert_gemm", [(wa, wbytes), (gstart, n_expert * 4), (gcount, n_expert * 4), (act_map, n_pairs * 4), (pslot, n_pairs * 4), (aq_rm, n_act * blocks * QK), (ad, n_act * blocks * 4), (oa, n_pairs * rows * 4)],
                ffi::llamd_fwd_expert_gemm(wa.ptr(), wbp, i(gstart), i(gcount), i(act_map), i(pslot), aq_rm.ptr(), f(ad), f(oa), obp, blocks as i32, rows as i32, n_expert as i32))
    }
    /// f32::exp as the CPU path evaluates it (the host libm's expf), elementwise.
    pub fn expf(x: &DevBuf, out: &DevBuf, n: usize) -> Result<()> {
        launch!("expf", [(x, n * 4), (out, n * 4)], ffi::llamd_fwd_expf(f(x), f(out), n))
    }
}
