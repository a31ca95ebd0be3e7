//! The resident model of the library (`llamd_model_*` of `include/llamd_cuda_model.h`) as an owned handle.
//!
//! The ROCm runtime type queues its ~600 launches per token from Rust through `op::*`. Here the same queue lives in
//! the library (`csrc/model.cu`), so that it can be captured into a CUDA graph together with the device-side token
//! feedback, and so that expert parallelism can wire peer memory into the launches. `llamd-runtime`'s `CudaModel`
//! (`crates/llamd-runtime/src/cuda_model.rs`) is a thin owner of this handle with `DeviceModel`'s methods.

use llamd_core::{Error, Result};

#[cfg(cuda)]
use crate::ffi;
use crate::not_built;

/// Architecture numbers the library needs, in the order of `llamd_hparams`.
#[derive(Debug, Clone, Copy, PartialEq)]
pub struct ModelDims {
    pub n_layer: usize,
    pub n_embd: usize,
    pub n_head: usize,
    pub n_head_kv: usize,
    pub head_dim: usize,
    pub n_expert: usize,
    pub n_expert_used: usize,
    pub n_ff_expert: usize,
    pub n_vocab: usize,
    pub rope_freq_base: f32,
    pub rms_eps: f32,
}

/// Tensor ids of `llamd_model_set_tensor` (`LLAMD_T_*`).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[repr(i32)]
pub enum TensorId {
    TokEmbd = 0,
    OutputNorm = 1,
    Output = 2,
    AttnNorm = 3,
    AttnQ = 4,
    AttnK = 5,
    AttnV = 6,
    AttnQNorm = 7,
    AttnKNorm = 8,
    AttnOut = 9,
    FfnNorm = 10,
    FfnGateInp = 11,
    FfnGateExps = 12,
    FfnUpExps = 13,
    FfnDownExps = 14,
}

pub struct CudaModelHandle {
    #[cfg(cuda)]
    h: *mut ffi::llamd_model,
    dims: ModelDims,
    max_kv: usize,
    max_seq: usize,
}

// SAFETY: the handle is used from one thread at a time (`&mut self` on every call that launches); the library's
// single stream serialises the work.
#[allow(unsafe_code)]
unsafe impl Send for CudaModelHandle {}

impl CudaModelHandle {
    /// Room for `max_seq` sequences of `max_kv` positions; weights arrive through [`CudaModelHandle::set_tensor`].
    pub fn create(dims: ModelDims, max_kv: usize, max_seq: usize) -> Result<Self> {
        if max_kv == 0 {
            return Err(Error::malformed("device model", "max_kv of 0"));
        }
        if max_seq == 0 || max_seq > crate::max_seq() {
            return Err(Error::malformed("device model", format!("max_seq {max_seq} outside 1..={}", crate::max_seq())));
        }
        #[cfg(not(cuda))]
        {
            let _ = dims;
            not_built()
        }
        #[cfg(cuda)]
        {
            if !crate::available() {
                return Err(Error::unsupported("cuda", "no device present (there is no CPU fallback)"));
            }
            let hp = ffi::llamd_hparams {
                n_layer: dims.n_layer as i32,
                n_embd: dims.n_embd as i32,
                n_head: dims.n_head as i32,
                n_head_kv: dims.n_head_kv as i32,
                head_dim: dims.head_dim as i32,
                n_expert: dims.n_expert as i32,
                n_expert_used: dims.n_expert_used as i32,
                n_ff_expert: dims.n_ff_expert as i32,
                n_vocab: dims.n_vocab as i32,
                rope_freq_base: dims.rope_freq_base,
                rms_eps: dims.rms_eps,
            };
            // SAFETY: `hp` is a live local of the layout the header declares; null on failure.
            #[allow(unsafe_code)]
            let h = unsafe { ffi::llamd_model_create(&hp, max_kv as i32, max_seq as i32) };
            if h.is_null() {
                return Err(Error::other(format!("model create failed: {}", crate::last_error_text())));
            }
            Ok(CudaModelHandle { h, dims, max_kv, max_seq })
        }
    }

    pub fn dims(&self) -> &ModelDims {
        &self.dims
    }
    pub fn max_kv(&self) -> usize {
        self.max_kv
    }
    pub fn max_seq(&self) -> usize {
        self.max_seq
    }

    #[cfg(cuda)]
    fn error_text(&self) -> String {
        // SAFETY: a NUL-terminated string owned by the model, copied at once.
        #[allow(unsafe_code)]
        unsafe {
            let p = ffi::llamd_model_error(self.h);
            if p.is_null() {
                String::new()
            } else {
                std::ffi::CStr::from_ptr(p).to_string_lossy().into_owned()
            }
        }
    }

    /// Upload (a slice of) one tensor in the reference's byte layout. Q6_K: `data` is whole 210-byte blocks landing at
    /// block `first_block`; f32: `data` is the whole tensor and `first_block` is 0. With expert parallelism only the
    /// experts this rank owns are kept.
    pub fn set_tensor(&mut self, layer: i32, which: TensorId, first_block: usize, data: &[u8]) -> Result<()> {
        let is_f32 = matches!(which, TensorId::OutputNorm | TensorId::AttnNorm | TensorId::AttnQNorm | TensorId::AttnKNorm | TensorId::FfnNorm | TensorId::FfnGateInp);
        let unit = if is_f32 { 4 } else { llamd_quant::Q6K_BLOCK_BYTES };
        if data.is_empty() || data.len() % unit != 0 {
            return Err(Error::malformed("set_tensor", format!("{} bytes is not a whole number of {unit}-byte units", data.len())));
        }
        #[cfg(not(cuda))]
        {
            let _ = (layer, first_block);
            not_built()
        }
        #[cfg(cuda)]
        {
            // SAFETY: `count` units of `unit` bytes are exactly `data`; the library checks the slice against the tensor.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_model_set_tensor(self.h, layer, which as i32, first_block, data.as_ptr() as *const _, data.len() / unit) };
            if rc != 0 {
                return Err(Error::other(format!("set_tensor: {}", self.error_text())));
            }
            Ok(())
        }
    }

    /// "use_graph", "trace", "prefill_tile", "prefill_gemm", "prefill_attn", "ep_poll_limit", ... (`llamd_model_set_option`).
    pub fn set_option(&mut self, name: &str, value: i32) -> Result<()> {
        #[cfg(not(cuda))]
        {
            let _ = (name, value);
            not_built()
        }
        #[cfg(cuda)]
        {
            let c = std::ffi::CString::new(name).map_err(|_| Error::malformed("set_option", "name contains NUL"))?;
            // SAFETY: a NUL-terminated name and an integer.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_model_set_option(self.h, c.as_ptr(), value) };
            if rc != 0 {
                return Err(Error::malformed("set_option", format!("{name} = {value} refused")));
            }
            Ok(())
        }
    }

    pub fn weight_bytes(&self) -> usize {
        #[cfg(cuda)]
        {
            // SAFETY: a live handle.
            #[allow(unsafe_code)]
            unsafe {
                ffi::llamd_model_weight_bytes(self.h)
            }
        }
        #[cfg(not(cuda))]
        0
    }

    fn check_token(&self, token: u32, pos: usize) -> Result<()> {
        if pos >= self.max_kv {
            return Err(Error::malformed("device forward", format!("position {pos} beyond the {} allocated", self.max_kv)));
        }
        if token as usize >= self.dims.n_vocab {
            return Err(Error::malformed("device forward", format!("token {token} outside a vocabulary of {}", self.dims.n_vocab)));
        }
        Ok(())
    }

    /// One token in, the greedy next token out: 8 bytes up, 4 bytes down, one synchronise.
    pub fn forward(&mut self, token: u32, pos: usize) -> Result<u32> {
        self.check_token(token, pos)?;
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let mut out = -1i32;
            // SAFETY: `out` is a live local.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_model_forward(self.h, token as i32, pos as i32, &mut out) };
            if rc != 0 || out < 0 {
                return Err(Error::other(format!("forward: {}", self.error_text())));
            }
            Ok(out as u32)
        }
    }

    /// `tokens.len()` independent sequences in one pass.
    pub fn forward_batch(&mut self, tokens: &[u32], positions: &[usize]) -> Result<Vec<u32>> {
        if tokens.len() != positions.len() || tokens.is_empty() || tokens.len() > self.max_seq {
            return Err(Error::malformed("forward_batch", format!("{} tokens, {} positions, max_seq {}", tokens.len(), positions.len(), self.max_seq)));
        }
        for (&t, &p) in tokens.iter().zip(positions) {
            self.check_token(t, p)?;
        }
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let t: Vec<i32> = tokens.iter().map(|&v| v as i32).collect();
            let p: Vec<i32> = positions.iter().map(|&v| v as i32).collect();
            let mut out = vec![-1i32; t.len()];
            // SAFETY: three arrays of `nseq` elements.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_model_forward_batch(self.h, t.as_ptr(), p.as_ptr(), t.len() as i32, out.as_mut_ptr()) };
            if rc != 0 {
                return Err(Error::other(format!("forward_batch: {}", self.error_text())));
            }
            Ok(out.into_iter().map(|v| v as u32).collect())
        }
    }

    /// Consume a prompt at positions `base_pos..`, in tiles; the greedy token after its last token.
    pub fn prefill(&mut self, tokens: &[u32], base_pos: usize) -> Result<u32> {
        if tokens.is_empty() {
            return Err(Error::malformed("prefill", "empty prompt"));
        }
        if base_pos + tokens.len() > self.max_kv {
            return Err(Error::malformed("prefill", format!("positions beyond the {} allocated", self.max_kv)));
        }
        if let Some(&bad) = tokens.iter().find(|&&t| t as usize >= self.dims.n_vocab) {
            return Err(Error::malformed("prefill", format!("token {bad} outside the vocabulary")));
        }
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let t: Vec<i32> = tokens.iter().map(|&v| v as i32).collect();
            let mut out = -1i32;
            // SAFETY: `t` holds `n_tokens` ids; `out` is a live local.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_model_prefill(self.h, t.as_ptr(), t.len() as i32, base_pos as i32, &mut out) };
            if rc != 0 || out < 0 {
                return Err(Error::other(format!("prefill: {}", self.error_text())));
            }
            Ok(out as u32)
        }
    }

    /// `n` greedy tokens with the token fed back on the device and one synchronise at the end; also the device time.
    pub fn decode(&mut self, first_token: u32, start_pos: usize, n: usize) -> Result<(Vec<u32>, f32)> {
        if n == 0 || start_pos + n > self.max_kv {
            return Err(Error::malformed("decode", format!("{n} tokens from position {start_pos} with {} allocated", self.max_kv)));
        }
        self.check_token(first_token, start_pos)?;
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let mut out = vec![-1i32; n];
            let mut ms = 0f32;
            // SAFETY: `out` holds `n` ids; `ms` is a live local.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_model_decode(self.h, first_token as i32, start_pos as i32, n as i32, out.as_mut_ptr(), &mut ms) };
            if rc != 0 {
                return Err(Error::other(format!("decode: {}", self.error_text())));
            }
            Ok((out.into_iter().map(|v| v as u32).collect(), ms))
        }
    }

    /// The logits of the last pass, `nseq` rows of `n_vocab`.
    pub fn logits(&self, nseq: usize) -> Result<Vec<f32>> {
        if nseq == 0 || nseq > self.max_seq {
            return Err(Error::malformed("logits", format!("{nseq} sequences of {}", self.max_seq)));
        }
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let mut out = vec![0f32; nseq * self.dims.n_vocab];
            // SAFETY: `out` holds nseq * n_vocab floats, what the callee copies.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_model_logits(self.h, out.as_mut_ptr(), nseq as i32) };
            if rc != 0 {
                return Err(Error::other(format!("logits: {}", self.error_text())));
            }
            Ok(out)
        }
    }
}

impl Drop for CudaModelHandle {
    fn drop(&mut self) {
        #[cfg(cuda)]
        {
            // SAFETY: created by `llamd_model_create`, freed once; the library drains its stream and drops a graph that
            // points at this model's buffers before freeing them.
            #[allow(unsafe_code)]
            unsafe {
                ffi::llamd_model_free(self.h)
            };
        }
    }
}
