//! The resident forward pass on the CUDA backend: `DeviceModel`'s surface (`device.rs`) plus `VulkanModel`'s prefill
//! (`vulkan_model.rs`), over `llamd_cuda::CudaModelHandle`.
//!
//! TO ADD THIS FILE TO `llamd-runtime`: `pub mod cuda_model;` in `lib.rs`, `llamd-cuda.workspace = true` in its
//! `Cargo.toml`, `"crates/llamd-cuda"` in the workspace members, and the `Cuda` arm of `backend.rs` shown in
//! `backend_cuda.patch` beside this file. NOT COMPILED where it was written (no Rust toolchain there); it follows the
//! Python runtime type of the same library (`llamd_rs_b200/model.py`), which the GPU parity tests drive.
//!
//! Unlike the ROCm type this one does not queue launches from Rust: the pass lives in the library, which captures it
//! into a CUDA graph once and replays it per token, feeds the token back on the device for `decode`, and cuts a prompt
//! into tiles for `prefill`. What crosses this boundary per token is what crosses it on ROCm: 8 bytes up, 4 bytes
//! down, one synchronise. Results are bit-identical to the CPU path (`forward` in `layer.rs`): expert ids, token ids,
//! logits.

use llamd_core::{Error, Result};
use llamd_cuda::model::{ModelDims, TensorId};
use llamd_cuda::CudaModelHandle;
use llamd_models::Model;

pub struct CudaModel {
    handle: CudaModelHandle,
    hparams: llamd_models::Hparams,
    /// Replay a captured graph instead of queueing every launch (default on), as `DeviceModel::use_graph`.
    pub use_graph: bool,
    /// Tokens per prefill tile, as `VulkanModel::prefill_tile` (default `min(max_kv, 512)`).
    pub prefill_tile: usize,
}

fn raw<'a>(model: &'a Model, name: &str) -> Result<&'a [u8]> {
    let info = model.info(name)?;
    model.gguf().tensor_data(info)
}

/// Norm vectors and the router matrix reach the device as f32; a file may hold them as F32 already (the usual case)
/// or F16, which widens exactly.
fn f32_bytes(model: &Model, name: &str) -> Result<Vec<u8>> {
    let t = model.tensor(name)?; // dequantizes whatever the file holds
    Ok(t.data().iter().flat_map(|v| v.to_le_bytes()).collect())
}

impl CudaModel {
    pub fn load(model: &Model, max_kv: usize) -> Result<Self> {
        Self::load_batched(model, max_kv, 1)
    }

    /// Room for `max_seq` concurrent sequences: activations and KV scale with it, the weights do not.
    pub fn load_batched(model: &Model, max_kv: usize, max_seq: usize) -> Result<Self> {
        llamd_cuda::stream_init()?;
        let hp = model.hparams.clone();
        if !hp.arch.is_moe() {
            return Err(Error::unsupported("device model", "only MoE models are wired up; a dense FFN has no expert path"));
        }
        if max_kv == 0 {
            return Err(Error::malformed("device model", "max_kv of 0"));
        }
        let dims = ModelDims {
            n_layer: hp.n_layer,
            n_embd: hp.n_embd,
            n_head: hp.n_head,
            n_head_kv: hp.n_head_kv,
            head_dim: hp.n_head_dim,
            n_expert: hp.n_expert,
            n_expert_used: hp.n_expert_used,
            n_ff_expert: hp.n_ff_expert,
            n_vocab: hp.n_vocab,
            rope_freq_base: hp.rope_freq_base,
            rms_eps: hp.rms_eps,
        };
        let mut handle = CudaModelHandle::create(dims, max_kv, max_seq)?;

        // Quantized tensors go up verbatim (the library repacks them on the device); every Q6_K check the ROCm loader
        // makes is made here too, before anything is uploaded.
        let q6k = |name: &str| -> Result<&[u8]> {
            let info = model.info(name)?;
            if info.ty != llamd_quant::QuantType::Q6K {
                return Err(Error::unsupported("device model", format!("{name} is {:?}; this backend takes Q6_K", info.ty)));
            }
            raw(model, name)
        };
        handle.set_tensor(-1, TensorId::TokEmbd, 0, q6k(&model.tok_embd)?)?;
        handle.set_tensor(-1, TensorId::OutputNorm, 0, &f32_bytes(model, &model.output_norm)?)?;
        if let Some(out) = &model.output {
            handle.set_tensor(-1, TensorId::Output, 0, q6k(out)?)?; // tied embeddings otherwise
        }
        for (il, l) in model.layers.iter().enumerate() {
            let il = il as i32;
            handle.set_tensor(il, TensorId::AttnNorm, 0, &f32_bytes(model, &l.attn_norm)?)?;
            handle.set_tensor(il, TensorId::AttnQ, 0, q6k(&l.attn_q)?)?;
            handle.set_tensor(il, TensorId::AttnK, 0, q6k(&l.attn_k)?)?;
            handle.set_tensor(il, TensorId::AttnV, 0, q6k(&l.attn_v)?)?;
            if let Some(n) = &l.attn_q_norm {
                handle.set_tensor(il, TensorId::AttnQNorm, 0, &f32_bytes(model, n)?)?;
            }
            if let Some(n) = &l.attn_k_norm {
                handle.set_tensor(il, TensorId::AttnKNorm, 0, &f32_bytes(model, n)?)?;
            }
            handle.set_tensor(il, TensorId::AttnOut, 0, q6k(&l.attn_out)?)?;
            handle.set_tensor(il, TensorId::FfnNorm, 0, &f32_bytes(model, &l.ffn_norm)?)?;
            let need = |n: &Option<String>, what: &str| -> Result<String> { n.clone().ok_or_else(|| Error::malformed("device model", format!("layer {il} has no {what}"))) };
            handle.set_tensor(il, TensorId::FfnGateInp, 0, &f32_bytes(model, &need(&l.ffn_gate_inp, "router")?)?)?;
            // the expert tensors are the large ones: sent in slices so that no second copy of 0.5 GB sits in memory
            for (which, name) in [(TensorId::FfnGateExps, &l.ffn_gate_exps), (TensorId::FfnUpExps, &l.ffn_up_exps), (TensorId::FfnDownExps, &l.ffn_down_exps)] {
                let bytes = q6k(&need(name, "expert tensor")?)?;
                let per_slice = (64 << 20) / llamd_quant::Q6K_BLOCK_BYTES * llamd_quant::Q6K_BLOCK_BYTES;
                let mut first = 0usize;
                for chunk in bytes.chunks(per_slice) {
                    handle.set_tensor(il, which, first, chunk)?;
                    first += chunk.len() / llamd_quant::Q6K_BLOCK_BYTES;
                }
            }
        }
        Ok(CudaModel { handle, hparams: hp, use_graph: true, prefill_tile: max_kv.min(512) })
    }

    pub fn weight_bytes(&self) -> usize {
        self.handle.weight_bytes()
    }
    pub fn hparams(&self) -> &llamd_models::Hparams {
        &self.hparams
    }

    fn push_knobs(&mut self) -> Result<()> {
        self.handle.set_option("use_graph", self.use_graph as i32)?;
        self.handle.set_option("prefill_tile", self.prefill_tile.clamp(1, 4096) as i32)
    }

    /// One token, the greedy next token.
    pub fn forward(&mut self, token: u32, pos: usize) -> Result<u32> {
        self.push_knobs()?;
        self.handle.forward(token, pos)
    }
    /// `tokens.len()` independent sequences, one pass.
    pub fn forward_batch(&mut self, tokens: &[u32], positions: &[usize]) -> Result<Vec<u32>> {
        self.push_knobs()?;
        self.handle.forward_batch(tokens, positions)
    }
    /// Consume a prompt in tiles; the greedy token after it. Equal to feeding the tokens one by one, bit for bit.
    pub fn prefill(&mut self, tokens: &[u32], base_pos: usize) -> Result<u32> {
        self.push_knobs()?;
        self.handle.prefill(tokens, base_pos)
    }
    /// `n` greedy tokens without returning to the host in between; also the device time in milliseconds.
    pub fn decode(&mut self, first_token: u32, start_pos: usize, n: usize) -> Result<(Vec<u32>, f32)> {
        self.push_knobs()?;
        self.handle.decode(first_token, start_pos, n)
    }
    pub fn logits(&self) -> Result<Vec<f32>> {
        self.handle.logits(1)
    }
}
