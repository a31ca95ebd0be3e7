//! The NVIDIA backend: B200 (sm_100a) kernels behind the surface `llamd-rocm` presents.
//!
//! WHAT THIS CRATE IS. `llamd-runtime` and `llamd-bench` drive the ROCm backend by name -- `DeviceWeights`,
//! `DevBuf`, `op::*`, `bop::*`, `graph::*`, `sync` -- and the quantized operator set is deliberately not abstracted
//! behind `llamd_tensor::Backend`. So the drop-in is a crate with the same names, argument meanings and error
//! behaviour over a different kernel library: `libllamd_cuda` (hand-written CUDA, `../../llamd_rs_b200/csrc`, C ABI
//! in `../../include`). Every f32 operation whose order is observable on the CPU path is reproduced in that order,
//! so results are bit-identical to `llamd-cpu`, not merely within the reduction tolerance.
//!
//! NOT COMPILED where it was written: that machine had no Rust toolchain. What keeps it honest instead: `ffi.rs` is
//! generated from the C headers (`gen_ffi.py`, checked by the repository's tests symbol by symbol and argument by
//! argument), and the wrappers below follow, call for call, the Python binding of the same library that the GPU
//! parity tests drive.
//!
//! UNSAFE POLICY, as in `llamd-rocm`: `unsafe` only to cross the FFI boundary, each call behind a safe function that
//! has checked lengths and ids first.
//!
//! AVAILABILITY IS A RUNTIME QUESTION. `build.rs` compiles the kernels when `nvcc` is present and a stub otherwise;
//! callers ask [`available`]. There is no CPU fallback inside this crate: without a device every call answers
//! `Error::Unsupported`.

#![deny(unsafe_code)]

pub mod batch;
#[cfg(cuda)]
#[allow(unsafe_code)]
pub(crate) mod ffi;
pub mod forward;
pub mod model;
pub use batch::{bop, max_seq};
pub use forward::{free_memory, graph, op, stream_init, sync, DevBuf};
pub use model::CudaModelHandle;

use llamd_core::{Error, Result};
use llamd_quant::{BlockQ8K, Q6K_BLOCK_BYTES, QK_K};

#[derive(Debug, Clone)]
pub struct DeviceInfo {
    pub index: i32,
    pub name: String,
    pub total_mem: usize,
    pub free_mem: usize,
    /// Streaming multiprocessors: 148 on a B200.
    pub sm_count: i32,
    /// Threads per warp: 32 on every NVIDIA part.
    pub warp_size: i32,
    /// The compiled-for target as the runtime names the device, e.g. "sm_100".
    pub arch: String,
}

impl std::fmt::Display for DeviceInfo {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        let gib = |b: usize| b as f64 / (1u64 << 30) as f64;
        write!(
            f,
            "{} -- {:.2} GiB ({:.2} free), {} SMs, warp{}, {}",
            self.name,
            gib(self.total_mem),
            gib(self.free_mem),
            self.sm_count,
            self.warp_size,
            self.arch
        )
    }
}

/// Host-facing entry points share grow-only device scratch inside the library (activations, results, expert ids),
/// exactly as the ROCm layer's do, and tests run concurrently: one lock for all of them.
pub(crate) static SCRATCH: std::sync::Mutex<()> = std::sync::Mutex::new(());

pub(crate) fn not_built<T>() -> Result<T> {
    Err(Error::unsupported("cuda", "not built with CUDA support"))
}

/// The library's sticky error text (first failure since it was last read).
#[cfg(cuda)]
pub(crate) fn last_error_text() -> String {
    // SAFETY: returns a NUL-terminated string owned by the library, valid until the next error is recorded; it is
    // copied out at once.
    #[allow(unsafe_code)]
    unsafe {
        let p = ffi::llamd_cuda_last_error_string();
        if p.is_null() {
            String::new()
        } else {
            std::ffi::CStr::from_ptr(p).to_string_lossy().into_owned()
        }
    }
}

/// Was this crate built against a CUDA toolkit?
pub const fn built_with_cuda() -> bool {
    cfg!(cuda)
}

/// Is a device present and usable now?
pub fn available() -> bool {
    device_count() > 0
}

pub fn device_count() -> i32 {
    #[cfg(cuda)]
    {
        // SAFETY: no arguments; answers 0 when the runtime is unusable.
        #[allow(unsafe_code)]
        unsafe {
            ffi::llamd_cuda_device_count()
        }
    }
    #[cfg(not(cuda))]
    0
}

/// One process drives one device. Must precede the first use of the stream; refused afterwards.
pub fn set_device(index: i32) -> Result<()> {
    #[cfg(not(cuda))]
    {
        let _ = index;
        not_built()
    }
    #[cfg(cuda)]
    {
        if index < 0 || index >= device_count() {
            return Err(Error::malformed("cuda device", format!("index {index} of {} devices", device_count())));
        }
        // SAFETY: a plain integer in, a status out.
        #[allow(unsafe_code)]
        let rc = unsafe { ffi::llamd_cuda_set_device(index) };
        if rc != 0 {
            return Err(Error::other(format!("cudaSetDevice({index}): {}", last_error_text())));
        }
        Ok(())
    }
}

pub fn device_info(index: i32) -> Result<DeviceInfo> {
    #[cfg(not(cuda))]
    {
        let _ = index;
        not_built()
    }
    #[cfg(cuda)]
    {
        if index < 0 || index >= device_count() {
            return Err(Error::malformed("cuda device", format!("index {index} of {} devices", device_count())));
        }
        let mut name = [0 as std::os::raw::c_char; 256];
        let mut arch = [0 as std::os::raw::c_char; 64];
        let (mut total, mut sms, mut warp) = (0usize, 0, 0);
        // SAFETY: both buffers travel with their lengths and the callee terminates within them; the out-pointers
        // target live locals.
        #[allow(unsafe_code)]
        let rc = unsafe {
            ffi::llamd_cuda_device_info(index, name.as_mut_ptr(), name.len() as i32, arch.as_mut_ptr(), arch.len() as i32, &mut total, &mut sms, &mut warp)
        };
        if rc != 0 {
            return Err(Error::other(format!("cudaGetDeviceProperties failed for device {index}")));
        }
        let text = |b: &[std::os::raw::c_char]| -> String {
            let bytes: Vec<u8> = b.iter().take_while(|&&c| c != 0).map(|&c| c as u8).collect();
            String::from_utf8_lossy(&bytes).into_owned()
        };
        // SAFETY: no arguments; 0 when the query fails.
        #[allow(unsafe_code)]
        let free = unsafe { ffi::llamd_cuda_free_mem() };
        Ok(DeviceInfo { index, name: text(&name), total_mem: total, free_mem: free, sm_count: sms, warp_size: warp, arch: text(&arch) })
    }
}

/// Split Q8_K blocks into the two planes the kernels read: quants in natural order, one scale per block.
pub(crate) fn split_blocks(act: &[BlockQ8K]) -> (Vec<i8>, Vec<f32>) {
    let mut aq = Vec::with_capacity(act.len() * QK_K);
    let mut ad = Vec::with_capacity(act.len());
    for b in act {
        aq.extend_from_slice(&b.qs);
        ad.push(b.d);
    }
    (aq, ad)
}

/// Q6_K weights resident on the device, uploaded once and kept in the library's tiled layout (a bit permutation of
/// the 210-byte blocks, done on the device at upload; [`DeviceWeights::unpack`] gives the bytes back).
pub struct DeviceWeights {
    #[cfg(cuda)]
    ptr: *mut std::ffi::c_void,
    rows: usize,
    blocks: usize,
}

// SAFETY: an opaque device pointer, dereferenced only inside library calls, freed exactly once by `Drop`; every use
// is a read.
#[allow(unsafe_code)]
unsafe impl Send for DeviceWeights {}
#[allow(unsafe_code)]
unsafe impl Sync for DeviceWeights {}

impl DeviceWeights {
    /// Upload packed Q6_K weights for `rows` rows of `blocks` blocks each (reference byte layout).
    pub fn upload(w: &[u8], rows: usize, blocks: usize) -> Result<Self> {
        let need = rows * blocks * Q6K_BLOCK_BYTES;
        if w.len() < need {
            return Err(Error::malformed("device weights", format!("need {need} bytes for {rows}x{blocks}, have {}", w.len())));
        }
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            if !available() {
                return Err(Error::unsupported("cuda", "no device present"));
            }
            // SAFETY: `w` holds at least `rows * blocks` whole blocks, which is what is read; null on failure.
            #[allow(unsafe_code)]
            let ptr = unsafe { ffi::llamd_cuda_upload_q6k(w.as_ptr() as *const _, rows * blocks) };
            if ptr.is_null() {
                return Err(Error::other(format!("device upload of {:.1} MiB of weights failed: {}", need as f64 / (1 << 20) as f64, last_error_text())));
            }
            Ok(DeviceWeights { ptr, rows, blocks })
        }
    }

    pub fn rows(&self) -> usize {
        self.rows
    }
    pub fn blocks(&self) -> usize {
        self.blocks
    }
    /// The device address, for the `op::*` functions that take weights by pointer.
    #[cfg(cuda)]
    pub fn ptr(&self) -> *const std::ffi::c_void {
        self.ptr
    }

    /// Matvec against the resident weights: only the activation and the result cross the bus.
    pub fn matvec(&self, act: &[BlockQ8K]) -> Result<Vec<f32>> {
        if act.len() != self.blocks {
            return Err(Error::Shape { expected: vec![self.blocks], got: vec![act.len()] });
        }
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let (aq, ad) = split_blocks(act);
            let mut out = vec![0f32; self.rows];
            let _guard = SCRATCH.lock().unwrap_or_else(|e| e.into_inner());
            // SAFETY: aq/ad hold `blocks` blocks, out holds `rows` floats, and those are the extents passed.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_cuda_matvec_q6k_resident(self.ptr, aq.as_ptr(), ad.as_ptr(), out.as_mut_ptr(), self.blocks as i32, self.rows as i32) };
            if rc != 0 {
                return Err(Error::other(format!("CUDA matvec failed: {}", last_error_text())));
            }
            Ok(out)
        }
    }

    fn check_grouped(&self, act_blocks: usize, expert_ids: &[i32], rows_per_expert: usize) -> Result<()> {
        if act_blocks != self.blocks {
            return Err(Error::Shape { expected: vec![self.blocks], got: vec![act_blocks] });
        }
        if expert_ids.is_empty() {
            return Err(Error::malformed("grouped matvec", "no expert ids"));
        }
        if rows_per_expert == 0 || self.rows % rows_per_expert != 0 {
            return Err(Error::malformed("grouped matvec", format!("{rows_per_expert} rows per expert does not divide {} rows", self.rows)));
        }
        let n_expert = (self.rows / rows_per_expert) as i32;
        if let Some(&bad) = expert_ids.iter().find(|&&e| e < 0 || e >= n_expert) {
            return Err(Error::malformed("grouped matvec", format!("expert id {bad} outside 0..{n_expert}")));
        }
        Ok(())
    }

    /// The expert gather: this buffer holds `rows / rows_per_expert` experts; row block `s` of the result is expert
    /// `expert_ids[s]` applied to the one shared activation. Ids are checked here, before the call.
    pub fn matvec_grouped(&self, act: &[BlockQ8K], expert_ids: &[i32], rows_per_expert: usize) -> Result<Vec<f32>> {
        self.check_grouped(act.len(), expert_ids, rows_per_expert)?;
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let (aq, ad) = split_blocks(act);
            let mut out = vec![0f32; rows_per_expert * expert_ids.len()];
            let _guard = SCRATCH.lock().unwrap_or_else(|e| e.into_inner());
            // SAFETY: every extent passed matches the slice it describes; the ids were range-checked above.
            #[allow(unsafe_code)]
            let rc = unsafe {
                ffi::llamd_cuda_matvec_grouped(self.ptr, expert_ids.as_ptr(), aq.as_ptr(), ad.as_ptr(), out.as_mut_ptr(), self.blocks as i32, rows_per_expert as i32, expert_ids.len() as i32)
            };
            if rc != 0 {
                return Err(Error::other(format!("CUDA grouped matvec failed: {}", last_error_text())));
            }
            Ok(out)
        }
    }

    /// Kernel-only milliseconds per launch: one warm launch, then `iters` back to back between two events.
    pub fn bench_kernel_only(&self, act: &[BlockQ8K], iters: u32) -> Result<f32> {
        if act.len() != self.blocks {
            return Err(Error::Shape { expected: vec![self.blocks], got: vec![act.len()] });
        }
        if iters == 0 {
            return Err(Error::malformed("bench", "zero iterations"));
        }
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let (aq, ad) = split_blocks(act);
            let mut ms = 0f32;
            let _guard = SCRATCH.lock().unwrap_or_else(|e| e.into_inner());
            // SAFETY: as in `matvec`; `ms` is a live local.
            #[allow(unsafe_code)]
            let rc = unsafe { ffi::llamd_cuda_matvec_bench(self.ptr, aq.as_ptr(), ad.as_ptr(), self.blocks as i32, self.rows as i32, iters as i32, &mut ms) };
            if rc != 0 {
                return Err(Error::other(format!("CUDA matvec bench failed: {}", last_error_text())));
            }
            Ok(ms / iters as f32)
        }
    }

    pub fn bench_grouped_kernel_only(&self, act: &[BlockQ8K], expert_ids: &[i32], rows_per_expert: usize, iters: u32) -> Result<f32> {
        self.check_grouped(act.len(), expert_ids, rows_per_expert)?;
        if iters == 0 {
            return Err(Error::malformed("bench", "zero iterations"));
        }
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let (aq, ad) = split_blocks(act);
            let mut ms = 0f32;
            let _guard = SCRATCH.lock().unwrap_or_else(|e| e.into_inner());
            // SAFETY: as in `matvec_grouped`.
            #[allow(unsafe_code)]
            let rc = unsafe {
                ffi::llamd_cuda_matvec_grouped_bench(self.ptr, expert_ids.as_ptr(), aq.as_ptr(), ad.as_ptr(), self.blocks as i32, rows_per_expert as i32, expert_ids.len() as i32, iters as i32, &mut ms)
            };
            if rc != 0 {
                return Err(Error::other(format!("CUDA grouped bench failed: {}", last_error_text())));
            }
            Ok(ms / iters as f32)
        }
    }

    /// The reference bytes back from the tiled layout: proves the upload is a permutation.
    pub fn unpack(&self) -> Result<Vec<u8>> {
        #[cfg(not(cuda))]
        {
            not_built()
        }
        #[cfg(cuda)]
        {
            let n = self.rows * self.blocks;
            let flat = DevBuf::new(n * Q6K_BLOCK_BYTES)?;
            // SAFETY: the tiled source holds `n` blocks and `flat` was sized for `n` blocks of 210 bytes.
            #[allow(unsafe_code)]
            unsafe {
                ffi::llamd_fwd_unpack_q6k(self.ptr, flat.ptr(), n)
            };
            sync()?;
            let mut out = vec![0u8; n * Q6K_BLOCK_BYTES];
            flat.download_bytes(&mut out)?;
            Ok(out)
        }
    }
}

impl Drop for DeviceWeights {
    fn drop(&mut self) {
        #[cfg(cuda)]
        {
            // SAFETY: the pointer came from `llamd_cuda_upload_q6k`, is released once, and is never used again.
            #[allow(unsafe_code)]
            unsafe {
                ffi::llamd_cuda_release(self.ptr)
            };
        }
    }
}

/// Quantize on the device; bit-identical to `llamd_quant::quantize_q8_k` (ties, clamp, zero blocks, negative peaks).
pub fn quantize_q8k_on_device(x: &[f32]) -> Result<Vec<BlockQ8K>> {
    if x.is_empty() || x.len() % QK_K != 0 {
        return Err(Error::malformed("q8_k input", format!("{} values is not a whole number of {QK_K}-element blocks", x.len())));
    }
    #[cfg(not(cuda))]
    {
        not_built()
    }
    #[cfg(cuda)]
    {
        let nb = x.len() / QK_K;
        let mut qs = vec![0i8; x.len()];
        let mut d = vec![0f32; nb];
        let mut bsums = vec![0i16; nb * 16];
        let _guard = SCRATCH.lock().unwrap_or_else(|e| e.into_inner());
        // SAFETY: the three outputs are sized for `nb` blocks, the count passed.
        #[allow(unsafe_code)]
        let rc = unsafe { ffi::llamd_cuda_quantize_q8k(x.as_ptr(), nb as i32, qs.as_mut_ptr(), d.as_mut_ptr(), bsums.as_mut_ptr()) };
        if rc != 0 {
            return Err(Error::other(format!("CUDA q8_k quantize failed: {}", last_error_text())));
        }
        let mut out = Vec::with_capacity(nb);
        for b in 0..nb {
            let mut blk = BlockQ8K::default();
            blk.d = d[b];
            blk.qs.copy_from_slice(&qs[b * QK_K..(b + 1) * QK_K]);
            blk.bsums.copy_from_slice(&bsums[b * 16..(b + 1) * 16]);
            out.push(blk);
        }
        Ok(out)
    }
}

/// Upload, multiply, release: the one-shot form.
pub fn matvec_q6k(w: &[u8], act: &[BlockQ8K], rows: usize) -> Result<Vec<f32>> {
    if rows == 0 || act.is_empty() {
        return Err(Error::malformed("matvec", "no rows or no activation blocks"));
    }
    DeviceWeights::upload(w, rows, act.len())?.matvec(act)
}

#[cfg(test)]
mod tests {
    use super::*;

    /// The stub build's contract, as `llamd-rocm` tests its own: bad arguments are refused before any FFI call, and
    /// without a device everything else answers `Unsupported`, never a wrong number.
    #[test]
    fn refuses_bad_arguments_without_a_device() {
        assert!(matches!(DeviceWeights::upload(&[0u8; 10], 1, 1), Err(Error::Malformed { .. })));
        assert!(matches!(quantize_q8k_on_device(&[0.0; 100]), Err(Error::Malformed { .. })));
        assert!(matches!(matvec_q6k(&[], &[], 0), Err(Error::Malformed { .. })));
        if !available() {
            assert!(matches!(DeviceWeights::upload(&[0u8; 210], 1, 1), Err(Error::Unsupported { .. })));
            assert!(device_info(0).is_err());
        }
    }
}
