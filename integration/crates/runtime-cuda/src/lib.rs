//! Safe Rust over the CUDA backend's C ABI (`ffi.rs`), shaped like `crates/runtime-cpu/src/lib.rs`: owning handles with
//! `Drop`, `Result<_, BackendError>` instead of status codes, slices instead of pointer + length. Device buffers are
//! plain `DeviceBuffer` values (an address and a byte length on one runtime); nothing here copies unless its name says so.
//!
//! The crate links `libetcuda.so` (built from this repository by `python -m effect_torch_b200.build`, or by any
//! build script that runs `nvcc -gencode arch=compute_100a,code=sm_100a` over `effect_torch_b200/csrc`), found through
//! `ETCUDA_LIB_DIR` in `build.rs`.
pub mod ffi;
#[cfg(feature = "napi")]
pub mod napi;

use std::ffi::{CStr, CString};
use std::os::raw::{c_int, c_void};
use std::ptr;
use std::sync::atomic::{AtomicI32, Ordering};
use std::sync::Arc;

/// The reason classes of `BackendError` (packages/core/src/Runtime.ts:129-143), one per non-zero `etc_status`.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum Reason {
    BackendUnavailable,
    UnsupportedOperation,
    InvalidHandle,
    CompilationFailed,
    ExecutionFailed,
    TransferFailed,
    Cancelled,
    ClosedRuntime,
    InvalidArgument,
}

#[derive(Clone, Debug)]
pub struct BackendError {
    pub reason: Reason,
    pub message: String,
}

impl std::fmt::Display for BackendError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "{:?}: {}", self.reason, self.message)
    }
}
impl std::error::Error for BackendError {}

pub type Result<T> = std::result::Result<T, BackendError>;

fn check(status: ffi::EtcStatus) -> Result<()> {
    let reason = match status {
        ffi::ETC_OK => return Ok(()),
        ffi::ETC_UNAVAILABLE => Reason::BackendUnavailable,
        ffi::ETC_UNSUPPORTED => Reason::UnsupportedOperation,
        ffi::ETC_INVALID_HANDLE => Reason::InvalidHandle,
        ffi::ETC_COMPILATION => Reason::CompilationFailed,
        ffi::ETC_TRANSFER => Reason::TransferFailed,
        ffi::ETC_CANCELLED => Reason::Cancelled,
        ffi::ETC_CLOSED => Reason::ClosedRuntime,
        ffi::ETC_INVALID_ARGUMENT => Reason::InvalidArgument,
        _ => Reason::ExecutionFailed,
    };
    // the message is thread local and stays valid until this thread's next call into the library
    let message = unsafe { CStr::from_ptr(ffi::etc_last_error_message()) }.to_string_lossy().into_owned();
    Err(BackendError { reason, message })
}

/// Cooperative cancellation flag shared with native calls (crates/napi/src/lib.rs:56-82: one winner between cancel
/// and commit; the library reads the flag once before it commits a step).
#[derive(Clone, Default)]
pub struct CancellationToken(Arc<AtomicI32>);

impl CancellationToken {
    pub fn new() -> Self {
        Self::default()
    }
    pub fn cancel(&self) {
        self.0.store(1, Ordering::SeqCst);
    }
    pub fn cancelled(&self) -> bool {
        self.0.load(Ordering::SeqCst) != 0
    }
    fn as_ptr(token: Option<&CancellationToken>) -> *const c_int {
        token.map_or(ptr::null(), |t| t.0.as_ptr() as *const c_int)
    }
}

/// Number of usable CUDA devices (0 when there is none: `isAvailable()` is `device_count()? > 0`).
pub fn device_count() -> Result<usize> {
    let mut n: c_int = 0;
    check(unsafe { ffi::etc_device_count(&mut n) })?;
    Ok(n as usize)
}

/// One device, one stream, one status word. `Send` (calls are serialised by `&mut self` or by the napi wrapper's mutex).
pub struct Runtime {
    raw: *mut ffi::EtcRuntime,
}
unsafe impl Send for Runtime {}

#[derive(Clone, Copy, Debug)]
pub struct DeviceBuffer {
    pub address: *mut c_void,
    pub bytes: usize,
}
unsafe impl Send for DeviceBuffer {}

impl Runtime {
    pub fn new(device_ordinal: usize) -> Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::etc_runtime_create(device_ordinal as c_int, &mut raw) })?;
        Ok(Self { raw })
    }
    pub fn raw(&self) -> *mut ffi::EtcRuntime {
        self.raw
    }
    /// Waits for the stream; a device-side status raised since the last call (index out of range, non-finite logit, a
    /// bounded wait that ran out) comes back as the error.
    pub fn synchronize(&self) -> Result<()> {
        check(unsafe { ffi::etc_runtime_synchronize(self.raw) })
    }
    pub fn memory_bytes(&self) -> Result<u64> {
        let mut out = 0u64;
        check(unsafe { ffi::etc_runtime_memory_bytes(self.raw, &mut out) })?;
        Ok(out)
    }
    pub fn capabilities(&self) -> Result<ffi::EtcCapabilities> {
        let mut out = std::mem::MaybeUninit::<ffi::EtcCapabilities>::zeroed();
        check(unsafe { ffi::etc_runtime_capabilities(self.raw, out.as_mut_ptr()) })?;
        Ok(unsafe { out.assume_init() })
    }
    pub fn alloc(&self, bytes: usize) -> Result<DeviceBuffer> {
        let mut address = ptr::null_mut();
        check(unsafe { ffi::etc_alloc(self.raw, bytes, &mut address) })?;
        Ok(DeviceBuffer { address, bytes })
    }
    pub fn free(&self, buffer: DeviceBuffer) -> Result<()> {
        check(unsafe { ffi::etc_free(self.raw, buffer.address) })
    }
    pub fn upload(&self, dst: DeviceBuffer, src: &[u8]) -> Result<()> {
        assert!(src.len() <= dst.bytes);
        check(unsafe { ffi::etc_upload(self.raw, dst.address, src.as_ptr() as *const c_void, src.len()) })
    }
    pub fn download(&self, dst: &mut [u8], src: DeviceBuffer) -> Result<()> {
        assert!(dst.len() <= src.bytes);
        check(unsafe { ffi::etc_download(self.raw, dst.as_mut_ptr() as *mut c_void, src.address, dst.len()) })
    }
    /// `quantized_linear_into` (crates/runtime-cpu/src/quantized.rs:419-499) over device buffers.
    #[allow(clippy::too_many_arguments)]
    pub fn qlinear_into(&self, codec: c_int, x: DeviceBuffer, vectors: i64, columns: i64, weight: DeviceBuffer, rows: i64,
                        bias: Option<DeviceBuffer>, out: DeviceBuffer, token: Option<&CancellationToken>) -> Result<()> {
        check(unsafe {
            ffi::etc_qlinear_into(self.raw, codec, x.address as *const f32, vectors, columns, weight.address, rows,
                                  bias.map_or(ptr::null(), |b| b.address as *const f32), out.address as *mut f32,
                                  CancellationToken::as_ptr(token))
        })
    }
    /// `sample_logits` (crates/runtime/src/sampling.rs:80-206) for one row of device logits.
    #[allow(clippy::too_many_arguments)]
    pub fn sample_row(&self, logits: DeviceBuffer, vocab: i64, temperature: f64, top_k: Option<usize>, top_p: f64, seed: u64,
                      counter: u64) -> Result<u32> {
        let mut token = 0u32;
        check(unsafe {
            ffi::etc_sample_row(self.raw, logits.address as *const f32, vocab, temperature, top_k.map_or(0, |k| k as i64), top_p, seed,
                                counter, &mut token)
        })?;
        Ok(token)
    }
}

impl Drop for Runtime {
    fn drop(&mut self) {
        unsafe { ffi::etc_runtime_destroy(self.raw) };
    }
}

/// Paged KV pool (crates/runtime-cpu/src/pool.rs:1-60): host-side page allocator, prefix cache and block tables; the K/V
/// slabs live in device memory.
pub struct KvPool {
    raw: *mut ffi::EtcPool,
}
unsafe impl Send for KvPool {}

impl KvPool {
    #[allow(clippy::too_many_arguments)]
    pub fn new(rt: &Runtime, layers: usize, kv_heads: usize, head_dim: usize, max_tokens: usize, block_size: usize,
               dtype: c_int) -> Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe {
            ffi::etc_pool_create(rt.raw, layers as c_int, kv_heads as c_int, head_dim as c_int, max_tokens as c_int, block_size as c_int,
                                 dtype, &mut raw)
        })?;
        Ok(Self { raw })
    }
    /// (capacity, free blocks, cached blocks)
    pub fn stats(&self) -> Result<(u32, u32, u32)> {
        let (mut a, mut b, mut c) = (0u32, 0u32, 0u32);
        check(unsafe { ffi::etc_pool_stats(self.raw, &mut a, &mut b, &mut c) })?;
        Ok((a, b, c))
    }
    pub fn make_sequence(&self) -> Result<KvSequence> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::etc_seq_create(self.raw, &mut raw) })?;
        Ok(KvSequence { raw })
    }
}
impl Drop for KvPool {
    fn drop(&mut self) {
        unsafe { ffi::etc_pool_destroy(self.raw) };
    }
}

pub struct KvSequence {
    raw: *mut ffi::EtcSeq,
}
unsafe impl Send for KvSequence {}

impl KvSequence {
    pub fn cursor(&self) -> Result<u32> {
        let mut c = 0u32;
        check(unsafe { ffi::etc_seq_cursor(self.raw, &mut c) })?;
        Ok(c)
    }
    /// Idempotent: returns the block references; the handle stays valid and empty.
    pub fn release(&self) -> Result<()> {
        check(unsafe { ffi::etc_seq_release(self.raw) })
    }
    /// Longest cached prefix of `tokens` adopted by this (empty) sequence, in tokens.
    pub fn prefill_match(&self, tokens: &[u32]) -> Result<u32> {
        let mut matched = 0u32;
        check(unsafe { ffi::etc_seq_prefill_match(self.raw, tokens.as_ptr(), tokens.len() as i64, &mut matched) })?;
        Ok(matched)
    }
}
impl Drop for KvSequence {
    fn drop(&mut self) {
        unsafe { ffi::etc_seq_destroy(self.raw) };
    }
}

/// The compiled stateful decode program: what `compile(roots, options, state)` returns for the Llama-family decode graph
/// once `specialize_decode` (crates/compiler/src/decode.rs:105-481) has recognised its layers.
pub struct Decoder {
    raw: *mut ffi::EtcDecoder,
    pub config: ffi::EtcDecoderConfig,
}
unsafe impl Send for Decoder {}

impl Decoder {
    pub fn new(rt: &Runtime, config: ffi::EtcDecoderConfig, max_advance: usize) -> Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::etc_decoder_create(rt.raw, &config, &mut raw) })?;
        let decoder = Self { raw, config };
        check(unsafe { ffi::etc_decoder_set_max_advance(raw, max_advance as c_int) })?;
        Ok(decoder)
    }
    /// Host bytes: dense f32 `[rows, columns]` or packed GGUF rows; uploaded and retained (constantWeights).
    pub fn set_weight(&self, slot: c_int, layer: usize, codec: c_int, data: &[u8], rows: i64, columns: i64) -> Result<()> {
        check(unsafe { ffi::etc_decoder_set_weight(self.raw, slot, layer as c_int, codec, data.as_ptr() as *const c_void, rows, columns) })
    }
    pub fn finalize(&self) -> Result<()> {
        check(unsafe { ffi::etc_decoder_finalize(self.raw) })
    }
    fn handles(sequences: &[&KvSequence]) -> Vec<*mut ffi::EtcSeq> {
        sequences.iter().map(|s| s.raw).collect()
    }
    /// One stateful invocation: `tokens` is `[active][advance]` row-major; returns LastTokenRow logits `[active][vocab]`.
    /// Sequence updates are committed only when this returns `Ok`.
    pub fn execute(&self, pool: &KvPool, sequences: &[&KvSequence], tokens: &[u32], advance: usize,
                   token: Option<&CancellationToken>) -> Result<Vec<f32>> {
        let active = sequences.len();
        assert_eq!(tokens.len(), active * advance);
        let mut logits = vec![0f32; active * self.config.vocab as usize];
        let handles = Self::handles(sequences);
        check(unsafe {
            ffi::etc_decoder_execute(self.raw, pool.raw, handles.as_ptr(), active as c_int, tokens.as_ptr(), advance as c_int,
                                     logits.as_mut_ptr(), CancellationToken::as_ptr(token))
        })?;
        Ok(logits)
    }
    /// The same transaction returning one greedy token per active sequence (`executeSampled`).
    pub fn execute_sampled(&self, pool: &KvPool, sequences: &[&KvSequence], tokens: &[u32], advance: usize,
                           token: Option<&CancellationToken>) -> Result<Vec<u32>> {
        let active = sequences.len();
        assert_eq!(tokens.len(), active * advance);
        let mut out = vec![0u32; active];
        let handles = Self::handles(sequences);
        check(unsafe {
            ffi::etc_decoder_execute_sampled(self.raw, pool.raw, handles.as_ptr(), active as c_int, tokens.as_ptr(), advance as c_int,
                                             out.as_mut_ptr(), CancellationToken::as_ptr(token))
        })?;
        Ok(out)
    }
    /// `steps` greedy steps with ids, tables and cursors resident on the device; `[steps][active]` tokens and the device time.
    pub fn generate_greedy(&self, pool: &KvPool, sequences: &[&KvSequence], first: &[u32], steps: usize) -> Result<(Vec<u32>, f32)> {
        let active = sequences.len();
        let mut out = vec![0u32; steps * active];
        let mut ms = 0f32;
        let handles = Self::handles(sequences);
        check(unsafe {
            ffi::etc_decoder_generate_greedy(self.raw, pool.raw, handles.as_ptr(), active as c_int, first.as_ptr(), steps as c_int,
                                             out.as_mut_ptr(), &mut ms)
        })?;
        Ok((out, ms))
    }
}
impl Drop for Decoder {
    fn drop(&mut self) {
        unsafe { ffi::etc_decoder_destroy(self.raw) };
    }
}

/// A parsed GGUF file (crates/runtime/src/gguf.rs:682-946): metadata and catalog only until a tensor is read.
pub struct Gguf {
    raw: *mut ffi::EtcGguf,
}
unsafe impl Send for Gguf {}

pub struct GgufTensor {
    pub name: String,
    pub codec: c_int,
    pub logical_shape: Vec<i64>,
    pub physical_shape: Vec<i64>,
    pub byte_len: u64,
}

impl Gguf {
    pub fn open(path: &str, token: Option<&CancellationToken>) -> Result<Self> {
        let c_path = CString::new(path).map_err(|_| BackendError { reason: Reason::InvalidArgument, message: "gguf: path contains a NUL byte".into() })?;
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::etc_gguf_open(c_path.as_ptr(), CancellationToken::as_ptr(token), &mut raw) })?;
        Ok(Self { raw })
    }
    pub fn tensor_count(&self) -> Result<usize> {
        let (mut arch, mut meta, mut tensors) = (ptr::null(), 0i64, 0i64);
        check(unsafe { ffi::etc_gguf_summary(self.raw, &mut arch, &mut meta, &mut tensors) })?;
        Ok(tensors as usize)
    }
    pub fn tensor(&self, index: usize) -> Result<GgufTensor> {
        let mut name = ptr::null();
        let (mut codec, mut rank) = (0 as c_int, 0 as c_int);
        let (mut logical, mut physical) = ([0i64; 4], [0i64; 4]);
        let (mut offset, mut byte_len) = (0u64, 0u64);
        check(unsafe {
            ffi::etc_gguf_tensor(self.raw, index as i64, &mut name, &mut codec, &mut rank, logical.as_mut_ptr(), physical.as_mut_ptr(),
                                 &mut offset, &mut byte_len)
        })?;
        let physical_rank = if codec == ffi::ETC_CODEC_F32 { rank as usize } else { 2 };
        Ok(GgufTensor {
            name: unsafe { CStr::from_ptr(name) }.to_string_lossy().into_owned(),
            codec,
            logical_shape: logical[..rank as usize].to_vec(),
            physical_shape: physical[..physical_rank].to_vec(),
            byte_len,
        })
    }
    /// Streams the payload into device memory through the library's pinned staging buffers.
    pub fn load_tensor_device(&self, rt: &Runtime, index: usize, dst: DeviceBuffer, token: Option<&CancellationToken>) -> Result<()> {
        check(unsafe { ffi::etc_gguf_load_tensor_device(rt.raw, self.raw, index as i64, dst.address, dst.bytes as u64, CancellationToken::as_ptr(token)) })
    }
}
impl Drop for Gguf {
    fn drop(&mut self) {
        unsafe { ffi::etc_gguf_close(self.raw) };
    }
}
