//! The napi-rs addon of the CUDA backend: the JavaScript classes `@effect-torch/backend-cuda` loads, with the names and
//! call shapes of the CPU addon (`crates/runtime-cpu/src/napi/mod.rs`; its JavaScript face is
//! `packages/backend-cpu/src/internal/native-addon.ts`) for everything on the compiled decode path:
//!
//!   CancellationToken, NativeTensor (a device buffer), NativeKvPool, NativeKvSequence, Executable, compileDecoder,
//!   inspectGguf, loadGguf, externalMemoryBytes, isAvailable.
//!
//! What the CPU addon builds from a traced graph (`compile(roots, options, state)`) this addon builds from the
//! decoder description that `specialize_decode` (crates/compiler/src/decode.rs:105-481) arrives at: layer count, widths,
//! head geometry, RoPE and norm constants, the KV state schema, and one weight tensor per slot. `Executable.execute` and
//! `executeSampled` keep the reference's transaction: sequences advance only when the returned Promise resolves.
use std::sync::{Arc, Mutex};

use napi::bindgen_prelude::*;
use napi_derive::napi;

use crate::ffi;
use crate::{BackendError, CancellationToken as Token, Decoder, DeviceBuffer, Gguf, KvPool, KvSequence, Reason, Runtime};

fn js_error(e: BackendError) -> Error {
    // napi Status::InvalidArg for argument validation, GenericFailure otherwise; the adapter reads the reason from the
    // "<reason>: " prefix exactly as it does for the CPU addon (packages/backend-cpu/src/internal/adapter.ts)
    let status = if e.reason == Reason::InvalidArgument { Status::InvalidArg } else { Status::GenericFailure };
    let reason = match e.reason {
        Reason::BackendUnavailable => "backend-unavailable",
        Reason::UnsupportedOperation => "unsupported-operation",
        Reason::InvalidHandle => "invalid-handle",
        Reason::CompilationFailed => "compilation-failed",
        Reason::ExecutionFailed => "execution-failed",
        Reason::TransferFailed => "transfer-failed",
        Reason::Cancelled => "cancelled",
        Reason::ClosedRuntime => "closed-runtime",
        Reason::InvalidArgument => "invalid-argument",
    };
    Error::new(status, format!("{reason}: {}", e.message))
}

/// The process-wide runtime on device 0 (the CPU addon is process-wide as well); made on first use.
fn runtime() -> Result<Arc<Mutex<Runtime>>> {
    static RUNTIME: Mutex<Option<Arc<Mutex<Runtime>>>> = Mutex::new(None);
    let mut slot = RUNTIME.lock().unwrap();
    if slot.is_none() {
        *slot = Some(Arc::new(Mutex::new(Runtime::new(0).map_err(js_error)?)));
    }
    Ok(slot.as_ref().unwrap().clone())
}

#[napi]
pub fn is_available() -> bool {
    crate::device_count().map(|n| n > 0).unwrap_or(false)
}

#[napi]
pub fn external_memory_bytes() -> Result<f64> {
    let rt = runtime()?;
    let bytes = rt.lock().unwrap().memory_bytes().map_err(js_error)?;
    Ok(bytes as f64)
}

#[napi]
pub struct CancellationToken {
    inner: Token,
}

#[napi]
impl CancellationToken {
    #[napi(constructor)]
    pub fn new() -> Self {
        Self { inner: Token::new() }
    }
    #[napi]
    pub fn cancel(&self) {
        self.inner.cancel();
    }
    #[napi(getter)]
    pub fn cancelled(&self) -> bool {
        self.inner.cancelled()
    }
}

/// A dense or packed tensor in device memory: shape, dtype ("f32" or "u8" for packed GGUF rows) and the buffer.
#[napi]
pub struct NativeTensor {
    buffer: Option<DeviceBuffer>,
    shape: Vec<i64>,
    dtype: String,
    codec: i32,
}

#[napi]
impl NativeTensor {
    /// Uploads host bytes (Float32Array / Uint8Array storage) into a new device tensor.
    #[napi(factory)]
    pub fn from_bytes(data: Uint8Array, shape: Vec<i64>, dtype: String) -> Result<Self> {
        let rt = runtime()?;
        let rt = rt.lock().unwrap();
        let buffer = rt.alloc(data.len()).map_err(js_error)?;
        rt.upload(buffer, &data).map_err(js_error)?;
        Ok(Self { buffer: Some(buffer), shape, dtype, codec: ffi::ETC_CODEC_F32 })
    }
    #[napi]
    pub fn clear(&mut self) -> Result<()> {
        if let Some(buffer) = self.buffer.take() {
            runtime()?.lock().unwrap().free(buffer).map_err(js_error)?;
        }
        Ok(())
    }
    #[napi(getter)]
    pub fn shape(&self) -> Vec<i64> {
        self.shape.clone()
    }
    #[napi(getter)]
    pub fn dtype(&self) -> String {
        self.dtype.clone()
    }
    #[napi(getter)]
    pub fn device(&self) -> String {
        "cuda:0".to_string()
    }
    #[napi]
    pub async fn readback(&self) -> Result<Buffer> {
        let buffer = self.buffer.ok_or_else(|| Error::new(Status::GenericFailure, "invalid-handle: tensor was cleared"))?;
        let mut host = vec![0u8; buffer.bytes];
        runtime()?.lock().unwrap().download(&mut host, buffer).map_err(js_error)?;
        Ok(host.into())
    }
    /// One token from a `[vocab]` f32 row on the device (crates/runtime/src/sampling.rs:80-206).
    #[napi]
    pub async fn sample(&self, temperature: f64, top_k: i64, top_p: f64, seed: BigInt, counter: BigInt) -> Result<u32> {
        let buffer = self.buffer.ok_or_else(|| Error::new(Status::GenericFailure, "invalid-handle: tensor was cleared"))?;
        let vocab = *self.shape.last().unwrap_or(&0);
        let top_k = if top_k > 0 { Some(top_k as usize) } else { None };
        runtime()?.lock().unwrap().sample_row(buffer, vocab, temperature, top_k, top_p, seed.get_u64().1, counter.get_u64().1).map_err(js_error)
    }
}

impl Drop for NativeTensor {
    fn drop(&mut self) {
        let _ = self.clear();
    }
}

#[napi(object)]
pub struct NativeKvStateSchema {
    pub max_tokens: u32,
    pub block_size: u32,
    pub kv_dtype: String,
    pub window: Option<i64>,
    pub batch: u32,
}

fn kv_dtype(name: &str) -> Result<i32> {
    match name {
        "f32" => Ok(ffi::ETC_KV_F32),
        "f16" => Ok(ffi::ETC_KV_F16),
        "bf16" => Ok(ffi::ETC_KV_BF16),
        "u8" => Ok(ffi::ETC_KV_U8),
        other => Err(Error::new(Status::InvalidArg, format!("kv state: dtype {other} is not a KV tier"))),
    }
}

#[napi]
pub struct NativeKvPool {
    inner: Arc<KvPool>,
}

#[napi]
impl NativeKvPool {
    #[napi(constructor)]
    pub fn new(layers: u32, kv_heads: u32, head_dim: u32, max_tokens: u32, block_size: Option<u32>, dtype: Option<String>) -> Result<Self> {
        let rt = runtime()?;
        let rt = rt.lock().unwrap();
        let tier = kv_dtype(dtype.as_deref().unwrap_or("f32"))?;
        let pool = KvPool::new(&rt, layers as usize, kv_heads as usize, head_dim as usize, max_tokens as usize, block_size.unwrap_or(16) as usize, tier)
            .map_err(js_error)?;
        Ok(Self { inner: Arc::new(pool) })
    }
    #[napi(getter)]
    pub fn capacity(&self) -> Result<u32> {
        Ok(self.inner.stats().map_err(js_error)?.0)
    }
    #[napi(getter)]
    pub fn free_blocks(&self) -> Result<u32> {
        Ok(self.inner.stats().map_err(js_error)?.1)
    }
    #[napi(getter)]
    pub fn cached_blocks(&self) -> Result<u32> {
        Ok(self.inner.stats().map_err(js_error)?.2)
    }
    #[napi]
    pub fn make_sequence(&self) -> Result<NativeKvSequence> {
        Ok(NativeKvSequence { inner: Arc::new(self.inner.make_sequence().map_err(js_error)?), pool: self.inner.clone() })
    }
}

#[napi]
pub struct NativeKvSequence {
    inner: Arc<KvSequence>,
    pool: Arc<KvPool>,
}

#[napi]
impl NativeKvSequence {
    #[napi(getter)]
    pub fn cursor(&self) -> Result<u32> {
        self.inner.cursor().map_err(js_error)
    }
    #[napi]
    pub fn release(&self) -> Result<()> {
        self.inner.release().map_err(js_error)
    }
    #[napi]
    pub fn prefill_match(&self, tokens: Vec<u32>) -> Result<u32> {
        self.inner.prefill_match(&tokens).map_err(js_error)
    }
}

/// What `specialize_decode` extracts from a Llama-family decode graph.
#[napi(object)]
pub struct NativeDecoderDescription {
    pub layers: u32,
    pub d_model: u32,
    pub q_heads: u32,
    pub kv_heads: u32,
    pub head_dim: u32,
    pub ffn: u32,
    pub vocab: u32,
    pub rms_eps: f64,
    pub rope_theta: f64,
    pub rope_layout: String, // "HalfSplit" | "InterleavedPairs"
    pub prefill_chunk: u32,
}

/// One bound weight: the slot name, its layer, and the tensor (dense f32, or packed rows with `format`).
#[napi(object)]
pub struct NativeDecoderWeight {
    pub slot: String, // tokEmbd attnNorm wq wk wv wo ffnNorm gate up down outNorm head
    pub layer: u32,
    pub format: String, // "F32" | "Q4_0" | "Q8_0" | "Q2_K" .. "Q6_K"
    pub rows: i64,
    pub columns: i64,
    pub data: Uint8Array,
}

fn slot_code(name: &str) -> Result<i32> {
    Ok(match name {
        "tokEmbd" => ffi::ETC_W_TOK_EMBD,
        "attnNorm" => ffi::ETC_W_ATTN_NORM,
        "wq" => ffi::ETC_W_Q,
        "wk" => ffi::ETC_W_K,
        "wv" => ffi::ETC_W_V,
        "wo" => ffi::ETC_W_O,
        "ffnNorm" => ffi::ETC_W_FFN_NORM,
        "gate" => ffi::ETC_W_GATE,
        "up" => ffi::ETC_W_UP,
        "down" => ffi::ETC_W_DOWN,
        "outNorm" => ffi::ETC_W_OUT_NORM,
        "head" => ffi::ETC_W_HEAD,
        other => return Err(Error::new(Status::InvalidArg, format!("compile: unknown weight slot {other}"))),
    })
}

fn codec_code(format: &str) -> Result<i32> {
    Ok(match format {
        "F32" => ffi::ETC_CODEC_F32,
        "Q4_0" => ffi::ETC_CODEC_Q4_0,
        "Q8_0" => ffi::ETC_CODEC_Q8_0,
        "Q2_K" => ffi::ETC_CODEC_Q2_K,
        "Q3_K" => ffi::ETC_CODEC_Q3_K,
        "Q4_K" => ffi::ETC_CODEC_Q4_K,
        "Q5_K" => ffi::ETC_CODEC_Q5_K,
        "Q6_K" => ffi::ETC_CODEC_Q6_K,
        other => return Err(Error::new(Status::InvalidArg, format!("compile: unknown tensor format {other}"))),
    })
}

#[napi]
pub struct Executable {
    inner: Arc<Mutex<Decoder>>,
    state: NativeKvStateSchemaCopy,
}

#[derive(Clone, Copy)]
struct NativeKvStateSchemaCopy {
    batch: u32,
    layers: u32,
    kv_heads: u32,
    head_dim: u32,
    window: Option<i64>,
}

/// Compiles the stateful decode program with constant weights (compile + NativeCompileOptions.constantWeights).
#[napi]
pub fn compile_decoder(description: NativeDecoderDescription, weights: Vec<NativeDecoderWeight>, state: NativeKvStateSchema) -> Result<Executable> {
    let rt = runtime()?;
    let rt = rt.lock().unwrap();
    let config = ffi::EtcDecoderConfig {
        layers: description.layers as i32,
        d_model: description.d_model as i32,
        q_heads: description.q_heads as i32,
        kv_heads: description.kv_heads as i32,
        head_dim: description.head_dim as i32,
        ffn: description.ffn as i32,
        vocab: description.vocab as i32,
        rms_eps: description.rms_eps,
        rope_theta: description.rope_theta,
        rope_layout: if description.rope_layout == "InterleavedPairs" { ffi::ETC_ROPE_INTERLEAVED_PAIRS } else { ffi::ETC_ROPE_HALF_SPLIT },
        window: state.window.unwrap_or(ffi::ETC_NO_WINDOW),
        batch: state.batch as i32,
        max_tokens: state.max_tokens as i32,
        block_size: state.block_size as i32,
        kv_dtype: kv_dtype(&state.kv_dtype)?,
        exact: 0,
    };
    let decoder = Decoder::new(&rt, config, description.prefill_chunk.max(1) as usize).map_err(js_error)?;
    for w in &weights {
        decoder.set_weight(slot_code(&w.slot)?, w.layer as usize, codec_code(&w.format)?, &w.data, w.rows, w.columns).map_err(js_error)?;
    }
    decoder.finalize().map_err(js_error)?;
    Ok(Executable {
        inner: Arc::new(Mutex::new(decoder)),
        state: NativeKvStateSchemaCopy { batch: state.batch, layers: description.layers, kv_heads: description.kv_heads, head_dim: description.head_dim, window: state.window },
    })
}

#[napi]
impl Executable {
    #[napi(getter)]
    pub fn batch(&self) -> u32 {
        self.state.batch
    }
    #[napi(getter)]
    pub fn stateful(&self) -> bool {
        true
    }
    #[napi(getter)]
    pub fn allows_window_eviction(&self) -> bool {
        self.state.window.is_some()
    }
    #[napi(getter)]
    pub fn layers(&self) -> u32 {
        self.state.layers
    }
    #[napi(getter)]
    pub fn kv_heads(&self) -> u32 {
        self.state.kv_heads
    }
    #[napi(getter)]
    pub fn head_dim(&self) -> u32 {
        self.state.head_dim
    }
    /// `tokens[i]` is sequence i's chunk; all chunks have one length. Resolves to `[active][vocab]` logits.
    #[napi]
    pub async fn execute(&self, pool: &NativeKvPool, sequences: Vec<&NativeKvSequence>, tokens: Vec<Vec<u32>>,
                         token: Option<&CancellationToken>) -> Result<Float32Array> {
        let advance = tokens.first().map_or(0, |t| t.len());
        let flat: Vec<u32> = tokens.into_iter().flatten().collect();
        let handles: Vec<&KvSequence> = sequences.iter().map(|s| s.inner.as_ref()).collect();
        let decoder = self.inner.lock().unwrap();
        let logits = decoder.execute(&pool.inner, &handles, &flat, advance, token.map(|t| &t.inner)).map_err(js_error)?;
        Ok(Float32Array::new(logits))
    }
    /// The same transaction returning one greedy token per active sequence.
    #[napi]
    pub async fn execute_sampled(&self, pool: &NativeKvPool, sequences: Vec<&NativeKvSequence>, tokens: Vec<Vec<u32>>,
                                 token: Option<&CancellationToken>) -> Result<Vec<u32>> {
        let advance = tokens.first().map_or(0, |t| t.len());
        let flat: Vec<u32> = tokens.into_iter().flatten().collect();
        let handles: Vec<&KvSequence> = sequences.iter().map(|s| s.inner.as_ref()).collect();
        let decoder = self.inner.lock().unwrap();
        decoder.execute_sampled(&pool.inner, &handles, &flat, advance, token.map(|t| &t.inner)).map_err(js_error)
    }
    /// `steps` greedy steps without leaving the device between them; resolves to `[steps][active]` tokens.
    #[napi]
    pub async fn generate_greedy(&self, pool: &NativeKvPool, sequences: Vec<&NativeKvSequence>, first: Vec<u32>, steps: u32) -> Result<Vec<u32>> {
        let handles: Vec<&KvSequence> = sequences.iter().map(|s| s.inner.as_ref()).collect();
        let decoder = self.inner.lock().unwrap();
        Ok(decoder.generate_greedy(&pool.inner, &handles, &first, steps as usize).map_err(js_error)?.0)
    }
}

#[napi(object)]
pub struct NativeGgufTensorDescriptor {
    pub name: String,
    pub format: String,
    pub logical_shape: Vec<i64>,
    pub logical_dtype: String,
    pub physical_shape: Vec<i64>,
    pub physical_dtype: String,
}

fn format_name(codec: i32) -> &'static str {
    match codec {
        ffi::ETC_CODEC_F32 => "F32",
        ffi::ETC_CODEC_Q4_0 => "Q4_0",
        ffi::ETC_CODEC_Q8_0 => "Q8_0",
        ffi::ETC_CODEC_Q2_K => "Q2_K",
        ffi::ETC_CODEC_Q3_K => "Q3_K",
        ffi::ETC_CODEC_Q4_K => "Q4_K",
        ffi::ETC_CODEC_Q5_K => "Q5_K",
        _ => "Q6_K",
    }
}

/// Parses and validates a GGUF file's catalog without loading payloads.
#[napi]
pub async fn inspect_gguf(path: String, token: Option<&CancellationToken>) -> Result<Vec<NativeGgufTensorDescriptor>> {
    let file = Gguf::open(&path, token.map(|t| &t.inner)).map_err(js_error)?;
    (0..file.tensor_count().map_err(js_error)?)
        .map(|i| {
            let t = file.tensor(i).map_err(js_error)?;
            Ok(NativeGgufTensorDescriptor {
                name: t.name,
                format: format_name(t.codec).to_string(),
                logical_shape: t.logical_shape,
                logical_dtype: "f32".to_string(),
                physical_shape: t.physical_shape,
                physical_dtype: if t.codec == ffi::ETC_CODEC_F32 { "f32" } else { "u8" }.to_string(),
            })
        })
        .collect()
}

#[napi(object)]
pub struct NativeGgufEntry {
    pub descriptor: NativeGgufTensorDescriptor,
    pub tensor: ClassInstance<NativeTensor>,
}

/// Loads every tensor's payload into device memory (file reads overlap the copies).
#[napi]
pub fn load_gguf(env: Env, path: String, token: Option<&CancellationToken>) -> Result<Vec<NativeGgufEntry>> {
    let file = Gguf::open(&path, token.map(|t| &t.inner)).map_err(js_error)?;
    let rt = runtime()?;
    let rt = rt.lock().unwrap();
    let mut entries = Vec::new();
    for i in 0..file.tensor_count().map_err(js_error)? {
        let t = file.tensor(i).map_err(js_error)?;
        let buffer = rt.alloc(t.byte_len as usize).map_err(js_error)?;
        file.load_tensor_device(&rt, i, buffer, token.map(|t| &t.inner)).map_err(js_error)?;
        let dense = t.codec == ffi::ETC_CODEC_F32;
        let tensor = NativeTensor {
            buffer: Some(buffer),
            shape: t.physical_shape.clone(),
            dtype: if dense { "f32" } else { "u8" }.to_string(),
            codec: t.codec,
        };
        entries.push(NativeGgufEntry {
            descriptor: NativeGgufTensorDescriptor {
                name: t.name,
                format: format_name(t.codec).to_string(),
                logical_shape: t.logical_shape,
                logical_dtype: "f32".to_string(),
                physical_shape: t.physical_shape,
                physical_dtype: if dense { "f32" } else { "u8" }.to_string(),
            },
            tensor: tensor.into_instance(env)?,
        });
    }
    Ok(entries)
}
