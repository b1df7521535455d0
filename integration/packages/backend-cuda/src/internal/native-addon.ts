/*
 * Source-only structural mirror of the JavaScript API napi-rs generates from `crates/runtime-cuda/src/napi/mod.rs`,
 * in the manner of packages/backend-cpu/src/internal/native-addon.ts: the adapter imports these declarations with
 * `import type`, the loader asserts the shape without validating it, so this file must stay in lockstep with the addon.
 */
/** Cooperative token polled by native work; cancel and commit have one winner. @internal */
export declare class CancellationToken {
  constructor()
  cancel(): void
  get cancelled(): boolean
}

/** A dense f32 or packed-u8 tensor in device memory. @internal */
export declare class NativeTensor {
  static fromBytes(data: Uint8Array, shape: Array<number>, dtype: string): NativeTensor
  clear(): void
  get shape(): Array<number>
  get dtype(): string
  get device(): string
  readback(): Promise<ArrayBuffer>
  sample(temperature: number, topK: number, topP: number, seed: bigint, counter: bigint): Promise<number>
}

/** Paged KV pool: pages and prefix cache on the host, K/V slabs on the device. @internal */
export declare class NativeKvPool {
  constructor(
    layers: number,
    kvHeads: number,
    headDim: number,
    maxTokens: number,
    blockSize?: number | undefined | null,
    dtype?: NativeDType | undefined | null
  )
  get capacity(): number
  get freeBlocks(): number
  get cachedBlocks(): number
  makeSequence(): NativeKvSequence
}

/** Sequence leased from one pool; `release` idempotently returns its block references. @internal */
export declare class NativeKvSequence {
  get cursor(): number
  release(): void
  prefillMatch(tokens: Array<number>): number
}

/**
 * Immutable compiled decode program. `execute` and `executeSampled` borrow the sequences until their Promise settles
 * and commit sequence updates only on success; `generateGreedy` runs whole steps on the device.
 *
 * @internal
 */
export declare class Executable {
  get batch(): number
  get stateful(): boolean
  get allowsWindowEviction(): boolean
  get layers(): number
  get kvHeads(): number
  get headDim(): number
  execute(
    pool: NativeKvPool,
    sequences: Array<NativeKvSequence>,
    tokens: Array<Array<number>>,
    token?: CancellationToken | undefined | null
  ): Promise<Float32Array>
  executeSampled(
    pool: NativeKvPool,
    sequences: Array<NativeKvSequence>,
    tokens: Array<Array<number>>,
    token?: CancellationToken | undefined | null
  ): Promise<Array<number>>
  generateGreedy(
    pool: NativeKvPool,
    sequences: Array<NativeKvSequence>,
    first: Array<number>,
    steps: number
  ): Promise<Array<number>>
}

/** KV tiers of the pool. @internal */
export type NativeDType = "f32" | "f16" | "bf16" | "u8"
/** Native spelling of the two supported rotary coordinate layouts. @internal */
export type NativeRotaryLayout = "HalfSplit" | "InterleavedPairs"
/** Tensor formats the decode path reads. @internal */
export type NativeTensorFormat = "F32" | "Q4_0" | "Q8_0" | "Q2_K" | "Q3_K" | "Q4_K" | "Q5_K" | "Q6_K"

/** Decode specialization request (packages/backend-cpu/src/internal/native-addon.ts:352-360). @internal */
export interface NativeKvStateSchema {
  maxTokens: number
  blockSize: number
  kvDtype: NativeDType
  window?: number
  batch: number
}

/** The Llama-family decode graph as `specialize_decode` describes it. @internal */
export interface NativeDecoderDescription {
  layers: number
  dModel: number
  qHeads: number
  kvHeads: number
  headDim: number
  ffn: number
  vocab: number
  rmsEps: number
  ropeTheta: number
  ropeLayout: NativeRotaryLayout
  prefillChunk: number
}

/** One constant weight of the program. @internal */
export interface NativeDecoderWeight {
  slot: "tokEmbd" | "attnNorm" | "wq" | "wk" | "wv" | "wo" | "ffnNorm" | "gate" | "up" | "down" | "outNorm" | "head"
  layer: number
  format: NativeTensorFormat
  rows: number
  columns: number
  data: Uint8Array
}

/** Logical f32 and physical storage geometry for one GGUF tensor. @internal */
export interface NativeGgufTensorDescriptor {
  name: string
  format: NativeTensorFormat
  logicalShape: Array<number>
  logicalDtype: "f32"
  physicalShape: Array<number>
  physicalDtype: "f32" | "u8"
}

/** Compiles the stateful decode program with constant weights. @internal */
export declare function compileDecoder(
  description: NativeDecoderDescription,
  weights: Array<NativeDecoderWeight>,
  state: NativeKvStateSchema
): Executable

/** Parses and validates GGUF metadata/catalog without loading payloads. @internal */
export declare function inspectGguf(
  path: string,
  token?: CancellationToken | undefined | null
): Promise<Array<NativeGgufTensorDescriptor>>

/** Loads GGUF F32 and packed payloads into device memory. @internal */
export declare function loadGguf(
  path: string,
  token?: CancellationToken | undefined | null
): Array<{ descriptor: NativeGgufTensorDescriptor; tensor: NativeTensor }>

/** Bytes of device memory held by live native handles. @internal */
export declare function externalMemoryBytes(): number

/** True when the driver answers and at least one device is usable. @internal */
export declare function isAvailable(): boolean

/** Complete runtime shape asserted over the object returned by `require`. @internal */
export interface NativeAddon {
  readonly CancellationToken: typeof CancellationToken
  readonly Executable: typeof Executable
  readonly NativeKvPool: typeof NativeKvPool
  readonly NativeKvSequence: typeof NativeKvSequence
  readonly NativeTensor: typeof NativeTensor
  readonly compileDecoder: typeof compileDecoder
  readonly externalMemoryBytes: typeof externalMemoryBytes
  readonly inspectGguf: typeof inspectGguf
  readonly isAvailable: typeof isAvailable
  readonly loadGguf: typeof loadGguf
}
