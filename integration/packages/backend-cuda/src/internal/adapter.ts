/*
 * RuntimeService adapter over the CUDA addon, the sibling of packages/backend-cpu/src/internal/adapter.ts. It fills the
 * members of `Runtime.RuntimeService` (packages/core/src/Runtime.ts:1228-1290) that the compiled decode path uses:
 *
 *   compile  (a stateful CompileRequest whose roots `specialize_decode` reduces to a decoder description)
 *   execute  (stateful invocations: sequences + token chunks -> LastTokenRow logits)
 *   readback / release
 *   extensions.decode    makePool, makeSequence, prefillMatch, sequenceCursor, releaseSequence
 *   extensions.sampling  sample, executeDecode
 *   extensions.gguf      inspect, load
 *
 * and turns native rejections into `Runtime.BackendError` with the reason class the library reported. Graph
 * construction, autodiff and safetensors stay with the CPU backend: those members fail with `unsupported-operation`.
 */
import { Runtime } from "@effect-torch/core"
import { Effect } from "effect"
import type * as Native from "./native-addon.js"

type Phase = Runtime.BackendError["phase"]
type Reason = Runtime.BackendError["reason"]

const reasons: ReadonlyArray<Reason> = [
  "backend-unavailable",
  "unsupported-operation",
  "invalid-handle",
  "compilation-failed",
  "execution-failed",
  "transfer-failed",
  "cancelled",
  "closed-runtime"
]

/** The addon prefixes every message with the library's reason class ("execution-failed: ..."). */
const toBackendError = (operation: string, phase: Phase) => (error: unknown): Runtime.BackendError => {
  if (error instanceof Runtime.BackendError) return error
  const text = error instanceof Error ? error.message : String(error)
  const cut = text.indexOf(": ")
  const head = cut > 0 ? text.slice(0, cut) : ""
  const known = reasons.find((r) => r === head)
  return new Runtime.BackendError({
    reason: known ?? "execution-failed", // "invalid-argument" has no class of its own in BackendError
    backend: "cuda",
    operation,
    phase,
    message: known || head === "invalid-argument" ? text.slice(cut + 2) : text
  })
}

const attempt = <A>(operation: string, phase: Phase, body: () => A): Effect.Effect<A, Runtime.BackendError> =>
  Effect.try({ try: body, catch: toBackendError(operation, phase) })

const attemptPromise = <A>(operation: string, phase: Phase, body: () => Promise<A>): Effect.Effect<A, Runtime.BackendError> =>
  Effect.tryPromise({ try: body, catch: toBackendError(operation, phase) })

const unsupported = (operation: string, phase: Phase) => (): Effect.Effect<never, Runtime.BackendError> =>
  Effect.fail(
    new Runtime.BackendError({
      reason: "unsupported-operation",
      backend: "cuda",
      operation,
      phase,
      message: `${operation} is not served by the CUDA decode backend`
    })
  )

/** Handles are the addon's own objects behind the core's opaque brands. */
const brand = <H>(value: unknown): H => value as H
const pool = (handle: Runtime.KvPoolHandle): Native.NativeKvPool => handle as unknown as Native.NativeKvPool
const sequence = (handle: Runtime.KvSequenceHandle): Native.NativeKvSequence => handle as unknown as Native.NativeKvSequence
const tensor = (handle: Runtime.ConcreteTensorHandle): Native.NativeTensor => handle as unknown as Native.NativeTensor

interface CompiledDecode {
  readonly executable: Native.Executable
}

export const makeRuntime = (native: Native.NativeAddon): Runtime.RuntimeService => {
  if (!native.isAvailable()) {
    throw new Runtime.BackendError({
      reason: "backend-unavailable",
      backend: "cuda",
      operation: "makeRuntime",
      phase: "graph",
      message: "no usable CUDA device"
    })
  }
  const identity = {}
  // Which pool a sequence was made from: a stateful invocation names sequences only, and all of them must share one pool
  // (the CPU adapter keeps the same record beside each sequence handle, packages/backend-cpu/src/internal/adapter.ts:661-662).
  const poolOf = new WeakMap<Native.NativeKvSequence, Native.NativeKvPool>()
  const sharedPool = (operation: string, sequences: ReadonlyArray<Native.NativeKvSequence>): Native.NativeKvPool => {
    const first = sequences.length > 0 ? poolOf.get(sequences[0]!) : undefined
    if (first === undefined) throw new Error(`invalid-handle: ${operation}: the invocation names no sequence of this runtime`)
    if (sequences.some((entry) => poolOf.get(entry) !== first)) {
      throw new Error(`execution-failed: ${operation}: the sequences of one invocation must come from one pool`)
    }
    return first
  }

  const decode: Runtime.DecodeRuntime = {
    makePool: (options) =>
      attempt("makePool", "execute", () => {
        if (options.kdaLayers !== 0 || options.convLayers !== 0) {
          throw new Error("unsupported-operation: recurrent state (KDA / short convolution) is not served by the CUDA decode backend")
        }
        return brand<Runtime.KvPoolHandle>(
          new native.NativeKvPool(
            options.layers,
            options.kvHeads,
            options.headDim,
            options.maxTokens,
            options.blockSize,
            options.dtype as Native.NativeDType
          )
        )
      }),
    makeSequence: (handle) =>
      attempt("makeSequence", "execute", () => {
        const made = pool(handle).makeSequence()
        poolOf.set(made, pool(handle))
        return brand<Runtime.KvSequenceHandle>(made)
      }),
    prefillMatch: (handle, tokens) => attempt("prefillMatch", "execute", () => sequence(handle).prefillMatch([...tokens])),
    sequenceCursor: (handle) => attempt("sequenceCursor", "execute", () => sequence(handle).cursor),
    releaseSequence: (handle) => attempt("releaseSequence", "execute", () => sequence(handle).release())
  }

  const compiled = (handle: Runtime.ExecutableHandle): CompiledDecode => handle as unknown as CompiledDecode

  return {
    identity,
    backend: { name: "cuda", version: "0.1.0" } as Runtime.BackendInfo,
    placement: { device: "cuda:0" } as Runtime.Placement,
    capabilities: { dtypes: ["f32", "u8", "u32", "i64"], features: ["decode", "gguf", "sampling"] } as unknown as Runtime.Capabilities,
    node: unsupported("node", "graph"),
    grad: unsupported("grad", "autodiff"),
    compile: (request) =>
      attempt("compile", "compile", () => {
        // The decode specialization (crates/compiler/src/decode.rs:105-481) runs in the core against the request's roots;
        // what reaches the addon is its result: the decoder description, one constant weight per slot, the state schema.
        const plan = Runtime.describeDecode(request)
        if (plan === undefined || request.state === undefined) {
          throw new Error("unsupported-operation: only stateful Llama-family decode graphs compile on the CUDA backend")
        }
        const executable = native.compileDecoder(plan.description, plan.weights, {
          maxTokens: request.state.maxTokens,
          blockSize: request.state.blockSize,
          kvDtype: request.state.kvDtype as Native.NativeDType,
          window: request.state.window,
          batch: request.state.batch
        })
        const entry: CompiledDecode = { executable }
        return brand<Runtime.ExecutableHandle>(entry)
      }),
    execute: (handle, invocation) =>
      attemptPromise("execute", "execute", async () => {
        const entry = compiled(handle)
        const sequences = (invocation.sequences ?? []).map(sequence)
        const tokens = (invocation.tokens ?? []).map((chunk) => [...chunk])
        const logits = await entry.executable.execute(sharedPool("execute", sequences), sequences, tokens)
        const bytes = new Uint8Array(logits.buffer, logits.byteOffset, logits.byteLength)
        return [brand<Runtime.ConcreteTensorHandle>(native.NativeTensor.fromBytes(bytes, [sequences.length, logits.length / sequences.length], "f32"))]
      }),
    readback: (handle) => attemptPromise("readback", "readback", () => tensor(handle).readback()),
    release: (handle) => attempt("release", "execute", () => tensor(handle).clear()),
    extensions: {
      pathSafetensors: {
        load: unsupported("loadTensors", "io"),
        save: unsupported("saveTensors", "io")
      } as unknown as Runtime.PathSafetensors,
      gguf: {
        inspect: (path) =>
          attemptPromise("inspectGguf", "io", async () => ({ metadata: [], tensors: await native.inspectGguf(path) }) as unknown as Runtime.GgufInspection),
        load: (path) => attempt("loadGguf", "io", () => ({ entries: native.loadGguf(path) }) as unknown as Runtime.GgufLoadArchive)
      },
      sampling: {
        sample: (logits, options) =>
          attemptPromise("sample", "execute", () =>
            tensor(logits).sample(options.temperature, options.topK, options.topP, BigInt(options.seed), BigInt(options.counter))
          ),
        executeDecode: (handle, invocation, options) =>
          attemptPromise("executeDecode", "execute", async () => {
            const entry = compiled(handle)
            const sequences = (invocation.sequences ?? []).map(sequence)
            const tokens = (invocation.tokens ?? []).map((chunk) => [...chunk])
            const shared = sharedPool("executeDecode", sequences)
            if (options.every((o) => o.temperature === 0)) {
              return entry.executable.executeSampled(shared, sequences, tokens)
            }
            // non-greedy draws: the logits come back once, one sampling launch per row
            const logits = await entry.executable.execute(shared, sequences, tokens)
            const vocab = logits.length / sequences.length
            return Promise.all(
              options.map((o, row) => {
                const bytes = new Uint8Array(logits.buffer, logits.byteOffset + row * vocab * 4, vocab * 4)
                const rowTensor = native.NativeTensor.fromBytes(bytes, [vocab], "f32")
                return rowTensor.sample(o.temperature, o.topK, o.topP, BigInt(o.seed), BigInt(o.counter)).finally(() => rowTensor.clear())
              })
            )
          })
      },
      decode,
      diagnostics: { externalMemoryBytes: () => native.externalMemoryBytes() } as unknown as Runtime.RuntimeDiagnostics
    }
  }
}
