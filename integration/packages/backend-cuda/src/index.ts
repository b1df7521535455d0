/**
 * CUDA (B200, sm_100a) package entry point, the sibling of `@effect-torch/backend-cpu`
 * (packages/backend-cpu/src/index.ts:27-41): importing this module loads the native addon built from
 * `crates/runtime-cuda`; {@link makeRuntime} and {@link layer} expose one module-memoized adapter as either a direct
 * service or an Effect dependency. The adapter serves the compiled stateful decode path (paged KV pool, sequences,
 * decode executables over GGUF block-quantized weights, sampling, GGUF loading); every other `RuntimeService` member
 * rejects with `unsupported-operation`, so a model can keep its non-decode work on the CPU layer.
 */
import { Runtime } from "@effect-torch/core"
import { Effect, Layer } from "effect"
import { makeRuntime as makeRuntimeAdapter } from "./internal/adapter.js"
import native from "./internal/native.js"

let runtime: Runtime.RuntimeService | undefined

/**
 * Returns the memoized CUDA runtime singleton for this package module. The addon is loaded at import time; a host
 * without the addon, without a CUDA driver or without a usable device fails here with `backend-unavailable`
 * (`native.isAvailable()` is false), and a failed construction can be retried.
 *
 * @since 0.1.0
 * @category constructors
 */
export const makeRuntime = (): Runtime.RuntimeService => runtime ??= makeRuntimeAdapter(native)

/**
 * A reusable Layer that provides the memoized CUDA runtime singleton.
 *
 * @since 0.1.0
 * @category layers
 */
export const layer: Layer.Layer<Runtime.Runtime> = Layer.effect(Runtime.Runtime, Effect.sync(makeRuntime))

/**
 * Whether this host can run the CUDA backend (addon loaded and at least one device answers).
 *
 * @since 0.1.0
 * @category guards
 */
export const isAvailable = (): boolean => native.isAvailable()
