/*
 * Loads the addon built from `crates/runtime-cuda` (cargo build --release --features napi). One Linux x86-64 / glibc
 * binary exists: a B200 host. Loading failures throw during module evaluation, as they do for the CPU package.
 */
import { createRequire } from "node:module"
import type { NativeAddon } from "./native-addon.js"

const require = createRequire(import.meta.url)

const load = (): NativeAddon => {
  if (process.platform !== "linux" || process.arch !== "x64") {
    throw new Error(`@effect-torch/backend-cuda: unsupported host ${process.platform}-${process.arch}`)
  }
  return require("../../effect-torch-backend-cuda.linux-x64-gnu.node") as NativeAddon
}

const native: NativeAddon = load()
export default native
