/-
  Hesper.Backend.B200 — routes Hesper's quantized-inference hot path to libhesper_b200.so.

  Mirrors Hesper/Backend/LlamaCppPTX.lean:383-432 (`installOverride` / `autoInstall`): the
  Q4_K / Q8_0 matvec goes through the hook that already exists,
  `Hesper.Layers.Linear.llamaCppDp4aOverride` (Hesper/Layers/Linear.lean:65-72, consulted at
  :5723-5740).  BitLinear and decode attention have no hook in Hesper; section 2 below holds
  the two `IO.Ref`s and the call-site lines a maintainer adds for them.

  Build: add this file and `HesperB200Extern.lean` to the `Hesper` library, compile
  `lean_ffi.cpp` into the native archive and append `-L<dir> -lhesper_b200` to `cudaExeArgs`
  (lakefile.lean:123-129).  Not compiled where this repository is developed (no Lean toolchain
  there); the C++ side is type-checked against a stand-in `lean.h` by the repository's tests.
-/
import Hesper.Layers.Linear
import Hesper.Backend.B200Extern  -- = HesperB200Extern.lean

namespace Hesper.Backend.B200

/-- GGUF type ids the C ABI speaks (Hesper/GGUF/Types.lean:86-132). -/
def fmtQ8_0 : UInt32 := 8
def fmtQ4_K : UInt32 := 12

/-- One library context per process, created on the CUDA context Hesper already made
    (`cuCtxCreate`, native/cuda_bridge.cpp:78-82) — call after `CUDAContext.init`. -/
initialize ctxRef : IO.Ref (Option USize) ← IO.mkRef none

def getCtx : IO USize := do
  match ← ctxRef.get with
  | some c => pure c
  | none =>
    let c ← ctxCreateCurrent
    ctxRef.set (some c)
    pure c

/-- The stream every launch must go to: the capture stream while a graph is being recorded
    (Hesper/Backend/LlamaCppPTX.lean:138-155), else the legacy default stream. -/
def currentStream : IO USize := do
  match ← Hesper.cudaCaptureStream.get with
  | some s => pure s
  | none => pure 0

def isEnabled : IO Bool := do
  match ← IO.getEnv "HESPER_USE_B200" with
  | some "1" => pure true
  | _ => pure false

/-! ## 1. Q4_K / Q8_0 matvec: the existing hook -/

/-- Same shape as `LlamaCppPTX.installOverride`.  Quant tags of the hook: 0 = Q4_K, 1 = Q6_K
    (not handled: falls through to Hesper's kernel), 2 = Q8_0. -/
def installOverride : IO Unit := do
  let ctx ← getCtx
  Hesper.Layers.Linear.llamaCppDp4aOverride.set (some fun inPtr wPtr outPtr inDim outDim tag => do
    let fmt ← match tag with
      | 0 => pure fmtQ4_K
      | 2 => pure fmtQ8_0
      | _ => return false
    if inDim % 256 != 0 then return false
    let stream ← currentStream
    kquantForward ctx fmt wPtr inDim.toUInt32 outDim.toUInt32 inPtr 1 0 0.0 0 outPtr stream
    return true)

/-- Auto-install if `HESPER_USE_B200=1`; returns `true` if the override is now live. -/
def autoInstall : IO Bool := do
  if ← isEnabled then
    installOverride
    IO.println "[hesper] HESPER_USE_B200=1 — B200 library override installed."
    return true
  else
    return false

/-! ## 2. BitLinear and decode attention: hooks to add

  Hesper has no override point for these.  The refs below belong next to the code that would
  consult them; they are declared here so that this file is the whole integration.  The
  call-site additions (three lines each) are:

  * Hesper/Layers/BitLinear.lean, top of `forward` (:1226), `forwardWithResidual` (:1308),
    `forwardFusedRMSNormResidual` (:1370):
      `if let some f ← Hesper.Backend.B200.bitLinearOverride.get then
         if ← f (rawPtr layer.weights) (rawPtr layer.scale) (rawPtr input) gammaPtr residualPtr
                (rawPtr output) layer.config.inDim layer.config.outDim numRows eps then return`
    (`rawPtr` = `GPUBackend.rawDevicePtr`, Hesper/Backend.lean:90; CUDA returns `some buf.ptr`,
    Hesper/Backend/CUDA.lean:832.)
  * the same in `forwardFusedGateUpReluSqrMul` (:1419) with `gateUpOverride`.
  * Hesper/WGSL/FlashAttentionExperiments.lean, top of `executeFlashAttentionV11` (:572):
      `if let some f ← Hesper.Backend.B200.attnOverride.get then
         if ← f qPtr kPtr vPtr outPtr numHeads numKVHeads headDim maxSeqLen cacheLen scale then return`
-/

/-- `(packed scale x gamma residual y : USize) (inDim outDim rows : Nat) (eps : Float)`;
    `gamma` / `residual` are 0 when absent. -/
initialize bitLinearOverride :
  IO.Ref (Option (USize → USize → USize → USize → USize → USize → Nat → Nat → Nat → Float → IO Bool)) ←
    IO.mkRef none

/-- `(packedGate scaleGate packedUp scaleUp x gamma y : USize) (inDim outDim rows : Nat) (eps : Float)`. -/
initialize gateUpOverride :
  IO.Ref (Option (USize → USize → USize → USize → USize → USize → USize → Nat → Nat → Nat → Float → IO Bool)) ←
    IO.mkRef none

/-- `(q kCache vCache out : USize) (heads kvHeads headDim maxSeq cacheLen : Nat) (scale : Float)`;
    q and out are f32 `[heads·headDim]`, the caches f16 `[kvHead][pos][headDim]`
    (Hesper/WGSL/FlashAttention.lean:590-597). -/
initialize attnOverride :
  IO.Ref (Option (USize → USize → USize → USize → Nat → Nat → Nat → Nat → Nat → Float → IO Bool)) ←
    IO.mkRef none

/-- Scratch of the attention hook: the cache length and the split-K workspace, both allocated
    once by the host (`CUDABuffer`s of Hesper's pool) and handed over here. -/
initialize attnScratch : IO.Ref (Option (USize × USize × USize)) ← IO.mkRef none  -- (lenPtr, wsPtr, wsBytes)

def installLayerOverrides : IO Unit := do
  let ctx ← getCtx
  bitLinearOverride.set (some fun packed scale x gamma residual y inDim outDim rows eps => do
    if inDim % 128 != 0 then return false
    let stream ← currentStream
    bitlinearForward ctx packed scale inDim.toUInt32 outDim.toUInt32 x rows.toUInt32 gamma eps
      residual 0 0 y stream
    return true)
  gateUpOverride.set (some fun pg sg pu su x gamma y inDim outDim rows eps => do
    if inDim % 128 != 0 then return false
    let stream ← currentStream
    bitlinearGateupRelu2 ctx pg sg pu su inDim.toUInt32 outDim.toUInt32 x rows.toUInt32 gamma eps
      y stream
    return true)
  attnOverride.set (some fun q k v out heads kvHeads headDim maxSeq _cacheLen scale => do
    if headDim != 64 && headDim != 128 && headDim != 256 then return false
    match ← attnScratch.get with
    | none => return false
    | some (lenPtr, wsPtr, wsBytes) =>
      let stream ← currentStream
      -- the host writes cacheLen to lenPtr (a one-element i32 device buffer) before the call,
      -- exactly as it fills the V11 kernel's params buffer (FlashAttentionExperiments.lean:586-597)
      attnDecode ctx q 0 k v lenPtr 1 heads.toUInt32 kvHeads.toUInt32 headDim.toUInt32
        maxSeq.toUInt32 0 scale wsPtr wsBytes out stream
      return true)

end Hesper.Backend.B200
