// Drop-in for MetalInferenceModel (Sources/MetalCompiler/Execution/MetalInferenceModel.swift:311,464,1897-1911):
// the same mutating surface and the same "-1 means failure" convention, over libswlm_cuda.so. Not compiled in the
// environment this library was built in (no Swift toolchain there).
import CSwlmCUDA

public struct CUDAPromptSnapshot {
    let handle: OpaquePointer
}

extension swlm_buffers_desc {
    /// InferencePolicy.kvCache (Sources/MetalCompiler/InferencePolicy.swift:55-86) into the plan description: the raw value
    /// of the resolved QuantizationSchemeIdentifier (0x01 bf16, 0x10 / 0x11 / 0x12, 0x40 / 0x41, rotated 0x70 / 0x71; one
    /// scheme for K and V) and the projection dimension of the rotated schemes' K residuals (0 = none, at most 64).
    public mutating func setKVCache(schemeRawValue: UInt8, qjlDimension: Int = 0) {
        kv_scheme = Int32(schemeRawValue)
        kv_qjl_dim = Int32(qjlDimension)
    }
}

public final class CUDAInferenceModel {
    let store: CUDAWeightStore
    let plan: OpaquePointer
    let state: OpaquePointer
    public let vocabularySize: Int

    public init(store: CUDAWeightStore, steps: [swlm_step], buffers: swlm_buffers_desc) throws {
        var p: OpaquePointer?
        var s: OpaquePointer?
        var desc = buffers
        try steps.withUnsafeBufferPointer {
            try swlmCheck(swlm_plan_build(store.ctx, $0.baseAddress, Int32($0.count), &desc, &p))
        }
        do { try swlmCheck(swlm_state_create(p, &s)) } catch { swlm_plan_destroy(p); throw error }
        self.store = store
        plan = p!
        state = s!
        vocabularySize = Int(buffers.vocab)
    }

    deinit {
        swlm_state_destroy(state)
        swlm_plan_destroy(plan)
    }

    public var position: Int { Int(swlm_position(state)) }
    public var launchesPerStep: Int { Int(swlm_plan_launch_count(plan)) }

    /// First generated token, or -1 (message in swlm_last_error()).
    public func prefill(tokens: [Int32]) -> Int32 {
        var first: Int32 = -1
        _ = tokens.withUnsafeBufferPointer { swlm_prefill(state, $0.baseAddress, Int32($0.count), &first) }
        return first
    }

    /// One greedy step: token in, token out, one synchronisation.
    public func decode(tokenID: Int32) -> Int32 {
        var tin = tokenID
        var tout: Int32 = -1
        _ = swlm_decode(state, &tin, &tout)
        return tout
    }

    /// `count` greedy steps without host round trips; the tokens come back together.
    public func decode(from tokenID: Int32, count: Int) throws -> [Int32] {
        var tin = tokenID
        var out = [Int32](repeating: -1, count: count)
        try out.withUnsafeMutableBufferPointer { try swlmCheck(swlm_decode_n(state, &tin, Int32(count), $0.baseAddress)) }
        return out
    }

    public func resetState() { _ = swlm_state_reset(state) }

    // ---- several sequences per step (swlm_buffers_desc.max_batch > 1; no counterpart in the reference) ----------
    /// Append a prompt to one sequence while the others keep their state; returns that sequence's next token (-1 on failure).
    public func prefill(sequence: Int, tokens: [Int32]) -> Int32 {
        var first: Int32 = -1
        _ = tokens.withUnsafeBufferPointer { swlm_prefill_seq(state, Int32(sequence), $0.baseAddress, Int32($0.count), &first) }
        return first
    }

    /// One decode step for all sequences, each at its own position.
    public func decode(tokenIDs: [Int32]) -> [Int32] {
        var out = [Int32](repeating: -1, count: tokenIDs.count)
        _ = tokenIDs.withUnsafeBufferPointer { swlm_decode(state, $0.baseAddress, &out) }
        return out
    }

    public func resetSequence(_ sequence: Int) throws { try swlmCheck(swlm_state_reset_seq(state, Int32(sequence))) }

    public func positions(count: Int) throws -> [Int32] {
        var out = [Int32](repeating: 0, count: count)
        try swlmCheck(swlm_get_positions(state, &out))
        return out
    }

    /// MetalInferenceModel.promptSnapshot / restore: KV cache, conv state, position and last tokens.
    public func promptSnapshot() throws -> CUDAPromptSnapshot {
        var h: OpaquePointer?
        try swlmCheck(swlm_state_snapshot(state, &h))
        return CUDAPromptSnapshot(handle: h!)
    }

    public func restore(_ snapshot: CUDAPromptSnapshot) throws { try swlmCheck(swlm_state_restore(state, snapshot.handle)) }

    public func discard(_ snapshot: CUDAPromptSnapshot) { swlm_snap_destroy(snapshot.handle) }

    /// Logits of the last step as bf16 bit patterns, for host-side sampling
    /// (Sources/SwiftLM/LanguageModelContext.swift:2197-2209 reads the decode plan's logits buffer the same way).
    public func logits() throws -> [UInt16] {
        var out = [UInt16](repeating: 0, count: vocabularySize)
        try out.withUnsafeMutableBufferPointer { try swlmCheck(swlm_read_logits(state, $0.baseAddress, $0.count)) }
        return out
    }

    public func setPrefillChunk(tokens: Int) throws { try swlmCheck(swlm_state_set_prefill_chunk(state, Int32(tokens))) }

    // ---- rotated KV schemes: MetalKVCache.rotorParameters (Buffer/MetalGraphAllocator.swift:258-262) --------------------

    /// fp16 bit patterns [kvLayers][kvHeads][ceil(headDimension / 3)][4] = (s, b12, b13, b23) per rotor.
    public func rotorParameters(count: Int) throws -> [UInt16] {
        var out = [UInt16](repeating: 0, count: count)
        try out.withUnsafeMutableBufferPointer { try swlmCheck(swlm_state_get_rotors(state, $0.baseAddress, $0.count)) }
        return out
    }

    /// Replaces every rotor; call before the first token is cached (rows already in the cache were turned by the old ones).
    public func setRotorParameters(_ values: [UInt16]) throws {
        try values.withUnsafeBufferPointer { try swlmCheck(swlm_state_set_rotors(state, $0.baseAddress, $0.count)) }
    }
}
