// DispatchEntry -> swlm_step: the CUDA backend's counterpart of MetalDispatchStepBuilder.buildDecodePlan
// (Sources/MetalCompiler/Compiler/MetalDispatchStepBuilder.swift:4-105) for the fragments of the hot path.
// MetalEntryCollector.collect (Compiler/MetalEntryCollector.swift:143-218) still produces the flat entry list and
// DecodeRoutingPlanner (MetalDispatchStepBuilder.swift:587-737) still assigns the buffer slots; this file turns each
// routed entry into one plan step. Kernel selection, launch fusion and buffer allocation happen behind the C ABI.
// Not compiled in the environment this library was built in (no Swift toolchain there): the entry description below
// is a plain value type a maintainer fills from DispatchEntry + DecodeRoutingPlanner's routing state.
import CSwlmCUDA

/// What the mapper needs to know of one routed dispatch entry.
public enum CUDAPlanEntry {
    /// GatherFragment (bf16 table) or the Q4 lookup when `table` names a quantized tensor (tied head).
    case embedding(table: String, hidden: Int)
    /// CopyFragment / ResidualAddFragment + Reduction, as MetalEntryCollector fuses them.
    case rmsNorm(kind: NormKind, weight: String, dimension: Int, epsilon: Float, weightBias: Float, input: Slot, output: Slot)
    /// LinearFragment over a 4-bit group-64 weight.
    case linear(weight: String, outputDimension: Int, inputDimension: Int, input: Slot, output: Slot)
    /// BatchedFragment[QKNormFragment x 2].
    case qkNorm(qWeight: String, kWeight: String, heads: Int, kvHeads: Int, headDimension: Int, epsilon: Float,
                weightBias: Float, q: Slot, k: Slot)
    /// FlashAttentionFragment (decode): inline RoPE, KV append, attention over [0, position].
    case attention(layer: Int, heads: Int, kvHeads: Int, headDimension: Int, ropeDimension: Int, ropeBase: Float,
                   scale: Float, windowLeft: Int?, q: Slot, k: Slot, v: Slot, output: Slot)
    /// ElementwiseFragment(.swiglu) or the gated activation with .geluTanh.
    case gatedActivation(gelu: Bool, dimension: Int, gate: Slot, up: Slot, output: Slot)
    /// Conv1dFragment: conv_state_update over the packed B|C|x projection.
    case shortConv(layer: Int, weight: String, dimension: Int, kernelSize: Int, input: Slot, output: Slot)
    /// SSMRecurrenceFragment (decode): gated delta rule over the projected q|k|v, z, beta and alpha buffers.
    case recurrence(layer: Int, heads: Int, groups: Int, keyDimension: Int, valueDimension: Int, convKernelSize: Int,
                    convWeight: String, normWeight: String, dtBias: String, aLog: String,
                    qkv: Slot, z: Slot, beta: Slot, alpha: Slot, output: Slot)
    /// ArgmaxFragment over the logits.
    case argmax(vocabulary: Int)

    public enum NormKind { case copy, residualAddCopy, residualAdd }

    /// Logical buffers of the decode plan (hidden, residual, scratch slots 0-4, logits).
    public enum Slot: Int32 {
        case hidden = 0, residual = 1, scratch0 = 2, scratch1 = 3, scratch2 = 4, scratch3 = 5, scratch4 = 6, logits = 7
    }
}

public struct CUDADispatchPlanBuilder {
    public init() {}

    public func steps(for entries: [CUDAPlanEntry]) throws -> [swlm_step] {
        try entries.map(step(for:))
    }

    func blank(_ kind: Int32) -> swlm_step {
        var s = swlm_step()
        s.kind = kind
        s.layer = -1
        s.in_buf = -1; s.in2_buf = -1; s.in3_buf = -1; s.in4_buf = -1; s.out_buf = -1
        return s
    }

    func setName(_ name: String, into field: inout swlm_step, second: Bool = false) throws {
        let bytes = Array(name.utf8)
        guard bytes.count < Int(SWLM_NAME_MAX) else { throw CUDACompilerError.unsupportedTensor(name) }
        withUnsafeMutableBytes(of: second ? &field.weight2 : &field.weight) { raw in
            raw.initializeMemory(as: UInt8.self, repeating: 0)
            raw.copyBytes(from: bytes)
        }
    }

    func setName<T>(_ name: String, into field: inout T) throws {
        let bytes = Array(name.utf8)
        guard bytes.count < Int(SWLM_NAME_MAX) else { throw CUDACompilerError.unsupportedTensor(name) }
        withUnsafeMutableBytes(of: &field) { raw in
            raw.initializeMemory(as: UInt8.self, repeating: 0)
            raw.copyBytes(from: bytes)
        }
    }

    func step(for entry: CUDAPlanEntry) throws -> swlm_step {
        switch entry {
        case let .embedding(table, hidden):
            var s = blank(Int32(SWLM_STEP_EMBED))
            s.out_buf = CUDAPlanEntry.Slot.hidden.rawValue
            s.n = Int32(hidden)
            try setName(table, into: &s)
            return s
        case let .rmsNorm(kind, weight, dimension, epsilon, weightBias, input, output):
            let k: Int   // anonymous C enum constants import as Int
            switch kind {
            case .copy: k = SWLM_STEP_COPY_RMSNORM
            case .residualAddCopy: k = SWLM_STEP_RESADD_COPY_RMSNORM
            case .residualAdd: k = SWLM_STEP_RESADD_RMSNORM
            }
            var s = blank(Int32(k))
            s.in_buf = input.rawValue; s.out_buf = output.rawValue
            s.n = Int32(dimension); s.eps = epsilon; s.weight_bias = weightBias
            try setName(weight, into: &s)
            return s
        case let .linear(weight, outputDimension, inputDimension, input, output):
            var s = blank(Int32(SWLM_STEP_QGEMV))
            s.in_buf = input.rawValue; s.out_buf = output.rawValue
            s.n = Int32(outputDimension); s.k = Int32(inputDimension)
            try setName(weight, into: &s)
            return s
        case let .qkNorm(qWeight, kWeight, heads, kvHeads, headDimension, epsilon, weightBias, q, k):
            var s = blank(Int32(SWLM_STEP_QK_NORM))
            s.in_buf = q.rawValue; s.in2_buf = k.rawValue
            s.heads = Int32(heads); s.kv_heads = Int32(kvHeads); s.head_dim = Int32(headDimension)
            s.eps = epsilon; s.weight_bias = weightBias
            try setName(qWeight, into: &s)
            try setName(kWeight, into: &s, second: true)
            return s
        case let .attention(layer, heads, kvHeads, headDimension, ropeDimension, ropeBase, scale, windowLeft, q, k, v, output):
            var s = blank(Int32(SWLM_STEP_ATTN_DECODE))
            s.layer = Int32(layer)
            s.in_buf = q.rawValue; s.in2_buf = k.rawValue; s.in3_buf = v.rawValue; s.out_buf = output.rawValue
            s.heads = Int32(heads); s.kv_heads = Int32(kvHeads); s.head_dim = Int32(headDimension)
            s.rope_dim = Int32(ropeDimension); s.rope_base = ropeBase; s.scale = scale
            s.window_left = Int32(windowLeft ?? 0)   // FlashAttentionFragment.windowLeft (nil = full attention)
            return s
        case let .gatedActivation(gelu, dimension, gate, up, output):
            var s = blank(Int32(gelu ? SWLM_STEP_GEGLU : SWLM_STEP_SWIGLU))
            s.in_buf = gate.rawValue; s.in2_buf = up.rawValue; s.out_buf = output.rawValue
            s.n = Int32(dimension)
            return s
        case let .shortConv(layer, weight, dimension, kernelSize, input, output):
            var s = blank(Int32(SWLM_STEP_CONV_STATE_UPDATE))
            s.layer = Int32(layer)
            s.in_buf = input.rawValue; s.out_buf = output.rawValue
            s.n = Int32(dimension); s.conv_kernel = Int32(kernelSize)
            try setName(weight, into: &s)
            return s
        case let .recurrence(layer, heads, groups, keyDimension, valueDimension, convKernelSize, convWeight, normWeight, dtBias, aLog,
                             qkv, z, beta, alpha, output):
            var s = blank(Int32(SWLM_STEP_SSM_RECURRENCE))
            s.layer = Int32(layer)
            s.in_buf = qkv.rawValue; s.in2_buf = z.rawValue; s.in3_buf = beta.rawValue; s.in4_buf = alpha.rawValue
            s.out_buf = output.rawValue
            s.heads = Int32(heads); s.groups = Int32(groups); s.key_dim = Int32(keyDimension); s.value_dim = Int32(valueDimension)
            s.conv_kernel = Int32(convKernelSize)
            try setName(convWeight, into: &s)
            try setName(normWeight, into: &s, second: true)
            try setName(dtBias, into: &s.weight3)
            try setName(aLog, into: &s.weight4)
            return s
        case let .argmax(vocabulary):
            var s = blank(Int32(SWLM_STEP_ARGMAX))
            s.in_buf = CUDAPlanEntry.Slot.logits.rawValue
            s.n = Int32(vocabulary)
            return s
        }
    }
}
