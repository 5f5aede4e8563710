// CUDA counterpart of STAFWeightStore (Sources/MetalCompiler/STAF/STAFLoader.swift:19-299): one context per
// device (and tensor-parallel rank) that owns the device-resident weights. Not compiled in the environment this
// library was built in (no Swift toolchain there); it only calls the C ABI declared in include/swlm.h.
import CSwlmCUDA
import Foundation

public enum CUDACompilerError: Error {
    case status(Int32, String)
    case unsupportedTensor(String)
}

@inline(__always) func swlmCheck(_ rc: Int32) throws {
    if rc != SWLM_OK { throw CUDACompilerError.status(rc, String(cString: swlm_last_error())) }
}

public final class CUDAWeightStore {
    let ctx: OpaquePointer

    public init(device: Int32 = 0, tensorParallelRank: Int32 = 0, tensorParallelSize: Int32 = 1) throws {
        var c: OpaquePointer?
        try swlmCheck(swlm_ctx_create(device, tensorParallelRank, tensorParallelSize, &c))
        ctx = c!
    }

    deinit { swlm_ctx_destroy(ctx) }

    public var residentBytes: Int64 { swlm_weights_bytes(ctx) }

    /// STAF payload of one tensor with scheme q4Group64ScaleF16 (0x40): `rows x cols` weights as interleaved
    /// 36-byte blocks, straight from the mmap of `model.staf`.
    public func addSTAFBlocks(name: String, rows: Int, cols: Int, blocks: UnsafeRawPointer,
                              shard: Int32 = Int32(SWLM_SHARD_REPLICATE)) throws {
        try swlmCheck(swlm_weights_add_q4g64_staf(ctx, name, Int32(rows), Int32(cols), blocks, shard))
    }

    /// MLX safetensors triple: words u32 [rows][cols/8], scales and biases bf16 [rows][cols/64].
    public func addMLX(name: String, rows: Int, cols: Int, weight: UnsafePointer<UInt32>,
                       scales: UnsafePointer<UInt16>, biases: UnsafePointer<UInt16>,
                       shard: Int32 = Int32(SWLM_SHARD_REPLICATE)) throws {
        try swlmCheck(swlm_weights_add_q4g64_mlx(ctx, name, Int32(rows), Int32(cols), weight, scales, biases, shard))
    }

    public func addDense(name: String, rows: Int, cols: Int, bf16: UnsafePointer<UInt16>,
                         shard: Int32 = Int32(SWLM_SHARD_REPLICATE)) throws {
        try swlmCheck(swlm_weights_add_dense_bf16(ctx, name, Int64(rows), Int64(cols), bf16, shard))
    }

    /// Upload every tensor of a loaded STAF file that the hot path holds. `entries` is what STAFLoader parsed
    /// (name, scheme, shape, payload offset and size); `base` is the start of the mapped file.
    /// `shardKind` maps tensor names to SWLM_SHARD_* for tensor-parallel contexts.
    public func load(staf entries: [(name: String, scheme: UInt8, shape: [Int], payloadOffset: Int, payloadSize: Int)],
                     base: UnsafeRawPointer, shardKind: (String) -> Int32 = { _ in Int32(SWLM_SHARD_REPLICATE) }) throws {
        for e in entries {
            let payload = base + e.payloadOffset
            switch e.scheme {
            case 0x40:  // q4Group64ScaleF16: shape is the packed safetensors shape [rows, cols / 8]
                guard e.shape.count == 2 else { throw CUDACompilerError.unsupportedTensor(e.name) }
                try addSTAFBlocks(name: e.name, rows: e.shape[0], cols: e.shape[1] * 8, blocks: payload, shard: shardKind(e.name))
            case 0x41:  // q4Group128ScaleF16: 68-byte blocks of 128 weights
                guard e.shape.count == 2 else { throw CUDACompilerError.unsupportedTensor(e.name) }
                try swlmCheck(swlm_weights_add_q4g128_staf(ctx, e.name, Int32(e.shape[0]), Int32(e.shape[1] * 8), payload, shardKind(e.name)))
            case 0x02 where e.name.hasSuffix(".linear_attn.norm.weight") || e.name.hasSuffix(".A_log"):
                // fp32RowMajor tensors the recurrent step reads as fp32 (STAFConversionPlanner.swift:117-140)
                try swlmCheck(swlm_weights_add_dense_f32(ctx, e.name, Int64(e.payloadSize / 4), payload.assumingMemoryBound(to: Float.self)))
            case 0x01:  // bf16RowMajor
                let cols = e.shape.last ?? 1
                let rows = e.shape.dropLast().reduce(1, *)
                try addDense(name: e.name, rows: rows, cols: cols, bf16: payload.assumingMemoryBound(to: UInt16.self),
                             shard: shardKind(e.name))
            default:
                continue  // other schemes are outside this path; the plan build reports a tensor it misses
            }
        }
    }
}
