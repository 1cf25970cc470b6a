// Swift wrapper with the call surface of FFAI's MoERouter / MoELayer
// (Sources/FFAI/Models/MoELayer.swift:88-205, 319-969) whose bodies call libffai_cuda.
// Device tensors are raw pointers plus a CUDA stream; FFAI's Tensor (MTLBuffer + offset) and
// MTLCommandBuffer have no counterpart on this side of the boundary.
import CFFAICuda

public enum MoEGatingMode: Sendable {
    case softmaxThenTopK
    case topKThenSoftmax
    var raw: Int32 { self == .softmaxThenTopK ? 0 : 1 }
}

public struct FFAICudaError: Error, CustomStringConvertible {
    public let status: Int32
    public let message: String
    public var description: String { "libffai_cuda status \(status): \(message)" }
}

/// Mirrors `MoERouter` (value type; validation as MoELayer.swift:109-118).
public struct MoERouter: Sendable {
    public let nExperts: Int
    public let topK: Int
    public let gatingMode: MoEGatingMode
    public let normTopKProb: Bool
    public let expertBias: [Float]?

    public init(nExperts: Int, topK: Int, gatingMode: MoEGatingMode,
                normTopKProb: Bool = true, expertBias: [Float]? = nil) {
        precondition(nExperts > 0, "MoERouter: nExperts must be positive")
        precondition(topK > 0 && topK <= nExperts, "MoERouter: topK must be in 1...nExperts")
        if let b = expertBias { precondition(b.count == nExperts, "MoERouter: expertBias count") }
        self.nExperts = nExperts; self.topK = topK; self.gatingMode = gatingMode
        self.normTopKProb = normTopKProb; self.expertBias = expertBias
    }
}

/// Mirrors `MoELayer` (and, through the config, `GPTOSSMoELayer` / `Qwen35MoEFFN`).
/// Not safe for concurrent calls on one instance (MoELayer.swift:311-318).
public final class MoELayer {
    private var handle: OpaquePointer?
    public let hidden: Int

    /// `config` and `weights` are the C structs of ffai_cuda.h; weights stay in FFAI's stacked
    /// layout (`StackedInt4Experts`, MoELayer.swift:347-391) and may be borrowed device pointers.
    public init(config: ffai_moe_config, weights: ffai_moe_weights) throws {
        var cfg = config, w = weights
        cfg.struct_size = UInt32(MemoryLayout<ffai_moe_config>.size)
        w.struct_size = UInt32(MemoryLayout<ffai_moe_weights>.size)
        hidden = Int(cfg.hidden)
        var h: OpaquePointer?
        var rc = ffai_moe_create(&cfg, &h)
        handle = h
        if rc == 0 { rc = ffai_moe_set_weights(h, &w) }
        if rc != 0 {
            let msg = String(cString: ffai_moe_last_error(h))
            ffai_moe_destroy(h); handle = nil
            throw FFAICudaError(status: rc, message: msg)
        }
    }

    deinit { if let h = handle { ffai_moe_destroy(h) } }

    /// decode(_:position:cache:cmd:device:) — MoELayer.swift:530-534.
    public func decode(_ h: UnsafePointer<UInt16>, out: UnsafeMutablePointer<UInt16>,
                       residual: UnsafePointer<UInt16>? = nil, stream: UnsafeMutableRawPointer?) throws {
        try decodeMany(h, t: 1, out: out, residual: residual, stream: stream)
    }

    /// decodeMany(_:t:cmd:device:) — MoELayer.swift:677-680.
    public func decodeMany(_ hFlat: UnsafePointer<UInt16>, t: Int, out: UnsafeMutablePointer<UInt16>,
                           residual: UnsafePointer<UInt16>? = nil, stream: UnsafeMutableRawPointer?) throws {
        precondition(t > 0, "MoELayer.decodeMany: T must be positive")
        let rc = ffai_moe_forward(handle, hFlat, Int32(t), out, residual, nil, stream)
        if rc != 0 { throw FFAICudaError(status: rc, message: String(cString: ffai_moe_last_error(handle))) }
    }
}
