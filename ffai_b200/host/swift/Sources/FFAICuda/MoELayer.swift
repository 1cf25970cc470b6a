// Swift wrapper with the call surface of FFAI's MoERouter / MoELayer
// (Sources/FFAI/Models/MoELayer.swift:88-205, 319-969) whose bodies call libffai_cuda.
// Device tensors are raw pointers plus a CUDA stream; FFAI's Tensor (MTLBuffer + offset) and
// MTLCommandBuffer have no counterpart on this side of the boundary.
import CFFAICuda

public enum MoEGatingMode: Sendable {
    case softmaxThenTopK
    case topKThenSoftmax
    case sigmoidTopK          // NemotronHMoELayer routing
    var raw: Int32 {
        switch self {
        case .softmaxThenTopK: return 0
        case .topKThenSoftmax: return 1
        case .sigmoidTopK: return 2
        }
    }
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

    /// Gemma4MoEFFN.forward — Gemma4Text.swift:928-980: the router reads its own normalised rows,
    /// the experts read `hExperts`.  `hRouter == nil` means `hExperts`.
    public func decodeManySplit(_ hExperts: UnsafePointer<UInt16>, router hRouter: UnsafePointer<UInt16>?, t: Int,
                                out: UnsafeMutablePointer<UInt16>, residual: UnsafePointer<UInt16>? = nil,
                                stream: UnsafeMutableRawPointer?) throws {
        precondition(t > 0, "MoELayer.decodeManySplit: T must be positive")
        let rc = ffai_moe_forward_split(handle, hExperts, hRouter, Int32(t), out, residual, nil, stream)
        if rc != 0 { throw FFAICudaError(status: rc, message: String(cString: ffai_moe_last_error(handle))) }
    }

    /// Execution options ("path", "ksplit", "tc_min_rows", …) — the `FFAI_MOE_*` environment
    /// switches of MoELayer.swift:486-497.
    public func setOption(_ name: String, _ value: Int) throws {
        let rc = name.withCString { ffai_moe_set_option(handle, $0, Int32(value)) }
        if rc != 0 { throw FFAICudaError(status: rc, message: "ffai_moe_set_option(\(name))") }
    }

    /// Expert parallelism over peer memory (no counterpart in the reference): every rank exports, the
    /// caller hands all blobs to every rank in rank order, every rank imports; release on every rank
    /// before any rank's layer is destroyed.
    public func exportPeerBuffers() throws -> [UInt8] {
        var blob = [UInt8](repeating: 0, count: Int(FFAI_EP_EXPORT_BYTES))
        let rc = ffai_moe_ep_export(handle, &blob)
        if rc != 0 { throw FFAICudaError(status: rc, message: String(cString: ffai_moe_last_error(handle))) }
        return blob
    }

    public func importPeerBuffers(_ allBlobs: [UInt8]) throws {
        precondition(!allBlobs.isEmpty && allBlobs.count % Int(FFAI_EP_EXPORT_BYTES) == 0,
                     "MoELayer.importPeerBuffers: expected ep_world blobs of FFAI_EP_EXPORT_BYTES")
        let rc = ffai_moe_ep_import(handle, allBlobs)
        if rc != 0 { throw FFAICudaError(status: rc, message: String(cString: ffai_moe_last_error(handle))) }
    }

    /// This rank sits out one step of the peer-memory exchange: its step counter moves on without a forward.
    public func skipPeerStep() throws {
        let rc = ffai_moe_ep_skip_step(handle)
        if rc != 0 { throw FFAICudaError(status: rc, message: String(cString: ffai_moe_last_error(handle))) }
    }

    public func releasePeerBuffers() throws {
        let rc = ffai_moe_ep_release(handle)
        if rc != 0 { throw FFAICudaError(status: rc, message: String(cString: ffai_moe_last_error(handle))) }
    }
}
