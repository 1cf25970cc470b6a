// C++ host mirror of FFAI's MoE-layer call surface over the C ABI of libffai_cuda.
//
// The reference's host code is Swift (Sources/FFAI/Models/MoELayer.swift).  No Swift toolchain
// exists where this library is built and tested, so this header is the executed host side: the
// same type names, argument meaning and error behaviour as the reference, with the reference's
// `precondition` traps surfaced as exceptions carrying the library's status and message.
// The Swift wrapper with the same surface is in host/swift/ (shipped, not compiled here).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "ffai_cuda.h"

namespace ffai_host {

struct Error : std::runtime_error {
    int status;
    Error(int s, const std::string& what) : std::runtime_error(what), status(s) {}
};

// MoEGatingMode — MoELayer.swift:71-78
enum class MoEGatingMode { softmaxThenTopK = FFAI_GATING_SOFTMAX_THEN_TOPK, topKThenSoftmax = FFAI_GATING_TOPK_THEN_SOFTMAX,
                           sigmoidTopK = FFAI_GATING_SIGMOID_TOPK /* NemotronHMoELayer routing */ };

// MoERouter — MoELayer.swift:88-205.  A value type; routing itself runs on the device inside
// MoELayer::decode / decodeMany (route() on a logits vector is ffai_op_moe_router_topk).
struct MoERouter {
    int nExperts;
    int topK;
    MoEGatingMode gatingMode;
    bool normTopKProb = true;
    std::vector<float> expertBias;  // empty: none (LFM2 load-balancing bias otherwise)

    MoERouter(int nExperts_, int topK_, MoEGatingMode mode, bool norm = true, std::vector<float> bias = {})
        : nExperts(nExperts_), topK(topK_), gatingMode(mode), normTopKProb(norm), expertBias(std::move(bias)) {
        // MoELayer.swift:109-118
        if (nExperts <= 0) throw Error(FFAI_ERR_INVALID_ARG, "MoERouter: nExperts must be positive");
        if (topK <= 0 || topK > nExperts) throw Error(FFAI_ERR_INVALID_ARG, "MoERouter: topK must be in 1...nExperts");
        if (!expertBias.empty() && (int)expertBias.size() != nExperts)
            throw Error(FFAI_ERR_INVALID_ARG, "MoERouter: expertBias has the wrong number of entries");
    }
};

// MoELayer — MoELayer.swift:319-969 (and, through the config, GPTOSSMoELayer and Qwen35MoEFFN).
// Not safe for concurrent calls on one instance (same contract as MoELayer.swift:311-318).
class MoELayer {
  public:
    MoELayer(const ffai_moe_config& config, const ffai_moe_weights& weights) {
        int rc = ffai_moe_create(&config, &h_);
        if (rc != FFAI_OK) fail(rc, "ffai_moe_create");
        rc = ffai_moe_set_weights(h_, &weights);
        if (rc != FFAI_OK) fail(rc, "ffai_moe_set_weights");
    }
    ~MoELayer() { if (h_) ffai_moe_destroy(h_); }
    MoELayer(const MoELayer&) = delete;
    MoELayer& operator=(const MoELayer&) = delete;

    // decode(_:position:cache:cmd:device:) — MoELayer.swift:530-534.  h, out: device bf16 [hidden].
    // The command buffer of the reference becomes the CUDA stream; nothing is committed or waited on.
    void decode(const uint16_t* h, uint16_t* out, void* stream, const uint16_t* residual = nullptr) {
        decodeMany(h, 1, out, stream, residual);
    }
    // decodeMany(_:t:cmd:device:) — MoELayer.swift:677-680.  hFlat, out: device bf16 [t, hidden].
    void decodeMany(const uint16_t* hFlat, int t, uint16_t* out, void* stream, const uint16_t* residual = nullptr,
                    const ffai_moe_debug* debug = nullptr) {
        if (t <= 0) throw Error(FFAI_ERR_INVALID_ARG, "MoELayer.decodeMany: T must be positive");  // :684
        int rc = ffai_moe_forward(h_, hFlat, t, out, residual, debug, stream);
        if (rc != FFAI_OK) fail(rc, "ffai_moe_forward");
    }
    // host buffers in and out (the reference's shared-storage MTLBuffers)
    void decodeManyHost(const uint16_t* hFlat, int t, uint16_t* out, const uint16_t* residual = nullptr,
                        const ffai_moe_debug* debug = nullptr) {
        int rc = ffai_moe_forward_host(h_, hFlat, t, out, residual, debug);
        if (rc != FFAI_OK) fail(rc, "ffai_moe_forward_host");
    }
    // Gemma4MoEFFN.forward — Gemma4Text.swift:928-980: the router reads its own normalised rows while the
    // experts read hExperts.  hRouter == nullptr means hExperts.
    void decodeManySplit(const uint16_t* hExperts, const uint16_t* hRouter, int t, uint16_t* out, void* stream,
                         const uint16_t* residual = nullptr, const ffai_moe_debug* debug = nullptr) {
        if (t <= 0) throw Error(FFAI_ERR_INVALID_ARG, "MoELayer.decodeManySplit: T must be positive");
        int rc = ffai_moe_forward_split(h_, hExperts, hRouter, t, out, residual, debug, stream);
        if (rc != FFAI_OK) fail(rc, "ffai_moe_forward_split");
    }

    // Loading one block the way the reference's loaders do (stacked triplets under `prefix`;
    // Qwen3xText.swift:605-650 for FFAI_ST_SWITCH_MLP, Gemma4Text.swift:540-554 for FFAI_ST_SWITCH_GLU).
    // `config` carries what the file does not: routing mode, activation, top_k, max_tokens, group sizes.
    static MoELayer fromSafetensors(const std::string& path, const std::string& prefix, int scheme,
                                    ffai_moe_config config) {
        ffai_st_file* f = nullptr;
        int rc = ffai_st_open(path.c_str(), &f);
        if (rc != FFAI_OK) {
            std::string msg = "ffai_st_open: " + std::string(ffai_status_string(rc)) + ": " + ffai_st_last_error(f);
            ffai_st_close(f);
            throw Error(rc, msg);
        }
        ffai_moe_weights w{};
        rc = ffai_st_moe_weights(f, prefix.c_str(), scheme, &config, &w);
        if (rc != FFAI_OK) {
            std::string msg = "ffai_st_moe_weights: " + std::string(ffai_status_string(rc)) + ": " + ffai_st_last_error(f);
            ffai_st_close(f);
            throw Error(rc, msg);
        }
        try {
            MoELayer layer(config, w);   // copies the mapped tensors to the device
            ffai_st_close(f);
            return layer;
        } catch (...) {
            ffai_st_close(f);
            throw;
        }
    }
    MoELayer(MoELayer&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }

    // Execution options ("path", "ksplit", "tc_min_rows", ...); unknown names are FFAI_ERR_INVALID_ARG.
    void setOption(const char* name, int value) {
        int rc = ffai_moe_set_option(h_, name, value);
        if (rc != FFAI_OK) throw Error(rc, std::string("ffai_moe_set_option(") + name + "): " + ffai_status_string(rc));
    }

    // Expert parallelism (no counterpart in the reference, which is single-device).  Either attach an
    // initialised NCCL communicator, or exchange over peer memory: every rank exports, the caller hands all
    // blobs (rank order) to every rank, every rank imports; release on every rank before any rank is destroyed.
    void setNcclComm(void* comm) {
        int rc = ffai_moe_set_nccl_comm(h_, comm);
        if (rc != FFAI_OK) throw Error(rc, std::string("ffai_moe_set_nccl_comm: ") + ffai_moe_last_error(h_));
    }
    std::vector<uint8_t> exportPeerBuffers() {
        std::vector<uint8_t> blob(FFAI_EP_EXPORT_BYTES);
        int rc = ffai_moe_ep_export(h_, blob.data());
        if (rc != FFAI_OK) throw Error(rc, std::string("ffai_moe_ep_export: ") + ffai_moe_last_error(h_));
        return blob;
    }
    void importPeerBuffers(const std::vector<uint8_t>& allBlobs) {
        if (allBlobs.empty() || allBlobs.size() % FFAI_EP_EXPORT_BYTES != 0)
            throw Error(FFAI_ERR_INVALID_ARG, "MoELayer.importPeerBuffers: expected ep_world blobs of FFAI_EP_EXPORT_BYTES");
        int rc = ffai_moe_ep_import(h_, allBlobs.data());
        if (rc != FFAI_OK) throw Error(rc, std::string("ffai_moe_ep_import: ") + ffai_moe_last_error(h_));
    }
    void releasePeerBuffers() {
        int rc = ffai_moe_ep_release(h_);
        if (rc != FFAI_OK) throw Error(rc, std::string("ffai_moe_ep_release: ") + ffai_moe_last_error(h_));
    }
    // This rank sits out one step of the peer-memory exchange: its step counter moves on without a forward.
    void skipPeerStep() {
        int rc = ffai_moe_ep_skip_step(h_);
        if (rc != FFAI_OK) throw Error(rc, std::string("ffai_moe_ep_skip_step: ") + ffai_moe_last_error(h_));
    }
    // Reads the device error word the bounded waits of the kernels write (0 = none).
    void checkDeviceStatus() {
        int rc = ffai_moe_check_device_status(h_);
        if (rc != FFAI_OK) throw Error(rc, std::string("device status: ") + ffai_moe_last_error(h_));
    }

    ffai_moe_layer* handle() const { return h_; }

  private:
    [[noreturn]] void fail(int rc, const char* where) {
        std::string msg = std::string(where) + ": " + ffai_status_string(rc);
        if (h_) { msg += ": "; msg += ffai_moe_last_error(h_); ffai_moe_destroy(h_); h_ = nullptr; }
        throw Error(rc, msg);
    }
    ffai_moe_layer* h_ = nullptr;
};

// The reference's other two block types are parameterisations of the same layer object here:
// GPTOSSMoELayer (GPTOSSText.swift:1246-1392: softmax over the selected logits, clamped SwiGLU, biased
// router and expert rows) and Qwen35MoEFFN (Qwen3xText.swift:928-1103: softmax-then-top-k, SwiGLU, a
// sigmoid-gated shared expert) differ only in the config fields, so they share the call surface.
using GPTOSSMoELayer = MoELayer;
using Qwen35MoEFFN = MoELayer;

// Ops.* — operator-level calls named as in Sources/FFAI/Ops/Ops.swift; device pointers, the command
// buffer argument becomes the stream.  Shape violations the reference traps on come back as Error.
namespace Ops {
inline void check(int rc, const char* what) {
    if (rc != FFAI_OK) throw Error(rc, std::string(what) + ": " + ffai_status_string(rc));
}
// Ops.moeRouterTopKMany — Ops.swift:2598-2661
inline void moeRouterTopK(const float* logits, uint32_t* indices, float* weights, int nTokens, const MoERouter& r,
                          void* stream) {
    check(ffai_op_moe_router_topk(logits, indices, weights, nTokens, r.nExperts, r.topK, (int)r.gatingMode,
                                  r.normTopKProb ? 1 : 0, nullptr, stream), "Ops.moeRouterTopK");
}
// Ops.gather — Ops.swift:308-346
inline void gather(const uint16_t* table, const uint32_t* ids, uint16_t* out, int nRows, int rowLen, void* stream) {
    check(ffai_op_gather_rows(table, ids, out, nRows, rowLen, stream), "Ops.gather");
}
// Ops.dequantGemv — Ops.swift:1489-1693
inline void dequantGemv(const uint16_t* x, const uint32_t* weight, const uint16_t* scales, const uint16_t* biases,
                        uint16_t* out, int outDim, int inDim, int bits, int groupSize, void* stream) {
    check(ffai_op_dequant_gemv(x, weight, scales, biases, out, outDim, inDim, bits, groupSize, stream), "Ops.dequantGemv");
}
// Ops.moeGatherDequantGemmInt4 — Ops.swift:4553-4708
inline void moeGatherDequantGemm(const uint16_t* x, const uint32_t* weight, const uint16_t* scales,
                                 const uint16_t* biases, const uint32_t* indices, uint16_t* out, int mTotal, int nOut,
                                 int kIn, int nExperts, int bits, int groupSize, void* stream) {
    check(ffai_op_moe_gather_dequant_gemm(x, weight, scales, biases, indices, out, mTotal, nOut, kIn, nExperts, bits,
                                          groupSize, stream), "Ops.moeGatherDequantGemm");
}
// Ops.moeUnpermute — Ops.swift:5030-5110
inline void moeUnpermute(const uint16_t* expertOut, const uint32_t* invPerm, const float* weights, uint16_t* out,
                         int nTokens, int hidden, int k, void* stream) {
    check(ffai_op_moe_unpermute(expertOut, invPerm, weights, out, nTokens, hidden, k, stream), "Ops.moeUnpermute");
}
// Ops.addAndRmsNorm — Ops.swift:658-760
inline void addAndRmsNorm(const uint16_t* a, const uint16_t* b, const uint16_t* weight, float eps, int nRows, int n,
                          uint16_t* residualOut, uint16_t* normedOut, void* stream) {
    check(ffai_op_add_rmsnorm(a, b, weight, eps, nRows, n, residualOut, normedOut, stream), "Ops.addAndRmsNorm");
}
}  // namespace Ops

}  // namespace ffai_host
