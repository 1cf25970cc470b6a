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
enum class MoEGatingMode { softmaxThenTopK = FFAI_GATING_SOFTMAX_THEN_TOPK, topKThenSoftmax = FFAI_GATING_TOPK_THEN_SOFTMAX };

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
    ffai_moe_layer* handle() const { return h_; }

  private:
    [[noreturn]] void fail(int rc, const char* where) {
        std::string msg = std::string(where) + ": " + ffai_status_string(rc);
        if (h_) { msg += ": "; msg += ffai_moe_last_error(h_); ffai_moe_destroy(h_); h_ = nullptr; }
        throw Error(rc, msg);
    }
    ffai_moe_layer* h_ = nullptr;
};

}  // namespace ffai_host
