// turbofieldfare.hpp — C++ host-side mirror of the reference's Swift operator classes over the C ABI.
//
// The reference's host code is Swift (Sources/TurboFieldfare/Kernels/...); where no Swift toolchain exists, this
// header is the host side above turbofieldfare_cuda.h: the same class and method names, the same argument meaning
// ((buffer, byte offset) pairs, a stream where Swift takes a command buffer), and the same error behaviour (a Swift
// `precondition` or `throw` becomes a thrown tf::Error carrying the status and tf_last_error's text). Every method
// is one call into the C ABI; nothing here computes or allocates on the device.
#pragma once

#include <stdexcept>
#include <string>

#include "turbofieldfare_cuda.h"

namespace turbofieldfare {

// SharedExpertError / PrefillMoEGroupingError / PrefillGroupedRoutedMoEError / MetalError in one type:
// `status` tells which (TF_ERR_DIMENSION_MISMATCH, TF_ERR_GROUPING_*, TF_ERR_OUT_OF_MEMORY, TF_ERR_NO_DEVICE, ...).
class Error : public std::runtime_error {
public:
    Error(tf_status s, const std::string& what) : std::runtime_error(what), status(s) {}
    tf_status status;
};

// MetalContext (Infrastructure/Metal/MetalContext.swift:51-214): device + error text; kernels are compiled ahead of time.
class Context {
public:
    explicit Context(int device = 0) {
        const tf_status s = tf_context_create(device, &ctx_);
        if (s != TF_OK) throw Error(s, tf_last_error(nullptr));
    }
    ~Context() { tf_context_destroy(ctx_); }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
    tf_context* handle() const { return ctx_; }
    void check(tf_status s) const { if (s != TF_OK) throw Error(s, tf_last_error(ctx_)); }
    // commandBuffer.waitUntilCompleted() + .error for kernels with bounded waits
    void waitUntilCompleted() const { uint32_t code = 0; check(tf_device_status(ctx_, &code)); }
private:
    tf_context* ctx_ = nullptr;
};

// A buffer + byte offset, the pair every Swift wrapper takes (TensorView, ModelTypes.swift:164-192).
struct BufferRef {
    const void* buffer = nullptr;
    uint64_t offset = 0;
};
struct MutableBufferRef {
    void* buffer = nullptr;
    uint64_t offset = 0;
};

// DequantInt4GEMV (Kernels/Quant/DequantInt4GEMV.swift:44-87)
class DequantInt4GEMV {
public:
    explicit DequantInt4GEMV(const Context& c) : c_(c) {}
    void encode(void* stream, BufferRef weights, BufferRef scales, BufferRef biases, BufferRef x, MutableBufferRef y,
                uint32_t m, uint32_t n, tf_dtype scaleBiasType = TF_BF16) const {
        c_.check(tf_int4_gemv(c_.handle(), stream, weights.buffer, weights.offset, scales.buffer, scales.offset, biases.buffer,
                              biases.offset, x.buffer, x.offset, y.buffer, y.offset, m, n, scaleBiasType));
    }
private:
    const Context& c_;
};

// DequantInt8GEMV (Kernels/Quant/DequantInt8GEMV.swift:50-81)
class DequantInt8GEMV {
public:
    explicit DequantInt8GEMV(const Context& c) : c_(c) {}
    void encode(void* stream, BufferRef weights, BufferRef scales, BufferRef biases, BufferRef x, MutableBufferRef y,
                uint32_t m, uint32_t n, tf_dtype scaleBiasType = TF_BF16) const {
        c_.check(tf_int8_gemv(c_.handle(), stream, weights.buffer, weights.offset, scales.buffer, scales.offset, biases.buffer,
                              biases.offset, x.buffer, x.offset, y.buffer, y.offset, m, n, scaleBiasType));
    }
private:
    const Context& c_;
};

// MoE (Kernels/MoE/MoE.swift:92-295): router and the reference-shaped decode phases over a table of blob pointers.
class MoE {
public:
    explicit MoE(const Context& c) : c_(c) {}
    void encodeRouterGemma4(void* stream, BufferRef weights, BufferRef scales, BufferRef biases, const void* hidden,
                            BufferRef effectiveScale, BufferRef perExpertScale, uint32_t* outIndices, void* outWeights,
                            uint32_t numExperts, uint32_t d, uint32_t topK = TF_MAX_TOP_K) const {
        c_.check(tf_router_gemma4(c_.handle(), stream, weights.buffer, weights.offset, scales.buffer, scales.offset, biases.buffer,
                                  biases.offset, hidden, effectiveScale.buffer, effectiveScale.offset, perExpertScale.buffer,
                                  perExpertScale.offset, outIndices, outWeights, nullptr, numExperts, d, topK));
    }
    void encodeRoutedPersistentPhase1U16Load(void* stream, const void* const* blobTable, const tf_expert_offsets& offsets,
                                             const void* x, void* acts, uint32_t d, uint32_t f, uint32_t topK) const {
        c_.check(tf_moe_phase1(c_.handle(), stream, blobTable, &offsets, x, acts, d, f, topK));
    }
    void encodeRoutedPersistentPhase2Reduce(void* stream, const void* const* blobTable, const tf_expert_offsets& offsets,
                                            const void* acts, const void* routingWeights, const void* residual, void* y,
                                            uint32_t d, uint32_t f, uint32_t topK) const {
        c_.check(tf_moe_phase2_reduce(c_.handle(), stream, blobTable, &offsets, acts, routingWeights, residual, y, d, f, topK));
    }
private:
    const Context& c_;
};

// PrefillRouter (Kernels/Prefill/MoE/PrefillRouter.swift:37-89)
class PrefillRouter {
public:
    explicit PrefillRouter(const Context& c) : c_(c) {}
    void encodeGemma4Block(void* stream, BufferRef weights, BufferRef scales, BufferRef biases, BufferRef hidden,
                           BufferRef effectiveScale, BufferRef perExpertScale, uint32_t* outIndices, void* outWeights,
                           uint32_t queryCount, uint32_t numExperts, uint32_t d, uint32_t topK, uint32_t hiddenStrideElements,
                           tf_dtype hiddenType = TF_FP16) const {
        c_.check(tf_router_gemma4_block(c_.handle(), stream, weights.buffer, weights.offset, scales.buffer, scales.offset,
                                        biases.buffer, biases.offset, hidden.buffer, hidden.offset, hiddenType, effectiveScale.buffer,
                                        effectiveScale.offset, perExpertScale.buffer, perExpertScale.offset, nullptr, outIndices, 0,
                                        outWeights, 0, nullptr, queryCount, numExperts, d, topK, hiddenStrideElements));
    }
private:
    const Context& c_;
};

// PrefillGroupedRoutedMoE (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:386-461) over the HBM-resident pool, with the
// grouping done on the device (PrefillMoEGrouping.groupTokenExpertPairs without the CPU read-back).
class PrefillGroupedRoutedMoE {
public:
    explicit PrefillGroupedRoutedMoE(const Context& c) : c_(c) {}
    void encodeGroupRoutes(void* stream, const uint32_t* indices, const void* weights, uint32_t queryCount, uint32_t topK,
                           uint32_t numExperts, const tf_device_routes& routes) const {
        c_.check(tf_group_routes_device(c_.handle(), stream, indices, weights, queryCount, topK, numExperts, &routes));
    }
    void encodeStreamedBatched(void* stream, BufferRef hidden, uint32_t hiddenStrideElements, const void* poolLayerBase,
                               uint64_t expertStride, const tf_expert_offsets& offsets, const tf_device_routes& routes,
                               void* actsScratch, void* routePartials, bool partialsF32, uint32_t queryCount, uint32_t d,
                               uint32_t f, uint32_t topK) const {
        c_.check(tf_grouped_moe_batched(c_.handle(), stream, hidden.buffer, hidden.offset, hiddenStrideElements, poolLayerBase,
                                        expertStride, &offsets, &routes, actsScratch, routePartials, partialsF32 ? 1 : 0, queryCount,
                                        d, f, topK));
    }
private:
    const Context& c_;
};

// PrefillMoE (Kernels/Prefill/MoE/PrefillMoE.swift:11-39)
class PrefillMoE {
public:
    explicit PrefillMoE(const Context& c) : c_(c) {}
    void encodeReduceTokenMajor(void* stream, const void* routePartials, bool partialsF32, const void* routeWeights, void* h2,
                                uint32_t queryCount, uint32_t topK, uint32_t d) const {
        c_.check(tf_moe_reduce_token_major(c_.handle(), stream, routePartials, partialsF32 ? 1 : 0, routeWeights, nullptr, d, h2, d,
                                           queryCount, topK, d));
    }
private:
    const Context& c_;
};

// PrefillSharedExpert (Kernels/Prefill/MoE/PrefillSharedExpert.swift:11-59)
class PrefillSharedExpert {
public:
    explicit PrefillSharedExpert(const Context& c) : c_(c) {}
    void encodeBlock(void* stream, BufferRef x, uint32_t xStrideElements, const tf_projection& gate, const tf_projection& up,
                     const tf_projection& down, MutableBufferRef y, uint32_t yStrideElements, void* scratchAct, uint32_t rows) const {
        c_.check(tf_shared_expert_int4_block(c_.handle(), stream, x.buffer, x.offset, xStrideElements, &gate, &up, &down, y.buffer,
                                             y.offset, yStrideElements, scratchAct, rows));
    }
private:
    const Context& c_;
};

// MPPPrefillInt4QMM (Kernels/TensorCore/MPPPrefillInt4QMM.swift:34-78): there is no `.unavailable` path here.
class MPPPrefillInt4QMM {
public:
    explicit MPPPrefillInt4QMM(const Context& c) : c_(c) {}
    void encode(void* stream, BufferRef weights, BufferRef scales, BufferRef biases, BufferRef x, MutableBufferRef y,
                uint32_t m, uint32_t n, uint32_t k) const {
        c_.check(tf_int4_qmm(c_.handle(), stream, weights.buffer, weights.offset, scales.buffer, scales.offset, biases.buffer,
                             biases.offset, x.buffer, x.offset, y.buffer, y.offset, m, n, k));
    }
private:
    const Context& c_;
};

// LMHeadChainInt4 (Kernels/Fusions/LMHeadChainInt4.swift:53-135): final RMSNorm, tied int4 LM head, greedy token.
class LMHeadChainInt4 {
public:
    explicit LMHeadChainInt4(const Context& c) : c_(c) {}
    void encodeGreedyDecode(void* stream, BufferRef hidden, BufferRef normWeight, BufferRef weights, BufferRef scales,
                            BufferRef biases, uint32_t* outToken, uint32_t d, uint32_t vocab, float rmsEps = 1e-6f) const {
        c_.check(tf_lm_head_greedy_int4(c_.handle(), stream, hidden.buffer, hidden.offset, normWeight.buffer, normWeight.offset,
                                        weights.buffer, weights.offset, scales.buffer, scales.offset, biases.buffer,
                                        biases.offset, outToken, d, vocab, rmsEps));
    }
private:
    const Context& c_;
};

// FusedPostAttentionSetup (Kernels/Fusions/FusedPostAttentionSetup.swift:26-60) and, with rows and strides,
// PrefillPostAttentionSetup (Kernels/Prefill/Epilogues/PrefillPostAttentionSetup.swift).
class FusedPostAttentionSetup {
public:
    explicit FusedPostAttentionSetup(const Context& c) : c_(c) {}
    void encode(void* stream, void* hidden, const void* attn, void* denseX, void* routedX, void* routerX,
                const void* postAttentionWeight, const void* preFFNWeight, const void* preFFN2Weight, uint32_t d, float eps,
                uint32_t rows = 1, uint32_t strideElements = 0) const {
        const uint32_t st = strideElements ? strideElements : d;
        c_.check(tf_post_attn_setup(c_.handle(), stream, hidden, st, attn, st, denseX, st, routedX, st, routerX, st,
                                    postAttentionWeight, preFFNWeight, preFFN2Weight, rows, d, eps));
    }
private:
    const Context& c_;
};

// ManifestReader + PackedExpertsLayoutReader + ResidentIndexReader in one handle
// (Infrastructure/ModelIO/ManifestReader.swift:64-152, PackedExpertsLayout.swift:57-119, ResidentIndex.swift:44-140):
// opening validates the three documents the way the Swift codecs do; ModelError / GTurboFormatError become Error
// with TF_ERR_FORMAT_* / TF_ERR_IO / TF_ERR_NOT_FOUND. No GPU is needed.
class GTurboDirectory {
public:
    explicit GTurboDirectory(const std::string& directory) {
        const tf_status s = tf_gturbo_open(directory.c_str(), &g_);
        if (s != TF_OK) throw Error(s, tf_last_error(nullptr));
    }
    // decode(data:) of the three codecs, from memory
    GTurboDirectory(const std::string& manifestJSON, const std::string& layoutJSON, const std::string& residentIndex) {
        const tf_status s = tf_gturbo_parse(manifestJSON.data(), manifestJSON.size(), layoutJSON.data(), layoutJSON.size(),
                                            residentIndex.data(), residentIndex.size(), &g_);
        if (s != TF_OK) throw Error(s, tf_last_error(nullptr));
    }
    ~GTurboDirectory() { tf_gturbo_close(g_); }
    GTurboDirectory(const GTurboDirectory&) = delete;
    GTurboDirectory& operator=(const GTurboDirectory&) = delete;
    const tf_gturbo* handle() const { return g_; }
    tf_gturbo_info info() const { tf_gturbo_info i; check(tf_gturbo_get_info(g_, &i)); return i; }
    // Model.routedExpertOffsets(layer:) (Runtime/Inference/ModelExpertIO.swift:21-40)
    tf_expert_offsets routedExpertOffsets(uint32_t layer) const {
        tf_expert_offsets o; check(tf_gturbo_expert_offsets(g_, layer, &o)); return o;
    }
    // PackedExpertsLayout.expert(layer:expert:).offset
    uint64_t expertOffset(uint32_t layer, uint32_t expert) const {
        uint64_t off = 0; check(tf_gturbo_expert_location(g_, layer, expert, nullptr, &off, nullptr, nullptr)); return off;
    }
    // Model.resident(name:) (Runtime/Inference/Model.swift:195-233)
    tf_gturbo_tensor resident(const std::string& name) const {
        tf_gturbo_tensor t; check(tf_gturbo_resident(g_, name.c_str(), &t)); return t;
    }
private:
    static void check(tf_status s) { if (s != TF_OK) throw Error(s, tf_last_error(nullptr)); }
    tf_gturbo* g_ = nullptr;
};

}  // namespace turbofieldfare
