// Entry points of the attention family and the choice of kernel behind each.
//
//   cuda_dispatch_multi_head_attention   device.Attention.MultiHeadAttention (device/interface.go:98-103)
//       float32, sliding window, or cuda_context_set_exact(1)   -> operation-order-exact kernel (attention_exact.cu)
//       bf16/f16, seqQ == 1, head_dim 128, group <= 16           -> split-KV decode kernel over contiguous K/V
//       bf16/f16, causal prefill, head_dim 128                   -> tensor-core prefill kernel (prefill_attention.cu)
//       anything else                                            -> exact kernel
//   cuda_dispatch_rope_attention_prefill  RoPE(q), RoPE(k), causal MultiHeadAttention per batch item, fused
#include <math.h>

#include "common.cuh"

namespace puter {
int launch_mha_exact(Context* ctx, int dt, const void* q, const void* k, const void* v, void* out, uint32_t seqQ, uint32_t seqK,
                     uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal, uint32_t window, CUDAStatus* status);
struct DecodeScratch;
int launch_paged_decode(Context* ctx, int dt, int kvDT, const void* q, const void* kPages, const void* vPages, const int32_t* pageTable,
                        const int32_t* ctxLens, int uniformCtx, const float* kScale, const float* vScale, void* out, int* errorFlag,
                        uint32_t batch, uint32_t maxPages, uint32_t pageCount, uint32_t pageSize, uint32_t numHeads, uint32_t kvHeads,
                        long long seqStrideKV, long long totalTilesHint, const DecodeScratch* fixed, CUDAStatus* status);
bool decode_supported(int dt, int kvDT, uint32_t numHeads, uint32_t kvHeads, uint32_t headDim);
bool prefill_supported(int dt, uint32_t seqQ, uint32_t seqK, uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal);
int launch_prefill(Context* ctx, int dt, const void* q, const void* k, const void* v, void* out, uint32_t batch, uint32_t seqLen,
                   uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal, int ropeMode, const float* ropeTable,
                   CUDAStatus* status);
int validate_rope(CUDAStatus* status, double base, uint32_t halfMode, uint32_t scaling, double factor, double low, double high,
                  uint32_t origCtx);
const float* cached_rope_table(Context* ctx, size_t seqLen, int headDim, double base, long long startPos, int scaling, double factor,
                               double low, double high, int origCtx, CUDAStatus* status);
}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_multi_head_attention(CUDADeviceRef contextRef, int elementDType, int variant, CUDABufferRef queryRef,
                                                  CUDABufferRef keyRef, CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t seqQ,
                                                  uint32_t seqK, uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t windowSize,
                                                  uint32_t causal, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (seqQ == 0 || seqK == 0 || numHeads == 0 || headDim == 0) return ok(status);
    if (kvHeads == 0) kvHeads = numHeads;  // device/cpu/attention/compute.go:37-41
    if (numHeads % kvHeads != 0) return fail(status, -2, "attention: %u heads are not a multiple of %u KV heads", numHeads, kvHeads);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "attention: MultiHeadAttention unsupported dtype");
    if (variant != CUDAAttentionVariantSlidingWindow) windowSize = 0;
    const size_t es = dtype_size(elementDType);
    PUTER_REQUIRE(queryRef, "query", (size_t)seqQ * numHeads * headDim * es);
    PUTER_REQUIRE(keyRef, "key", (size_t)seqK * kvHeads * headDim * es);
    PUTER_REQUIRE(valueRef, "value", (size_t)seqK * kvHeads * headDim * es);
    PUTER_REQUIRE(outRef, "out", (size_t)seqQ * numHeads * headDim * es);
    const void* q = dev_ptr(queryRef);
    const void* k = dev_ptr(keyRef);
    const void* v = dev_ptr(valueRef);
    void* o = dev_ptr(outRef);
    const bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15u) == 0;
    if (!ctx->exact && windowSize == 0 && aligned) {
        if (seqQ == 1 && decode_supported(elementDType, elementDType, numHeads, kvHeads, headDim)) {
            // one sequence, contiguous K/V: the context length travels as a kernel argument
            return launch_paged_decode(ctx, elementDType, elementDType, q, k, v, nullptr, nullptr, (int)seqK, nullptr, nullptr, o, nullptr, 1,
                                       0, (seqK + 15) / 16, 16, numHeads, kvHeads, 0, (long long)((seqK + 15) / 16), nullptr, status);
        }
        if (prefill_supported(elementDType, seqQ, seqK, numHeads, kvHeads, headDim, causal))
            return launch_prefill(ctx, elementDType, q, k, v, o, 1, seqQ, numHeads, kvHeads, headDim, causal, 2, nullptr, status);
    }
    return launch_mha_exact(ctx, elementDType, q, k, v, o, seqQ, seqK, numHeads, kvHeads, headDim, causal, windowSize, status);
}

extern "C" int cuda_dispatch_rope_f64(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef,
                                      uint32_t seqLen, uint32_t numHeads, uint32_t headDim, double baseFreq, int64_t startPosition,
                                      uint32_t halfMode, uint32_t scaling, double scalingFactor, double lowFreqFactor,
                                      double highFreqFactor, uint32_t originalContext, uint64_t completionToken, CUDAStatus* status);

extern "C" int cuda_dispatch_rope_attention_prefill(CUDADeviceRef contextRef, int elementDType, CUDABufferRef queryRef, CUDABufferRef keyRef,
                                                    CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t batch, uint32_t seqLen,
                                                    uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal, uint32_t ropeMode,
                                                    double baseFreq, int64_t startPosition, uint32_t scaling, double scalingFactor,
                                                    double lowFreqFactor, double highFreqFactor, uint32_t originalContext,
                                                    uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (batch == 0 || seqLen == 0 || numHeads == 0 || headDim == 0) return ok(status);
    if (kvHeads == 0) kvHeads = numHeads;
    if (numHeads % kvHeads != 0) return fail(status, -2, "attention: %u heads are not a multiple of %u KV heads", numHeads, kvHeads);
    if (elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "prefill attention: supported dtypes are bf16 and f16 (got %d)", elementDType);
    if (ropeMode > 2) return fail(status, -2, "rope: unsupported mode %u", ropeMode);
    if (ropeMode != 2) {
        int rc = validate_rope(status, baseFreq, ropeMode, scaling, scalingFactor, lowFreqFactor, highFreqFactor, originalContext);
        if (rc != 0) return rc;
        if (headDim % 2 != 0) return fail(status, -2, "rope: head dimension must be even");
    }
    const size_t es = 2;
    const size_t qElems = (size_t)seqLen * numHeads * headDim, kvElems = (size_t)seqLen * kvHeads * headDim;
    PUTER_REQUIRE(queryRef, "query", batch * qElems * es);
    PUTER_REQUIRE(keyRef, "key", batch * kvElems * es);
    PUTER_REQUIRE(valueRef, "value", batch * kvElems * es);
    PUTER_REQUIRE(outRef, "out", batch * qElems * es);
    const char* q = (const char*)dev_ptr(queryRef);
    const char* k = (const char*)dev_ptr(keyRef);
    const char* v = (const char*)dev_ptr(valueRef);
    char* o = (char*)dev_ptr(outRef);
    const bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15u) == 0;

    if (!ctx->exact && aligned && prefill_supported(elementDType, seqLen, seqLen, numHeads, kvHeads, headDim, causal)) {
        const float* table = nullptr;
        if (ropeMode != 2) {
            // scratch for the rotated K; the cos/sin table comes from the context's cache
            if (!ensure_workspace(ctx, batch * kvElems * es + 1024, status)) return status ? status->code : -7;
            table = cached_rope_table(ctx, seqLen, (int)headDim, baseFreq, (long long)startPosition, (int)scaling, scalingFactor,
                                      lowFreqFactor, highFreqFactor, (int)originalContext, status);
            if (!table) return status ? status->code : -7;
        }
        return launch_prefill(ctx, elementDType, q, k, v, o, batch, seqLen, numHeads, kvHeads, headDim, causal, (int)ropeMode, table, status);
    }

    // general path: rotate into scratch with the standalone RoPE kernels, then attend one batch item at a time
    const char* qr = q;
    const char* kr = k;
    CUDABufferRef qTmp = nullptr, kTmp = nullptr;
    if (ropeMode != 2) {
        qTmp = cuda_buffer_alloc(contextRef, (long long)(batch * qElems * es));
        kTmp = cuda_buffer_alloc(contextRef, (long long)(batch * kvElems * es));
        if (!qTmp || !kTmp) {
            cuda_buffer_release(qTmp);
            cuda_buffer_release(kTmp);
            return fail(status, -7, "prefill attention: scratch allocation failed");
        }
        qr = (const char*)dev_ptr(qTmp);
        kr = (const char*)dev_ptr(kTmp);
    }
    int rc = 0;
    for (uint32_t b = 0; b < batch && rc == 0; b++) {
        CUDABufferRef qi = cuda_buffer_wrap(contextRef, (void*)(q + b * qElems * es), (long long)(qElems * es));
        CUDABufferRef ki = cuda_buffer_wrap(contextRef, (void*)(k + b * kvElems * es), (long long)(kvElems * es));
        CUDABufferRef qo = cuda_buffer_wrap(contextRef, (void*)(qr + b * qElems * es), (long long)(qElems * es));
        CUDABufferRef ko = cuda_buffer_wrap(contextRef, (void*)(kr + b * kvElems * es), (long long)(kvElems * es));
        if (ropeMode != 2) {
            rc = cuda_dispatch_rope_f64(contextRef, elementDType, qi, qo, seqLen, numHeads, headDim, baseFreq, startPosition, ropeMode,
                                        scaling, scalingFactor, lowFreqFactor, highFreqFactor, originalContext, 0, status);
            if (rc == 0)
                rc = cuda_dispatch_rope_f64(contextRef, elementDType, ki, ko, seqLen, kvHeads, headDim, baseFreq, startPosition, ropeMode,
                                            scaling, scalingFactor, lowFreqFactor, highFreqFactor, originalContext, 0, status);
        }
        if (rc == 0)
            rc = launch_mha_exact(ctx, elementDType, qr + b * qElems * es, kr + b * kvElems * es, v + b * kvElems * es,
                                  o + b * qElems * es, seqLen, seqLen, numHeads, kvHeads, headDim, causal, 0, status);
        cuda_buffer_release(qi);
        cuda_buffer_release(ki);
        cuda_buffer_release(qo);
        cuda_buffer_release(ko);
    }
    if (qTmp || kTmp) {
        cudaStreamSynchronize(ctx->stream);  // scratch is freed below
        cuda_buffer_release(qTmp);
        cuda_buffer_release(kTmp);
    }
    return rc;
}
