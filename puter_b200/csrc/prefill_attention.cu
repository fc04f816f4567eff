// Placeholder translation unit for the tensor-core prefill kernel (filled in below).
#include "common.cuh"

namespace puter {

bool prefill_supported(int dt, uint32_t seqQ, uint32_t seqK, uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal) {
    (void)dt; (void)seqQ; (void)seqK; (void)numHeads; (void)kvHeads; (void)headDim; (void)causal;
    return false;
}

int launch_prefill(Context* ctx, int dt, const void* q, const void* k, const void* v, void* out, uint32_t batch, uint32_t seqLen,
                   uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal, int ropeMode, const float* ropeTable,
                   CUDAStatus* status) {
    (void)ctx; (void)dt; (void)q; (void)k; (void)v; (void)out; (void)batch; (void)seqLen; (void)numHeads; (void)kvHeads;
    (void)headDim; (void)causal; (void)ropeMode; (void)ropeTable;
    return fail(status, -6, "prefill attention: tensor-core kernel not available for this shape");
}

}  // namespace puter
