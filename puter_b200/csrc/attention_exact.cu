// Attention kernels that reproduce the operation ORDER of the reference CPU implementation, so that the
// float32 path agrees to the last bits and the 16-bit paths reproduce every intermediate rounding.
//
//   MultiHeadAttention  device/cpu/attention/compute.go:70-90, typed_compute.go:142-237, softmax.go:5-85
//       score[k] = dot(q, k) * (1/sqrt(headDim));  f32: dot accumulated in float64 in index order;
//       bf16/f16: dot accumulated in float32 in index order and ROUNDED to the storage type
//       (device/cpu/dot/bf16_generic.go:9-21); causal mask is bottom-right (key > q + seqK - seqQ),
//       sliding window masks q - key >= window; softmax = max, exp through float64, sequential float32 sum,
//       divide; +Inf / all -Inf rows handled as softmax.go:32-73; out[d] = sequential float32 sum over keys.
//   FlashAttention / ScaledDotProductAttention (single head)  typed_compute.go:31-97, select_flash_amd64.go:133-177
//       online softmax, one key at a time, top-left causal mask (key > row skipped), exp = the reference's
//       polynomial FastExp32 with the guards of flash_attention.go:171-189, multiplies and adds unfused.
//
// These are the kernels behind float32 attention and behind every shape the tensor-core / split-KV kernels
// do not cover; they favour exactness over speed: one block per (query row, head), the scores of the row live
// in shared memory, sums over keys are sequential per thread.
#include "common.cuh"

namespace puter {

template <int DT> __device__ __forceinline__ float load_el(const void* p, size_t i) {
    return Storage<DT>::load((const typename Storage<DT>::type*)p, i);
}
template <int DT> __device__ __forceinline__ void store_el(void* p, size_t i, float v) {
    Storage<DT>::store((typename Storage<DT>::type*)p, i, v);
}

// dot of a shared-memory f32 row with a global row, in index order, with the reference's accumulation type
template <int DT> __device__ __forceinline__ float ordered_dot(const float* __restrict__ qs, const void* __restrict__ k, size_t kOff, int n) {
    if (DT == DT_F32) {
        double s = 0.0;
        for (int i = 0; i < n; i++) s = fma((double)qs[i], (double)((const float*)k)[kOff + i], s);  // product exact in f64
        return (float)s;
    }
    float s = 0.f;
    for (int i = 0; i < n; i++) s = fmaf(qs[i], load_el<DT>(k, kOff + i), s);  // product of two 16-bit values is exact in f32
    return Storage<DT>::widen(Storage<DT>::narrow(s));
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    __syncthreads();
    return t;
}

template <int DT>
__global__ void __launch_bounds__(256) mha_exact_kernel(const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                                                       void* __restrict__ out, int seqQ, int seqK, int numHeads, int kvHeads, int headDim,
                                                       int causal, int window, float scale) {
    extern __shared__ float smem[];
    float* scores = smem;               // [seqK]
    float* qs = smem + seqK;            // [headDim]
    __shared__ float red[32];
    __shared__ float sumShared;
    __shared__ int infCount;
    const int qi = blockIdx.x, head = blockIdx.y;
    const int kvHead = head / (numHeads / kvHeads);
    const size_t qStride = (size_t)numHeads * headDim, kvStride = (size_t)kvHeads * headDim;
    const size_t qOff = (size_t)qi * qStride + (size_t)head * headDim;
    const size_t kvOff = (size_t)kvHead * headDim;
    for (int d = threadIdx.x; d < headDim; d += blockDim.x) qs[d] = load_el<DT>(q, qOff + d);
    if (threadIdx.x == 0) infCount = 0;
    __syncthreads();
    const int absq = qi + seqK - seqQ;
    float localMax = -INFINITY;
    bool sawNaN = false;
    for (int ki = threadIdx.x; ki < seqK; ki += blockDim.x) {
        float sc = mul(ordered_dot<DT>(qs, k, (size_t)ki * kvStride + kvOff, headDim), scale);
        if (causal && ki > absq) sc = -INFINITY;
        if (window > 0 && qi - ki >= window) sc = -INFINITY;
        scores[ki] = sc;
        localMax = fmaxf(localMax, sc);
        sawNaN |= (sc != sc);
    }
    (void)sawNaN;
    const float mx = block_max(localMax, red);
    if (isinf(mx)) {
        // softmax.go:32-73: all -Inf -> zeros; +Inf entries share the weight equally
        if (mx > 0) {
            int c = 0;
            for (int ki = threadIdx.x; ki < seqK; ki += blockDim.x) c += (scores[ki] == INFINITY);
            if (c) atomicAdd(&infCount, c);
        }
        __syncthreads();
        float w = (mx > 0 && infCount > 0) ? divf(1.0f, (float)infCount) : 0.0f;
        for (int ki = threadIdx.x; ki < seqK; ki += blockDim.x) scores[ki] = (mx > 0 && scores[ki] == INFINITY) ? w : 0.0f;
        __syncthreads();
    } else {
        for (int ki = threadIdx.x; ki < seqK; ki += blockDim.x) scores[ki] = (float)exp((double)sub(scores[ki], mx));
        __syncthreads();
        if (threadIdx.x == 0) {
            float sum = 0.f;
            for (int ki = 0; ki < seqK; ki++) sum = add(sum, scores[ki]);  // sequential, as SoftmaxRowFillExpsNative
            sumShared = sum;
        }
        __syncthreads();
        const float sum = sumShared;
        if (sum != 0.f)
            for (int ki = threadIdx.x; ki < seqK; ki += blockDim.x) scores[ki] = divf(scores[ki], sum);
        __syncthreads();
    }
    for (int d = threadIdx.x; d < headDim; d += blockDim.x) {
        float acc = 0.f;
        for (int ki = 0; ki < seqK; ki++) acc = add(acc, mul(scores[ki], load_el<DT>(v, (size_t)ki * kvStride + kvOff + d)));
        store_el<DT>(out, qOff + d, acc);
    }
}

__device__ __forceinline__ float flash_exp32(float v) {  // flash_attention.go:171-189
    if (v == -INFINITY || v < -88.0f) return 0.0f;
    if (v == INFINITY) return INFINITY;
    return fast_exp32(v);
}

template <int DT>
__global__ void __launch_bounds__(128) sdpa_exact_kernel(const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                                                        void* __restrict__ out, int seqQ, int seqK, int depth, int valueDim, int causal,
                                                        float scale) {
    extern __shared__ float smem[];
    float* scores = smem;          // [seqK]
    float* qs = smem + seqK;       // [depth]
    const int row = blockIdx.x;
    for (int d = threadIdx.x; d < depth; d += blockDim.x) qs[d] = load_el<DT>(q, (size_t)row * depth + d);
    __syncthreads();
    int limit = causal ? min(seqK, row + 1) : seqK;  // keys with index > row are skipped entirely
    for (int ki = threadIdx.x; ki < limit; ki += blockDim.x) scores[ki] = mul(ordered_dot<DT>(qs, k, (size_t)ki * depth, depth), scale);
    __syncthreads();
    for (int d = threadIdx.x; d < valueDim; d += blockDim.x) {
        float maxScore = -INFINITY, normalizer = 0.f, acc = 0.f;
        for (int ki = 0; ki < limit; ki++) {
            float score = scores[ki];
            float oldMax = maxScore;
            if (score > maxScore) maxScore = score;
            float alpha = flash_exp32(sub(oldMax, maxScore));
            float shifted = flash_exp32(sub(score, maxScore));
            normalizer = add(mul(normalizer, alpha), shifted);
            acc = add(mul(acc, alpha), mul(load_el<DT>(v, (size_t)ki * valueDim + d), shifted));
        }
        float o = 0.f;
        if (normalizer != 0.f) o = mul(acc, divf(1.0f, normalizer));
        store_el<DT>(out, (size_t)row * valueDim + d, o);
    }
}

static const size_t kMaxDynSmem = 227 * 1024 - 1024;

int launch_mha_exact(Context* ctx, int dt, const void* q, const void* k, const void* v, void* out, uint32_t seqQ, uint32_t seqK,
                     uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal, uint32_t window, CUDAStatus* status) {
    size_t smem = ((size_t)seqK + headDim) * sizeof(float);
    if (smem > kMaxDynSmem)
        return fail(status, -6, "attention: exact kernel holds one score row in shared memory; seqK=%u exceeds its limit of %zu keys",
                    seqK, kMaxDynSmem / 4 - headDim);
    float scale = (float)(1.0 / sqrt((double)headDim));
    dim3 grid(seqQ, numHeads);
#define MHA_LAUNCH(DT)                                                                                                   \
    do {                                                                                                                 \
        cudaFuncSetAttribute(mha_exact_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem);       \
        mha_exact_kernel<DT><<<grid, 256, smem, ctx->stream>>>(q, k, v, out, (int)seqQ, (int)seqK, (int)numHeads, (int)kvHeads, \
                                                               (int)headDim, (int)causal, (int)window, scale);           \
    } while (0)
    if (dt == DT_F32) MHA_LAUNCH(DT_F32);
    else if (dt == DT_BF16) MHA_LAUNCH(DT_BF16);
    else if (dt == DT_F16) MHA_LAUNCH(DT_F16);
    else return fail(status, -6, "attention: MultiHeadAttention unsupported dtype");
#undef MHA_LAUNCH
    return check_launch(ctx, status, "multi-head attention (exact)");
}

}  // namespace puter

using namespace puter;

static int flash_entry(CUDADeviceRef contextRef, int dt, CUDABufferRef queryRef, CUDABufferRef keyRef, CUDABufferRef valueRef,
                       CUDABufferRef outRef, uint32_t seqQ, uint32_t seqK, uint32_t depth, uint32_t valueDim, uint32_t causal,
                       CUDAStatus* status) {
    PUTER_ENTER(ctx);
    if (seqQ == 0 || seqK == 0) return ok(status);
    if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16) return fail(status, -6, "attention: ScaledDotProductAttention unsupported dtype");
    size_t es = dtype_size(dt);
    PUTER_REQUIRE(queryRef, "query", (size_t)seqQ * depth * es);
    PUTER_REQUIRE(keyRef, "key", (size_t)seqK * depth * es);
    PUTER_REQUIRE(valueRef, "value", (size_t)seqK * valueDim * es);
    PUTER_REQUIRE(outRef, "out", (size_t)seqQ * valueDim * es);
    size_t smem = ((size_t)seqK + depth) * sizeof(float);
    if (smem > kMaxDynSmem) return fail(status, -6, "attention: flash kernel limit is %zu keys, got %u", kMaxDynSmem / 4 - depth, seqK);
    float scale = (float)(1.0 / sqrt((double)depth));
    const void* q = dev_ptr(queryRef);
    const void* k = dev_ptr(keyRef);
    const void* v = dev_ptr(valueRef);
    void* o = dev_ptr(outRef);
#define SDPA_LAUNCH(DT)                                                                                                   \
    do {                                                                                                                  \
        cudaFuncSetAttribute(sdpa_exact_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem);       \
        sdpa_exact_kernel<DT><<<seqQ, 128, smem, ctx->stream>>>(q, k, v, o, (int)seqQ, (int)seqK, (int)depth, (int)valueDim, (int)causal, scale); \
    } while (0)
    if (dt == DT_F32) SDPA_LAUNCH(DT_F32);
    else if (dt == DT_BF16) SDPA_LAUNCH(DT_BF16);
    else SDPA_LAUNCH(DT_F16);
#undef SDPA_LAUNCH
    return check_launch(ctx, status, "flash attention (exact)");
}

extern "C" int cuda_dispatch_flash_attention(CUDADeviceRef contextRef, int elementDType, CUDABufferRef queryRef, CUDABufferRef keyRef,
                                             CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t seqQ, uint32_t seqK, uint32_t depth,
                                             uint32_t valueDim, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    return flash_entry(contextRef, elementDType, queryRef, keyRef, valueRef, outRef, seqQ, seqK, depth, valueDim, 0, status);
}

extern "C" int cuda_dispatch_flash_attention_causal(CUDADeviceRef contextRef, int elementDType, CUDABufferRef queryRef, CUDABufferRef keyRef,
                                                    CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t seqQ, uint32_t seqK,
                                                    uint32_t depth, uint32_t valueDim, uint32_t causal, uint64_t completionToken,
                                                    CUDAStatus* status) {
    (void)completionToken;
    return flash_entry(contextRef, elementDType, queryRef, keyRef, valueRef, outRef, seqQ, seqK, depth, valueDim, causal, status);
}
