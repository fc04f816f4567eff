// C++ host-side mirror of the hot-path subset of puter's `device.Backend` (device/interface.go) over the C ABI.
//
// The reference's host code is Go; where no Go toolchain is available this header is the compiled-language host side:
// the same method names, argument order and error behaviour as the Go interface.  Void methods throw
// `puter::DeviceError` on failure (the counterpart of the panic in device/cuda/compute_host.go:42-46); zero-sized
// problems are silent no-ops.  Tensor arguments are `DeviceTensor*` whose `DispatchPointer()` is what the dispatcher
// hands to a backend (execution/dispatch.go:616-640); the backend unwraps it to the buffer handle.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/puter_b200.h"

namespace puter {

struct DeviceError : std::runtime_error {
    int code;
    DeviceError(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

// dtype.DType values used on this path, mapped to CUDAElementDType
enum class DType : int { Float32 = 0, Float16 = 1, BFloat16 = 2, Float64 = 3, Float8E4M3 = 4, Float8E5M2 = 5 };

// device/config.go:82-92
struct RMSNormConfig {
    double Epsilon = 1e-5;
};
// device/config.go:94-109
struct ModulatedLayerNormConfig {
    double Epsilon = 1e-6;
    int Set = 0;
};
// device/config.go:111-134
enum class RoPEMode : int { Interleaved = 0, Half = 1 };
enum class RoPEScaling : int { None = 0, Llama3 = 1 };
struct RoPEConfig {
    double BaseFreq = 10000.0;
    int StartPosition = 0;
    RoPEMode Mode = RoPEMode::Interleaved;
    RoPEScaling Scaling = RoPEScaling::None;
    double ScalingFactor = 1.0, LowFreqFactor = 0.0, HighFreqFactor = 0.0;
    int OriginalContext = 0;
};
// device/config.go:278-290
struct FlashAttentionConfig {
    int BlockSize = 64;
    bool Causal = false;
};
struct MultiHeadAttentionConfig {
    int NumHeads = 1, HeadDim = 1;
    bool Causal = false;
    int WindowSize = 0;
    float ALiBiSlope = 0.f;
    int KVHeadCount = 0;
};

class Backend;

// Device-resident tensor: owns (or wraps) one buffer handle.  DispatchPointer() returns the address of this object.
class DeviceTensor {
   public:
    DeviceTensor(CUDADeviceRef ctx, long long bytes) : ref_(cuda_buffer_alloc(ctx, bytes)), bytes_(bytes) {
        if (!ref_ && bytes > 0) throw DeviceError(-7, "cuda: device allocation failed");
    }
    DeviceTensor(CUDADeviceRef ctx, void* devicePtr, long long bytes) : ref_(cuda_buffer_wrap(ctx, devicePtr, bytes)), bytes_(bytes) {}
    DeviceTensor(const DeviceTensor&) = delete;
    DeviceTensor& operator=(const DeviceTensor&) = delete;
    ~DeviceTensor() { cuda_buffer_release(ref_); }
    void* DispatchPointer() { return this; }
    bool ValidDispatchPointer() const { return ref_ != nullptr; }
    CUDABufferRef Ref() const { return ref_; }
    long long Bytes() const { return bytes_; }

   private:
    CUDABufferRef ref_;
    long long bytes_;
};

class Backend {
   public:
    explicit Backend(int ordinal = 0) {
        CUDAStatus st;
        if (cuda_open_device_index(ordinal, &ctx_, &st) != 0) throw DeviceError(st.code, st.message);  // tensor.ErrNeedsPlatformSetup
    }
    Backend(const Backend&) = delete;
    ~Backend() { cuda_close_device(ctx_); }
    CUDADeviceRef Context() const { return ctx_; }

    // tensor.Backend (device/cuda/backend.go:101-234)
    void Upload(DeviceTensor& dst, const void* host, long long bytes) {
        CUDAStatus st;
        check(cuda_memcpy_async_h2d(dst.Ref(), host, bytes, cuda_context_default_stream(ctx_), &st), st);
    }
    void Download(void* host, DeviceTensor& src, long long bytes) {
        CUDAStatus st;
        check(cuda_memcpy_async_d2h(host, src.Ref(), bytes, cuda_context_default_stream(ctx_), &st), st);
        check(cuda_stream_synchronize(cuda_context_default_stream(ctx_), &st), st);
    }
    // batchExecutionDevice (execution/dispatch.go:120-123)
    void BeginBatch() {}
    void EndBatch() {
        CUDAStatus st;
        int flag = 0;
        check(cuda_context_take_error(ctx_, &flag, &st), st);
        if (flag) throw DeviceError(-2, "cuda: a kernel skipped an out-of-range page id, offset or context length");
    }

    // ---- device.Activation ----
    void Silu(void* dst, void* src, int count, DType f) { unary(CUDAUnaryFloat32Silu, dst, src, count, f); }
    void Gelu(void* dst, void* src, int count, DType f) { unary(CUDAUnaryFloat32Gelu, dst, src, count, f); }
    void GeluTanh(void* dst, void* src, int count, DType f) { unary(CUDAUnaryFloat32GeluTanh, dst, src, count, f); }
    void Sigmoid(void* dst, void* src, int count, DType f) { unary(CUDAUnaryFloat32Sigmoid, dst, src, count, f); }
    // the rest of the unary set (device/interface.go:18-74): one bridge op code each
#define PUTER_UNARY_METHOD(Name, Code) \
    void Name(void* dst, void* src, int count, DType f) { unary(Code, dst, src, count, f); }
    PUTER_UNARY_METHOD(ReLU, CUDAUnaryFloat32Relu)
    PUTER_UNARY_METHOD(Tanh, CUDAUnaryFloat32Tanh)
    PUTER_UNARY_METHOD(Exp, CUDAUnaryFloat32Exp)
    PUTER_UNARY_METHOD(Log, CUDAUnaryFloat32Log)
    PUTER_UNARY_METHOD(Log1p, CUDAUnaryFloat32Log1p)
    PUTER_UNARY_METHOD(Expm1, CUDAUnaryFloat32Expm1)
    PUTER_UNARY_METHOD(Swish, CUDAUnaryFloat32Swish)
    PUTER_UNARY_METHOD(Softsign, CUDAUnaryFloat32Softsign)
    PUTER_UNARY_METHOD(ELU, CUDAUnaryFloat32ELU)
    PUTER_UNARY_METHOD(CELU, CUDAUnaryFloat32CELU)
    PUTER_UNARY_METHOD(SELU, CUDAUnaryFloat32SELU)
    PUTER_UNARY_METHOD(LeakyReLU, CUDAUnaryFloat32LeakyReLU)
    PUTER_UNARY_METHOD(HardSigmoid, CUDAUnaryFloat32HardSigmoid)
    PUTER_UNARY_METHOD(HardSwish, CUDAUnaryFloat32HardSwish)
    PUTER_UNARY_METHOD(HardTanh, CUDAUnaryFloat32HardTanh)
    PUTER_UNARY_METHOD(HardGelu, CUDAUnaryFloat32HardGelu)
    PUTER_UNARY_METHOD(QuickGelu, CUDAUnaryFloat32QuickGelu)
    PUTER_UNARY_METHOD(Softplus, CUDAUnaryFloat32Softplus)
    PUTER_UNARY_METHOD(Mish, CUDAUnaryFloat32Mish)
    PUTER_UNARY_METHOD(LogSigmoid, CUDAUnaryFloat32LogSigmoid)
    PUTER_UNARY_METHOD(TanhShrink, CUDAUnaryFloat32TanhShrink)
#undef PUTER_UNARY_METHOD
    void Softmax(void* dst, void* src, int count, DType f) {  // one vector (device/interface.go:65)
        CUDAStatus st;
        check(cuda_dispatch_softmax(ctx_, (int)f, ref(src), ref(dst), 1, (uint32_t)count, 0, &st), st);
    }
    void LogSoftmax(void* dst, void* src, int count, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_log_softmax(ctx_, (int)f, ref(src), ref(dst), 1, (uint32_t)count, 0, &st), st);
    }
    void SeGLUTensors(void* dst, void* gate, void* up, int count, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_seglu(ctx_, (int)f, ref(dst), ref(gate), ref(up), (uint32_t)count, 0, &st), st);
    }
    void LinGLUTensors(void* dst, void* gate, void* up, int count, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_linglu(ctx_, (int)f, ref(dst), ref(gate), ref(up), (uint32_t)count, 0, &st), st);
    }
    void SwiGLU(void* dst, void* packed, int batch, int halfCount, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_swiglu_packed(ctx_, (int)f, ref(dst), ref(packed), (uint32_t)halfCount, (uint32_t)batch, 0, &st), st);
    }
    void SwiGLUTensors(void* dst, void* gate, void* up, int count, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_swiglu(ctx_, (int)f, ref(dst), ref(gate), ref(up), (uint32_t)count, 0, &st), st);
    }
    void GeGLUTensors(void* dst, void* gate, void* up, int count, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_geglu(ctx_, (int)f, ref(dst), ref(gate), ref(up), (uint32_t)count, 0, &st), st);
    }
    // ---- device.Elementwise ----
    void Add(void* dst, void* left, void* right, int count, DType f) { binary(CUDABinaryFloat32Add, dst, left, right, count, f); }
    void Mul(void* dst, void* left, void* right, int count, DType f) { binary(CUDABinaryFloat32Mul, dst, left, right, count, f); }
    // ---- device.LayerNorm ----
    void RMSNorm(RMSNormConfig config, void* input, void* scale, void* output, int rows, int lastDim, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_rmsnorm_f64(ctx_, (int)f, ref(input), ref(scale), ref(output), (uint32_t)rows, (uint32_t)lastDim,
                                        config.Epsilon, 0, &st), st);
    }
    // device.LayerNorm.LayerNorm / AdaptiveRMSNorm / ModulatedLayerNorm (device/interface.go:355-372)
    void LayerNorm(void* input, void* scale, void* bias, void* output, int rows, int lastDim, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_layernorm(ctx_, (int)f, ref(input), ref(scale), ref(bias), ref(output), (uint32_t)rows, (uint32_t)lastDim, 0.0f, 0,
                                      &st), st);
    }
    // the catalog's fused layernorm + add (fusion/catalog.go:183-205)
    void LayerNormResidual(void* input, void* scale, void* bias, void* residual, void* output, int rows, int lastDim, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_layernorm_residual(ctx_, (int)f, ref(input), ref(scale), ref(bias), ref(residual), ref(output), (uint32_t)rows,
                                               (uint32_t)lastDim, 0.0f, 0, &st), st);
    }
    // device.Shape.LastToken (device/interface.go:622) and the shape.last_token device hook (execution/shape_intrinsic.go:12-19)
    void LastToken(void* input, void* output, int batch, int seq, int hidden, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_last_token(ctx_, (int)f, ref(input), ref(output), (uint32_t)batch, (uint32_t)seq, (uint32_t)hidden, 0, &st), st);
    }
    void IntrinsicLastToken(void* input, void* output, int seq, int hiddenBytes, int outBytes, DType f) {
        const int es = (f == DType::Float32) ? 4 : (f == DType::Float64) ? 8 : (f == DType::Float16 || f == DType::BFloat16) ? 2 : 1;
        if (hiddenBytes <= 0) return;
        LastToken(input, output, outBytes / hiddenBytes, seq, hiddenBytes / es, f);
    }
    void AdaptiveRMSNorm(RMSNormConfig config, void* input, void* modulation, void* output, int rows, int lastDim, int rowsPerBatch,
                         int modulationCols, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_adaptive_rmsnorm(ctx_, (int)f, ref(input), ref(modulation), ref(output), (uint32_t)rows, (uint32_t)lastDim,
                                             (uint32_t)rowsPerBatch, (uint32_t)modulationCols, config.Epsilon, 0, &st), st);
    }
    void ModulatedLayerNorm(ModulatedLayerNormConfig config, void* input, void* modulation, void* output, int rows, int lastDim,
                            int rowsPerBatch, int modulationCols, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_modulated_layernorm(ctx_, (int)f, ref(input), ref(modulation), ref(output), (uint32_t)rows, (uint32_t)lastDim,
                                                (uint32_t)rowsPerBatch, (uint32_t)modulationCols, (uint32_t)config.Set, config.Epsilon, 0,
                                                &st), st);
    }
    // gatedResidualDevice (execution/math_gated_residual_intrinsic.go:11-17)
    void GatedResidual(void* residual, void* branch, void* modulation, void* output, int rows, int lastDim, int rowsPerBatch,
                       int modulationCols, int set, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_gated_residual(ctx_, (int)f, ref(residual), ref(branch), ref(modulation), ref(output), (uint32_t)rows,
                                           (uint32_t)lastDim, (uint32_t)rowsPerBatch, (uint32_t)modulationCols, (uint32_t)set, 0, &st), st);
    }
    // ---- device.RoPE ----
    void RoPE(RoPEConfig c, void* input, void* output, int seqLen, int numHeads, int headDim, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_rope_f64(ctx_, (int)f, ref(input), ref(output), (uint32_t)seqLen, (uint32_t)numHeads, (uint32_t)headDim,
                                     c.BaseFreq, c.StartPosition, (uint32_t)c.Mode, (uint32_t)c.Scaling, c.ScalingFactor, c.LowFreqFactor,
                                     c.HighFreqFactor, (uint32_t)c.OriginalContext, 0, &st), st);
    }
    void RoPEPairs(void* output, void* input, void* cosBuffer, void* sinBuffer, int halfDim, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_rope_pairs(ctx_, (int)f, ref(input), ref(output), ref(cosBuffer), ref(sinBuffer), (uint32_t)halfDim, 0, &st), st);
    }
    // ---- pageIntrinsicDevice (execution/page_intrinsic.go:13-24) ----
    void KVPageWrite(void* storage, void* values, void* pageIDs, void* offsets, void* output, int pageCount, int pageSize, int inner,
                     int valueRows, int storageOffset, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_kv_page_write(ctx_, (int)f, ref(storage), ref(values), ref(pageIDs), ref(offsets), ref(output),
                                          (uint32_t)pageCount, (uint32_t)pageSize, (uint32_t)inner, (uint32_t)valueRows,
                                          (uint64_t)storageOffset, 0, &st), st);
    }
    // KV-cache producer: RoPE(k) at positions[row] -> [e4m3 of value / scale] -> KVPageWrite of K and V, one launch (no single
    // reference counterpart; kScale / vScale may be null unless kvFormat is Float8E4M3)
    void RoPEKVPageWrite(RoPEConfig c, void* k, void* v, void* positions, void* pageIDs, void* offsets, void* kPages, void* vPages,
                         void* kScale, void* vScale, int rows, int kvHeads, int headDim, int pageCount, int pageSize, int maxPositions,
                         DType f, DType kvFormat) {
        CUDAStatus st;
        check(cuda_dispatch_rope_kv_page_write(ctx_, (int)f, (int)kvFormat, ref(k), ref(v), ref(positions), ref(pageIDs), ref(offsets),
                                               ref(kPages), ref(vPages), kScale ? ref(kScale) : nullptr, vScale ? ref(vScale) : nullptr, (uint32_t)rows,
                                               (uint32_t)kvHeads,
                                               (uint32_t)headDim, (uint32_t)pageCount, (uint32_t)pageSize, (uint32_t)maxPositions,
                                               c.BaseFreq, (uint32_t)c.Mode, (uint32_t)c.Scaling, c.ScalingFactor, c.LowFreqFactor,
                                               c.HighFreqFactor, (uint32_t)c.OriginalContext, 0, &st), st);
    }
    void KVPageGather(void* storage, void* pageTable, void* output, int pageCount, int pageSize, int inner, int outRows,
                      int storageOffset, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_kv_page_gather(ctx_, (int)f, ref(storage), ref(pageTable), ref(output), (uint32_t)pageCount,
                                           (uint32_t)pageSize, (uint32_t)inner, (uint32_t)outRows, (uint64_t)storageOffset, 0, &st), st);
    }
    // ---- device.Attention ----
    void MultiHeadAttention(MultiHeadAttentionConfig c, void* query, void* key, void* value, void* output, int seqQ, int seqK, DType f) {
        if (c.ALiBiSlope != 0.f) throw DeviceError(-6, "attention: ALiBi is not on this library's path");
        const int kv = c.KVHeadCount > 0 ? c.KVHeadCount : c.NumHeads;  // device/cpu/attention/compute.go:37-41
        const int variant = c.WindowSize > 0 ? CUDAAttentionVariantSlidingWindow
                                             : (kv != c.NumHeads ? CUDAAttentionVariantGroupedQuery : CUDAAttentionVariantMultiHead);
        CUDAStatus st;
        check(cuda_dispatch_multi_head_attention(ctx_, (int)f, variant, ref(query), ref(key), ref(value), ref(output), (uint32_t)seqQ,
                                                 (uint32_t)seqK, (uint32_t)c.NumHeads, (uint32_t)kv, (uint32_t)c.HeadDim,
                                                 (uint32_t)c.WindowSize, c.Causal ? 1u : 0u, 0, &st), st);
    }
    void FlashAttention(FlashAttentionConfig c, void* query, void* key, void* value, void* output, int seqQ, int seqK, int depth,
                        int valueDim, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_flash_attention_causal(ctx_, (int)f, ref(query), ref(key), ref(value), ref(output), (uint32_t)seqQ,
                                                   (uint32_t)seqK, (uint32_t)depth, (uint32_t)valueDim, c.Causal ? 1u : 0u, 0, &st), st);
    }
    void ScaledDotProductAttention(FlashAttentionConfig c, void* q, void* k, void* v, void* o, int seqQ, int seqK, int depth, int valueDim,
                                   DType f) {
        FlashAttention(c, q, k, v, o, seqQ, seqK, depth, valueDim, f);
    }
    void PagedDecodeAttention(MultiHeadAttentionConfig c, void* query, void* kPages, void* vPages, void* pageTable, void* ctxLens,
                              void* kScale, void* vScale, void* output, int batch, int maxPagesPerSeq, int pageCount, int pageSize,
                              DType f, DType kvFormat) {
        const int kv = c.KVHeadCount > 0 ? c.KVHeadCount : c.NumHeads;
        CUDAStatus st;
        check(cuda_dispatch_paged_decode_attention(ctx_, (int)f, (int)kvFormat, ref(query), ref(kPages), ref(vPages), ref(pageTable),
                                                   ref(ctxLens), kScale ? ref(kScale) : nullptr, vScale ? ref(vScale) : nullptr,
                                                   ref(output), nullptr, (uint32_t)batch, (uint32_t)maxPagesPerSeq, (uint32_t)pageCount,
                                                   (uint32_t)pageSize, (uint32_t)c.NumHeads, (uint32_t)kv, (uint32_t)c.HeadDim, 0, &st), st);
    }
    // convert package on device memory (execution/shape_cast_intrinsic.go:57-114)
    void Convert(void* dst, void* src, long long count, DType dstFormat, DType srcFormat) {
        CUDAStatus st;
        check(cuda_dispatch_convert(ctx_, (int)srcFormat, (int)dstFormat, ref(src), ref(dst), (uint64_t)count, 0, &st), st);
    }

   private:
    static CUDABufferRef ref(void* dispatchPointer) {
        if (!dispatchPointer) throw DeviceError(-2, "cuda: nil tensor");
        return static_cast<DeviceTensor*>(dispatchPointer)->Ref();
    }
    static void check(int code, const CUDAStatus& st) {
        if (code != 0) throw DeviceError(st.code, st.message);
    }
    void unary(int op, void* dst, void* src, int count, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_unary_elementwise(ctx_, op, (int)f, ref(src), ref(dst), (uint32_t)count, 0, &st), st);
    }
    void binary(int op, void* dst, void* l, void* r, int count, DType f) {
        CUDAStatus st;
        check(cuda_dispatch_binary_elementwise(ctx_, op, (int)f, ref(l), ref(r), ref(dst), (uint32_t)count, 0, &st), st);
    }
    CUDADeviceRef ctx_ = nullptr;
};

// convert package (convert/bf16_f32.go:11-22, f16_f32.go:10-20, fp8_f32.go:8-65): host slices in, host slices out.
// Returns false for unequal lengths (ErrLenMismatch, convert/errors.go:10-15); throws on device failure.
namespace convert {
inline bool run(Backend& b, DType src, DType dst, const void* s, uint64_t ns, void* d, uint64_t nd) {
    CUDAStatus st;
    int rc = cuda_convert_host(b.Context(), (int)src, (int)dst, s, ns, d, nd, &st);
    if (rc == -2 && ns != nd) return false;
    if (rc != 0) throw DeviceError(st.code, st.message);
    return true;
}
inline bool Float32ToBFloat16(Backend& b, uint16_t* dst, size_t nd, const float* src, size_t ns) { return run(b, DType::Float32, DType::BFloat16, src, ns, dst, nd); }
inline bool BFloat16ToFloat32(Backend& b, float* dst, size_t nd, const uint16_t* src, size_t ns) { return run(b, DType::BFloat16, DType::Float32, src, ns, dst, nd); }
inline bool Float32ToFloat16(Backend& b, uint16_t* dst, size_t nd, const float* src, size_t ns) { return run(b, DType::Float32, DType::Float16, src, ns, dst, nd); }
inline bool Float16ToFloat32(Backend& b, float* dst, size_t nd, const uint16_t* src, size_t ns) { return run(b, DType::Float16, DType::Float32, src, ns, dst, nd); }
inline bool Float32ToFloat8E4M3(Backend& b, uint8_t* dst, size_t nd, const float* src, size_t ns) { return run(b, DType::Float32, DType::Float8E4M3, src, ns, dst, nd); }
inline bool Float8E4M3ToFloat32(Backend& b, float* dst, size_t nd, const uint8_t* src, size_t ns) { return run(b, DType::Float8E4M3, DType::Float32, src, ns, dst, nd); }
inline bool Float32ToFloat8E5M2(Backend& b, uint8_t* dst, size_t nd, const float* src, size_t ns) { return run(b, DType::Float32, DType::Float8E5M2, src, ns, dst, nd); }
inline bool Float8E5M2ToFloat32(Backend& b, float* dst, size_t nd, const uint8_t* src, size_t ns) { return run(b, DType::Float8E5M2, DType::Float32, src, ns, dst, nd); }
}  // namespace convert

}  // namespace puter
