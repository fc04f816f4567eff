/*
 * puter_b200.h — C ABI of libputer_b200.so, a Blackwell (sm_100a) implementation of
 * puter's LLM-execution hot path: attention (prefill, paged decode), RoPE, RMSNorm
 * (+ fused residual / gated residual), SwiGLU/GELU activations and the dtype converters.
 *
 * The library is what a Go `device.Backend` binds over cgo.  Handle types, the status
 * struct, dtype / op enums and the `cuda_dispatch_*` names and argument orders are the
 * ones of the reference CUDA bridge (device/cuda/internal/bridge/core.h), so the
 * reference's Go wrappers (device/cuda/<family>/dispatch_cuda.go) bind unchanged.
 * Each declaration cites the reference interface it replaces (paths relative to the
 * reference project root).  Entry points marked NEW have no counterpart in the
 * reference's C bridge; they back `device.Backend` methods or execution intrinsics
 * the reference only implements on CPU or Metal.
 *
 * Conventions (reference: core.h:21-24, status.c:5-27, runtime.c):
 *   - every call returns 0 on success or a negative code and fills `status`
 *     (-1 no device/context, -2 nil buffer / bad argument, -6 unknown dtype or
 *     unsupported combination, -7 launch / memcpy / driver failure);
 *   - buffers are opaque `CUDABufferRef` handles owned by the caller; the callee keeps
 *     no pointer beyond the call; zero-sized problems are silent no-ops;
 *   - launches are stream-ordered on the context's default stream and do not
 *     synchronise; `cuda_stream_synchronize` is the explicit fence;
 *   - `completionToken` is accepted and ignored, as in the reference;
 *   - there is no CPU fallback: without a CUDA device every call fails with -1.
 */
#ifndef PUTER_B200_H
#define PUTER_B200_H

#include <stddef.h>
#include <stdint.h>

#define CUDA_STATUS_MESSAGE_BYTES 1024

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with -fvisibility=hidden; these are its exports */
#endif

/* ---- handles, status, enums: device/cuda/internal/bridge/core.h:14-70 ---- */
typedef void* CUDADeviceRef;
typedef void* CUDABufferRef;
typedef void* CUDAStreamRef;

typedef struct CUDAStatus {
    int code;
    char message[CUDA_STATUS_MESSAGE_BYTES];
} CUDAStatus;

typedef enum CUDAElementDType {
    CUDAElementDTypeFloat32 = 0,
    CUDAElementDTypeFloat16 = 1,
    CUDAElementDTypeBFloat16 = 2,
    CUDAElementDTypeFloat64 = 3,
    CUDAElementDTypeFloat8E4M3 = 4,
    CUDAElementDTypeFloat8E5M2 = 5,
} CUDAElementDType;

/* CUDAUnaryFloat32Op (core.h:35-70).  Implemented: every activation of device.Activation (device/interface.go:18-74) that has a
   code here; the plain math codes 1-7, 10, 11 (Abs .. Cos) belong to another op family and return -6. */
typedef enum CUDAUnaryFloat32Op {
    CUDAUnaryFloat32Relu = 0,
    CUDAUnaryFloat32Exp = 8,
    CUDAUnaryFloat32Log = 9,
    CUDAUnaryFloat32Tanh = 12,
    CUDAUnaryFloat32Sigmoid = 13,
    CUDAUnaryFloat32Silu = 14,
    CUDAUnaryFloat32Swish = 15,
    CUDAUnaryFloat32Softsign = 16,
    CUDAUnaryFloat32ELU = 17,
    CUDAUnaryFloat32SELU = 18,
    CUDAUnaryFloat32LeakyReLU = 19,
    CUDAUnaryFloat32HardSigmoid = 20,
    CUDAUnaryFloat32HardSwish = 21,
    CUDAUnaryFloat32Gelu = 22,
    CUDAUnaryFloat32Log1p = 23,
    CUDAUnaryFloat32Expm1 = 24,
    CUDAUnaryFloat32CELU = 25,
    CUDAUnaryFloat32Softplus = 26,
    CUDAUnaryFloat32Mish = 27,
    CUDAUnaryFloat32LogSigmoid = 28,
    CUDAUnaryFloat32GeluTanh = 29,
    CUDAUnaryFloat32HardTanh = 30,
    CUDAUnaryFloat32HardGelu = 31,
    CUDAUnaryFloat32QuickGelu = 32,
    CUDAUnaryFloat32TanhShrink = 33,
} CUDAUnaryFloat32Op;

/* device/cuda/elementwise/arithmetic.h */
typedef enum CUDABinaryFloat32Op {
    CUDABinaryFloat32Add = 0,
    CUDABinaryFloat32Sub = 1,
    CUDABinaryFloat32Mul = 2,
    CUDABinaryFloat32Div = 3,
    CUDABinaryFloat32Max = 4,
    CUDABinaryFloat32Min = 5,
} CUDABinaryFloat32Op;

/* variant codes of cuda_dispatch_multi_head_attention (device/cuda/attention/native/multihead.c:50-66) */
typedef enum CUDAAttentionVariant {
    CUDAAttentionVariantMultiHead = 0,
    CUDAAttentionVariantGroupedQuery = 1,
    CUDAAttentionVariantSlidingWindow = 2,
} CUDAAttentionVariant;

void cuda_status_clear(CUDAStatus* status);                              /* core.h:72 */
void cuda_status_set(CUDAStatus* status, int code, const char* message); /* core.h:74 */

/* ---- runtime: device/cuda/bridge_real.go:11-21, internal/bridge/runtime.c, core_private.h:85-97 ---- */
int cuda_open_device(CUDADeviceRef* outDevice, CUDAStatus* status); /* runtime.c:18 (device 0) */
/* NEW: one context per GPU ordinal (the reference hard-codes cudaSetDevice(0), runtime.c:36) */
int cuda_open_device_index(int ordinal, CUDADeviceRef* outDevice, CUDAStatus* status);
void cuda_close_device(CUDADeviceRef device);                         /* runtime.c:68 */
long long cuda_device_total_memory(CUDADeviceRef device);             /* runtime.c:90 */
int cuda_device_capability_major(CUDADeviceRef device);               /* runtime.c:105 */
CUDABufferRef cuda_buffer_alloc(CUDADeviceRef device, long long bytes); /* runtime.c:120 */
void cuda_buffer_release(CUDABufferRef buffer);                       /* runtime.c:138 */
void* cuda_buffer_device_ptr(CUDABufferRef buffer);                   /* runtime.c:152 */
/* NEW: non-owning handle over device memory allocated elsewhere (a framework's allocator);
   release frees only the handle */
CUDABufferRef cuda_buffer_wrap(CUDADeviceRef device, void* devicePtr, long long bytes);
int cuda_memcpy_async_h2d(CUDABufferRef dst, const void* src, long long bytes, CUDAStreamRef stream, CUDAStatus* status); /* runtime.c:162 */
int cuda_memcpy_async_d2h(void* dst, CUDABufferRef src, long long bytes, CUDAStreamRef stream, CUDAStatus* status);       /* runtime.c:184 */
int cuda_memcpy_async_d2d(CUDABufferRef dst, CUDABufferRef src, long long bytes, CUDAStreamRef stream, CUDAStatus* status); /* runtime.c:206 */
int cuda_stream_synchronize(CUDAStreamRef stream, CUDAStatus* status); /* runtime.c:235 */
CUDADeviceRef cuda_default_context(void);                             /* runtime.c:244 */
CUDAStreamRef cuda_context_upload_stream(CUDADeviceRef device);       /* runtime.c:248 */
CUDAStreamRef cuda_context_default_stream(CUDADeviceRef device);      /* core_private.h:97 */
/* NEW: sharing one allocation between the per-GPU processes of a box (CUDA IPC), for the kernels below that write their
   results straight into the peers' gathered tensors.  export fills a 64-byte handle for a buffer from cuda_buffer_alloc;
   import maps the peer's allocation into this process (release unmaps it).  Peer access is enabled on first use. */
int cuda_buffer_ipc_export(CUDABufferRef buffer, void* outHandle64, CUDAStatus* status);
CUDABufferRef cuda_buffer_ipc_import(CUDADeviceRef device, const void* handle64, long long bytes, CUDAStatus* status);
/* NEW: launch on a stream owned by the embedding framework; NULL is the legacy default stream (stream 0) */
int cuda_context_set_stream(CUDADeviceRef device, void* cudaStream, CUDAStatus* status);
/* NEW: go back to the context's own non-blocking stream */
int cuda_context_reset_stream(CUDADeviceRef device, CUDAStatus* status);
/* NEW: 1 = always use the kernels that reproduce device/cpu operation order exactly
   (sequential sums); 0 (default) = use the tensor-core / split-KV kernels where they apply */
int cuda_context_set_exact(CUDADeviceRef device, int exact, CUDAStatus* status);
/* NEW: synchronises the context's stream, returns the device-side error flag in *outFlag and clears it:
   1 = some call since the last read met an out-of-range page id / offset or an over-long context and skipped it;
   3 = a bounded wait on a row copy ran out (row-pipeline kernels); 4 = a bounded wait between the CTAs of a paged decode
   step ran out (an owner of a split sequence never arrived): the outputs of that call are not valid */
int cuda_context_take_error(CUDADeviceRef device, int* outFlag, CUDAStatus* status);
/* NEW: number of kernels this context has launched (diagnostics / benchmarks) */
unsigned long long cuda_context_launch_count(CUDADeviceRef device);
/* NEW: page-locked host staging memory for Upload/Download paths */
void* cuda_host_alloc(long long bytes);
void cuda_host_free(void* ptr);

/* ---- converters: convert package (convert/bf16_f32.go:11-22, f16_f32.go:10-20, fp8_f32.go:8-65);
        device-side cast for execution/shape_cast_intrinsic.go:57-114 ---- */
/* NEW: dst[i] = cast(src[i]); one side must be Float32.  Bit rules: RNE narrowing, fp8 saturating,
   exact widening; NaN handling is documented in convert.cu. */
int cuda_dispatch_convert(CUDADeviceRef contextRef, int srcDType, int dstDType, CUDABufferRef srcRef, CUDABufferRef dstRef,
                          uint64_t count, uint64_t completionToken, CUDAStatus* status);
/* NEW: the convert package's own shape — caller-owned HOST slices of equal length; chunks are staged
   through pinned memory and overlapped (H2D, kernel, D2H).  srcCount != dstCount -> -2 (ErrLenMismatch,
   convert/errors.go:10-15).  Synchronous on return. */
int cuda_convert_host(CUDADeviceRef contextRef, int srcDType, int dstDType, const void* srcHost, uint64_t srcCount,
                      void* dstHost, uint64_t dstCount, CUDAStatus* status);

/* ---- elementwise / activations ---- */
/* device/cuda/activation/standard.h (device.Activation.Silu/Gelu/GeluTanh, device/interface.go:59,29,30) */
int cuda_dispatch_unary_elementwise(CUDADeviceRef contextRef, int operation, int elementDType, CUDABufferRef inputRef,
                                    CUDABufferRef outRef, uint32_t count, uint64_t completionToken, CUDAStatus* status);
/* device/cuda/elementwise/arithmetic.h (device.Elementwise.Add, device/interface.go:219) */
int cuda_dispatch_binary_elementwise(CUDADeviceRef contextRef, int operation, int elementDType, CUDABufferRef leftRef,
                                     CUDABufferRef rightRef, CUDABufferRef outRef, uint32_t count, uint64_t completionToken,
                                     CUDAStatus* status);
/* device/cuda/activation/gated.h (device.Activation.SwiGLUTensors / SwiGLU, device/interface.go:68-69);
   packed: `inner` = half row length, `count` = rows (Go passes halfCount, batch: compute_host.go:1215-1231) */
#define PUTER_DECLARE_GATED(name)                                                                                         \
    int cuda_dispatch_##name(CUDADeviceRef contextRef, int elementDType, CUDABufferRef destinationRef, CUDABufferRef gateRef, \
                             CUDABufferRef upRef, uint32_t count, uint64_t completionToken, CUDAStatus* status);           \
    int cuda_dispatch_##name##_packed(CUDADeviceRef contextRef, int elementDType, CUDABufferRef destinationRef,            \
                                      CUDABufferRef packedRef, uint32_t inner, uint32_t count, uint64_t completionToken,    \
                                      CUDAStatus* status);
PUTER_DECLARE_GATED(swiglu)
PUTER_DECLARE_GATED(geglu)
PUTER_DECLARE_GATED(glu)
PUTER_DECLARE_GATED(reglu)
PUTER_DECLARE_GATED(siglu)
PUTER_DECLARE_GATED(geglu_tanh)
PUTER_DECLARE_GATED(seglu)
PUTER_DECLARE_GATED(linglu)
#undef PUTER_DECLARE_GATED
/* device/cuda/activation/softmax.h:10-19 (device.Activation.Softmax, device/interface.go:65; CPU device/cpu/math/softmax.go:7-33):
   per row of `cols` elements: max, FastExp32(x - max), sum, multiply by 1 / sum; 16-bit rows are widened, computed in
   float32 and rounded (device/cpu/activation/softmax.go:43-68).  The Go method takes one vector: rows = 1, cols = count. */
int cuda_dispatch_softmax(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t rows,
                          uint32_t cols, uint64_t completionToken, CUDAStatus* status);
/* NEW (CPU-only in the reference): device.Activation.LogSoftmax, device/interface.go:46; device/cpu/math/softmax.go:38-60:
   x - max - FastLog32(sum FastExp32(x - max)) */
int cuda_dispatch_log_softmax(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t rows,
                              uint32_t cols, uint64_t completionToken, CUDAStatus* status);
/* NEW: gated residual out = residual + modulation[b, set*3*C + 2*C + c] * branch, b = row / rowsPerBatch
   (execution/math_gated_residual_intrinsic.go:11-17,206-223; device kernel only on Metal) */
int cuda_dispatch_gated_residual(CUDADeviceRef contextRef, int elementDType, CUDABufferRef residualRef, CUDABufferRef branchRef,
                                 CUDABufferRef modulationRef, CUDABufferRef outputRef, uint32_t rows, uint32_t lastDim,
                                 uint32_t rowsPerBatch, uint32_t modulationCols, uint32_t set, uint64_t completionToken,
                                 CUDAStatus* status);

/* ---- norms ---- */
/* device/cuda/layernorm/native/layer.c:216-227 (device.LayerNorm.RMSNorm, device/interface.go:373-378) */
int cuda_dispatch_rmsnorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                          CUDABufferRef outputRef, uint32_t rows, uint32_t cols, float epsilon, uint64_t completionToken,
                          CUDAStatus* status);
/* NEW: same with the float64 epsilon of device.RMSNormConfig (device/config.go:82-92) */
int cuda_dispatch_rmsnorm_f64(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                              CUDABufferRef outputRef, uint32_t rows, uint32_t cols, double epsilon, uint64_t completionToken,
                              CUDAStatus* status);
/* device/cuda/layernorm/native/layer.h:14-25, called with a float epsilon by device/cuda/layernorm/dispatch_cuda.go:100-112
   (device.LayerNorm.LayerNorm, device/interface.go:362-366).  The CPU op has no epsilon argument and uses 1e-5
   (device/cpu/layernorm/compute.go:11); epsilon <= 0 selects that value. */
int cuda_dispatch_layernorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                            CUDABufferRef biasRef, CUDABufferRef outputRef, uint32_t rows, uint32_t cols, float epsilon,
                            uint64_t completionToken, CUDAStatus* status);
/* The catalog's fused entry layernorm + add -> layernorm_residual (fusion/catalog.go:183-205; four inputs; ULP bound 2; no CUDA
   kernel in the reference): out = LayerNorm(x, scale, bias) + residual.  The LayerNorm result is rounded to the storage
   type before the add, as the two separate ops would, so fused and unfused results are equal. */
int cuda_dispatch_layernorm_residual(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                                     CUDABufferRef biasRef, CUDABufferRef residualRef, CUDABufferRef outputRef, uint32_t rows,
                                     uint32_t cols, float epsilon, uint64_t completionToken, CUDAStatus* status);
/* NEW (CPU-only in the reference): device.LayerNorm.AdaptiveRMSNorm, device/interface.go:356-361;
   device/cpu/layernorm/compute.go:209-264,387-482.  modulation is [rows / rowsPerBatch, modulationCols] = [scale | shift | ...]. */
int cuda_dispatch_adaptive_rmsnorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef modulationRef,
                                   CUDABufferRef outputRef, uint32_t rows, uint32_t cols, uint32_t rowsPerBatch,
                                   uint32_t modulationCols, double epsilon, uint64_t completionToken, CUDAStatus* status);
/* NEW (CPU-only in the reference): device.LayerNorm.ModulatedLayerNorm, device/interface.go:367-372;
   device/cpu/layernorm/compute.go:266-333,513-570.  The [shift | scale] pair of modulation set `set` starts at column
   set * 3 * cols of the batch's modulation row (device.ModulatedLayerNormConfig, device/config.go:94-109). */
int cuda_dispatch_modulated_layernorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef modulationRef,
                                      CUDABufferRef outputRef, uint32_t rows, uint32_t cols, uint32_t rowsPerBatch,
                                      uint32_t modulationCols, uint32_t set, double epsilon, uint64_t completionToken,
                                      CUDAStatus* status);
/* NEW: fused residual add + RMSNorm (+ gated residual), one pass over the rows:
     h = x + residual;  normOut = RMSNorm(h, scale);  hOut = h (may be NULL);
     gatedOut = h + modulation[...] * branch   (skipped when branchRef == NULL)
   each result rounded to the storage dtype where the unfused ops would round (catalog-style fusion,
   fusion/catalog.go:183-205).
   Aliasing (also for cuda_dispatch_rmsnorm*): an output may be exactly the buffer of x or of residual (an in-place
   residual stream); an output that overlaps them only partly, that overlaps scale, branch or modulation, or that
   overlaps another output is refused with -2. */
int cuda_dispatch_add_rmsnorm_gated_residual(CUDADeviceRef contextRef, int elementDType, CUDABufferRef xRef, CUDABufferRef residualRef,
                                             CUDABufferRef scaleRef, CUDABufferRef branchRef, CUDABufferRef modulationRef,
                                             CUDABufferRef hOutRef, CUDABufferRef normOutRef, CUDABufferRef gatedOutRef, uint32_t rows,
                                             uint32_t cols, double epsilon, uint32_t rowsPerBatch, uint32_t modulationCols,
                                             uint32_t set, uint64_t completionToken, CUDAStatus* status);
/* NEW: the same kernel with the all-gather of its two outputs folded into its stores (config 5 across GPUs).  normAll and
   gatedAll are arrays of `world` (<= 8) handles: entry r is rank r's gathered tensor [world * rows, cols] as mapped into this
   process (cuda_buffer_ipc_import for r != rank).  This rank's rows are written at row offset rank * rows of every one, with
   plain 16-byte stores over NVLink (no TMA, no multicast).  A consumer on another GPU needs a cross-rank barrier after it. */
int cuda_dispatch_add_rmsnorm_gated_residual_gather(CUDADeviceRef contextRef, int elementDType, CUDABufferRef xRef,
                                                    CUDABufferRef residualRef, CUDABufferRef scaleRef, CUDABufferRef branchRef,
                                                    CUDABufferRef modulationRef, const CUDABufferRef* normAll,
                                                    const CUDABufferRef* gatedAll, uint32_t world, uint32_t rank, uint32_t rows,
                                                    uint32_t cols, double epsilon, uint32_t rowsPerBatch, uint32_t modulationCols,
                                                    uint32_t set, uint64_t completionToken, CUDAStatus* status);
/* NEW: SwiGLUTensors with the all-gather of its output folded into the stores: dstAll[r] is rank r's gathered tensor
   [world * count]; this rank's results land at element offset rank * count of every one. */
int cuda_dispatch_swiglu_gather(CUDADeviceRef contextRef, int elementDType, const CUDABufferRef* dstAll, uint32_t world, uint32_t rank,
                                CUDABufferRef gateRef, CUDABufferRef upRef, uint32_t count, uint64_t completionToken, CUDAStatus* status);

/* ---- RoPE ---- */
/* device/cuda/rope/rotate.h:10-28 (device.RoPE.RoPE, device/interface.go:599-604); float parameters as in the reference.
   ropeFactor <= 0 or originalContext == 0 selects no scaling, otherwise Llama-3 scaling. */
int cuda_dispatch_rope(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t seqLen,
                       uint32_t numHeads, uint32_t headDim, uint32_t pairCount, float theta, float ropeFactor, float lowFreqFactor,
                       float highFreqFactor, uint32_t originalContext, uint32_t halfMode, uint32_t positionOffset,
                       uint64_t completionToken, CUDAStatus* status);
/* NEW: float64 parameters of device.RoPEConfig (device/config.go:123-134); scaling 0 none / 1 llama3 */
int cuda_dispatch_rope_f64(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t seqLen,
                           uint32_t numHeads, uint32_t headDim, double baseFreq, int64_t startPosition, uint32_t halfMode,
                           uint32_t scaling, double scalingFactor, double lowFreqFactor, double highFreqFactor,
                           uint32_t originalContext, uint64_t completionToken, CUDAStatus* status);
/* device/cuda/rope/rotate.h:29-40 (device.RoPE.RoPEPairs, f32 only) */
int cuda_dispatch_rope_pairs(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef,
                             CUDABufferRef cosRef, CUDABufferRef sinRef, uint32_t halfDim, uint64_t completionToken,
                             CUDAStatus* status);

/* ---- paged KV (device.Shape.PageWrite/PageGather, device/interface.go:625-635;
        execution/page_intrinsic.go:13-24; no CUDA kernel in the reference) ---- */
/* NEW: storageOffset in elements (layer_index * layer elements).  outputRef == storageRef updates in place.
   Value rows aimed at the same (page, offset) within one call race (the CPU loop keeps the last one). */
int cuda_dispatch_kv_page_write(CUDADeviceRef contextRef, int elementDType, CUDABufferRef storageRef, CUDABufferRef valuesRef,
                                CUDABufferRef pageIDsRef, CUDABufferRef offsetsRef, CUDABufferRef outputRef, uint32_t pageCount,
                                uint32_t pageSize, uint32_t inner, uint32_t valueRows, uint64_t storageOffset,
                                uint64_t completionToken, CUDAStatus* status);
int cuda_dispatch_kv_page_gather(CUDADeviceRef contextRef, int elementDType, CUDABufferRef storageRef, CUDABufferRef pageTableRef,
                                 CUDABufferRef outputRef, uint32_t pageCount, uint32_t pageSize, uint32_t inner, uint32_t outRows,
                                 uint64_t storageOffset, uint64_t completionToken, CUDAStatus* status);
/* NEW: device.Shape.LastToken (device/interface.go:622; CPU device/cpu/shape/ops.go:133-160) and the device hook of the
   shape.last_token intrinsic (execution/shape_intrinsic.go:12-19,489-543): output[b] = input[b, seq - 1, :] for b < batch,
   rows of `hidden` elements.  `seq` is the LIVE sequence length of a possibly larger allocation. */
int cuda_dispatch_last_token(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t batch,
                             uint32_t seq, uint32_t hidden, uint64_t completionToken, CUDAStatus* status);
/* NEW, no single counterpart in the reference: the KV-cache producer step of a decoder layer in one launch.  Equals
   RoPE(k) (device/interface.go RoPE; device/cpu/rope/compute.go:55-193) at the per-row position positions[row], the result
   rounded to elementDType, then, when kvDType is e4m3, the cast of value / scale[kv head] (convert package rules), then
   KVPageWrite (execution/page_intrinsic.go:361-438) of K and of V into pools [pageCount, pageSize, kvHeads * headDim] updated
   in place.  positions, pageIDs and offsets are int32 device arrays of `rows` entries, so placing a new token needs no host
   read (the reference reads the RoPE start position on the host: execution/bind_resolver.go:108-121).  Rows whose page, offset
   or position (>= maxPositions) is out of range are skipped and raise the context's error flag.  kvDType is elementDType
   (f16/bf16) or 4 (e4m3, with kScaleRef / vScaleRef f32 per KV head; otherwise they may be NULL). */
int cuda_dispatch_rope_kv_page_write(CUDADeviceRef contextRef, int elementDType, int kvDType, CUDABufferRef kRef, CUDABufferRef vRef,
                                     CUDABufferRef positionsRef, CUDABufferRef pageIDsRef, CUDABufferRef offsetsRef,
                                     CUDABufferRef kPagesRef, CUDABufferRef vPagesRef, CUDABufferRef kScaleRef, CUDABufferRef vScaleRef,
                                     uint32_t rows, uint32_t kvHeads, uint32_t headDim, uint32_t pageCount, uint32_t pageSize,
                                     uint32_t maxPositions, double baseFreq, uint32_t halfMode, uint32_t scaling, double scalingFactor,
                                     double lowFreqFactor, double highFreqFactor, uint32_t originalContext, uint64_t completionToken,
                                     CUDAStatus* status);

/* ---- attention ---- */
/* device/cuda/attention/multihead.h:10-27 (device.Attention.MultiHeadAttention, device/interface.go:98-103).
   Layout q/out [seqQ, numHeads*headDim], k/v [seqK, kvHeads*headDim]; causal mask is bottom-right
   (key > q + seqK - seqQ masked), as device/cpu/attention/typed_compute.go:166-170. */
int cuda_dispatch_multi_head_attention(CUDADeviceRef contextRef, int elementDType, int variant, CUDABufferRef queryRef,
                                       CUDABufferRef keyRef, CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t seqQ,
                                       uint32_t seqK, uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t windowSize,
                                       uint32_t causal, uint64_t completionToken, CUDAStatus* status);
/* device/cuda/attention/flash.h:10-22 (device.Attention.FlashAttention, single head, non-causal) */
int cuda_dispatch_flash_attention(CUDADeviceRef contextRef, int elementDType, CUDABufferRef queryRef, CUDABufferRef keyRef,
                                  CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t seqQ, uint32_t seqK, uint32_t depth,
                                  uint32_t valueDim, uint64_t completionToken, CUDAStatus* status);
/* NEW: same with FlashAttentionConfig.Causal (device/config.go:278-281; top-left mask, key > row skipped) */
int cuda_dispatch_flash_attention_causal(CUDADeviceRef contextRef, int elementDType, CUDABufferRef queryRef, CUDABufferRef keyRef,
                                         CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t seqQ, uint32_t seqK, uint32_t depth,
                                         uint32_t valueDim, uint32_t causal, uint64_t completionToken, CUDAStatus* status);
/* NEW: batched prefill, RoPE fused into the Q/K load.  q/out [batch, seq, numHeads*headDim], k/v [batch, seq, kvHeads*headDim]
   (bf16 or f16).  Equivalent per batch item to RoPE(q), RoPE(k) (device.RoPE.RoPE, positions startPosition..)
   followed by causal MultiHeadAttention.  ropeMode: 0 interleaved, 1 half, 2 = inputs already rotated. */
int cuda_dispatch_rope_attention_prefill(CUDADeviceRef contextRef, int elementDType, CUDABufferRef queryRef, CUDABufferRef keyRef,
                                         CUDABufferRef valueRef, CUDABufferRef outRef, uint32_t batch, uint32_t seqLen,
                                         uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal, uint32_t ropeMode,
                                         double baseFreq, int64_t startPosition, uint32_t scaling, double scalingFactor,
                                         double lowFreqFactor, double highFreqFactor, uint32_t originalContext,
                                         uint64_t completionToken, CUDAStatus* status);
/* NEW: paged decode attention, one new token per sequence, reading KV pages in place
   (= KVPageGather(K), KVPageGather(V), MultiHeadAttention(seqQ=1, seqK=ctx, causal) per sequence).
     q/out       [batch, numHeads*headDim]                      elementDType (bf16 / f16)
     k/v pages   [pageCount, pageSize, kvHeads*headDim]         kvDType: elementDType, or Float8E4M3 with
                                                                 per-KV-head f32 scales kScale/vScale [kvHeads]
     pageTable   [batch, maxPagesPerSeq] int32, ctxLens [batch] int32
   ctxLens[i] == 0 leaves row i of out untouched.  A page id outside [0,pageCount) is never dereferenced (page 0 is
   read in its place) and a context longer than maxPages*pageSize is cut to that length; either way *errorFlag
   (device int32; NULL = the context's own flag, read with cuda_context_take_error) is set to 1 and the output
   row of that sequence is not valid.
   The step is one kernel, launched cooperatively (at most one CTA per SM, all resident at once) so that the CTAs which
   share a long sequence can wait for one another, bounded, and merge it together; if the device refuses a cooperative
   launch of that size (SMs reserved for other work), or the environment variable PUTER_DECODE_NO_COOPERATIVE is set,
   it is launched plainly and the last CTA to finish a sequence merges it alone.  Same results up to the order of the
   float32 sums. */
int cuda_dispatch_paged_decode_attention(CUDADeviceRef contextRef, int elementDType, int kvDType, CUDABufferRef queryRef,
                                         CUDABufferRef kPagesRef, CUDABufferRef vPagesRef, CUDABufferRef pageTableRef,
                                         CUDABufferRef ctxLensRef, CUDABufferRef kScaleRef, CUDABufferRef vScaleRef,
                                         CUDABufferRef outRef, CUDABufferRef errorFlagRef, uint32_t batch, uint32_t maxPagesPerSeq,
                                         uint32_t pageCount, uint32_t pageSize, uint32_t numHeads, uint32_t kvHeads,
                                         uint32_t headDim, uint64_t completionToken, CUDAStatus* status);

/* No counterpart in the reference.  For callers that cannot allocate device memory when a decode step runs: a
   server whose GPU memory is fully pre-planned and owned by its own arena, code in a latency-critical section that
   cannot afford the device-wide synchronisation hidden in cudaMalloc/cudaFree, or a runtime that forbids driver
   allocations after start-up.  Same operation and arguments as cuda_dispatch_paged_decode_attention, but the
   split-KV scratch is a fixed 8 MiB array that is part of the library image (held by every GPU that loads the
   library until exit) and the call performs no cudaMalloc/cudaFree.  Problems that need more scratch are refused
   with -2 (32 query heads, 148 SMs: batch <= 355).  The first call on a device resolves the array's address;
   make it before any stream capture.  All calls on a GPU share the array: calls that can overlap on the GPU race. */
int cuda_dispatch_paged_decode_attention_noalloc(CUDADeviceRef contextRef, int elementDType, int kvDType, CUDABufferRef queryRef,
                                                 CUDABufferRef kPagesRef, CUDABufferRef vPagesRef, CUDABufferRef pageTableRef,
                                                 CUDABufferRef ctxLensRef, CUDABufferRef kScaleRef, CUDABufferRef vScaleRef,
                                                 CUDABufferRef outRef, CUDABufferRef errorFlagRef, uint32_t batch, uint32_t maxPagesPerSeq,
                                                 uint32_t pageCount, uint32_t pageSize, uint32_t numHeads, uint32_t kvHeads,
                                                 uint32_t headDim, uint64_t completionToken, CUDAStatus* status);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif
