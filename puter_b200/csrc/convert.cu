// dtype converters: bf16 / f16 / fp8(e4m3, e5m2) <-> f32.
//
// Replaces the scalar loops of the reference's convert package (convert/bf16_f32.go:24-38,
// f16_f32.go:28-42, fp8_f32.go:8-65) and the host-side cast of execution/shape_cast_intrinsic.go:57-114.
// Pure HBM streaming: every thread moves 16-byte vectors on the narrow side (8 or 16 elements)
// and the matching 32..64 bytes on the f32 side, read-once data bypasses L1, the grid is a
// multiple of the SM count with a grid-stride loop.
//
// Bit rules (the arithmetic of the reference lives in an external Go module, so these follow the
// in-tree evidence: SIMD macros, Metal kernels, F16C):
//   f32->bf16  round-to-nearest-even; NaN -> (bits >> 16) | 0x0040
//   f32->f16   IEEE round-to-nearest-even, overflow -> Inf; NaN -> sign | 0x7E00 | payload >> 13
//   f32->fp8   saturating round-to-nearest-even (overflow and Inf -> largest finite); NaN -> sign | 0x7F
//   widening   exact; f16/e5m2 NaN keep sign and payload with the quiet bit set; e4m3 0x7F/0xFF -> quiet NaN
#include "common.cuh"

namespace puter {

template <int DT> __device__ __forceinline__ float widen_bits(uint32_t b);
template <> __device__ __forceinline__ float widen_bits<DT_BF16>(uint32_t b) { return bf16_bits_to_f32(b); }
template <> __device__ __forceinline__ float widen_bits<DT_F16>(uint32_t b) { return f16_bits_to_f32(b); }
template <> __device__ __forceinline__ float widen_bits<DT_E4M3>(uint32_t b) { return e4m3_bits_to_f32(b); }
template <> __device__ __forceinline__ float widen_bits<DT_E5M2>(uint32_t b) { return e5m2_bits_to_f32(b); }

template <int DT> __device__ __forceinline__ uint32_t narrow_bits(float f);
template <> __device__ __forceinline__ uint32_t narrow_bits<DT_BF16>(float f) { return f32_to_bf16_bits(f); }
template <> __device__ __forceinline__ uint32_t narrow_bits<DT_F16>(float f) { return f32_to_f16_bits(f); }
template <> __device__ __forceinline__ uint32_t narrow_bits<DT_E4M3>(float f) { return f32_to_e4m3_bits(f); }
template <> __device__ __forceinline__ uint32_t narrow_bits<DT_E5M2>(float f) { return f32_to_e5m2_bits(f); }

template <int DT> struct Narrow { static constexpr int kBytes = (DT == DT_BF16 || DT == DT_F16) ? 2 : 1; };

// narrow -> f32.  Writes dominate (4 output bytes per 1-2 input bytes), so the work is laid out for the stores: a thread
// produces ONE 16-byte output vector from 4 input elements (8 or 4 input bytes), which makes every warp-wide store a
// contiguous 512-byte run; four independent vectors per iteration keep enough loads in flight.
template <int DT>
__global__ void __launch_bounds__(256) widen_kernel(const uint8_t* __restrict__ src, float* __restrict__ dst, size_t n) {
    constexpr int EB = Narrow<DT>::kBytes;
    constexpr int UNROLL = 4;
    const size_t quads = n / 4;  // groups of 4 elements
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; q + (UNROLL - 1) * stride < quads; q += UNROLL * stride) {
        uint32_t lo[UNROLL], hi[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const size_t g = q + u * stride;
            if (EB == 2) {
                asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(lo[u]), "=r"(hi[u]) : "l"(src + g * 8));
            } else {
                asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(lo[u]) : "l"(src + g * 4));
                hi[u] = 0;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            Vec16 out;
            if (EB == 2) {
                out.w[0] = __float_as_uint(widen_bits<DT>(lo[u] & 0xFFFFu));
                out.w[1] = __float_as_uint(widen_bits<DT>(lo[u] >> 16));
                out.w[2] = __float_as_uint(widen_bits<DT>(hi[u] & 0xFFFFu));
                out.w[3] = __float_as_uint(widen_bits<DT>(hi[u] >> 16));
            } else {
                out.w[0] = __float_as_uint(widen_bits<DT>(lo[u] & 0xFFu));
                out.w[1] = __float_as_uint(widen_bits<DT>((lo[u] >> 8) & 0xFFu));
                out.w[2] = __float_as_uint(widen_bits<DT>((lo[u] >> 16) & 0xFFu));
                out.w[3] = __float_as_uint(widen_bits<DT>(lo[u] >> 24));
            }
            st_stream(dst + (q + u * stride) * 4, out);
        }
    }
    for (; q < quads; q += stride) {
        Vec16 out;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t bits = EB == 2 ? ((const uint16_t*)src)[q * 4 + i] : src[q * 4 + i];
            out.w[i] = __float_as_uint(widen_bits<DT>(bits));
        }
        st_stream(dst + q * 4, out);
    }
    // ragged tail (< 4 elements)
    size_t tail = quads * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tail < n) {
        uint32_t bits = EB == 2 ? ((const uint16_t*)src)[tail] : src[tail];
        dst[tail] = widen_bits<DT>(bits);
    }
}

// f32 -> narrow.
template <int DT>
__global__ void __launch_bounds__(256) narrow_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst, size_t n) {
    constexpr int EB = Narrow<DT>::kBytes;
    constexpr int PER = 16 / EB;
    size_t vecs = n / PER;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += stride) {
        const float* s = src + v * PER;
        Vec16 in[PER / 4];
#pragma unroll
        for (int w = 0; w < PER / 4; w++) in[w] = ld_stream(s + 4 * w);
        Vec16 out;
#pragma unroll
        for (int w = 0; w < PER / 4; w++) {
            uint32_t a = narrow_bits<DT>(__uint_as_float(in[w].w[0]));
            uint32_t b = narrow_bits<DT>(__uint_as_float(in[w].w[1]));
            uint32_t c = narrow_bits<DT>(__uint_as_float(in[w].w[2]));
            uint32_t d = narrow_bits<DT>(__uint_as_float(in[w].w[3]));
            if (DT == DT_BF16) {
                out.w[2 * w] = f32x2_to_bf16x2(__uint_as_float(in[w].w[0]), __uint_as_float(in[w].w[1]));
                out.w[2 * w + 1] = f32x2_to_bf16x2(__uint_as_float(in[w].w[2]), __uint_as_float(in[w].w[3]));
            } else if (EB == 2) {
                out.w[2 * w] = a | (b << 16);
                out.w[2 * w + 1] = c | (d << 16);
            } else {
                out.w[w] = a | (b << 8) | (c << 16) | (d << 24);
            }
        }
        st_stream(dst + v * 16, out);
    }
    size_t tail = vecs * PER + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tail < n) {
        uint32_t b = narrow_bits<DT>(src[tail]);
        if (EB == 2) ((uint16_t*)dst)[tail] = (uint16_t)b;
        else dst[tail] = (uint8_t)b;
    }
}

// element-at-a-time variants for buffers that are not 16-byte aligned
template <int DT>
__global__ void widen_scalar_kernel(const uint8_t* __restrict__ src, float* __restrict__ dst, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t b = Narrow<DT>::kBytes == 2 ? ((const uint16_t*)src)[i] : src[i];
        dst[i] = widen_bits<DT>(b);
    }
}
template <int DT>
__global__ void narrow_scalar_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t b = narrow_bits<DT>(src[i]);
        if (Narrow<DT>::kBytes == 2) ((uint16_t*)dst)[i] = (uint16_t)b;
        else dst[i] = (uint8_t)b;
    }
}

static int grid_for(Context* ctx, size_t vecs) {
    size_t blocks = (vecs + 255) / 256;
    size_t cap = (size_t)ctx->smCount * 16;  // 16 resident 256-thread blocks per SM worth of work in flight
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// launches one conversion on `stream`; pointers are device pointers
int launch_convert(Context* ctx, int srcDT, int dstDT, const void* src, void* dst, size_t n, cudaStream_t stream, CUDAStatus* status) {
    if (n == 0) return ok(status);
    bool aligned = (((uintptr_t)src | (uintptr_t)dst) & 15u) == 0;
#define WIDEN(DT)                                                                                                        \
    do {                                                                                                                 \
        if (aligned) {                                                                                                   \
            int g = grid_for(ctx, n / 16 + 256);                                                                         \
            widen_kernel<DT><<<g, 256, 0, stream>>>((const uint8_t*)src, (float*)dst, n);                               \
        } else {                                                                                                         \
            widen_scalar_kernel<DT><<<grid_for(ctx, n), 256, 0, stream>>>((const uint8_t*)src, (float*)dst, n);         \
        }                                                                                                                \
    } while (0)
#define NARROW(DT)                                                                                                       \
    do {                                                                                                                 \
        if (aligned) {                                                                                                   \
            int g = grid_for(ctx, n / (16 / Narrow<DT>::kBytes) + 256);                                                  \
            narrow_kernel<DT><<<g, 256, 0, stream>>>((const float*)src, (uint8_t*)dst, n);                              \
        } else {                                                                                                         \
            narrow_scalar_kernel<DT><<<grid_for(ctx, n), 256, 0, stream>>>((const float*)src, (uint8_t*)dst, n);        \
        }                                                                                                                \
    } while (0)
    if (dstDT == DT_F32) {
        switch (srcDT) {
            case DT_BF16: WIDEN(DT_BF16); break;
            case DT_F16: WIDEN(DT_F16); break;
            case DT_E4M3: WIDEN(DT_E4M3); break;
            case DT_E5M2: WIDEN(DT_E5M2); break;
            case DT_F32:
                if (cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
                    return fail(status, -7, "cuda: convert f32->f32 copy failed");
                return ok(status);
            default: return fail(status, -6, "cuda: convert: unsupported source dtype %d", srcDT);
        }
    } else if (srcDT == DT_F32) {
        switch (dstDT) {
            case DT_BF16: NARROW(DT_BF16); break;
            case DT_F16: NARROW(DT_F16); break;
            case DT_E4M3: NARROW(DT_E4M3); break;
            case DT_E5M2: NARROW(DT_E5M2); break;
            default: return fail(status, -6, "cuda: convert: unsupported destination dtype %d", dstDT);
        }
    } else {
        return fail(status, -6, "cuda: convert: one side must be float32 (got %d -> %d)", srcDT, dstDT);
    }
#undef WIDEN
#undef NARROW
    return check_launch(ctx, status, "convert");
}

}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_convert(CUDADeviceRef contextRef, int srcDType, int dstDType, CUDABufferRef srcRef, CUDABufferRef dstRef,
                                     uint64_t count, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (count == 0) return ok(status);
    size_t ss = dtype_size(srcDType), ds = dtype_size(dstDType);
    if (ss == 0 || ds == 0) return fail(status, -6, "cuda: convert: unknown dtype (%d -> %d)", srcDType, dstDType);
    PUTER_REQUIRE(srcRef, "src", count * ss);
    PUTER_REQUIRE(dstRef, "dst", count * ds);
    return launch_convert(ctx, srcDType, dstDType, dev_ptr(srcRef), dev_ptr(dstRef), count, ctx->stream, status);
}

// Host slices in, host slices out: the shape of the convert package itself.  The input is cut into
// chunks that alternate between two pinned staging buffers and two streams so that the upload of
// chunk i+1, the kernel of chunk i and the download of chunk i-1 overlap.
extern "C" int cuda_convert_host(CUDADeviceRef contextRef, int srcDType, int dstDType, const void* srcHost, uint64_t srcCount,
                                 void* dstHost, uint64_t dstCount, CUDAStatus* status) {
    PUTER_ENTER(ctx);
    if (srcCount != dstCount) return fail(status, -2, "convert: destination length does not match source");
    if (srcCount == 0) return ok(status);
    if (!srcHost || !dstHost) return fail(status, -2, "convert: nil host slice");
    size_t ss = dtype_size(srcDType), ds = dtype_size(dstDType);
    if (ss == 0 || ds == 0 || (srcDType != DT_F32 && dstDType != DT_F32))
        return fail(status, -6, "cuda: convert: unsupported pair (%d -> %d)", srcDType, dstDType);
    const size_t chunk = (size_t)1 << 24;  // elements per chunk (16 Mi)
    size_t per = chunk * (ss + ds);
    char* ws = (char*)ensure_workspace(ctx, 2 * per, status);
    if (!ws) return status ? status->code : -7;
    cudaStream_t streams[2] = {ctx->stream, ctx->uploadStream};
    // the workspace may still be read by work queued earlier on the main stream
    cudaEventRecord(ctx->stageEvents[0], ctx->stream);
    cudaStreamWaitEvent(ctx->uploadStream, ctx->stageEvents[0], 0);
    size_t done = 0;
    int slot = 0;
    // pageable host memory: cudaMemcpyAsync stages internally; pinned callers get true overlap
    while (done < srcCount) {
        size_t n = srcCount - done < chunk ? (size_t)(srcCount - done) : chunk;
        char* dsrc = ws + (size_t)slot * per;
        char* ddst = dsrc + chunk * ss;
        cudaStream_t st = streams[slot];
        if (cudaMemcpyAsync(dsrc, (const char*)srcHost + done * ss, n * ss, cudaMemcpyHostToDevice, st) != cudaSuccess)
            return fail(status, -7, "cuda: convert: upload failed: %s", cudaGetErrorString(cudaGetLastError()));
        int rc = launch_convert(ctx, srcDType, dstDType, dsrc, ddst, n, st, status);
        if (rc != 0) return rc;
        if (cudaMemcpyAsync((char*)dstHost + done * ds, ddst, n * ds, cudaMemcpyDeviceToHost, st) != cudaSuccess)
            return fail(status, -7, "cuda: convert: download failed: %s", cudaGetErrorString(cudaGetLastError()));
        done += n;
        slot ^= 1;
    }
    cudaEventRecord(ctx->stageEvents[1], ctx->uploadStream);
    cudaStreamWaitEvent(ctx->stream, ctx->stageEvents[1], 0);
    cudaError_t e0 = cudaStreamSynchronize(streams[0]);
    cudaError_t e1 = cudaStreamSynchronize(streams[1]);
    if (e0 != cudaSuccess || e1 != cudaSuccess) return fail(status, -7, "cuda: convert: synchronize failed");
    return ok(status);
}
