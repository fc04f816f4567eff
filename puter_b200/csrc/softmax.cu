// Row softmax and log-softmax: device.Activation.Softmax / LogSoftmax (device/interface.go:65,46).
//
// Reference semantics (device/cpu/math/softmax.go:7-60, device/cpu/activation/softmax.go:17-68), per row:
//   softmax     max = largest element; e[i] = FastExp32(x[i] - max); sum = sum of e[i]; out[i] = e[i] * (1 / sum)
//   log-softmax out[i] = x[i] - max - FastLog32(sum of FastExp32(x[i] - max))
// all in float32; bf16 / f16 rows are widened first and the result rounded once.  The CPU sums left to right, the kernels
// in a tree, so a result can differ in its last float32 bits (tests allow 1e-5 relative, one unit in the last place for the
// 16-bit types).  NaN ordering is the reference's too: the maximum is found with `>`, so a NaN never becomes the maximum.
//
// Rows that can travel as bulk copies go through the per-warp shared-memory row pipeline (row_pipeline.cuh): the row is read
// from HBM once, visited three times in shared memory (max, sum of exponentials, result) and written once.  Other rows take
// one CTA per row with scalar accesses.
#include <math.h>

#include "common.cuh"
#include "row_pipeline.cuh"

namespace puter {

namespace {

template <int DT> struct SPer { static constexpr int kPer = DT == DT_F32 ? 4 : 8; };
// (every 16-bit value here goes through float32 arithmetic before it is stored: the hardware conversions of pack16_arith apply)
template <int DT> __device__ __forceinline__ void s_unpack(const Vec16& v, float* f) {
    if (DT == DT_F32) {
#pragma unroll
        for (int i = 0; i < 4; i++) f[i] = __uint_as_float(v.w[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) unpack16_arith<DT>(v.w[i], f[2 * i], f[2 * i + 1]);
    }
}
template <int DT> __device__ __forceinline__ Vec16 s_pack(const float* f) {
    Vec16 v;
    if (DT == DT_F32) {
#pragma unroll
        for (int i = 0; i < 4; i++) v.w[i] = __float_as_uint(f[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) v.w[i] = pack16_arith<DT>(f[2 * i], f[2 * i + 1]);
    }
    return v;
}

// the reference's running maximum: `if x > max { max = x }` starting from the first element
__device__ __forceinline__ float ref_max(float a, float b) { return b > a ? b : a; }

struct SoftmaxParams {
    const void* in;
    void* out;
    size_t rows, cols;
    int* errorFlag;
};

template <int DT, bool LOG>
__global__ void __launch_bounds__(ROWPIPE_MAX_WARPS * 32) softmax_ring_kernel(SoftmaxParams p, int stages) {
    using T = typename Storage<DT>::type;
    constexpr int PER = SPer<DT>::kPer;
    constexpr int UN = ROWPIPE_UN;  // vectors per lane handled together: independent chains of maxima, exponentials and sums
    extern __shared__ __align__(128) unsigned char ringSmem[];
    const size_t cols = p.cols, nvec = cols / PER, rowBytes = cols * sizeof(T);
    const int lane = threadIdx.x & 31;
    // 16-bit softmax rows: the stage has room for the row's float32 exponentials (cols * 4 bytes); the 16-bit row lands in its
    // upper half and the exponentials are written from the start of the stage.  The exponentials of vector v overwrite the input
    // vectors 2v - nvec and 2v - nvec + 1, which are never beyond v: each round loads its vectors first, then stores.
    constexpr bool WIDE = DT != DT_F32 && !LOG;
    rowpipe::Ring ring(ringSmem, blockDim.x >> 5, stages, rowBytes, p.in, p.rows, WIDE ? cols * 4 : 0, WIDE ? rowBytes : 0);
    for (size_t row = ring.first(); row < p.rows; row = ring.next_row(row)) {
        const unsigned char* stageBase = ring.acquire(p.errorFlag);
        if (!stageBase) return;
        const unsigned char* x = stageBase + (WIDE ? rowBytes : 0);
        float* ex = (float*)const_cast<unsigned char*>(stageBase);
        char* o = (char*)((T*)p.out + row * cols);
        float part[UN];
        const float first = Storage<DT>::widen(*(const T*)x);  // the first element seeds the maximum
#pragma unroll
        for (int u = 0; u < UN; u++) part[u] = first;
        for (size_t v0 = lane; v0 < nvec; v0 += 32 * UN) {
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const size_t v = v0 + 32 * (size_t)u;
                if (v < nvec) {
                    float f[PER];
                    s_unpack<DT>(*(const Vec16*)(x + v * 16), f);
#pragma unroll
                    for (int i = 0; i < PER; i++) part[u] = ref_max(part[u], f[i]);
                }
            }
        }
        float mx = part[0];
#pragma unroll
        for (int u = 1; u < UN; u++) mx = ref_max(mx, part[u]);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) mx = ref_max(mx, __shfl_xor_sync(0xffffffffu, mx, s));
#pragma unroll
        for (int u = 0; u < UN; u++) part[u] = 0.f;
        for (size_t vb = 0; vb < nvec; vb += 32 * UN) {  // the same trip count for every lane: the round has a warp barrier
            const size_t v0 = vb + lane;
            Vec16 in[UN];
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const size_t v = v0 + 32 * (size_t)u;
                if (v < nvec) in[u] = *(const Vec16*)(x + v * 16);
            }
            if (WIDE) __syncwarp();  // every lane has read this round's inputs before any lane overwrites them
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const size_t v = v0 + 32 * (size_t)u;
                if (v < nvec) {
                    float f[PER];
                    s_unpack<DT>(in[u], f);
#pragma unroll
                    for (int i = 0; i < PER; i++) {
                        f[i] = fast_exp32(sub(f[i], mx));
                        part[u] = add(part[u], f[i]);
                    }
                    // the exponentials stay in the stage: the input values are not needed again
                    if (!LOG && DT == DT_F32) *(Vec16*)(const_cast<unsigned char*>(x) + v * 16) = s_pack<DT>(f);
                    if (WIDE) {
                        *(float4*)(ex + v * 8) = make_float4(f[0], f[1], f[2], f[3]);
                        *(float4*)(ex + v * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
                    }
                }
            }
        }
        float sum = part[0];
#pragma unroll
        for (int u = 1; u < UN; u++) sum = add(sum, part[u]);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) sum = add(sum, __shfl_xor_sync(0xffffffffu, sum, s));
        const float k = LOG ? fast_log32(sum) : divf(1.0f, sum);
        for (size_t v0 = lane; v0 < nvec; v0 += 32 * UN) {
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const size_t v = v0 + 32 * (size_t)u;
                if (v < nvec) {
                    float f[PER];
                    if (WIDE) {
                        const float4 a = *(const float4*)(ex + v * 8), b = *(const float4*)(ex + v * 8 + 4);
                        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4 % PER] = b.x; f[5 % PER] = b.y; f[6 % PER] = b.z; f[7 % PER] = b.w;
                    } else {
                        s_unpack<DT>(*(const Vec16*)(x + v * 16), f);
                    }
#pragma unroll
                    for (int i = 0; i < PER; i++) f[i] = LOG ? sub(sub(f[i], mx), k) : mul(f[i], k);
                    st_stream(o + v * 16, s_pack<DT>(f));
                }
            }
        }
        ring.release();
    }
}

// Rows of up to 256 * VPT vectors (4096 columns): one 256-thread block per row, the row widened into registers (16 values per
// thread), every exponential computed once and kept there, the block's NEXT row already in flight.  No shared-memory passes: the
// operator is bound by the instruction count of the reference's polynomial exponential, and three resident blocks per SM (24
// warps) keep the issue slots fuller than the 12-16 warps of the ring kernel, which still serves longer rows.
// Maximum as the reference's loop `if x > max { max = x }` seeded with the row's first element: a NaN never replaces the
// maximum, and a row that STARTS with a NaN keeps it as its maximum.
template <int DT, bool LOG, int VPT>
__global__ void __launch_bounds__(256, 3) softmax_block_kernel(SoftmaxParams p) {
    using T = typename Storage<DT>::type;
    constexpr int PER = SPer<DT>::kPer;
    __shared__ float red[2][2][8];  // [row parity][max | sum][warp]
    __shared__ float firstOf[2];    // [row parity] the row's first element
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t cols = p.cols, nvec = cols / PER;
    bool has[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) has[k] = (size_t)tid + 256 * (size_t)k < nvec;
    Vec16 cur[VPT], nxt[VPT];
    auto fetch = [&](size_t row, Vec16* dst) {
        const char* x = (const char*)((const T*)p.in + row * cols);
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) dst[k] = ld_stream(x + ((size_t)tid + 256 * k) * 16);
    };
    if (blockIdx.x < p.rows) fetch(blockIdx.x, cur);
    int par = 0;
    for (size_t row = blockIdx.x; row < p.rows; row += gridDim.x, par ^= 1) {
        if (row + gridDim.x < p.rows) fetch(row + gridDim.x, nxt);
        float f[VPT][PER];
        float mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                s_unpack<DT>(cur[k], f[k]);
#pragma unroll
                for (int i = 0; i < PER; i++) mx = ref_max(mx, f[k][i]);
            }
        if (tid == 0) firstOf[par] = f[0][0];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) mx = ref_max(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        if (lane == 0) red[par][0][warp] = mx;
        __syncthreads();
        {
            const float* r = red[par][0];
            mx = ref_max(ref_max(ref_max(r[0], r[1]), ref_max(r[2], r[3])), ref_max(ref_max(r[4], r[5]), ref_max(r[6], r[7])));
            const float first = firstOf[par];
            if (first != first) mx = first;  // the reference's running maximum never leaves a leading NaN
        }
        float part[4] = {0.f, 0.f, 0.f, 0.f};
        float e[VPT][PER];
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                if (DT == DT_F32) {
#pragma unroll
                    for (int i = 0; i < PER; i++) e[k][i] = fast_exp32(sub(f[k][i], mx));
                } else {
                    // 16-bit rows: two exponentials at a time on packed fused multiply-adds (the same polynomial and exponent
                    // splice, each Horner step rounded once instead of twice: within one float32 unit in the last place, far
                    // below the rounding of the 16-bit result)
#pragma unroll
                    for (int i = 0; i < PER; i += 2) fast_exp32x2_fused(sub(f[k][i], mx), sub(f[k][i + 1], mx), e[k][i], e[k][i + 1]);
                }
#pragma unroll
                for (int i = 0; i < PER; i++) part[i & 3] = add(part[i & 3], e[k][i]);
            }
        float sum = add(add(part[0], part[1]), add(part[2], part[3]));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) sum = add(sum, __shfl_xor_sync(0xffffffffu, sum, s));
        if (lane == 0) red[par][1][warp] = sum;
        __syncthreads();
        {
            const float* r = red[par][1];
            sum = add(add(add(r[0], r[4]), add(r[2], r[6])), add(add(r[1], r[5]), add(r[3], r[7])));
        }
        const float kk = LOG ? fast_log32(sum) : divf(1.0f, sum);
        char* o = (char*)((T*)p.out + row * cols);
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                float r[PER];
#pragma unroll
                for (int i = 0; i < PER; i++) r[i] = LOG ? sub(sub(f[k][i], mx), kk) : mul(e[k][i], kk);
                st_stream(o + ((size_t)tid + 256 * k) * 16, s_pack<DT>(r));
            }
#pragma unroll
        for (int k = 0; k < VPT; k++) cur[k] = nxt[k];
    }
}

// any alignment, any length: one CTA per row, scalar accesses, the row re-read from memory (L2) in every pass
template <int DT, bool LOG>
__global__ void __launch_bounds__(256) softmax_scalar_kernel(SoftmaxParams p) {
    using T = typename Storage<DT>::type;
    __shared__ float red[32];
    auto block_reduce = [&](float v, bool isMax) {
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, v, s);
            v = isMax ? ref_max(v, o) : add(v, o);
        }
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        __syncthreads();
        if (lane == 0) red[warp] = v;
        __syncthreads();
        float t = red[0];
        for (int w = 1; w < nw; w++) t = isMax ? ref_max(t, red[w]) : add(t, red[w]);
        return t;
    };
    for (size_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T* x = (const T*)p.in + row * p.cols;
        T* o = (T*)p.out + row * p.cols;
        float mx = Storage<DT>::load(x, 0);
        for (size_t i = threadIdx.x; i < p.cols; i += blockDim.x) mx = ref_max(mx, Storage<DT>::load(x, i));
        mx = block_reduce(mx, true);
        float sum = 0.f;
        for (size_t i = threadIdx.x; i < p.cols; i += blockDim.x) sum = add(sum, fast_exp32(sub(Storage<DT>::load(x, i), mx)));
        sum = block_reduce(sum, false);
        const float k = LOG ? fast_log32(sum) : divf(1.0f, sum);
        for (size_t i = threadIdx.x; i < p.cols; i += blockDim.x) {
            const float v = Storage<DT>::load(x, i);
            Storage<DT>::store(o, i, LOG ? sub(sub(v, mx), k) : mul(fast_exp32(sub(v, mx)), k));
        }
        __syncthreads();
    }
}

template <bool LOG>
int softmax_entry(CUDADeviceRef contextRef, int dt, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t rows, uint32_t cols,
                  CUDAStatus* status) {
    PUTER_ENTER(ctx);
    if (rows == 0 || cols == 0) return ok(status);
    const char* what = LOG ? "log-softmax" : "softmax";
    if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16) return fail(status, -6, "%s: unsupported dtype %d", what, dt);
    const size_t es = dtype_size(dt);
    PUTER_REQUIRE(inputRef, "input", (size_t)rows * cols * es);
    PUTER_REQUIRE(outRef, "out", (size_t)rows * cols * es);
    SoftmaxParams p{dev_ptr(inputRef), dev_ptr(outRef), rows, cols, ctx->errorFlag};
    const bool vec = ((size_t)cols * es) % 16 == 0 && (((uintptr_t)p.in | (uintptr_t)p.out) & 15u) == 0;
    // (16-bit softmax stages also hold the row's float32 exponentials)
    const rowpipe::Plan plan = vec ? rowpipe::plan((size_t)cols * ((es == 2 && !LOG) ? 4 : es)) : rowpipe::Plan{0, 0, 0};
#define SOFTMAX_LAUNCH(DT)                                                                                                  \
    do {                                                                                                                    \
        constexpr int kVpt = DT == DT_F32 ? 4 : 2;                                                                          \
        const size_t nvecRow = (size_t)cols * es / 16;                                                                      \
        if (vec && nvecRow > 128u * kVpt && nvecRow <= 256u * kVpt) {                                                       \
            const size_t resident = (size_t)ctx->smCount * 3;                                                               \
            softmax_block_kernel<DT, LOG, kVpt><<<(unsigned)(rows < resident ? rows : resident), 256, 0, ctx->stream>>>(p); \
        } else if (plan.warps) {                                                                                                   \
            size_t perSm = (220 * 1024) / (plan.smem + 1024);                                                               \
            perSm = perSm < 1 ? 1 : (perSm > 4 ? 4 : perSm);                                                                \
            size_t blocks = ((size_t)rows + plan.warps - 1) / plan.warps;                                                   \
            if (blocks > (size_t)ctx->smCount * perSm) blocks = (size_t)ctx->smCount * perSm;                               \
            cudaFuncSetAttribute(softmax_ring_kernel<DT, LOG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem); \
            softmax_ring_kernel<DT, LOG><<<(unsigned)blocks, plan.warps * 32, plan.smem, ctx->stream>>>(p, plan.stages);    \
        } else {                                                                                                            \
            size_t blocks = rows, cap = (size_t)ctx->smCount * 8;                                                           \
            softmax_scalar_kernel<DT, LOG><<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(p);            \
        }                                                                                                                   \
    } while (0)
    if (dt == DT_F32) SOFTMAX_LAUNCH(DT_F32);
    else if (dt == DT_BF16) SOFTMAX_LAUNCH(DT_BF16);
    else SOFTMAX_LAUNCH(DT_F16);
#undef SOFTMAX_LAUNCH
    return check_launch(ctx, status, what);
}

}  // namespace

}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_softmax(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t rows,
                                     uint32_t cols, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    return softmax_entry<false>(contextRef, elementDType, inputRef, outRef, rows, cols, status);
}

extern "C" int cuda_dispatch_log_softmax(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef,
                                         uint32_t rows, uint32_t cols, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    return softmax_entry<true>(contextRef, elementDType, inputRef, outRef, rows, cols, status);
}
