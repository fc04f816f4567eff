// Elementwise hot-path ops: the unary activations of device.Activation (Silu / Gelu / GeluTanh and the other
// 22 that carry a bridge op code), binary arithmetic (Add is the residual add), the eight gated
// activations (SwiGLU & friends, two-tensor and packed) and the gated residual.
//
// Semantics follow the scalar Go code of the reference operation by operation:
//   f32 unary      FastSilu32 / FastGelu32 / FastGeluTanh32 ...   device/cpu/math/f32.go, activation.go:50-57
//   16-bit unary   65536-entry lookup tables built from the f64 variants, exactly like
//                  device/cpu/activation/lut.go:48-61 (here the tables live in device memory)
//   gated          f32 math on widened inputs, RNE store           device/cpu/activation/compute.go:72-176
//   binary 16-bit  widen, f32 op, RNE narrow                       device/cpu/elementwise/uint16_generic.go:148-156
//   gated residual out = res + mod * branch (f32 mul then add)     execution/math_gated_residual_intrinsic.go:206-223
// All kernels stream 16-byte vectors with a grid-stride loop sized in multiples of the SM count.
#include "common.cuh"

namespace puter {

enum : int { G_SWIGLU = 0, G_GEGLU = 1, G_GLU = 2, G_REGLU = 3, G_SIGLU = 4, G_GEGLU_TANH = 5, G_SEGLU = 6, G_LINGLU = 7 };

// every activation of device.Activation that has a code in CUDAUnaryFloat32Op (device/cuda/internal/bridge/core.h:35-70)
#define PUTER_UNARY_OPS(X)                                                                                                   \
    X(CUDAUnaryFloat32Relu) X(CUDAUnaryFloat32Exp) X(CUDAUnaryFloat32Log) X(CUDAUnaryFloat32Tanh) X(CUDAUnaryFloat32Sigmoid)  \
    X(CUDAUnaryFloat32Silu) X(CUDAUnaryFloat32Swish) X(CUDAUnaryFloat32Softsign) X(CUDAUnaryFloat32ELU) X(CUDAUnaryFloat32SELU) \
    X(CUDAUnaryFloat32LeakyReLU) X(CUDAUnaryFloat32HardSigmoid) X(CUDAUnaryFloat32HardSwish) X(CUDAUnaryFloat32Gelu)           \
    X(CUDAUnaryFloat32Log1p) X(CUDAUnaryFloat32Expm1) X(CUDAUnaryFloat32CELU) X(CUDAUnaryFloat32Softplus) X(CUDAUnaryFloat32Mish) \
    X(CUDAUnaryFloat32LogSigmoid) X(CUDAUnaryFloat32GeluTanh) X(CUDAUnaryFloat32HardTanh) X(CUDAUnaryFloat32HardGelu)          \
    X(CUDAUnaryFloat32QuickGelu) X(CUDAUnaryFloat32TanhShrink)

// float32: one math.Fast*32 per element (device/cpu/activation/f32_generic.go:9-222); Swish runs the Silu kernel (ops.go:41-43),
// CELU with its default alpha of 1 is exp(v / 1) - 1 (math/activation.go:84-90)
template <int OP> __device__ __forceinline__ float unary32(float v) {
    if (OP == CUDAUnaryFloat32Relu) return fast_relu32(v);
    if (OP == CUDAUnaryFloat32Exp) return fast_exp32(v);
    if (OP == CUDAUnaryFloat32Log) return fast_log32(v);
    if (OP == CUDAUnaryFloat32Tanh) return fast_tanh32(v);
    if (OP == CUDAUnaryFloat32Sigmoid) return fast_sigmoid32(v);
    if (OP == CUDAUnaryFloat32Silu || OP == CUDAUnaryFloat32Swish) return fast_silu32(v);
    if (OP == CUDAUnaryFloat32Softsign) return fast_softsign32(v);
    if (OP == CUDAUnaryFloat32ELU || OP == CUDAUnaryFloat32CELU) return fast_elu32(v);
    if (OP == CUDAUnaryFloat32SELU) return fast_selu32(v);
    if (OP == CUDAUnaryFloat32LeakyReLU) return fast_leaky_relu32(v);
    if (OP == CUDAUnaryFloat32HardSigmoid) return fast_hard_sigmoid32(v);
    if (OP == CUDAUnaryFloat32HardSwish) return fast_hard_swish32(v);
    if (OP == CUDAUnaryFloat32Gelu) return fast_gelu32(v);
    if (OP == CUDAUnaryFloat32Log1p) return fast_log32(add(1.0f, v));
    if (OP == CUDAUnaryFloat32Expm1) return sub(fast_exp32(v), 1.0f);
    if (OP == CUDAUnaryFloat32Softplus) return fast_softplus32(v);
    if (OP == CUDAUnaryFloat32Mish) return fast_mish32(v);
    if (OP == CUDAUnaryFloat32LogSigmoid) return -fast_softplus32(-v);
    if (OP == CUDAUnaryFloat32GeluTanh) return fast_gelu_tanh32(v);
    if (OP == CUDAUnaryFloat32HardTanh) return fast_hard_tanh32(v);
    if (OP == CUDAUnaryFloat32HardGelu) return fast_hard_gelu32(v);
    if (OP == CUDAUnaryFloat32QuickGelu) return fast_quick_gelu32(v);
    return fast_tanh_shrink32(v);
}
// fill functions of the 16-bit tables (device/cpu/activation/lut.go:14-41); HardGelu, QuickGelu and TanhShrink go through
// their float32 forms (math/extra_activation.go:19-37)
__device__ __forceinline__ double unary64(int op, double v) {
    switch (op) {
        case CUDAUnaryFloat32Relu: return v > 0.0 ? v : 0.0;
        case CUDAUnaryFloat32Exp: return fast_exp64(v);
        case CUDAUnaryFloat32Log: return fast_log64(v);
        case CUDAUnaryFloat32Tanh: return fast_tanh64(v);
        case CUDAUnaryFloat32Sigmoid: return fast_sigmoid64(v);
        case CUDAUnaryFloat32Silu: case CUDAUnaryFloat32Swish: return fast_silu64(v);
        case CUDAUnaryFloat32Softsign: return __ddiv_rn(v, __dadd_rn(1.0, fabs(v)));
        case CUDAUnaryFloat32ELU: case CUDAUnaryFloat32CELU: return v > 0.0 ? v : __dsub_rn(fast_exp64(v), 1.0);
        case CUDAUnaryFloat32SELU:
            return v > 0.0 ? __dmul_rn(1.0507009873554805, v)
                           : __dmul_rn(1.0507009873554805 * 1.6732632423543772, __dsub_rn(fast_exp64(v), 1.0));
        case CUDAUnaryFloat32LeakyReLU: return v > 0.0 ? v : __dmul_rn(0.01, v);
        case CUDAUnaryFloat32HardSigmoid: return fast_hard_sigmoid64(v);
        case CUDAUnaryFloat32HardSwish: return __dmul_rn(v, fast_hard_sigmoid64(__dadd_rn(v, 3.0)));
        case CUDAUnaryFloat32Gelu: return fast_gelu64(v);
        case CUDAUnaryFloat32Log1p: return fast_log64(__dadd_rn(1.0, v));
        case CUDAUnaryFloat32Expm1: return __dsub_rn(fast_exp64(v), 1.0);
        case CUDAUnaryFloat32Softplus: return fast_softplus64(v);
        case CUDAUnaryFloat32Mish: return __dmul_rn(v, fast_tanh64(fast_softplus64(v)));
        case CUDAUnaryFloat32LogSigmoid: return -fast_softplus64(-v);
        case CUDAUnaryFloat32GeluTanh: return fast_gelu_tanh64(v);
        case CUDAUnaryFloat32HardTanh: return v < -1.0 ? -1.0 : (v > 1.0 ? 1.0 : v);
        case CUDAUnaryFloat32HardGelu: return (double)fast_hard_gelu32(f64_to_f32_host(v));
        case CUDAUnaryFloat32QuickGelu: return (double)fast_quick_gelu32(f64_to_f32_host(v));
        default: return (double)fast_tanh_shrink32(f64_to_f32_host(v));
    }
}
// variant asymmetry of the reference (math/activation.go:286-308, extra_activation.go:84-90): SwiGLU/SiGLU/SeGLU activate the
// gate, GLU/GeGLU/ReGLU/GeGLUTanh activate `up`, LinGLU is the plain product.
template <int OP> __device__ __forceinline__ float gated32(float gate, float up) {
    if (OP == G_SWIGLU) return mul(fast_silu32(gate), up);
    if (OP == G_GEGLU) return mul(gate, fast_gelu32(up));
    if (OP == G_GLU) return mul(gate, fast_sigmoid32(up));
    if (OP == G_REGLU) return mul(gate, fast_relu32(up));
    if (OP == G_SIGLU) return mul(fast_sigmoid32(gate), up);
    if (OP == G_SEGLU) return mul(up, fast_sigmoid32(gate));
    if (OP == G_LINGLU) return mul(gate, up);
    return mul(gate, fast_gelu_tanh32(up));
}
template <int OP> __device__ __forceinline__ float binary32(float a, float b) {
    if (OP == CUDABinaryFloat32Add) return add(a, b);
    if (OP == CUDABinaryFloat32Sub) return sub(a, b);
    if (OP == CUDABinaryFloat32Mul) return mul(a, b);
    if (OP == CUDABinaryFloat32Div) return divf(a, b);
    if (OP == CUDABinaryFloat32Max) return a > b ? a : b;
    return a < b ? a : b;
}

// ---- vector helpers: a Vec16 holds 4 f32 or 8 16-bit elements ----
template <int DT> struct Lanes { static constexpr int kPer = DT == DT_F32 ? 4 : 8; };

template <int DT> __device__ __forceinline__ void unpack(const Vec16& v, float* f) {
    if (DT == DT_F32) {
#pragma unroll
        for (int i = 0; i < 4; i++) f[i] = __uint_as_float(v.w[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            f[2 * i] = Storage<DT>::widen((uint16_t)(v.w[i] & 0xFFFFu));
            f[2 * i + 1] = Storage<DT>::widen((uint16_t)(v.w[i] >> 16));
        }
    }
}
template <int DT> __device__ __forceinline__ Vec16 pack(const float* f) {
    Vec16 v;
    if (DT == DT_F32) {
#pragma unroll
        for (int i = 0; i < 4; i++) v.w[i] = __float_as_uint(f[i]);
    } else if (DT == DT_BF16) {
#pragma unroll
        for (int i = 0; i < 4; i++) v.w[i] = f32x2_to_bf16x2(f[2 * i], f[2 * i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++)
            v.w[i] = (uint32_t)Storage<DT>::narrow(f[2 * i]) | ((uint32_t)Storage<DT>::narrow(f[2 * i + 1]) << 16);
    }
    return v;
}
template <int DT> __device__ __forceinline__ float load1(const void* p, size_t i) {
    return Storage<DT>::load((const typename Storage<DT>::type*)p, i);
}
template <int DT> __device__ __forceinline__ void store1(void* p, size_t i, float v) {
    Storage<DT>::store((typename Storage<DT>::type*)p, i, v);
}

// applies a gated variant to PER lanes.  16-bit SwiGLU goes two lanes at a time through packed f32x2 arithmetic (bf16: with
// the exponential and the reciprocal on the special-function unit); results stay within one unit in the last place of the
// reference.  float32 keeps the scalar unfused operations and is bit-identical.
template <int OP, int PER, int DT> __device__ __forceinline__ void gated_lanes(float* fa, const float* fb) {
    if (OP == G_SWIGLU && DT == DT_BF16) {
        // 8 significant bits: the special-function form rounds to the reference's result on all but ~3 in 10 000 elements
#pragma unroll
        for (int i = 0; i < PER; i += 2) fast_swiglu16x2_sfu(fa[i], fa[i + 1], fb[i], fb[i + 1], fa[i], fa[i + 1]);
    } else if (OP == G_SWIGLU && DT == DT_F16) {
        // 11 significant bits: the reference's polynomial on packed fused multiply-adds (differs on ~1 element in a million)
#pragma unroll
        for (int i = 0; i < PER; i += 2) fast_swiglu32x2_fused(fa[i], fa[i + 1], fb[i], fb[i + 1], fa[i], fa[i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < PER; i++) fa[i] = gated32<OP>(fa[i], fb[i]);
    }
}

// ---- kernels ----
template <int DT, int OP>
__global__ void __launch_bounds__(256) unary_f32_kernel(const void* __restrict__ src, void* __restrict__ dst, size_t n, int vec) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t vecs = vec ? n / 4 : 0;
    for (size_t v = tid; v < vecs; v += stride) {
        Vec16 in = ld_stream((const char*)src + v * 16);
        float f[4];
        unpack<DT_F32>(in, f);
#pragma unroll
        for (int i = 0; i < 4; i++) f[i] = unary32<OP>(f[i]);
        st_stream((char*)dst + v * 16, pack<DT_F32>(f));
    }
    for (size_t i = vecs * 4 + tid; i < n; i += stride) ((float*)dst)[i] = unary32<OP>(((const float*)src)[i]);
}

// table[bits] = narrow(float32(op64(float64(widen(bits)))))
template <int DT>
__global__ void build_lut_kernel(uint16_t* __restrict__ lut, int op) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536u) return;
    float x = Storage<DT>::widen((uint16_t)i);
    lut[i] = Storage<DT>::narrow(f64_to_f32_host(unary64(op, (double)x)));
}

__global__ void __launch_bounds__(256) lut_apply_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                                       const uint16_t* __restrict__ lut, size_t n, int vec) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t vecs = vec ? n / 8 : 0;
    for (size_t v = tid; v < vecs; v += stride) {
        Vec16 in = ld_stream((const char*)src + v * 16);
        Vec16 out;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t lo = __ldg(lut + (in.w[i] & 0xFFFFu));
            uint32_t hi = __ldg(lut + (in.w[i] >> 16));
            out.w[i] = lo | (hi << 16);
        }
        st_stream((char*)dst + v * 16, out);
    }
    for (size_t i = vecs * 8 + tid; i < n; i += stride) dst[i] = __ldg(lut + src[i]);
}

// Large inputs: the whole 128 KB table is copied into the block's shared memory first (one block of 1024 threads per SM).
// A warp's 32 two-byte lookups then cost a few bank cycles instead of up to 32 cache-line tag checks: random bf16 data,
// the worst case for the cache, goes from 5.0 to 5.4 TB/s.
__global__ void __launch_bounds__(1024, 1) lut_apply_smem_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                                                const uint16_t* __restrict__ lut, size_t n) {
    extern __shared__ __align__(16) uint16_t sLut[];
    for (int i = threadIdx.x; i < 65536 / 8; i += blockDim.x) ((Vec16*)sLut)[i] = ((const Vec16*)lut)[i];
    __syncthreads();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t vecs = n / 8;
    for (size_t v = tid; v < vecs; v += 2 * stride) {
        // two vectors per round: both loads are on their way before the first lookup
        const bool two = v + stride < vecs;
        const Vec16 in0 = ld_stream((const char*)src + v * 16);
        Vec16 in1 = in0;
        if (two) in1 = ld_stream((const char*)src + (v + stride) * 16);
        Vec16 out;
#pragma unroll
        for (int i = 0; i < 4; i++) out.w[i] = (uint32_t)sLut[in0.w[i] & 0xFFFFu] | ((uint32_t)sLut[in0.w[i] >> 16] << 16);
        st_stream((char*)dst + v * 16, out);
        if (two) {
#pragma unroll
            for (int i = 0; i < 4; i++) out.w[i] = (uint32_t)sLut[in1.w[i] & 0xFFFFu] | ((uint32_t)sLut[in1.w[i] >> 16] << 16);
            st_stream((char*)dst + (v + stride) * 16, out);
        }
    }
    for (size_t i = vecs * 8 + tid; i < n; i += stride) dst[i] = sLut[src[i]];
}

template <int DT, int OP>
__global__ void __launch_bounds__(256) binary_kernel(const void* __restrict__ l, const void* __restrict__ r, void* __restrict__ dst,
                                                    size_t n, int vec) {
    constexpr int PER = Lanes<DT>::kPer;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t vecs = vec ? n / PER : 0;
    for (size_t v = tid; v < vecs; v += stride) {
        Vec16 a = ld_stream((const char*)l + v * 16), b = ld_stream((const char*)r + v * 16);
        float fa[PER], fb[PER];
        unpack<DT>(a, fa);
        unpack<DT>(b, fb);
#pragma unroll
        for (int i = 0; i < PER; i++) fa[i] = binary32<OP>(fa[i], fb[i]);
        st_stream((char*)dst + v * 16, pack<DT>(fa));
    }
    for (size_t i = vecs * PER + tid; i < n; i += stride) store1<DT>(dst, i, binary32<OP>(load1<DT>(l, i), load1<DT>(r, i)));
}

template <int DT, int OP>
__global__ void __launch_bounds__(256) gated_tensors_kernel(void* __restrict__ dst, const void* __restrict__ gate,
                                                           const void* __restrict__ up, size_t n, int vec) {
    constexpr int PER = Lanes<DT>::kPer;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t vecs = vec ? n / PER : 0;
    for (size_t v = tid; v < vecs; v += stride) {
        Vec16 a = ld_stream((const char*)gate + v * 16), b = ld_stream((const char*)up + v * 16);
        float fa[PER], fb[PER];
        unpack<DT>(a, fa);
        unpack<DT>(b, fb);
        gated_lanes<OP, PER, DT>(fa, fb);
        st_stream((char*)dst + v * 16, pack<DT>(fa));
    }
    for (size_t i = vecs * PER + tid; i < n; i += stride) store1<DT>(dst, i, gated32<OP>(load1<DT>(gate, i), load1<DT>(up, i)));
}

// the two-tensor form with the all-gather of its output folded into the stores: every finished vector goes to the same
// offset of `n` destinations (this rank's own gathered tensor and up to 7 peers', plain 16-byte stores over NVLink)
struct GatherDst {
    char* dst[8];
    int n;
};
template <int DT, int OP>
__global__ void __launch_bounds__(256) gated_tensors_gather_kernel(GatherDst d, const void* __restrict__ gate, const void* __restrict__ up,
                                                                  size_t n) {
    constexpr int PER = Lanes<DT>::kPer;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t v = tid; v < n / PER; v += stride) {
        Vec16 a = ld_stream((const char*)gate + v * 16), b = ld_stream((const char*)up + v * 16);
        float fa[PER], fb[PER];
        unpack<DT>(a, fa);
        unpack<DT>(b, fb);
        gated_lanes<OP, PER, DT>(fa, fb);
        const Vec16 o = pack<DT>(fa);
        for (int r = 0; r < d.n; r++) st_stream(d.dst[r] + v * 16, o);
    }
}

// packed rows: [gate(half) | up(half)] -> dst[half].  vec != 0 requires half % PER == 0 and aligned bases.
template <int DT, int OP>
__global__ void __launch_bounds__(256) gated_packed_kernel(void* __restrict__ dst, const void* __restrict__ packed, size_t batch,
                                                          size_t half, int vec) {
    constexpr int PER = Lanes<DT>::kPer;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr size_t ES = DT == DT_F32 ? 4 : 2;
    if (vec) {
        size_t perRow = half / PER;
        size_t total = batch * perRow;
        for (size_t v = tid; v < total; v += stride) {
            size_t row = v / perRow, c = (v % perRow) * PER;
            const char* g = (const char*)packed + (row * half * 2 + c) * ES;
            Vec16 a = ld_stream(g), b = ld_stream(g + half * ES);
            float fa[PER], fb[PER];
            unpack<DT>(a, fa);
            unpack<DT>(b, fb);
            gated_lanes<OP, PER, DT>(fa, fb);
            st_stream((char*)dst + (row * half + c) * ES, pack<DT>(fa));
        }
    } else {
        size_t total = batch * half;
        for (size_t i = tid; i < total; i += stride) {
            size_t row = i / half, c = i % half;
            store1<DT>(dst, i, gated32<OP>(load1<DT>(packed, row * half * 2 + c), load1<DT>(packed, row * half * 2 + half + c)));
        }
    }
}

template <int DT>
__global__ void __launch_bounds__(256) gated_residual_kernel(const void* __restrict__ res, const void* __restrict__ branch,
                                                            const void* __restrict__ mod, void* __restrict__ out, size_t rows,
                                                            size_t lastDim, size_t rowsPerBatch, size_t modCols, size_t set, int vec) {
    constexpr int PER = Lanes<DT>::kPer;
    constexpr size_t ES = DT == DT_F32 ? 4 : 2;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        size_t perRow = lastDim / PER;
        size_t total = rows * perRow;
        for (size_t v = tid; v < total; v += stride) {
            size_t row = v / perRow, c = (v % perRow) * PER;
            size_t mo = (row / rowsPerBatch) * modCols + set * lastDim * 3 + lastDim * 2 + c;
            Vec16 a = ld_stream((const char*)res + (row * lastDim + c) * ES);
            Vec16 b = ld_stream((const char*)branch + (row * lastDim + c) * ES);
            Vec16 m = *(const Vec16*)((const char*)mod + mo * ES);  // reused by every row of the batch: keep cached
            float fa[PER], fb[PER], fm[PER];
            unpack<DT>(a, fa);
            unpack<DT>(b, fb);
            unpack<DT>(m, fm);
#pragma unroll
            for (int i = 0; i < PER; i++) fa[i] = add(fa[i], mul(fm[i], fb[i]));
            st_stream((char*)out + (row * lastDim + c) * ES, pack<DT>(fa));
        }
    } else {
        size_t total = rows * lastDim;
        for (size_t i = tid; i < total; i += stride) {
            size_t row = i / lastDim, c = i % lastDim;
            size_t mo = (row / rowsPerBatch) * modCols + set * lastDim * 3 + lastDim * 2 + c;
            store1<DT>(out, i, add(load1<DT>(res, i), mul(load1<DT>(mod, mo), load1<DT>(branch, i))));
        }
    }
}

static int stream_grid(Context* ctx, size_t items) {
    size_t blocks = (items + 255) / 256;
    size_t cap = (size_t)ctx->smCount * 16;
    if (blocks > cap) blocks = cap;
    return blocks < 1 ? 1 : (int)blocks;
}
static bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr) {
    return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d) & 15u) == 0;
}

// lookup tables for the 16-bit unary activations, built on first use and kept for the life of the process
struct LutKey { int device, dt, op; uint16_t* table; };
static LutKey g_luts[512];
static int g_lutCount = 0;

static uint16_t* get_lut(Context* ctx, int dt, int op, CUDAStatus* status) {
    for (int i = 0; i < g_lutCount; i++)
        if (g_luts[i].device == ctx->device && g_luts[i].dt == dt && g_luts[i].op == op) return g_luts[i].table;
    if (g_lutCount >= 512) { fail(status, -7, "cuda: activation table cache full"); return nullptr; }
    uint16_t* t = nullptr;
    if (cudaMalloc((void**)&t, 65536 * 2) != cudaSuccess) { cudaGetLastError(); fail(status, -7, "cuda: activation table allocation failed"); return nullptr; }
    if (dt == DT_BF16) build_lut_kernel<DT_BF16><<<256, 256, 0, ctx->stream>>>(t, op);
    else build_lut_kernel<DT_F16><<<256, 256, 0, ctx->stream>>>(t, op);
    if (check_launch(ctx, status, "activation table") != 0) return nullptr;
    g_luts[g_lutCount++] = LutKey{ctx->device, dt, op, t};
    return t;
}

template <int OP>
static int launch_unary_f32(Context* ctx, const void* src, void* dst, size_t n, CUDAStatus* status) {
    int vec = aligned16(src, dst);
    unary_f32_kernel<DT_F32, OP><<<stream_grid(ctx, n / 4 + 1), 256, 0, ctx->stream>>>(src, dst, n, vec);
    return check_launch(ctx, status, "unary activation");
}

template <int DT, int OP>
static int launch_binary(Context* ctx, const void* l, const void* r, void* d, size_t n, CUDAStatus* status) {
    int vec = aligned16(l, r, d);
    binary_kernel<DT, OP><<<stream_grid(ctx, n / Lanes<DT>::kPer + 1), 256, 0, ctx->stream>>>(l, r, d, n, vec);
    return check_launch(ctx, status, "binary elementwise");
}
template <int DT>
static int dispatch_binary(Context* ctx, int op, const void* l, const void* r, void* d, size_t n, CUDAStatus* status) {
    switch (op) {
        case CUDABinaryFloat32Add: return launch_binary<DT, CUDABinaryFloat32Add>(ctx, l, r, d, n, status);
        case CUDABinaryFloat32Sub: return launch_binary<DT, CUDABinaryFloat32Sub>(ctx, l, r, d, n, status);
        case CUDABinaryFloat32Mul: return launch_binary<DT, CUDABinaryFloat32Mul>(ctx, l, r, d, n, status);
        case CUDABinaryFloat32Div: return launch_binary<DT, CUDABinaryFloat32Div>(ctx, l, r, d, n, status);
        case CUDABinaryFloat32Max: return launch_binary<DT, CUDABinaryFloat32Max>(ctx, l, r, d, n, status);
        case CUDABinaryFloat32Min: return launch_binary<DT, CUDABinaryFloat32Min>(ctx, l, r, d, n, status);
    }
    return fail(status, -6, "cuda: binary elementwise: unsupported operation %d", op);
}

template <int DT, int OP>
static int launch_gated(Context* ctx, void* dst, const void* gate, const void* up, size_t n, CUDAStatus* status) {
    int vec = aligned16(dst, gate, up);
    gated_tensors_kernel<DT, OP><<<stream_grid(ctx, n / Lanes<DT>::kPer + 1), 256, 0, ctx->stream>>>(dst, gate, up, n, vec);
    return check_launch(ctx, status, "gated activation");
}
template <int DT, int OP>
static int launch_gated_packed(Context* ctx, void* dst, const void* packed, size_t batch, size_t half, CUDAStatus* status) {
    int vec = aligned16(dst, packed) && (half % Lanes<DT>::kPer == 0);
    gated_packed_kernel<DT, OP><<<stream_grid(ctx, batch * half / Lanes<DT>::kPer + 1), 256, 0, ctx->stream>>>(dst, packed, batch, half, vec);
    return check_launch(ctx, status, "packed gated activation");
}

template <int OP>
int gated_entry(CUDADeviceRef contextRef, int dt, CUDABufferRef dstRef, CUDABufferRef gateRef, CUDABufferRef upRef, uint32_t count,
                CUDAStatus* status) {
    PUTER_ENTER(ctx);
    if (count == 0) return ok(status);
    size_t es = dtype_size(dt);
    if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16) return fail(status, -6, "cuda: gated activation: unsupported dtype %d", dt);
    PUTER_REQUIRE(dstRef, "destination", count * es);
    PUTER_REQUIRE(gateRef, "gate", count * es);
    PUTER_REQUIRE(upRef, "up", count * es);
    void* d = dev_ptr(dstRef);
    const void* g = dev_ptr(gateRef);
    const void* u = dev_ptr(upRef);
    if (dt == DT_F32) return launch_gated<DT_F32, OP>(ctx, d, g, u, count, status);
    if (dt == DT_BF16) return launch_gated<DT_BF16, OP>(ctx, d, g, u, count, status);
    return launch_gated<DT_F16, OP>(ctx, d, g, u, count, status);
}
template <int OP>
int gated_packed_entry(CUDADeviceRef contextRef, int dt, CUDABufferRef dstRef, CUDABufferRef packedRef, uint32_t inner, uint32_t count,
                       CUDAStatus* status) {
    PUTER_ENTER(ctx);
    if (count == 0 || inner == 0) return ok(status);
    size_t es = dtype_size(dt);
    if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16) return fail(status, -6, "cuda: gated activation: unsupported dtype %d", dt);
    PUTER_REQUIRE(dstRef, "destination", (size_t)count * inner * es);
    PUTER_REQUIRE(packedRef, "packed", (size_t)count * inner * 2 * es);
    void* d = dev_ptr(dstRef);
    const void* p = dev_ptr(packedRef);
    if (dt == DT_F32) return launch_gated_packed<DT_F32, OP>(ctx, d, p, count, inner, status);
    if (dt == DT_BF16) return launch_gated_packed<DT_BF16, OP>(ctx, d, p, count, inner, status);
    return launch_gated_packed<DT_F16, OP>(ctx, d, p, count, inner, status);
}

}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_unary_elementwise(CUDADeviceRef contextRef, int operation, int elementDType, CUDABufferRef inputRef,
                                               CUDABufferRef outRef, uint32_t count, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (count == 0) return ok(status);
    bool known = false;
#define PUTER_KNOWN(OP) known |= operation == OP;
    PUTER_UNARY_OPS(PUTER_KNOWN)
#undef PUTER_KNOWN
    if (!known) return fail(status, -6, "cuda: unary elementwise: operation %d is not on this library's path", operation);
    size_t es = dtype_size(elementDType);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "cuda: unary elementwise: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(inputRef, "input", count * es);
    PUTER_REQUIRE(outRef, "out", count * es);
    const void* src = dev_ptr(inputRef);
    void* dst = dev_ptr(outRef);
    if (elementDType == DT_F32) {
        switch (operation) {
#define PUTER_CASE(OP) case OP: return launch_unary_f32<OP>(ctx, src, dst, count, status);
            PUTER_UNARY_OPS(PUTER_CASE)
#undef PUTER_CASE
        }
    }
    uint16_t* lut = get_lut(ctx, elementDType, operation, status);
    if (!lut) return status ? status->code : -7;
    int vec = aligned16(src, dst);
    if (vec && count >= (1u << 22) && (((uintptr_t)lut) & 15u) == 0) {  // 8 MB and up: the table copy per block pays for itself
        cudaFuncSetAttribute(lut_apply_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2);
        lut_apply_smem_kernel<<<ctx->smCount, 1024, 65536 * 2, ctx->stream>>>((const uint16_t*)src, (uint16_t*)dst, lut, count);
    } else {
        lut_apply_kernel<<<stream_grid(ctx, count / 8 + 1), 256, 0, ctx->stream>>>((const uint16_t*)src, (uint16_t*)dst, lut, count, vec);
    }
    return check_launch(ctx, status, "unary activation (table)");
}

extern "C" int cuda_dispatch_binary_elementwise(CUDADeviceRef contextRef, int operation, int elementDType, CUDABufferRef leftRef,
                                                CUDABufferRef rightRef, CUDABufferRef outRef, uint32_t count, uint64_t completionToken,
                                                CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (count == 0) return ok(status);
    size_t es = dtype_size(elementDType);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "cuda: binary elementwise: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(leftRef, "left", count * es);
    PUTER_REQUIRE(rightRef, "right", count * es);
    PUTER_REQUIRE(outRef, "out", count * es);
    const void* l = dev_ptr(leftRef);
    const void* r = dev_ptr(rightRef);
    void* d = dev_ptr(outRef);
    if (elementDType == DT_F32) return dispatch_binary<DT_F32>(ctx, operation, l, r, d, count, status);
    if (elementDType == DT_BF16) return dispatch_binary<DT_BF16>(ctx, operation, l, r, d, count, status);
    return dispatch_binary<DT_F16>(ctx, operation, l, r, d, count, status);
}

#define PUTER_DEFINE_GATED(name, OP)                                                                                              \
    extern "C" int cuda_dispatch_##name(CUDADeviceRef contextRef, int elementDType, CUDABufferRef destinationRef, CUDABufferRef gateRef, \
                                        CUDABufferRef upRef, uint32_t count, uint64_t completionToken, CUDAStatus* status) {      \
        (void)completionToken;                                                                                                    \
        return gated_entry<OP>(contextRef, elementDType, destinationRef, gateRef, upRef, count, status);                          \
    }                                                                                                                             \
    extern "C" int cuda_dispatch_##name##_packed(CUDADeviceRef contextRef, int elementDType, CUDABufferRef destinationRef,         \
                                                 CUDABufferRef packedRef, uint32_t inner, uint32_t count, uint64_t completionToken, \
                                                 CUDAStatus* status) {                                                            \
        (void)completionToken;                                                                                                    \
        return gated_packed_entry<OP>(contextRef, elementDType, destinationRef, packedRef, inner, count, status);                 \
    }
PUTER_DEFINE_GATED(swiglu, G_SWIGLU)
PUTER_DEFINE_GATED(geglu, G_GEGLU)
PUTER_DEFINE_GATED(glu, G_GLU)
PUTER_DEFINE_GATED(reglu, G_REGLU)
PUTER_DEFINE_GATED(siglu, G_SIGLU)
PUTER_DEFINE_GATED(geglu_tanh, G_GEGLU_TANH)
PUTER_DEFINE_GATED(seglu, G_SEGLU)
PUTER_DEFINE_GATED(linglu, G_LINGLU)

extern "C" int cuda_dispatch_gated_residual(CUDADeviceRef contextRef, int elementDType, CUDABufferRef residualRef, CUDABufferRef branchRef,
                                            CUDABufferRef modulationRef, CUDABufferRef outputRef, uint32_t rows, uint32_t lastDim,
                                            uint32_t rowsPerBatch, uint32_t modulationCols, uint32_t set, uint64_t completionToken,
                                            CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (rows == 0 || lastDim == 0) return ok(status);
    size_t es = dtype_size(elementDType);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "cuda: gated residual: unsupported dtype %d", elementDType);
    if (rowsPerBatch == 0) return fail(status, -2, "gated residual: rows per batch must be positive");
    if ((uint64_t)modulationCols < ((uint64_t)set * 3 + 3) * lastDim)
        return fail(status, -2, "gated residual: modulation has %u columns, set %u needs %llu", modulationCols, set,
                    (unsigned long long)(((uint64_t)set * 3 + 3) * lastDim));
    size_t batches = ((size_t)rows + rowsPerBatch - 1) / rowsPerBatch;
    PUTER_REQUIRE(residualRef, "residual", (size_t)rows * lastDim * es);
    PUTER_REQUIRE(branchRef, "branch", (size_t)rows * lastDim * es);
    PUTER_REQUIRE(modulationRef, "modulation", batches * modulationCols * es);
    PUTER_REQUIRE(outputRef, "output", (size_t)rows * lastDim * es);
    const void* r = dev_ptr(residualRef);
    const void* b = dev_ptr(branchRef);
    const void* m = dev_ptr(modulationRef);
    void* o = dev_ptr(outputRef);
    int per = elementDType == DT_F32 ? 4 : 8;
    int vec = aligned16(r, b, m, o) && lastDim % per == 0 && modulationCols % per == 0;
    int grid = stream_grid(ctx, (size_t)rows * lastDim / per + 1);
    if (elementDType == DT_F32)
        gated_residual_kernel<DT_F32><<<grid, 256, 0, ctx->stream>>>(r, b, m, o, rows, lastDim, rowsPerBatch, modulationCols, set, vec);
    else if (elementDType == DT_BF16)
        gated_residual_kernel<DT_BF16><<<grid, 256, 0, ctx->stream>>>(r, b, m, o, rows, lastDim, rowsPerBatch, modulationCols, set, vec);
    else
        gated_residual_kernel<DT_F16><<<grid, 256, 0, ctx->stream>>>(r, b, m, o, rows, lastDim, rowsPerBatch, modulationCols, set, vec);
    return check_launch(ctx, status, "gated residual");
}

// SwiGLUTensors with the all-gather of its output folded into the stores: dstAll[r] is rank r's gathered tensor
// [world * count] as mapped into this process; this rank's `count` results land at element offset rank * count of every one.
// A consumer on another GPU needs a cross-rank barrier after the call.  count must be a multiple of the 16-byte vector.
extern "C" int cuda_dispatch_swiglu_gather(CUDADeviceRef contextRef, int elementDType, const CUDABufferRef* dstAll, uint32_t world,
                                           uint32_t rank, CUDABufferRef gateRef, CUDABufferRef upRef, uint32_t count,
                                           uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (count == 0) return ok(status);
    if (world == 0 || world > 8 || rank >= world || !dstAll) return fail(status, -2, "gathered swiglu: rank %u of %u (at most 8 ranks)", rank, world);
    size_t es = dtype_size(elementDType);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "cuda: gated activation: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(gateRef, "gate", count * es);
    PUTER_REQUIRE(upRef, "up", count * es);
    const void* g = dev_ptr(gateRef);
    const void* u = dev_ptr(upRef);
    GatherDst d{};
    d.n = (int)world;
    const size_t per = 16 / es;
    bool vec = count % per == 0 && aligned16(g, u);
    for (uint32_t r = 0; r < world; r++) {
        PUTER_REQUIRE(dstAll[r], "dstAll[r]", (size_t)world * count * es);
        d.dst[r] = (char*)dev_ptr(dstAll[r]) + (size_t)rank * count * es;
        vec = vec && aligned16(d.dst[r]);
    }
    if (!vec) return fail(status, -2, "gathered swiglu: buffers must be 16-byte aligned and count a multiple of %zu", per);
    const int grid = stream_grid(ctx, count / per + 1);
    if (elementDType == DT_F32) gated_tensors_gather_kernel<DT_F32, G_SWIGLU><<<grid, 256, 0, ctx->stream>>>(d, g, u, count);
    else if (elementDType == DT_BF16) gated_tensors_gather_kernel<DT_BF16, G_SWIGLU><<<grid, 256, 0, ctx->stream>>>(d, g, u, count);
    else gated_tensors_gather_kernel<DT_F16, G_SWIGLU><<<grid, 256, 0, ctx->stream>>>(d, g, u, count);
    return check_launch(ctx, status, "gathered swiglu");
}
