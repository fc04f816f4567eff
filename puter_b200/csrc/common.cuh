// Shared device helpers: status/context plumbing, storage-dtype load/store with the exact
// rounding rules of the reference's convert package, and the reference's polynomial math.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <string.h>
#include <stdio.h>

#include "../../include/puter_b200.h"

namespace puter {

// ---------------------------------------------------------------------------------------------
// host-side context (one per GPU ordinal)
// ---------------------------------------------------------------------------------------------
struct Buffer {
    void* ptr;
    long long bytes;
    int owned;
    int device;
};

struct Context {
    int device;
    int ccMajor;
    int smCount;
    long long totalMem;
    cudaStream_t ownStream;
    cudaStream_t uploadStream;
    cudaStream_t stream;  // the stream launches go to (ownStream or an adopted one)
    int exact;
    unsigned long long launches;
    // grow-only scratch for split-KV partials, RoPE tables and staged conversions
    void* workspace;
    size_t workspaceBytes;
    void* pinned[2];
    size_t pinnedBytes;
    cudaEvent_t stageEvents[4];
    int* errorFlag;  // device int32 owned by the context
    // arrival counters of the split-KV decode kernels: zeroed once here, every launch returns them to zero
    int* decodeCounters;
    size_t decodeCounterBytes;
    // cos/sin table of the last RoPE configuration (positions x headDim/2, cos then sin), reused while the config repeats
    float* ropeTable;
    size_t ropeTableBytes;
    double ropeKey[10];
    int ropeKeyValid;
    cudaEvent_t streamSwitchEvent;  // orders work of a newly adopted stream after what the previous stream still has queued
};

int fail(CUDAStatus* status, int code, const char* fmt, ...);
int ok(CUDAStatus* status);
Context* ctx_of(CUDADeviceRef ref, CUDAStatus* status);
// device pointer of a handle, or nullptr (and status -2) when the handle is null
void* dev_ptr(CUDABufferRef ref);
int check_buffer(CUDAStatus* status, CUDABufferRef ref, const char* name, size_t needBytes);
int check_launch(Context* ctx, CUDAStatus* status, const char* what);
void* ensure_workspace(Context* ctx, size_t bytes, CUDAStatus* status);

inline size_t dtype_size(int dt) {
    switch (dt) {
        case CUDAElementDTypeFloat32: return 4;
        case CUDAElementDTypeFloat16:
        case CUDAElementDTypeBFloat16: return 2;
        case CUDAElementDTypeFloat64: return 8;
        case CUDAElementDTypeFloat8E4M3:
        case CUDAElementDTypeFloat8E5M2: return 1;
    }
    return 0;
}

#define PUTER_ENTER(ctxVar)                          \
    cuda_status_clear(status);                       \
    puter::Context* ctxVar = puter::ctx_of(contextRef, status); \
    if (!ctxVar) return status ? status->code : -1;  \
    cudaSetDevice(ctxVar->device);

#define PUTER_REQUIRE(ref, name, bytes)                                   \
    do {                                                                  \
        int _rc = puter::check_buffer(status, ref, name, (size_t)(bytes)); \
        if (_rc != 0) return _rc;                                         \
    } while (0)

// ---------------------------------------------------------------------------------------------
// device-side conversions (bit rules identical to the CPU oracle / the reference's convert package)
// ---------------------------------------------------------------------------------------------
enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_F64 = 3, DT_E4M3 = 4, DT_E5M2 = 5 };

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

// RNE by bits + 0x7FFF + lsb; NaN quieted as (bits >> 16) | 0x40.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    uint32_t r = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
    return ((u & 0x7FFFFFFFu) > 0x7F800000u) ? ((u >> 16) | 0x40u) : r;
}

// exact widening; NaN keeps sign + payload with the quiet bit set.
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    float f = __half2float(__ushort_as_half((unsigned short)h));
    if ((h & 0x7FFFu) > 0x7C00u) f = __uint_as_float(((h & 0x8000u) << 16) | 0x7FC00000u | ((h & 0x3FFu) << 13));
    return f;
}

// IEEE RNE (overflow -> Inf, gradual underflow); NaN -> sign | 0x7E00 | payload >> 13.
__device__ __forceinline__ uint32_t f32_to_f16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    uint32_t r = __half_as_ushort(__float2half_rn(f));
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) r = ((u >> 16) & 0x8000u) | 0x7E00u | ((u >> 13) & 0x3FFu);
    return r;
}

// E4M3 "FN": 0x7F / 0xFF are NaN, no Inf.  Every other code is exact in f16, so widen through it.
__device__ __forceinline__ float e4m3_bits_to_f32(uint32_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    float f = __half2float(__half(h));
    if ((b & 0x7Fu) == 0x7Fu) f = __uint_as_float(((b & 0x80u) << 24) | 0x7FC00000u);
    return f;
}
// E5M2 is the top byte of an f16.
__device__ __forceinline__ float e5m2_bits_to_f32(uint32_t b) { return f16_bits_to_f32(b << 8); }

// saturating RNE: finite overflow and +-Inf -> largest finite code, NaN -> sign | 0x7F.
__device__ __forceinline__ uint32_t f32_to_e4m3_bits(float f) {
    uint32_t u = __float_as_uint(f);
    uint32_t r = __nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) r = ((u >> 24) & 0x80u) | 0x7Fu;
    return r;
}
__device__ __forceinline__ uint32_t f32_to_e5m2_bits(float f) {
    uint32_t u = __float_as_uint(f);
    uint32_t r = __nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E5M2);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) r = ((u >> 24) & 0x80u) | 0x7Fu;
    return r;
}

template <int DT> struct Storage;
template <> struct Storage<DT_F32> {
    using type = float;
    static __device__ __forceinline__ float load(const float* p, size_t i) { return p[i]; }
    static __device__ __forceinline__ void store(float* p, size_t i, float v) { p[i] = v; }
    static __device__ __forceinline__ float widen(float v) { return v; }
    static __device__ __forceinline__ float narrow(float v) { return v; }
};
template <> struct Storage<DT_BF16> {
    using type = uint16_t;
    static __device__ __forceinline__ float load(const uint16_t* p, size_t i) { return bf16_bits_to_f32(p[i]); }
    static __device__ __forceinline__ void store(uint16_t* p, size_t i, float v) { p[i] = (uint16_t)f32_to_bf16_bits(v); }
    static __device__ __forceinline__ float widen(uint16_t v) { return bf16_bits_to_f32(v); }
    static __device__ __forceinline__ uint16_t narrow(float v) { return (uint16_t)f32_to_bf16_bits(v); }
};
template <> struct Storage<DT_F16> {
    using type = uint16_t;
    static __device__ __forceinline__ float load(const uint16_t* p, size_t i) { return f16_bits_to_f32(p[i]); }
    static __device__ __forceinline__ void store(uint16_t* p, size_t i, float v) { p[i] = (uint16_t)f32_to_f16_bits(v); }
    static __device__ __forceinline__ float widen(uint16_t v) { return f16_bits_to_f32(v); }
    static __device__ __forceinline__ uint16_t narrow(float v) { return (uint16_t)f32_to_f16_bits(v); }
};

// ---------------------------------------------------------------------------------------------
// the reference's scalar math, reproduced operation by operation with unfused multiplies and adds
// (the Go compiler on amd64 never contracts a*b+c)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float divf(float a, float b) { return __fdiv_rn(a, b); }

// FastExp32 (device/cpu/math/f32.go:21-47): 2^k * degree-5 polynomial in the fractional part.
__device__ __forceinline__ float fast_exp32(float x) {
    if (x < -87.33654f) return 0.0f;
    if (x > 88.72283f) return 3.40282346638528859812e+38f;
    float z = mul(x, 1.4426950408889634f);
    int k = (int)z;
    if (z < 0.0f) k--;
    float f = sub(z, (float)k);
    float p = mul(f, 0.00133389f);
    p = mul(f, add(0.00961812f, p));
    p = mul(f, add(0.05550410f, p));
    p = mul(f, add(0.24022650f, p));
    p = mul(f, add(0.69314718f, p));
    p = add(1.0f, p);
    return __uint_as_float(__float_as_uint(p) + ((uint32_t)k << 23));
}
// Packed f32x2 arithmetic (Blackwell): two float32 lanes per instruction.  The assembler contracts a packed multiply
// followed by a packed add into one fused multiply-add, so these helpers are used only where one rounding more or less
// is acceptable: the 16-bit gated activations, whose result is rounded to bf16/f16 anyway.  The float32 paths keep the
// scalar, never-fused operations and stay bit-identical to the reference.
__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void un2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// Two FastExp32 (device/cpu/math/f32.go:21-47) with the polynomial in Horner form on fused packed multiply-adds: the same
// polynomial and exponent splice as the reference, each step rounded once instead of twice (<= 1 float32 ulp apart).
__device__ __forceinline__ void fast_exp32x2_fused(float x0, float x1, float& e0, float& e1) {
    float z0, z1;
    un2(mul2(pk2(x0, x1), pk2(1.4426950408889634f, 1.4426950408889634f)), z0, z1);
    int k0 = (int)z0, k1 = (int)z1;
    if (z0 < 0.0f) k0--;
    if (z1 < 0.0f) k1--;
    const uint64_t f = add2(pk2(z0, z1), pk2(-(float)k0, -(float)k1));
    uint64_t p = fma2(f, pk2(0.00133389f, 0.00133389f), pk2(0.00961812f, 0.00961812f));
    p = fma2(f, p, pk2(0.05550410f, 0.05550410f));
    p = fma2(f, p, pk2(0.24022650f, 0.24022650f));
    p = fma2(f, p, pk2(0.69314718f, 0.69314718f));
    p = fma2(f, p, pk2(1.0f, 1.0f));
    float p0, p1;
    un2(p, p0, p1);
    e0 = __uint_as_float(__float_as_uint(p0) + ((uint32_t)k0 << 23));
    e1 = __uint_as_float(__float_as_uint(p1) + ((uint32_t)k1 << 23));
    if (x0 < -87.33654f) e0 = 0.0f;
    if (x1 < -87.33654f) e1 = 0.0f;
    if (x0 > 88.72283f) e0 = 3.40282346638528859812e+38f;
    if (x1 > 88.72283f) e1 = 3.40282346638528859812e+38f;
}
// two FastSwiGLU32 (silu(gate) * up) for 16-bit storage types
__device__ __forceinline__ void fast_swiglu32x2_fused(float g0, float g1, float u0, float u1, float& r0, float& r1) {
    float e0, e1, d0, d1;
    fast_exp32x2_fused(-g0, -g1, e0, e1);
    un2(add2(pk2(1.0f, 1.0f), pk2(e0, e1)), d0, d1);
    // reciprocal-multiply division (2 ulp) where the quotient is about to be rounded to 16 bits anyway; the IEEE divide
    // only for denominators near the top of the float range, which the fast form would flush to zero
    const float q0 = d0 > 8.0e37f ? divf(g0, d0) : __fdividef(g0, d0);
    const float q1 = d1 > 8.0e37f ? divf(g1, d1) : __fdividef(g1, d1);
    un2(mul2(pk2(q0, q1), pk2(u0, u1)), r0, r1);
}
// Two silu(gate) * up for 16-bit storage types through the special-function unit: 2^(-gate * log2 e) by ex2.approx (2^-22
// relative), the quotient by rcp.approx.  The reference's polynomial is itself about 1e-6 away from exp, so after rounding to
// bf16 / f16 the two agree except on the few results that sit within that distance of a rounding boundary (measured: one
// unit in the last place on about 3 in 10 000 elements).  The exponent is clamped so that the denominator stays finite and the
// results for |gate| beyond the reference's clamps (-87.3, 88.7) stay within one unit in the last place of its constants.
__device__ __forceinline__ void fast_swiglu16x2_sfu(float g0, float g1, float u0, float u1, float& r0, float& r1) {
    float z0, z1, d0, d1;
    un2(mul2(pk2(g0, g1), pk2(-1.4426950408889634f, -1.4426950408889634f)), z0, z1);
    z0 = fminf(fmaxf(z0, -126.0f), 127.99f);
    z1 = fminf(fmaxf(z1, -126.0f), 127.99f);
    float e0, e1, q0, q1;
    asm("ex2.approx.f32 %0, %1;" : "=f"(e0) : "f"(z0));
    asm("ex2.approx.f32 %0, %1;" : "=f"(e1) : "f"(z1));
    un2(add2(pk2(1.0f, 1.0f), pk2(e0, e1)), d0, d1);
    asm("rcp.approx.f32 %0, %1;" : "=f"(q0) : "f"(d0));
    asm("rcp.approx.f32 %0, %1;" : "=f"(q1) : "f"(d1));
    // (gate * 1/d) * up, in the reference's order
    un2(mul2(mul2(pk2(g0, g1), pk2(q0, q1)), pk2(u0, u1)), r0, r1);
}
// two f32 -> one word of two bf16 with the library's rounding rule (hardware RNE; NaN payload rule applied on the rare NaN)
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
    uint32_t w;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
    if (lo != lo || hi != hi) w = f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
    return w;
}

// Conversions for RESULTS OF ARITHMETIC in the 16-bit row kernels, done by the hardware.  Widening is exact; narrowing is
// cvt.rn (round to nearest even, overflow to infinity, gradual underflow), the same rounding as the bit arithmetic of
// Storage<DT>::narrow.  The two differ only in which NaN comes out, and a NaN that has been through float32 arithmetic is the
// canonical 0x7FFFFFFF on this hardware, which both map to 0x7FFF: the payload rule of Storage<DT>::narrow has nothing left
// to preserve.  Pure conversions and copies of caller data must not use these.
template <int DT> __device__ __forceinline__ uint32_t pack16_arith(float lo, float hi) {
    uint32_t w;
    if (DT == DT_BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
    return w;
}
template <int DT> __device__ __forceinline__ void unpack16_arith(uint32_t w, float& lo, float& hi) {
    if (DT == DT_BF16) {
        lo = __uint_as_float(w << 16);
        hi = __uint_as_float(w & 0xFFFF0000u);
    } else {
        const float2 t = __half22float2(*(const __half2*)&w);
        lo = t.x;
        hi = t.y;
    }
}
// rounds two results to the 16-bit storage type in place and returns the packed word
template <int DT> __device__ __forceinline__ uint32_t round_pair_arith(float& a, float& b) {
    const uint32_t w = pack16_arith<DT>(a, b);
    unpack16_arith<DT>(w, a, b);
    return w;
}

// rounds two float32 to the 16-bit storage type: returns the packed word and replaces the inputs by the rounded values
template <int DT> __device__ __forceinline__ uint32_t round_pair(float& a, float& b) {
    if (DT == DT_BF16) {
        const uint32_t w = f32x2_to_bf16x2(a, b);
        a = __uint_as_float(w << 16);
        b = __uint_as_float(w & 0xFFFF0000u);
        return w;
    }
    const uint32_t lo = f32_to_f16_bits(a), hi = f32_to_f16_bits(b);
    a = f16_bits_to_f32(lo);
    b = f16_bits_to_f32(hi);
    return lo | (hi << 16);
}

__device__ __forceinline__ float fast_tanh32(float x) {  // f32.go:71-86
    if (x > 4.92f) return 1.0f;
    if (x < -4.92f) return -1.0f;
    float x2 = mul(x, x);
    float num = mul(x, add(135135.0f, mul(x2, add(17325.0f, mul(x2, add(378.0f, x2))))));
    float den = add(135135.0f, mul(x2, add(62370.0f, mul(x2, add(3150.0f, mul(x2, 28.0f))))));
    return divf(num, den);
}
__device__ __forceinline__ float fast_sigmoid32(float v) {  // f32.go:88-95
    if (v >= 0.0f) return divf(1.0f, add(1.0f, fast_exp32(-v)));
    float e = fast_exp32(v);
    return divf(e, add(1.0f, e));
}
__device__ __forceinline__ float fast_silu32(float v) { return divf(v, add(1.0f, fast_exp32(-v))); }  // f32.go:97-99
__device__ __forceinline__ float fast_gelu32(float v) {  // math/activation.go:54-57
    double x = (double)v;
    return (float)__dmul_rn(__dmul_rn(0.5, x), __dadd_rn(1.0, erf(__dmul_rn(x, 0.7071067811865475))));
}
__device__ __forceinline__ float fast_gelu_tanh32(float v) {  // f32.go:101-105
    double x = (double)v;
    double cube = __dmul_rn(__dmul_rn(__dmul_rn(0.044715, x), x), x);
    double inner = __dmul_rn(0.7978845608028654, __dadd_rn(x, cube));
    return (float)__dmul_rn(__dmul_rn(0.5, x), __dadd_rn(1.0, (double)fast_tanh32((float)inner)));
}
__device__ __forceinline__ float fast_relu32(float v) { return v > 0.0f ? v : 0.0f; }

// ---- the rest of the activation set (device/cpu/math/f32.go:50-69, activation.go:34-270, extra_activation.go:3-37) ----
__device__ __forceinline__ float nan32_ref() { return __uint_as_float(0x7FC00001u); }  // math/constant.go:5: what the log family returns for x <= 0
__device__ __forceinline__ float fast_log32(float x) {
    if (x <= 0.0f) return nan32_ref();
    const uint32_t bits = __float_as_uint(x);
    const int e = (int)(bits >> 23) - 127;
    const float m = __uint_as_float((bits & 0x007FFFFFu) | (127u << 23));
    const float y = sub(m, 1.0f);
    float p = mul(y, 0.14449244f);
    p = mul(y, add(-0.2407338084f, p));
    p = mul(y, add(0.3317990258f, p));
    p = mul(y, add(-0.4998741238f, p));
    p = mul(y, add(0.9999964239f, p));
    return add(p, mul((float)e, 0.6931471805599453f));
}
__device__ __forceinline__ float fast_leaky_relu32(float v) { return v > 0.0f ? v : mul(0.01f, v); }
__device__ __forceinline__ float fast_elu32(float v) { return v > 0.0f ? v : sub(fast_exp32(v), 1.0f); }
__device__ __forceinline__ float fast_selu32(float v) {
    return v > 0.0f ? mul(1.0507009873554805f, v) : mul((float)(1.0507009873554805 * 1.6732632423543772), sub(fast_exp32(v), 1.0f));
}
__device__ __forceinline__ float fast_softplus32(float v) { return v > 20.0f ? v : fast_log32(add(1.0f, fast_exp32(v))); }
__device__ __forceinline__ float fast_mish32(float v) { return mul(v, fast_tanh32(fast_softplus32(v))); }
__device__ __forceinline__ float fast_softsign32(float v) { return v >= 0.0f ? divf(v, add(1.0f, v)) : divf(v, sub(1.0f, v)); }
__device__ __forceinline__ float fast_hard_sigmoid32(float v) {
    const float s = add(divf(v, 6.0f), 0.5f);
    return s < 0.0f ? 0.0f : (s > 1.0f ? 1.0f : s);
}
__device__ __forceinline__ float fast_hard_swish32(float v) { return mul(v, fast_hard_sigmoid32(add(v, 3.0f))); }
__device__ __forceinline__ float fast_hard_tanh32(float v) { return v < -1.0f ? -1.0f : (v > 1.0f ? 1.0f : v); }
__device__ __forceinline__ float fast_hard_gelu32(float v) {
    float inner = add(v, 3.0f);
    if (inner < 0.0f) inner = 0.0f;
    if (inner > 6.0f) inner = 6.0f;
    return mul(v, divf(inner, 6.0f));
}
__device__ __forceinline__ float fast_quick_gelu32(float v) { return mul(v, fast_sigmoid32(mul(1.702f, v))); }
__device__ __forceinline__ float fast_tanh_shrink32(float v) { return sub(v, fast_tanh32(v)); }

// f64 variants used by the 16-bit LUT semantics (device/cpu/activation/lut.go:48-61, math/f64.go)
__device__ __forceinline__ double fast_exp64(double x) {
    if (x < -708.3964185322641) return 0.0;
    if (x > 709.782712893384) return 1.7976931348623157e+308;
    double z = __dmul_rn(x, 1.4426950408889634);
    long long k = (long long)z;
    if (z < 0.0) k--;
    double f = __dsub_rn(z, (double)k);
    double p = __dmul_rn(f, 0.001333899727232439);
    p = __dmul_rn(f, __dadd_rn(0.009618127167766223, p));
    p = __dmul_rn(f, __dadd_rn(0.05550410706910451, p));
    p = __dmul_rn(f, __dadd_rn(0.2402265069591007, p));
    p = __dmul_rn(f, __dadd_rn(0.6931471805599453, p));
    p = __dadd_rn(1.0, p);
    return ldexp(p, (int)k);
}
__device__ __forceinline__ double fast_tanh64(double x) {
    if (x > 4.92) return 1.0;
    if (x < -4.92) return -1.0;
    double x2 = __dmul_rn(x, x);
    double num = __dmul_rn(x, __dadd_rn(135135.0, __dmul_rn(x2, __dadd_rn(17325.0, __dmul_rn(x2, __dadd_rn(378.0, x2))))));
    double den = __dadd_rn(13.0, x2);
    den = __dadd_rn(693.0, __dmul_rn(x2, den));
    den = __dadd_rn(7335.0, __dmul_rn(x2, den));
    den = __dadd_rn(31185.0, __dmul_rn(x2, den));
    den = __dadd_rn(62370.0, __dmul_rn(x2, den));
    den = __dadd_rn(135135.0, __dmul_rn(x2, den));
    return __ddiv_rn(num, den);
}
__device__ __forceinline__ double fast_sigmoid64(double v) {
    if (v >= 0.0) return __ddiv_rn(1.0, __dadd_rn(1.0, fast_exp64(-v)));
    double e = fast_exp64(v);
    return __ddiv_rn(e, __dadd_rn(1.0, e));
}
__device__ __forceinline__ double fast_silu64(double v) { return __ddiv_rn(v, __dadd_rn(1.0, fast_exp64(-v))); }
__device__ __forceinline__ double fast_gelu64(double v) {
    return __dmul_rn(__dmul_rn(0.5, v), __dadd_rn(1.0, erf(__dmul_rn(v, 0.7071067811865475))));
}
__device__ __forceinline__ double fast_gelu_tanh64(double v) {
    double cube = __dmul_rn(__dmul_rn(__dmul_rn(0.044715, v), v), v);
    double inner = __dmul_rn(0.7978845608028654, __dadd_rn(v, cube));
    return __dmul_rn(__dmul_rn(0.5, v), __dadd_rn(1.0, fast_tanh64(inner)));
}

__device__ __forceinline__ double fast_log64(double x) {  // math/f64.go:35-55
    if (x <= 0.0) return __longlong_as_double(0x7FF8000000000001ll);
    const unsigned long long bits = (unsigned long long)__double_as_longlong(x);
    const long long e = (long long)(bits >> 52) - 1023;
    const double m = __longlong_as_double((long long)((bits & 0x000FFFFFFFFFFFFFull) | (1023ull << 52)));
    const double y = __dsub_rn(m, 1.0);
    double p = __dmul_rn(y, 0.14449244);
    p = __dmul_rn(y, __dadd_rn(-0.2407338084, p));
    p = __dmul_rn(y, __dadd_rn(0.3317990258, p));
    p = __dmul_rn(y, __dadd_rn(-0.4998741238, p));
    p = __dmul_rn(y, __dadd_rn(0.9999964239, p));
    return __dadd_rn(p, __dmul_rn((double)e, 0.6931471805599453));
}
__device__ __forceinline__ double fast_softplus64(double v) { return v > 20.0 ? v : fast_log64(__dadd_rn(1.0, fast_exp64(v))); }
__device__ __forceinline__ double fast_hard_sigmoid64(double v) {
    const double s = __dadd_rn(__ddiv_rn(v, 6.0), 0.5);
    return s < 0.0 ? 0.0 : (s > 1.0 ? 1.0 : s);
}
// float64 -> float32 the way the host (amd64 CVTSD2SS) does it, NaN included: the payload's top bits survive, where the
// GPU's own conversion would return the canonical NaN
__device__ __forceinline__ float f64_to_f32_host(double d) {
    if (d != d) {
        const unsigned long long b = (unsigned long long)__double_as_longlong(d);
        return __uint_as_float((uint32_t)((b >> 32) & 0x80000000u) | 0x7FC00000u | (uint32_t)((b >> 29) & 0x003FFFFFu));
    }
    return (float)d;
}

// 16-byte vector of raw storage elements
struct __align__(16) Vec16 { uint32_t w[4]; };

__device__ __forceinline__ Vec16 ld_stream(const void* p) {  // read-once data: bypass L1 allocation
    Vec16 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(void* p, const Vec16& v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
}

}  // namespace puter
