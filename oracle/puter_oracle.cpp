// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of the scalar ("generic") Go code of puter's device/cpu backend
// and convert package for the LLM-execution hot path.  It exists only as the
// checker for the CUDA kernels (tests, the smoke check, and the cpu_baseline leg
// of the benchmark).  Nothing in the shipped library links or calls it.
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fopenmp -shared -fPIC
//   -ffp-contract=off because Go on amd64 never fuses a multiply with an add;
//   `double` is used exactly where the Go code uses float64.
//
// Parity status: the op semantics (attention, softmax, RoPE, RMSNorm, gated
// residual, page ops, activations) are pinned by the literal known-answer
// fixtures of the reference's own tests (replayed in tests/test_oracle_golden.py).
// The dtype converters are PARITY UNPINNED at bit level: their arithmetic lives
// in github.com/theapemachine/manifesto v1.2.3 (package dtype), which is not part
// of the reference tree; the rules below follow the in-tree evidence cited at each
// function and are cross-checked against ml_dtypes and torch CPU casts.
//
// Every function cites the reference file:line it follows (paths relative to the
// reference project root).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {

// dtype codes = CUDAElementDType, device/cuda/internal/bridge/core.h:26-33
enum DType { F32 = 0, F16 = 1, BF16 = 2, F64 = 3, E4M3 = 4, E5M2 = 5 };

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// ---------------------------------------------------------------------------
// dtype converters (convert/bf16_f32.go:24-38, convert/f16_f32.go:28-42,
// convert/fp8_f32.go:8-65; arithmetic = manifesto/dtype, absent -> rules below)
// ---------------------------------------------------------------------------

// bf16 -> f32: bits << 16 (exact).  convert/bf16_f32.go:24-30
inline float bf16_to_f32(uint16_t b) { return u2f(uint32_t(b) << 16); }

// f32 -> bf16: round-to-nearest-even by bits + 0x7FFF + lsb, the rule of the
// parity-tested SIMD macros (device/cpu/avx512_bf16_macros.inc:47-59); NaN is
// quieted as (bits >> 16) | 0x0040 (device/metal/layernorm/layernorm_common.metalinc:17-27).
inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((u >> 16) | 0x0040u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}

// f16 -> f32: exact widening; NaN keeps sign and payload with the quiet bit set,
// which is what VCVTPH2PS produces (device/cpu/f16c_fp16_macros.inc).
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = uint32_t(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0x1Fu) {
        if (man == 0) return u2f(sign | 0x7F800000u);
        return u2f(sign | 0x7FC00000u | (man << 13));
    }
    if (exp == 0) {
        if (man == 0) return u2f(sign);
        // subnormal: man * 2^-24
        float v = float(man) * 5.9604644775390625e-08f;
        return u2f(f2u(v) | sign);
    }
    return u2f(sign | ((exp + 112u) << 23) | (man << 13));
}

// f32 -> f16: IEEE round-to-nearest-even, overflow -> Inf, gradual underflow
// (VCVTPS2PH imm 0, device/cpu/f16c_fp16_macros.inc:4-5); NaN -> sign|0x7E00|payload>>13.
inline uint16_t f32_to_f16(float f) {
    uint32_t u = f2u(f);
    uint16_t sign = uint16_t((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return uint16_t(sign | 0x7E00u | ((a >> 13) & 0x3FFu));
    if (a >= 0x47800000u) {  // >= 65536 -> Inf (values in [65520,65536) round below)
        return uint16_t(sign | 0x7C00u);
    }
    if (a < 0x33000000u) {  // < 2^-25 -> 0 (2^-25 itself ties to even = 0)
        return sign;
    }
    int e = int(a >> 23) - 127;
    uint32_t man = (a & 0x7FFFFFu) | 0x800000u;
    int shift;  // number of low bits dropped from the 24-bit significand
    uint32_t base;
    if (e < -14) {
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = uint32_t(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    uint32_t r = base + q;
    if (rem > half || (rem == half && (q & 1u))) r += 1;
    return uint16_t(sign | r);  // carry into the exponent (and to Inf) is the correct encoding
}

// fp8 E4M3 ("FN": no Inf, NaN = 0x7F/0xFF; device/cpu/elementwise/fp8_test.go:24-29) -> f32
inline float e4m3_to_f32(uint8_t b) {
    uint32_t sign = uint32_t(b & 0x80u) << 24;
    uint32_t exp = (b >> 3) & 0xFu;
    uint32_t man = b & 7u;
    if ((b & 0x7Fu) == 0x7Fu) return u2f(sign | 0x7FC00000u);
    if (exp == 0) {
        float v = float(man) * 0.001953125f;  // man * 2^-9
        return u2f(f2u(v) | sign);
    }
    return u2f(sign | ((exp + 120u) << 23) | (man << 20));
}

// fp8 E5M2 (IEEE-like, exp 0x1F = Inf/NaN; fp8_test.go:46-49) -> f32 == f16 widening of byte<<8
inline float e5m2_to_f32(uint8_t b) { return f16_to_f32(uint16_t(b) << 8); }

// f32 -> fp8, "saturating round-to-nearest-even" (convert/fp8_f32.go:20-23,51-54):
// finite overflow and +-Inf clamp to the largest finite code, NaN -> sign|0x7F.
inline uint8_t f32_to_fp8(float f, int mbits, int bias, uint8_t max_code) {
    uint32_t u = f2u(f);
    uint8_t sign = uint8_t((u >> 24) & 0x80u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return uint8_t(sign | 0x7Fu);
    if (a == 0x7F800000u) return uint8_t(sign | max_code);
    int e = int(a >> 23) - 127;
    int emin = 1 - bias;
    uint32_t man = (a & 0x7FFFFFu) | 0x800000u;
    if ((a >> 23) == 0) return sign;  // f32 subnormal: far below the fp8 range
    int shift;
    uint32_t base;
    if (e < emin) {
        shift = (23 - mbits) + (emin - e);
        if (shift > 25) return sign;
        base = 0;
    } else {
        shift = 23 - mbits;
        base = uint32_t(e + bias) << mbits;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    uint32_t r = base + q;
    if (rem > half || (rem == half && (q & 1u))) r += 1;
    if (r > max_code) r = max_code;
    return uint8_t(sign | r);
}
inline uint8_t f32_to_e4m3(float f) { return f32_to_fp8(f, 3, 7, 0x7E); }
inline uint8_t f32_to_e5m2(float f) { return f32_to_fp8(f, 2, 15, 0x7B); }

// typed load/store: device/cpu/attention/dtype_load.go:9-52 (same in rope/, activation/)
inline float load_typed(const void* p, size_t i, int dt) {
    switch (dt) {
        case F32: return ((const float*)p)[i];
        case F16: return f16_to_f32(((const uint16_t*)p)[i]);
        case BF16: return bf16_to_f32(((const uint16_t*)p)[i]);
        case E4M3: return e4m3_to_f32(((const uint8_t*)p)[i]);
        case E5M2: return e5m2_to_f32(((const uint8_t*)p)[i]);
    }
    return 0.f;
}
inline void store_typed(void* p, size_t i, float v, int dt) {
    switch (dt) {
        case F32: ((float*)p)[i] = v; break;
        case F16: ((uint16_t*)p)[i] = f32_to_f16(v); break;
        case BF16: ((uint16_t*)p)[i] = f32_to_bf16(v); break;
        case E4M3: ((uint8_t*)p)[i] = f32_to_e4m3(v); break;
        case E5M2: ((uint8_t*)p)[i] = f32_to_e5m2(v); break;
    }
}
inline float round_typed(float v, int dt) {
    if (dt == BF16) return bf16_to_f32(f32_to_bf16(v));
    if (dt == F16) return f16_to_f32(f32_to_f16(v));
    return v;
}
inline size_t esize(int dt) {
    switch (dt) { case F32: return 4; case F16: case BF16: return 2; case F64: return 8; default: return 1; }
}

// ---------------------------------------------------------------------------
// scalar math (device/cpu/math/f32.go, f64.go, activation.go)
// ---------------------------------------------------------------------------

// device/cpu/math/f32.go:21-47
inline float fast_exp32(float x) {
    if (x < -87.33654f) return 0.0f;
    if (x > 88.72283f) return std::numeric_limits<float>::max();
    float z = x * 1.4426950408889634f;
    int32_t k = (int32_t)z;
    if (z < 0) k--;
    float f = z - (float)k;
    float poly = 1.0f + f * (0.69314718f + f * (0.24022650f + f * (0.05550410f + f * (0.00961812f + f * 0.00133389f))));
    uint32_t bits = f2u(poly);
    bits += uint32_t(k) << 23;
    return u2f(bits);
}

// device/cpu/math/f64.go:11-33
inline double fast_exp64(double x) {
    if (x < -708.3964185322641) return 0.0;
    if (x > 709.782712893384) return std::numeric_limits<double>::max();
    double z = x * 1.4426950408889634;
    int64_t k = (int64_t)z;
    if (z < 0) k--;
    double f = z - (double)k;
    double poly = 1.0 + f * (0.6931471805599453 + f * (0.2402265069591007 + f * (0.05550410706910451 + f * (0.009618127167766223 + f * 0.001333899727232439))));
    return std::ldexp(poly, (int)k);
}

// device/cpu/math/f32.go:71-86
inline float fast_tanh32(float x) {
    if (x > 4.92f) return 1.0f;
    if (x < -4.92f) return -1.0f;
    float x2 = x * x;
    float num = x * (135135.0f + x2 * (17325.0f + x2 * (378.0f + x2)));
    float den = 135135.0f + x2 * (62370.0f + x2 * (3150.0f + x2 * 28.0f));
    return num / den;
}

// device/cpu/math/f64.go:57-71
inline double fast_tanh64(double x) {
    if (x > 4.92) return 1.0;
    if (x < -4.92) return -1.0;
    double x2 = x * x;
    double num = x * (135135.0 + x2 * (17325.0 + x2 * (378.0 + x2)));
    double den = 135135.0 + x2 * (62370.0 + x2 * (31185.0 + x2 * (7335.0 + x2 * (693.0 + x2 * (13.0 + x2)))));
    return num / den;
}

constexpr double kGeluTanhAlpha = 0.7978845608028654;  // device/cpu/math/constant.go:20-21
constexpr double kGeluTanhBeta = 0.044715;
constexpr double kSqrtTwoOverTwo = 0.7071067811865475;  // device/cpu/math/activation.go:15

// device/cpu/math/f32.go:88-99
inline float fast_sigmoid32(float v) {
    if (v >= 0) return 1.0f / (1.0f + fast_exp32(-v));
    float e = fast_exp32(v);
    return e / (1.0f + e);
}
inline float fast_silu32(float v) { return v / (1.0f + fast_exp32(-v)); }
// device/cpu/math/f32.go:101-105
inline float fast_gelu_tanh32(float v) {
    double x = (double)v;
    double inner = kGeluTanhAlpha * (x + kGeluTanhBeta * x * x * x);
    return (float)(0.5 * x * (1.0 + (double)fast_tanh32((float)inner)));
}
// device/cpu/math/activation.go:50-57
inline double fast_gelu64(double v) { return 0.5 * v * (1.0 + std::erf(v * kSqrtTwoOverTwo)); }
inline float fast_gelu32(float v) {
    double x = (double)v;
    return (float)(0.5 * x * (1.0 + std::erf(x * kSqrtTwoOverTwo)));
}
// device/cpu/math/f64.go:73-97
inline double fast_sigmoid64(double v) {
    if (v >= 0) return 1.0 / (1.0 + fast_exp64(-v));
    double e = fast_exp64(v);
    return e / (1.0 + e);
}
inline double fast_silu64(double v) { return v / (1.0 + fast_exp64(-v)); }
inline double fast_gelu_tanh64(double v) {
    double inner = kGeluTanhAlpha * (v + kGeluTanhBeta * v * v * v);
    return 0.5 * v * (1.0 + fast_tanh64(inner));
}
inline float fast_relu32(float v) { return v > 0 ? v : 0.0f; }

// device/cpu/math/constant.go:3-6: the NaN the log family returns for x <= 0
inline float nan32() { return u2f(0x7FC00001u); }
inline double nan64() { uint64_t u = 0x7FF8000000000001ull; double d; std::memcpy(&d, &u, 8); return d; }

// device/cpu/math/f32.go:50-69
inline float fast_log32(float x) {
    if (x <= 0) return nan32();
    uint32_t bits = f2u(x);
    int32_t e = (int32_t)(bits >> 23) - 127;
    float m = u2f((bits & 0x007FFFFFu) | (127u << 23));
    float y = m - 1.0f;
    float poly = y * (0.9999964239f + y * (-0.4998741238f + y * (0.3317990258f + y * (-0.2407338084f + y * 0.14449244f))));
    return poly + (float)e * 0.6931471805599453f;
}
// device/cpu/math/f64.go:35-55
inline double fast_log64(double x) {
    if (x <= 0) return nan64();
    uint64_t bits;
    std::memcpy(&bits, &x, 8);
    int64_t e = (int64_t)(bits >> 52) - 1023;
    uint64_t mb = (bits & 0x000FFFFFFFFFFFFFull) | (1023ull << 52);
    double m;
    std::memcpy(&m, &mb, 8);
    double y = m - 1.0;
    double poly = y * (0.9999964239 + y * (-0.4998741238 + y * (0.3317990258 + y * (-0.2407338084 + y * 0.14449244))));
    return poly + (double)e * 0.6931471805599453;
}

// device/cpu/math/activation.go:7-16 (Go converts an untyped constant to the type of the expression it sits in)
constexpr double kSeluAlpha = 1.6732632423543772, kSeluScale = 1.0507009873554805, kLeakySlope = 0.01;

// device/cpu/math/activation.go:34-270, extra_activation.go:3-37: float32 forms
inline float fast_leaky_relu32(float v) { return v > 0 ? v : (float)kLeakySlope * v; }
inline float fast_elu32(float v) { return v > 0 ? v : 1.0f * (fast_exp32(v) - 1.0f); }
inline float fast_celu32(float v) { return v > 0 ? v : 1.0f * (fast_exp32(v / 1.0f) - 1.0f); }
inline float fast_selu32(float v) { return v > 0 ? (float)kSeluScale * v : (float)(kSeluScale * kSeluAlpha) * (fast_exp32(v) - 1.0f); }
inline float fast_softplus32(float v) { return v > 20 ? v : fast_log32(1.0f + fast_exp32(v)); }
inline float fast_mish32(float v) { return v * fast_tanh32(fast_softplus32(v)); }
inline float fast_softsign32(float v) { return v >= 0 ? v / (1.0f + v) : v / (1.0f - v); }
inline float fast_hard_sigmoid32(float v) {
    float s = v / 6.0f + 0.5f;
    return s < 0 ? 0.0f : (s > 1 ? 1.0f : s);
}
inline float fast_hard_swish32(float v) { return v * fast_hard_sigmoid32(v + 3.0f); }
inline float fast_hard_tanh32(float v) { return v < -1.0f ? -1.0f : (v > 1.0f ? 1.0f : v); }
inline float fast_log1p32(float v) { return fast_log32(1.0f + v); }
inline float fast_expm1_32(float v) { return fast_exp32(v) - 1.0f; }
inline float fast_log_sigmoid32(float v) { return -fast_softplus32(-v); }
inline float fast_hard_gelu32(float v) {
    float inner = v + 3.0f;
    if (inner < 0) inner = 0;
    if (inner > 6) inner = 6;
    return v * (inner / 6.0f);
}
inline float fast_quick_gelu32(float v) { return v * fast_sigmoid32(1.702f * v); }
inline float fast_tanh_shrink32(float v) { return v - fast_tanh32(v); }

// float64 forms, the fill functions of the 16-bit lookup tables (device/cpu/activation/lut.go:14-41)
inline double fast_leaky_relu64(double v) { return v > 0 ? v : kLeakySlope * v; }
inline double fast_elu64(double v) { return v > 0 ? v : 1.0 * (fast_exp64(v) - 1.0); }
inline double fast_celu64(double v) { return v > 0 ? v : 1.0 * (fast_exp64(v / 1.0) - 1.0); }
inline double fast_selu64(double v) { return v > 0 ? kSeluScale * v : kSeluScale * kSeluAlpha * (fast_exp64(v) - 1.0); }
inline double fast_softplus64(double v) { return v > 20 ? v : fast_log64(1.0 + fast_exp64(v)); }
inline double fast_mish64(double v) { return v * fast_tanh64(fast_softplus64(v)); }
inline double fast_softsign64(double v) { return v / (1.0 + std::fabs(v)); }
inline double fast_hard_sigmoid64(double v) {
    double s = v / 6.0 + 0.5;
    return s < 0 ? 0.0 : (s > 1 ? 1.0 : s);
}
inline double fast_hard_swish64(double v) { return v * fast_hard_sigmoid64(v + 3.0); }
inline double fast_hard_tanh64(double v) { return v < -1.0 ? -1.0 : (v > 1.0 ? 1.0 : v); }

// unary op codes = CUDAUnaryFloat32Op, device/cuda/internal/bridge/core.h:35-70
enum UnaryOp {
    U_RELU = 0, U_EXP = 8, U_LOG = 9, U_TANH = 12, U_SIGMOID = 13, U_SILU = 14, U_SWISH = 15, U_SOFTSIGN = 16, U_ELU = 17, U_SELU = 18,
    U_LEAKY_RELU = 19, U_HARD_SIGMOID = 20, U_HARD_SWISH = 21, U_GELU = 22, U_LOG1P = 23, U_EXPM1 = 24, U_CELU = 25, U_SOFTPLUS = 26,
    U_MISH = 27, U_LOG_SIGMOID = 28, U_GELU_TANH = 29, U_HARD_TANH = 30, U_HARD_GELU = 31, U_QUICK_GELU = 32, U_TANH_SHRINK = 33
};

// float32 kernels: device/cpu/activation/f32_generic.go:9-222 (one math.Fast*32 call per element; Swish runs the Silu kernel,
// device/cpu/activation/ops.go:41-43)
inline float unary32(int op, float v) {
    switch (op) {
        case U_RELU: return fast_relu32(v);
        case U_EXP: return fast_exp32(v);
        case U_LOG: return fast_log32(v);
        case U_TANH: return fast_tanh32(v);
        case U_SIGMOID: return fast_sigmoid32(v);
        case U_SILU: case U_SWISH: return fast_silu32(v);
        case U_SOFTSIGN: return fast_softsign32(v);
        case U_ELU: return fast_elu32(v);
        case U_SELU: return fast_selu32(v);
        case U_LEAKY_RELU: return fast_leaky_relu32(v);
        case U_HARD_SIGMOID: return fast_hard_sigmoid32(v);
        case U_HARD_SWISH: return fast_hard_swish32(v);
        case U_GELU: return fast_gelu32(v);
        case U_LOG1P: return fast_log1p32(v);
        case U_EXPM1: return fast_expm1_32(v);
        case U_CELU: return fast_celu32(v);
        case U_SOFTPLUS: return fast_softplus32(v);
        case U_MISH: return fast_mish32(v);
        case U_LOG_SIGMOID: return fast_log_sigmoid32(v);
        case U_GELU_TANH: return fast_gelu_tanh32(v);
        case U_HARD_TANH: return fast_hard_tanh32(v);
        case U_HARD_GELU: return fast_hard_gelu32(v);
        case U_QUICK_GELU: return fast_quick_gelu32(v);
        case U_TANH_SHRINK: return fast_tanh_shrink32(v);
    }
    return std::numeric_limits<float>::quiet_NaN();
}
// table fill functions: device/cpu/activation/lut.go:14-41 (HardGelu, QuickGelu and TanhShrink go through their float32 forms,
// device/cpu/math/extra_activation.go:19-37)
inline double unary64(int op, double v) {
    switch (op) {
        case U_RELU: return v > 0 ? v : 0.0;
        case U_EXP: return fast_exp64(v);
        case U_LOG: return fast_log64(v);
        case U_TANH: return fast_tanh64(v);
        case U_SIGMOID: return fast_sigmoid64(v);
        case U_SILU: case U_SWISH: return fast_silu64(v);
        case U_SOFTSIGN: return fast_softsign64(v);
        case U_ELU: return fast_elu64(v);
        case U_SELU: return fast_selu64(v);
        case U_LEAKY_RELU: return fast_leaky_relu64(v);
        case U_HARD_SIGMOID: return fast_hard_sigmoid64(v);
        case U_HARD_SWISH: return fast_hard_swish64(v);
        case U_GELU: return fast_gelu64(v);
        case U_LOG1P: return fast_log64(1.0 + v);
        case U_EXPM1: return fast_exp64(v) - 1.0;
        case U_CELU: return fast_celu64(v);
        case U_SOFTPLUS: return fast_softplus64(v);
        case U_MISH: return fast_mish64(v);
        case U_LOG_SIGMOID: return -fast_softplus64(-v);
        case U_GELU_TANH: return fast_gelu_tanh64(v);
        case U_HARD_TANH: return fast_hard_tanh64(v);
        case U_HARD_GELU: return (double)fast_hard_gelu32((float)v);
        case U_QUICK_GELU: return (double)fast_quick_gelu32((float)v);
        case U_TANH_SHRINK: return (double)fast_tanh_shrink32((float)v);
    }
    return std::numeric_limits<double>::quiet_NaN();
}

// gated variants (device/cpu/math/activation.go:286-308): SwiGLU/SiGLU activate
// the gate, GLU/GeGLU/ReGLU/GeGLUTanh activate `up`.
enum GatedOp { G_SWIGLU = 0, G_GEGLU = 1, G_GLU = 2, G_REGLU = 3, G_SIGLU = 4, G_GEGLU_TANH = 5, G_SEGLU = 6, G_LINGLU = 7 };
inline float gated32(int op, float gate, float up) {
    switch (op) {
        case G_SWIGLU: return fast_silu32(gate) * up;
        case G_GEGLU: return gate * fast_gelu32(up);
        case G_GLU: return gate * fast_sigmoid32(up);
        case G_REGLU: return gate * fast_relu32(up);
        case G_SIGLU: return fast_sigmoid32(gate) * up;
        case G_GEGLU_TANH: return gate * fast_gelu_tanh32(up);
        case G_SEGLU: return up * fast_sigmoid32(gate);  // device/cpu/math/extra_activation.go:88-90
        case G_LINGLU: return gate * up;                 // extra_activation.go:84-86
    }
    return std::numeric_limits<float>::quiet_NaN();
}

// ---------------------------------------------------------------------------
// dot products (device/cpu/dot/f32_generic.go:5-15, bf16_generic.go:9-21, fp16_generic.go)
// ---------------------------------------------------------------------------
// f32: f64 accumulate, result cast to f32.  bf16/f16: f32 accumulate, result
// ROUNDED TO THE STORAGE DTYPE, then widened again by the caller
// (device/cpu/attention/typed_compute.go:10-29).
inline float typed_row_dot(const void* l, size_t lo, const void* r, size_t ro, int n, int dt) {
    if (dt == F32) {
        const float* a = (const float*)l + lo;
        const float* b = (const float*)r + ro;
        double s = 0.0;
        for (int i = 0; i < n; i++) s += (double)a[i] * (double)b[i];
        return (float)s;
    }
    float s = 0.f;
    for (int i = 0; i < n; i++) s += load_typed(l, lo + i, dt) * load_typed(r, ro + i, dt);
    if (dt == BF16) return bf16_to_f32(f32_to_bf16(s));
    return f16_to_f32(f32_to_f16(s));
}

// ---------------------------------------------------------------------------
// softmax row (device/cpu/attention/softmax.go:5-85)
// ---------------------------------------------------------------------------
void stable_softmax_row(float* s, int n) {
    if (n == 0) return;
    float mx = s[0];
    for (int i = 1; i < n; i++) if (s[i] > mx) mx = s[i];
    if (std::isinf(mx)) {
        if (mx < 0) { for (int i = 0; i < n; i++) s[i] = 0; return; }
        int cnt = 0;
        for (int i = 0; i < n; i++) if (std::isinf(s[i]) && s[i] > 0) cnt++;
        if (cnt == 0) { for (int i = 0; i < n; i++) s[i] = 0; return; }
        float w = 1.0f / (float)cnt;
        for (int i = 0; i < n; i++) s[i] = (std::isinf(s[i]) && s[i] > 0) ? w : 0.f;
        return;
    }
    float sum = 0.f;
    for (int i = 0; i < n; i++) {
        float e = (float)std::exp((double)(s[i] - mx));
        s[i] = e;
        sum += e;
    }
    if (sum == 0) return;
    for (int i = 0; i < n; i++) s[i] /= sum;
}

// device/cpu/attention/flash_attention.go:171-189 (Exp kernel = FastExp32, activation/f32_generic.go:9-16)
inline float flash_exp32(float v) {
    if ((std::isinf(v) && v < 0) || v < -88.f) return 0.f;
    if (std::isinf(v) && v > 0) return std::numeric_limits<float>::infinity();
    return fast_exp32(v);
}

// one (query row, head) of MultiHeadAttention:
// device/cpu/attention/typed_compute.go:142-204 (scores, causal bottom-right, window, ALiBi, P.V)
void mha_row(const void* q, const void* k, const void* v, void* out, int qi, int seqQ, int seqK,
             int headDim, int numHeads, int kvHeads, int head, int causal, int window, float alibi,
             int dt, float scale, float* scores) {
    int kvHead = head / (numHeads / kvHeads);
    size_t qStride = (size_t)numHeads * headDim, kvStride = (size_t)kvHeads * headDim;
    size_t qOff = (size_t)qi * qStride + (size_t)head * headDim;
    size_t kvOff = (size_t)kvHead * headDim;
    for (int ki = 0; ki < seqK; ki++) {
        float sc = typed_row_dot(q, qOff, k, (size_t)ki * kvStride + kvOff, headDim, dt) * scale;
        int absq = qi + seqK - seqQ;
        if (causal && ki > absq) sc = -std::numeric_limits<float>::infinity();
        if (window > 0 && qi - ki >= window) sc = -std::numeric_limits<float>::infinity();
        if (alibi != 0.f) sc += alibi * (float)(ki - qi);
        scores[ki] = sc;
    }
    stable_softmax_row(scores, seqK);
    for (int d = 0; d < headDim; d++) {
        float sum = 0.f;
        for (int ki = 0; ki < seqK; ki++) sum += scores[ki] * load_typed(v, (size_t)ki * kvStride + kvOff + d, dt);
        store_typed(out, qOff + d, sum, dt);
    }
}

// device/cpu/rope/compute.go:98-126
double rope_inv_freq(double base, int pair, int headDim, int scaling, double factor, double low, double high, int orig) {
    double exponent = -(double)(2 * pair) / (double)headDim;
    double inv = std::pow(base, exponent);
    if (scaling != 1) return inv;
    double wavelength = (2.0 * M_PI) / inv;
    double lowW = (double)orig / low;
    double highW = (double)orig / high;
    if (wavelength > lowW) return inv / factor;
    if (wavelength < highW) return inv;
    double smooth = ((double)orig / wavelength - low) / (high - low);
    return (1.0 - smooth) * (inv / factor) + smooth * inv;
}

}  // namespace

// ===========================================================================
// exported entry points
// ===========================================================================

ORACLE_API void oracle_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n > 0 ? n : 1);
#else
    (void)n;
#endif
}
ORACLE_API int oracle_max_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API float oracle_fast_exp32(float x) { return fast_exp32(x); }
ORACLE_API float oracle_fast_tanh32(float x) { return fast_tanh32(x); }
ORACLE_API float oracle_fast_silu32(float x) { return fast_silu32(x); }
ORACLE_API double oracle_fast_exp64(double x) { return fast_exp64(x); }

// convert package: element-wise conversion between equal-length buffers.
// Returns 0, or -1 for an unsupported pair (the Go API returns ErrLenMismatch for
// unequal lengths, convert/errors.go:10-15 — lengths are the caller's here).
ORACLE_API int oracle_convert(int srcDT, int dstDT, const void* src, void* dst, long long n) {
    if (dstDT == F32) {
        float* d = (float*)dst;
        switch (srcDT) {
            case BF16:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) d[i] = bf16_to_f32(((const uint16_t*)src)[i]);
                return 0;
            case F16:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) d[i] = f16_to_f32(((const uint16_t*)src)[i]);
                return 0;
            case E4M3:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) d[i] = e4m3_to_f32(((const uint8_t*)src)[i]);
                return 0;
            case E5M2:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) d[i] = e5m2_to_f32(((const uint8_t*)src)[i]);
                return 0;
            case F32:
                std::memcpy(dst, src, (size_t)n * 4);
                return 0;
        }
        return -1;
    }
    if (srcDT == F32) {
        const float* s = (const float*)src;
        switch (dstDT) {
            case BF16:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) ((uint16_t*)dst)[i] = f32_to_bf16(s[i]);
                return 0;
            case F16:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) ((uint16_t*)dst)[i] = f32_to_f16(s[i]);
                return 0;
            case E4M3:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) ((uint8_t*)dst)[i] = f32_to_e4m3(s[i]);
                return 0;
            case E5M2:
#pragma omp parallel for schedule(static)
                for (long long i = 0; i < n; i++) ((uint8_t*)dst)[i] = f32_to_e5m2(s[i]);
                return 0;
        }
        return -1;
    }
    return -1;
}

// device.Activation.{Silu,Gelu,GeluTanh,...}: device/cpu/activation/ops.go:37-50,
// f32_apply.go:128-147.  f32 = Fast*32; f16/bf16 = 65536-entry LUT semantics
// (lut.go:48-61): table[bits] = narrow(float32(op64(float64(widen(bits))))).
ORACLE_API int oracle_unary(int op, int dt, const void* src, void* dst, long long n) {
    if (dt == F32) {
#pragma omp parallel for schedule(static)
        for (long long i = 0; i < n; i++) ((float*)dst)[i] = unary32(op, ((const float*)src)[i]);
        return 0;
    }
    if (dt == BF16 || dt == F16) {
#pragma omp parallel for schedule(static)
        for (long long i = 0; i < n; i++) {
            float x = load_typed(src, i, dt);
            store_typed(dst, i, (float)unary64(op, (double)x), dt);
        }
        return 0;
    }
    return -1;
}

// device.Activation.SwiGLUTensors etc.: device/cpu/activation/compute.go:148-176
// device.Activation.Softmax / LogSoftmax over each row of `cols` elements: device/cpu/math/softmax.go:7-60 in float32
// (sequential sum in index order); 16-bit rows are widened into a float32 scratch row and the result rounded
// (device/cpu/activation/softmax.go:43-68).  The Go method works on one vector: rows = 1.
ORACLE_API int oracle_softmax_rows(int dt, const void* src, void* dst, long long rows, long long cols, int logSpace) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        std::vector<float> x((size_t)cols), y((size_t)cols);
        for (long long i = 0; i < cols; i++) x[i] = load_typed(src, (size_t)(r * cols + i), dt);
        float mx = x[0];
        for (long long i = 1; i < cols; i++) if (x[i] > mx) mx = x[i];
        float sum = 0.f;
        if (logSpace) {
            for (long long i = 0; i < cols; i++) sum += fast_exp32(x[i] - mx);
            float ls = fast_log32(sum);
            for (long long i = 0; i < cols; i++) y[i] = x[i] - mx - ls;
        } else {
            for (long long i = 0; i < cols; i++) { y[i] = fast_exp32(x[i] - mx); sum += y[i]; }
            float inv = 1.0f / sum;
            for (long long i = 0; i < cols; i++) y[i] *= inv;
        }
        for (long long i = 0; i < cols; i++) store_typed(dst, (size_t)(r * cols + i), y[i], dt);
    }
    return 0;
}

// device.Shape.LastToken: device/cpu/shape/ops.go:133-160 (byte copy of the final sequence row of every batch item)
ORACLE_API int oracle_last_token(const void* src, void* dst, long long batch, long long seq, long long hiddenBytes) {
    if (batch == 0 || seq == 0 || hiddenBytes == 0) return 0;
    for (long long b = 0; b < batch; b++)
        std::memcpy((char*)dst + b * hiddenBytes, (const char*)src + ((b * seq + seq - 1) * hiddenBytes), (size_t)hiddenBytes);
    return 0;
}

ORACLE_API int oracle_gated_tensors(int op, int dt, void* dst, const void* gate, const void* up, long long n) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++) store_typed(dst, i, gated32(op, load_typed(gate, i, dt), load_typed(up, i, dt)), dt);
    return 0;
}

// device.Activation.SwiGLU etc. (packed rows: gate half then up half):
// device/cpu/activation/compute.go:72-116, gated_packed_f32_generic.go:5-17
ORACLE_API int oracle_gated_packed(int op, int dt, void* dst, const void* packed, long long batch, long long half) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
#pragma omp parallel for schedule(static)
    for (long long b = 0; b < batch; b++) {
        size_t rb = (size_t)b * half * 2, db = (size_t)b * half;
        for (long long i = 0; i < half; i++)
            store_typed(dst, db + i, gated32(op, load_typed(packed, rb + i, dt), load_typed(packed, rb + half + i, dt)), dt);
    }
    return 0;
}

// device.Elementwise.{Add,Sub,Mul,Div,Max,Min}: device/cpu/elementwise/f32_generic.go,
// uint16_generic.go:148-156 (16-bit: widen, f32 op, RNE narrow).
// op codes = CUDABinaryFloat32Op (device/cuda/elementwise/arithmetic.h).
ORACLE_API int oracle_binary(int op, int dt, const void* l, const void* r, void* dst, long long n) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (op < 0 || op > 5) return -1;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++) {
        float a = load_typed(l, i, dt), b = load_typed(r, i, dt), c;
        switch (op) {
            case 0: c = a + b; break;
            case 1: c = a - b; break;
            case 2: c = a * b; break;
            case 3: c = a / b; break;
            case 4: c = a > b ? a : b; break;
            default: c = a < b ? a : b; break;
        }
        store_typed(dst, i, c, dt);
    }
    return 0;
}

// device.LayerNorm.RMSNorm: device/cpu/layernorm/compute.go:35-59,129-143,177-207,350-385
ORACLE_API int oracle_rmsnorm(int dt, const void* in, const void* scale, void* out, long long rows, long long cols, double eps) {
    if (rows == 0 || cols == 0) return 0;
    if (!(eps > 0)) return -2;  // device/config.go:86-92
    if (dt == F32) {
        const float* x = (const float*)in;
        const float* g = (const float*)scale;
        float* o = (float*)out;
#pragma omp parallel for schedule(static)
        for (long long r = 0; r < rows; r++) {
            const float* row = x + r * cols;
            double s = 0.0;
            for (long long i = 0; i < cols; i++) s += (double)row[i] * (double)row[i];
            float ss = (float)s;
            double ms = (double)ss / (double)cols;
            float inv = (float)(1.0 / std::sqrt(ms + eps));
            for (long long i = 0; i < cols; i++) o[r * cols + i] = row[i] * (inv * g[i]);
        }
        return 0;
    }
    if (dt == BF16 || dt == F16) {
#pragma omp parallel for schedule(static)
        for (long long r = 0; r < rows; r++) {
            size_t base = (size_t)r * cols;
            float ss = typed_row_dot(in, base, in, base, (int)cols, dt);  // rounded to storage dtype
            float ms = ss / (float)cols;
            float inv = (float)(1.0 / std::sqrt((double)ms + eps));
            for (long long i = 0; i < cols; i++) {
                float v = load_typed(in, base + i, dt) * inv * load_typed(scale, i, dt);
                store_typed(out, base + i, v, dt);
            }
        }
        return 0;
    }
    return -1;
}

// device.LayerNorm.LayerNorm: device/cpu/layernorm/compute.go:109-127 (f32: row sum in float32, mean and variance carried in
// float64, 1/sqrt in float64; apply = ((x - mean) * inv) * scale + bias with every product rounded, f32_generic.go:14-24),
// :484-511 (16-bit: bf16 mean from the float32 row sum rounded to bf16, reduction/bf16_kernels.go:41-51; f16 mean from the plain
// float32 sum, :572-580; float32 variance :582-602; epsilon 1e-5 added in float32).
static const float kLayerNormEps = 1e-5f;
ORACLE_API int oracle_layernorm(int dt, const void* in, const void* scale, const void* bias, void* out, long long rows, long long cols) {
    if (rows == 0 || cols == 0) return 0;
    if (dt == F32) {
        const float* x = (const float*)in;
        const float* g = (const float*)scale;
        const float* b = (const float*)bias;
        float* o = (float*)out;
#pragma omp parallel for schedule(static)
        for (long long r = 0; r < rows; r++) {
            const float* row = x + r * cols;
            float sum = 0.f;
            for (long long i = 0; i < cols; i++) sum += row[i];
            const double mean = (double)sum / (double)cols;
            const float mean32 = (float)mean;
            float sq = 0.f;
            for (long long i = 0; i < cols; i++) {
                const float d = row[i] - mean32;
                sq += d * d;
            }
            const double var = (double)sq / (double)cols;
            const float inv = (float)(1.0 / std::sqrt(var + 1e-5));
            for (long long i = 0; i < cols; i++) {
                float d = row[i] - mean32;
                d *= inv;
                d *= g[i];
                o[r * cols + i] = d + b[i];
            }
        }
        return 0;
    }
    if (dt == BF16 || dt == F16) {
#pragma omp parallel for schedule(static)
        for (long long r = 0; r < rows; r++) {
            const size_t base = (size_t)r * cols;
            float sum = 0.f;
            for (long long i = 0; i < cols; i++) sum += load_typed(in, base + i, dt);
            if (dt == BF16) sum = round_typed(sum, dt);  // SumBFloat16Native returns a bf16
            const float mean = sum / (float)cols;
            float var = 0.f;
            for (long long i = 0; i < cols; i++) {
                const float d = load_typed(in, base + i, dt) - mean;
                var += d * d;
            }
            var = var / (float)cols;
            const float inv = (float)(1.0 / std::sqrt((double)(var + kLayerNormEps)));
            for (long long i = 0; i < cols; i++) {
                const float nrm = (load_typed(in, base + i, dt) - mean) * inv;
                store_typed(out, base + i, nrm * load_typed(scale, i, dt) + load_typed(bias, i, dt), dt);
            }
        }
        return 0;
    }
    return -1;
}

// device.LayerNorm.AdaptiveRMSNorm: device/cpu/layernorm/compute.go:209-264,387-482 (mean square from 256 strided float32
// partial sums folded pairwise; out = (x * inv) * (1 + scale) + shift with modulation row [scale | shift] of the row's batch).
ORACLE_API int oracle_adaptive_rmsnorm(int dt, const void* in, const void* mod, void* out, long long rows, long long cols,
                                       long long rowsPerBatch, long long modCols, double eps) {
    if (!(eps > 0) || rowsPerBatch <= 0 || rows % rowsPerBatch != 0 || modCols < 2 * cols) return -2;  // :625-644
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (rows == 0 || cols == 0) return 0;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        const size_t base = (size_t)r * cols, mbase = (size_t)(r / rowsPerBatch) * modCols;
        float partial[256];
        for (int l = 0; l < 256; l++) {
            partial[l] = 0.f;
            for (long long i = l; i < cols; i += 256) {
                const float v = load_typed(in, base + i, dt);
                partial[l] += v * v;
            }
        }
        for (int stride = 128; stride > 0; stride >>= 1)
            for (int l = 0; l < stride; l++) partial[l] += partial[l + stride];
        const float ms = partial[0] / (float)cols;
        const float inv = (float)(1.0 / std::sqrt((double)ms + eps));
        for (long long i = 0; i < cols; i++) {
            const float nrm = load_typed(in, base + i, dt) * inv;
            const float sc = load_typed(mod, mbase + i, dt), sh = load_typed(mod, mbase + cols + i, dt);
            store_typed(out, base + i, nrm * (1.0f + sc) + sh, dt);
        }
    }
    return 0;
}

// device.LayerNorm.ModulatedLayerNorm: device/cpu/layernorm/compute.go:266-333,513-570 (statistics as LayerNorm but with the
// configured epsilon added in float64; modulation row of the batch at offset set*3*cols holds [shift | scale];
// out = ((x - mean) * inv) * (1 + scale) + shift).
ORACLE_API int oracle_modulated_layernorm(int dt, const void* in, const void* mod, void* out, long long rows, long long cols,
                                          long long rowsPerBatch, long long modCols, double eps, long long set) {
    if (!(eps > 0) || set < 0 || rowsPerBatch <= 0 || rows % rowsPerBatch != 0 || modCols < (set * 3 + 2) * cols) return -2;  // :604-648
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (rows == 0 || cols == 0) return 0;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        const size_t base = (size_t)r * cols, mbase = (size_t)(r / rowsPerBatch) * modCols + (size_t)set * cols * 3;
        float mean, inv;
        if (dt == F32) {
            const float* row = (const float*)in + base;
            float sum = 0.f;
            for (long long i = 0; i < cols; i++) sum += row[i];
            const double mean64 = (double)sum / (double)cols;
            mean = (float)mean64;
            float sq = 0.f;
            for (long long i = 0; i < cols; i++) {
                const float d = row[i] - mean;
                sq += d * d;
            }
            inv = (float)(1.0 / std::sqrt((double)sq / (double)cols + eps));
        } else {
            float sum = 0.f;
            for (long long i = 0; i < cols; i++) sum += load_typed(in, base + i, dt);
            if (dt == BF16) sum = round_typed(sum, dt);
            mean = sum / (float)cols;
            float var = 0.f;
            for (long long i = 0; i < cols; i++) {
                const float d = load_typed(in, base + i, dt) - mean;
                var += d * d;
            }
            var = var / (float)cols;
            inv = (float)(1.0 / std::sqrt((double)var + eps));
        }
        for (long long i = 0; i < cols; i++) {
            const float nrm = (load_typed(in, base + i, dt) - mean) * inv;
            const float sh = load_typed(mod, mbase + i, dt), sc = load_typed(mod, mbase + cols + i, dt);
            store_typed(out, base + i, nrm * (1.0f + sc) + sh, dt);
        }
    }
    return 0;
}

// gated residual: execution/math_gated_residual_intrinsic.go:206-223 (f32);
// 16-bit formats follow the Metal kernel: f32 math, RNE store
// (device/metal/layernorm/layernorm.metal:152-174).
ORACLE_API int oracle_gated_residual(int dt, const void* res, const void* branch, const void* mod, void* out,
                                     long long rows, long long lastDim, long long rowsPerBatch, long long modCols, long long set) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (rowsPerBatch <= 0 || modCols < (set * 3 + 3) * lastDim) return -2;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        long long b = r / rowsPerBatch;
        size_t ro = (size_t)r * lastDim;
        size_t mo = (size_t)b * modCols + (size_t)set * lastDim * 3 + (size_t)lastDim * 2;
        for (long long c = 0; c < lastDim; c++) {
            float v = load_typed(res, ro + c, dt) + load_typed(mod, mo + c, dt) * load_typed(branch, ro + c, dt);
            store_typed(out, ro + c, v, dt);
        }
    }
    return 0;
}

// device.RoPE.RoPE: device/cpu/rope/compute.go:11-31,55-96,128-193
// mode: 0 interleaved, 1 half.  scaling: 0 none, 1 llama3.  Layout [seq, heads, headDim].
ORACLE_API int oracle_rope(int dt, const void* in, void* out, long long seqLen, long long numHeads, long long headDim,
                           double base, long long startPos, int mode, int scaling, double factor, double low,
                           double high, long long origCtx) {
    if (seqLen == 0 || numHeads == 0 || headDim == 0 || headDim % 2 != 0) return 0;
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (!(base > 0) || (mode != 0 && mode != 1) || (scaling != 0 && scaling != 1)) return -2;
    if (scaling == 1 && (!(factor > 0) || !(low > 0) || !(high > low) || origCtx <= 0)) return -2;  // device/config.go:215-258
    int half = (int)(headDim / 2);
    std::vector<double> inv(half);
    for (int p = 0; p < half; p++) inv[p] = rope_inv_freq(base, p, (int)headDim, scaling, factor, low, high, (int)origCtx);
#pragma omp parallel for schedule(static)
    for (long long s = 0; s < seqLen; s++) {
        std::vector<float> c(half), sn(half);
        double pos = (double)(s + startPos);
        for (int p = 0; p < half; p++) {
            double th = pos * inv[p];
            c[p] = (float)std::cos(th);
            sn[p] = (float)std::sin(th);
        }
        for (long long h = 0; h < numHeads; h++) {
            size_t ro = ((size_t)s * numHeads + h) * headDim;
            for (int p = 0; p < half; p++) {
                size_t ei = mode == 1 ? ro + p : ro + 2 * (size_t)p;
                size_t oi = mode == 1 ? ro + half + p : ei + 1;
                float e = load_typed(in, ei, dt), o = load_typed(in, oi, dt);
                float re = e * c[p] - o * sn[p];
                float rd = e * sn[p] + o * c[p];
                store_typed(out, ei, re, dt);
                store_typed(out, oi, rd, dt);
            }
        }
    }
    return 0;
}

// device.RoPE.RoPEPairs (f32 only): device/cpu/rope/ops.go:25-38, f32_generic.go:3-11
ORACLE_API int oracle_rope_pairs(float* out, const float* in, const float* cosb, const float* sinb, long long half) {
    for (long long p = 0; p < half; p++) {
        float e = in[2 * p], o = in[2 * p + 1];
        out[2 * p] = e * cosb[p] - o * sinb[p];
        out[2 * p + 1] = e * sinb[p] + o * cosb[p];
    }
    return 0;
}

// device.Shape.PageWrite / KVPageWrite: device/cpu/shape/page_generic.go:5-29, page.go:104-150
// (validation), execution/page_intrinsic.go:361-438 (storageOffset in elements).
// When out != storage the whole layer is copied first, as the CPU op does.
ORACLE_API int oracle_page_write(int dt, const void* storage, const void* values, const int32_t* pageIDs, const int32_t* offsets,
                                 void* out, long long pageCount, long long pageSize, long long inner, long long valueRows,
                                 long long storageOffset) {
    size_t es = esize(dt);
    for (long long r = 0; r < valueRows; r++)
        if (pageIDs[r] < 0 || pageIDs[r] >= pageCount || offsets[r] < 0 || offsets[r] >= pageSize) return -2;
    const char* s = (const char*)storage + (size_t)storageOffset * es;
    char* o = (char*)out + (size_t)storageOffset * es;
    if (o != s) std::memmove(o, s, (size_t)pageCount * pageSize * inner * es);
    for (long long r = 0; r < valueRows; r++) {
        size_t row = ((size_t)pageIDs[r] * pageSize + offsets[r]) * inner;
        std::memcpy(o + row * es, (const char*)values + (size_t)r * inner * es, (size_t)inner * es);
    }
    return 0;
}

// device.Shape.PageGather / KVPageGather: device/cpu/shape/page_generic.go:30-50, page.go:156-211
ORACLE_API int oracle_page_gather(int dt, const void* storage, const int32_t* pageTable, void* out, long long pageCount,
                                  long long pageSize, long long inner, long long outRows, long long storageOffset) {
    size_t es = esize(dt);
    long long tables = (outRows + pageSize - 1) / pageSize;
    for (long long t = 0; t < tables; t++)
        if (pageTable[t] < 0 || pageTable[t] >= pageCount) return -2;
    const char* s = (const char*)storage + (size_t)storageOffset * es;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < outRows; r++) {
        size_t row = ((size_t)pageTable[r / pageSize] * pageSize + (size_t)(r % pageSize)) * inner;
        std::memcpy((char*)out + (size_t)r * inner * es, s + row * es, (size_t)inner * es);
    }
    return 0;
}

ORACLE_API void oracle_stable_softmax_row(float* scores, long long n) { stable_softmax_row(scores, (int)n); }

// device.Attention.MultiHeadAttention: device/cpu/attention/ops.go:33-40, compute.go:31-52,70-90,
// typed_compute.go:142-237.  Layout q/out [seqQ, numHeads*headDim], k/v [seqK, kvHeads*headDim].
ORACLE_API int oracle_mha(int dt, const void* q, const void* k, const void* v, void* out, long long seqQ, long long seqK,
                          long long numHeads, long long kvHeads, long long headDim, int causal, long long window, float alibi) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (kvHeads <= 0) kvHeads = numHeads;
    if (seqQ == 0 || seqK == 0) return 0;
    float scale = (float)(1.0 / std::sqrt((double)headDim));
    long long units = numHeads * seqQ;
#pragma omp parallel
    {
        std::vector<float> scores(seqK);
#pragma omp for schedule(dynamic, 4)
        for (long long u = 0; u < units; u++) {
            int head = (int)(u / seqQ), qi = (int)(u % seqQ);
            mha_row(q, k, v, out, qi, (int)seqQ, (int)seqK, (int)headDim, (int)numHeads, (int)kvHeads, head, causal,
                    (int)window, alibi, dt, scale, scores.data());
        }
    }
    return 0;
}

// Same op restricted to a list of (query row, head) pairs: used to check very large
// prefill problems on a row sample.  Rows not listed are left untouched in `out`.
ORACLE_API int oracle_mha_rows(int dt, const void* q, const void* k, const void* v, void* out, long long seqQ, long long seqK,
                               long long numHeads, long long kvHeads, long long headDim, int causal,
                               const int32_t* rowIdx, const int32_t* headIdx, long long nPairs) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (kvHeads <= 0) kvHeads = numHeads;
    float scale = (float)(1.0 / std::sqrt((double)headDim));
#pragma omp parallel
    {
        std::vector<float> scores(seqK);
#pragma omp for schedule(dynamic, 1)
        for (long long u = 0; u < nPairs; u++)
            mha_row(q, k, v, out, rowIdx[u], (int)seqQ, (int)seqK, (int)headDim, (int)numHeads, (int)kvHeads, headIdx[u],
                    causal, 0, 0.f, dt, scale, scores.data());
    }
    return 0;
}

// device.Attention.{FlashAttention,ScaledDotProductAttention} (single head, online softmax,
// causal = top-left key>row skipped): device/cpu/attention/compute.go:54-68,
// typed_compute.go:31-97, select_flash_amd64.go:133-177.
ORACLE_API int oracle_sdpa(int dt, const void* q, const void* k, const void* v, void* out, long long seqQ, long long seqK,
                           long long depth, long long valueDim, int causal) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    if (seqQ == 0 || seqK == 0) return 0;
    float scale = (float)(1.0 / std::sqrt((double)depth));
#pragma omp parallel
    {
        std::vector<float> acc(valueDim);
#pragma omp for schedule(dynamic, 4)
        for (long long row = 0; row < seqQ; row++) {
            float maxScore = -std::numeric_limits<float>::infinity();
            float normalizer = 0.f;
            std::fill(acc.begin(), acc.end(), 0.f);
            for (long long ki = 0; ki < seqK; ki++) {
                if (causal && ki > row) continue;
                float score = typed_row_dot(q, (size_t)row * depth, k, (size_t)ki * depth, (int)depth, dt) * scale;
                float oldMax = maxScore;
                if (score > maxScore) maxScore = score;
                float alpha = flash_exp32(oldMax - maxScore);
                float shifted = flash_exp32(score - maxScore);
                normalizer = normalizer * alpha + shifted;
                for (long long d = 0; d < valueDim; d++) {
                    float ve = load_typed(v, (size_t)ki * valueDim + d, dt);
                    acc[d] = acc[d] * alpha + ve * shifted;
                }
            }
            if (normalizer == 0.f) {
                for (long long d = 0; d < valueDim; d++) store_typed(out, (size_t)row * valueDim + d, 0.f, dt);
                continue;
            }
            float invN = 1.0f / normalizer;
            for (long long d = 0; d < valueDim; d++) store_typed(out, (size_t)row * valueDim + d, acc[d] * invN, dt);
        }
    }
    return 0;
}

// Paged decode attention = the reference's composition for one new token per sequence:
// page_gather(K), page_gather(V) (execution/page_intrinsic.go:217-352) then
// MultiHeadAttention with seqQ = 1, seqK = ctx, causal (bottom-right, so every live key is visible).
//   q, out      [B, numHeads*headDim]         dt (f32 / f16 / bf16)
//   kPages/vPages [pageCount, pageSize, kvHeads*headDim]   kvDT
//   pageTable   [B, maxPages] int32, ctxLens [B] int32
// kvDT == dt: the reference path verbatim.  kvDT == E4M3/E5M2 (extension; the CPU ops reject fp8,
// device/cpu/shape/page.go:302-304): K/V bytes are widened (Float8*ToFloat32 semantics), multiplied by the
// per-KV-head f32 scale, q is widened to f32, the f32 MultiHeadAttention runs, and the row is narrowed to dt.
ORACLE_API int oracle_paged_decode(int dt, int kvDT, const void* q, const void* kPages, const void* vPages,
                                   const int32_t* pageTable, const int32_t* ctxLens, const float* kScale, const float* vScale,
                                   void* out, long long batch, long long maxPages, long long pageCount, long long pageSize,
                                   long long numHeads, long long kvHeads, long long headDim) {
    if (dt != F32 && dt != BF16 && dt != F16) return -1;
    long long inner = kvHeads * headDim;
    size_t kes = esize(kvDT), qes = esize(dt);
    int rc = 0;
    const float scale = (float)(1.0 / std::sqrt((double)headDim));
    // phase 1: the two page gathers of every sequence (parallel over sequences)
    std::vector<std::vector<char>> kg(batch), vg(batch);
    std::vector<std::vector<float>> kf(batch), vf(batch), qf(batch), of(batch);
    std::vector<char> live(batch, 0);
#pragma omp parallel for schedule(dynamic, 1)
    for (long long b = 0; b < batch; b++) {
        long long ctx = ctxLens[b];
        if (ctx <= 0) continue;  // seqK == 0: silent no-op (device/cpu/attention/compute.go:16-18)
        if ((ctx + pageSize - 1) / pageSize > maxPages) { rc = -2; continue; }
        const int32_t* table = pageTable + b * maxPages;
        kg[b].resize((size_t)ctx * inner * kes);
        vg[b].resize((size_t)ctx * inner * kes);
        if (oracle_page_gather(kvDT, kPages, table, kg[b].data(), pageCount, pageSize, inner, ctx, 0) != 0 ||
            oracle_page_gather(kvDT, vPages, table, vg[b].data(), pageCount, pageSize, inner, ctx, 0) != 0) { rc = -2; continue; }
        if (kvDT != dt) {
            kf[b].resize((size_t)ctx * inner);
            vf[b].resize((size_t)ctx * inner);
            qf[b].resize(numHeads * headDim);
            of[b].resize(numHeads * headDim);
            for (size_t i = 0; i < (size_t)ctx * inner; i++) {
                int kvh = (int)((i % inner) / headDim);
                kf[b][i] = load_typed(kg[b].data(), i, kvDT) * (kScale ? kScale[kvh] : 1.0f);
                vf[b][i] = load_typed(vg[b].data(), i, kvDT) * (vScale ? vScale[kvh] : 1.0f);
            }
            const char* qb = (const char*)q + (size_t)b * numHeads * headDim * qes;
            for (long long i = 0; i < numHeads * headDim; i++) qf[b][i] = load_typed(qb, i, dt);
        }
        live[b] = 1;
    }
    // phase 2: MultiHeadAttention rows, one (sequence, head) per task
#pragma omp parallel
    {
        std::vector<float> scores;
#pragma omp for schedule(dynamic, 1)
        for (long long u = 0; u < batch * numHeads; u++) {
            long long b = u / numHeads;
            int h = (int)(u % numHeads);
            if (!live[b]) continue;
            int ctx = ctxLens[b];
            scores.resize(ctx);
            const char* qb = (const char*)q + (size_t)b * numHeads * headDim * qes;
            char* ob = (char*)out + (size_t)b * numHeads * headDim * qes;
            if (kvDT == dt)
                mha_row(qb, kg[b].data(), vg[b].data(), ob, 0, 1, ctx, (int)headDim, (int)numHeads, (int)kvHeads, h, 1, 0, 0.f, dt, scale,
                        scores.data());
            else
                mha_row(qf[b].data(), kf[b].data(), vf[b].data(), of[b].data(), 0, 1, ctx, (int)headDim, (int)numHeads, (int)kvHeads, h,
                        1, 0, 0.f, F32, scale, scores.data());
        }
    }
    if (kvDT != dt) {
        for (long long b = 0; b < batch; b++) {
            if (!live[b]) continue;
            char* ob = (char*)out + (size_t)b * numHeads * headDim * qes;
            for (long long i = 0; i < numHeads * headDim; i++) store_typed(ob, i, of[b][i], dt);
        }
    }
    return rc;
}
