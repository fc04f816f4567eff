// Rotary position embedding (device.RoPE.RoPE / RoPEPairs).
//
// Reference semantics (device/cpu/rope/compute.go:55-193): per position the angle
// theta = float64(seq + StartPosition) * inverseFrequency(pair) is formed in float64, with
// inverseFrequency = BaseFreq^(-2*pair/headDim) optionally rescaled by the Llama-3 rule (:109-126);
// cos/sin are taken in float64 and cast to float32; pairs are rotated in float32 with separate
// multiplies and a subtract/add (no fused multiply-add): e' = e*c - o*s, o' = e*s + o*c.
// Interleaved mode pairs (2i, 2i+1); half mode pairs (i, i + headDim/2).  Layout [seq, heads, headDim].
//
// Two kernels: a table kernel evaluates the float64 angles once per (position, pair) into a
// float32 cos/sin table (a few MB, L2-resident); the rotate kernel streams the activations with
// 16-byte vectors and reads the table through the cache.
#include <math.h>

#include "common.cuh"

namespace puter {

struct InvFreq {
    double v[128];  // head dimensions up to 256
};

__global__ void rope_table_kernel(float* __restrict__ cosT, float* __restrict__ sinT, InvFreq inv, int half, long long seqLen,
                                  long long startPos) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= seqLen * half) return;
    long long s = i / half;
    int p = (int)(i % half);
    double theta = __dmul_rn((double)(s + startPos), inv.v[p]);
    double sn, cs;
    sincos(theta, &sn, &cs);
    cosT[i] = (float)cs;
    sinT[i] = (float)sn;
}

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
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++)
            v.w[i] = (uint32_t)Storage<DT>::narrow(f[2 * i]) | ((uint32_t)Storage<DT>::narrow(f[2 * i + 1]) << 16);
    }
    return v;
}

// vector path: headDim % (2*PER) == 0 and 16-byte aligned buffers
template <int DT, bool HALF>
__global__ void __launch_bounds__(256) rope_rotate_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                         const float* __restrict__ cosT, const float* __restrict__ sinT,
                                                         size_t seqLen, size_t heads, size_t headDim) {
    constexpr int PER = Lanes<DT>::kPer;
    constexpr size_t ES = DT == DT_F32 ? 4 : 2;
    const size_t half = headDim / 2;
    // HALF: a work item rotates PER pairs (two vectors PER apart by `half`); interleaved: PER/2 pairs (one vector)
    const size_t itemsPerHead = HALF ? half / PER : headDim / PER;
    const size_t total = seqLen * heads * itemsPerHead;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += stride) {
        size_t j = it % itemsPerHead;
        size_t sh = it / itemsPerHead;  // seq * heads + head
        size_t s = sh / heads;
        size_t base = sh * headDim;
        if (HALF) {
            size_t p0 = j * PER;
            Vec16 ve = ld_stream((const char*)in + (base + p0) * ES);
            Vec16 vo = ld_stream((const char*)in + (base + half + p0) * ES);
            float e[PER], o[PER], re[PER], ro[PER];
            unpack<DT>(ve, e);
            unpack<DT>(vo, o);
#pragma unroll
            for (int i = 0; i < PER; i++) {
                float c = __ldg(cosT + s * half + p0 + i), sn = __ldg(sinT + s * half + p0 + i);
                re[i] = sub(mul(e[i], c), mul(o[i], sn));
                ro[i] = add(mul(e[i], sn), mul(o[i], c));
            }
            st_stream((char*)out + (base + p0) * ES, pack<DT>(re));
            st_stream((char*)out + (base + half + p0) * ES, pack<DT>(ro));
        } else {
            size_t p0 = j * (PER / 2);
            Vec16 v = ld_stream((const char*)in + (base + 2 * p0) * ES);
            float f[PER], r[PER];
            unpack<DT>(v, f);
#pragma unroll
            for (int i = 0; i < PER / 2; i++) {
                float c = __ldg(cosT + s * half + p0 + i), sn = __ldg(sinT + s * half + p0 + i);
                r[2 * i] = sub(mul(f[2 * i], c), mul(f[2 * i + 1], sn));
                r[2 * i + 1] = add(mul(f[2 * i], sn), mul(f[2 * i + 1], c));
            }
            st_stream((char*)out + (base + 2 * p0) * ES, pack<DT>(r));
        }
    }
}

// The usual shapes (the work items of a head are a power of two <= 256 and the rotation has fewer than 2^32 items): a thread keeps
// its place inside the head for the whole launch and walks (position, head) rows, so the only division per item is one 32-bit
// position = row / heads; the cos / sin values of an item arrive as 16-byte vectors; results are rounded by the hardware
// conversion (they come out of float32 arithmetic).  The generic kernel above spent most of its instructions on three
// 64-bit divisions per item and scalar table loads: 4.1 TB/s on [16384, 32, 128] bf16 against 5.7 here.
template <int DT, bool HALF>
__global__ void __launch_bounds__(256) rope_rotate_pow2_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                              const float* __restrict__ cosT, const float* __restrict__ sinT,
                                                              uint32_t seqHeads, uint32_t heads, uint32_t headDim, int itemShift) {
    constexpr int PER = Lanes<DT>::kPer;
    constexpr size_t ES = DT == DT_F32 ? 4 : 2;
    const uint32_t half = headDim / 2;
    const uint32_t j = threadIdx.x & ((1u << itemShift) - 1);
    const uint32_t rowsPerBlock = 256u >> itemShift;
    auto pack_arith = [](const float* f) {
        Vec16 v;
        if (DT == DT_F32) {
#pragma unroll
            for (int i = 0; i < 4; i++) v.w[i] = __float_as_uint(f[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) v.w[i] = pack16_arith<DT == DT_F32 ? DT_BF16 : DT>(f[2 * i], f[2 * i + 1]);
        }
        return v;
    };
    for (uint32_t sh = blockIdx.x * rowsPerBlock + (threadIdx.x >> itemShift); sh < seqHeads; sh += gridDim.x * rowsPerBlock) {
        const uint32_t s = sh / heads;
        const size_t base = (size_t)sh * headDim;
        if (HALF) {
            const uint32_t p0 = j * PER;
            const Vec16 ve = ld_stream((const char*)in + (base + p0) * ES);
            const Vec16 vo = ld_stream((const char*)in + (base + half + p0) * ES);
            float c[PER], sn[PER], e[PER], o[PER], re[PER], ro[PER];
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                *(float4*)(c + i) = __ldg((const float4*)(cosT + (size_t)s * half + p0 + i));
                *(float4*)(sn + i) = __ldg((const float4*)(sinT + (size_t)s * half + p0 + i));
            }
            unpack<DT>(ve, e);
            unpack<DT>(vo, o);
#pragma unroll
            for (int i = 0; i < PER; i++) {
                re[i] = sub(mul(e[i], c[i]), mul(o[i], sn[i]));
                ro[i] = add(mul(e[i], sn[i]), mul(o[i], c[i]));
            }
            st_stream((char*)out + (base + p0) * ES, pack_arith(re));
            st_stream((char*)out + (base + half + p0) * ES, pack_arith(ro));
        } else {
            constexpr int PAIRS = PER / 2;
            const uint32_t p0 = j * PAIRS;
            const Vec16 v = ld_stream((const char*)in + (base + 2 * p0) * ES);
            float c[PAIRS], sn[PAIRS], f[PER], r[PER];
            if (PAIRS == 4) {
                *(float4*)c = __ldg((const float4*)(cosT + (size_t)s * half + p0));
                *(float4*)sn = __ldg((const float4*)(sinT + (size_t)s * half + p0));
            } else {
                *(float2*)c = __ldg((const float2*)(cosT + (size_t)s * half + p0));
                *(float2*)sn = __ldg((const float2*)(sinT + (size_t)s * half + p0));
            }
            unpack<DT>(v, f);
#pragma unroll
            for (int i = 0; i < PAIRS; i++) {
                r[2 * i] = sub(mul(f[2 * i], c[i]), mul(f[2 * i + 1], sn[i]));
                r[2 * i + 1] = add(mul(f[2 * i], sn[i]), mul(f[2 * i + 1], c[i]));
            }
            st_stream((char*)out + (base + 2 * p0) * ES, pack_arith(r));
        }
    }
}

// KV-cache producer: RoPE(k) at a per-row position, optional e4m3 quantisation with a per-head scale, and the paged write of K
// and V, in one pass (no reference counterpart as one op: it equals RoPE -> [convert] -> KVPageWrite for K and
// [convert] -> KVPageWrite for V; device/cpu/rope/compute.go:55-193, execution/page_intrinsic.go:361-438).  Positions, page
// ids and offsets are device arrays, so a decode step needs no host read to place its new token.  A work item is 8
// elements of V, or of K in interleaved mode, or 8 + 8 elements (a vector and its partner `half` further on) of K in half mode.
template <int DT, bool HALF, bool FP8>
__global__ void __launch_bounds__(256) rope_kv_page_write_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                                                                const int32_t* __restrict__ positions, const int32_t* __restrict__ pageIDs,
                                                                const int32_t* __restrict__ offsets, void* __restrict__ kPages,
                                                                void* __restrict__ vPages, const float* __restrict__ kScale,
                                                                const float* __restrict__ vScale, const float* __restrict__ cosT,
                                                                const float* __restrict__ sinT, size_t rows, size_t heads, size_t headDim,
                                                                size_t pageCount, size_t pageSize, size_t maxPositions,
                                                                int* __restrict__ errorFlag) {
    const size_t half = headDim / 2;
    const size_t kItemsPerHead = HALF ? half / 8 : headDim / 8, vItemsPerHead = headDim / 8;
    const size_t kItems = rows * heads * kItemsPerHead, total = kItems + rows * heads * vItemsPerHead;
    const size_t inner = heads * headDim;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    auto store8 = [&](void* pool, size_t elem, const float* f, float scale) {
        if (FP8) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                w0 |= f32_to_e4m3_bits(__fdiv_rn(f[i], scale)) << (8 * i);
                w1 |= f32_to_e4m3_bits(__fdiv_rn(f[4 + i], scale)) << (8 * i);
            }
            *(uint2*)((char*)pool + elem) = make_uint2(w0, w1);
        } else {
            *(Vec16*)((char*)pool + elem * 2) = pack<DT>(f);
        }
    };
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += stride) {
        const bool isK = it < kItems;
        const size_t local = isK ? it : it - kItems;
        const size_t perHead = isK ? kItemsPerHead : vItemsPerHead;
        const size_t j = local % perHead, rh = local / perHead, h = rh % heads, row = rh / heads;
        const long long page = pageIDs[row], off = offsets[row], pos = positions[row];
        if (page < 0 || page >= (long long)pageCount || off < 0 || off >= (long long)pageSize || pos < 0 || pos >= (long long)maxPositions) {
            if (j == 0 && h == 0) atomicExch(errorFlag, 1);
            continue;
        }
        const size_t src = row * inner + h * headDim;
        const size_t dst = ((size_t)page * pageSize + (size_t)off) * inner + h * headDim;
        if (!isK) {
            float f[8];
            unpack<DT>(ld_stream((const char*)v + (src + j * 8) * 2), f);
            if (FP8) store8(vPages, dst + j * 8, f, vScale[h]);
            else *(Vec16*)((char*)vPages + (dst + j * 8) * 2) = ld_stream((const char*)v + (src + j * 8) * 2);
        } else if (HALF) {
            const size_t p0 = j * 8;
            float e[8], o[8], re[8], ro[8];
            unpack<DT>(ld_stream((const char*)k + (src + p0) * 2), e);
            unpack<DT>(ld_stream((const char*)k + (src + half + p0) * 2), o);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float c = __ldg(cosT + (size_t)pos * half + p0 + i), sn = __ldg(sinT + (size_t)pos * half + p0 + i);
                // rounded to the storage type first, as the separate RoPE op would have stored it
                re[i] = Storage<DT>::widen(Storage<DT>::narrow(sub(mul(e[i], c), mul(o[i], sn))));
                ro[i] = Storage<DT>::widen(Storage<DT>::narrow(add(mul(e[i], sn), mul(o[i], c))));
            }
            store8(kPages, dst + p0, re, FP8 ? kScale[h] : 1.f);
            store8(kPages, dst + half + p0, ro, FP8 ? kScale[h] : 1.f);
        } else {
            const size_t p0 = j * 4;
            float f[8], r[8];
            unpack<DT>(ld_stream((const char*)k + (src + 2 * p0) * 2), f);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float c = __ldg(cosT + (size_t)pos * half + p0 + i), sn = __ldg(sinT + (size_t)pos * half + p0 + i);
                r[2 * i] = Storage<DT>::widen(Storage<DT>::narrow(sub(mul(f[2 * i], c), mul(f[2 * i + 1], sn))));
                r[2 * i + 1] = Storage<DT>::widen(Storage<DT>::narrow(add(mul(f[2 * i], sn), mul(f[2 * i + 1], c))));
            }
            store8(kPages, dst + 2 * p0, r, FP8 ? kScale[h] : 1.f);
        }
    }
}

// The same producer with one WARP per row, for head dimensions whose work items per head are a power of two: the row's page,
// offset and position are looked up once, a lane derives (head, item) with shifts, the cos / sin values of an item arrive as
// 16-byte vectors and the rotated values are rounded by the hardware conversion.  The element-wise kernel above pays four
// 64-bit divisions, three row lookups and 8-16 scalar table loads per 16-byte item: 3.6 TB/s on [131072, 8 x 128] bf16
// against 5.8 here.
template <int DT, bool HALF, bool FP8>
__global__ void __launch_bounds__(256) rope_kv_page_write_rows_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                                                                     const int32_t* __restrict__ positions, const int32_t* __restrict__ pageIDs,
                                                                     const int32_t* __restrict__ offsets, void* __restrict__ kPages,
                                                                     void* __restrict__ vPages, const float* __restrict__ kScale,
                                                                     const float* __restrict__ vScale, const float* __restrict__ cosT,
                                                                     const float* __restrict__ sinT, size_t rows, uint32_t heads, uint32_t headDim,
                                                                     size_t pageCount, size_t pageSize, size_t maxPositions, int kShift, int vShift,
                                                                     int* __restrict__ errorFlag) {
    const int lane = threadIdx.x & 31;
    const uint32_t half = headDim / 2;
    const uint32_t inner = heads * headDim;
    const uint32_t kItems = heads << kShift, vItems = heads << vShift;  // per row
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    auto store8 = [&](void* pool, size_t elem, float* f, float scale) {  // f: values already rounded to the 16-bit type
        if (FP8) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                w0 |= f32_to_e4m3_bits(__fdiv_rn(f[i], scale)) << (8 * i);
                w1 |= f32_to_e4m3_bits(__fdiv_rn(f[4 + i], scale)) << (8 * i);
            }
            *(uint2*)((char*)pool + elem) = make_uint2(w0, w1);
        } else {
            Vec16 o;
#pragma unroll
            for (int i = 0; i < 4; i++) o.w[i] = pack16_arith<DT>(f[2 * i], f[2 * i + 1]);
            *(Vec16*)((char*)pool + elem * 2) = o;
        }
    };
    for (size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
        const long long page = pageIDs[row], off = offsets[row], pos = positions[row];
        if (page < 0 || page >= (long long)pageCount || off < 0 || off >= (long long)pageSize || pos < 0 || pos >= (long long)maxPositions) {
            if (lane == 0) atomicExch(errorFlag, 1);
            continue;
        }
        const size_t src = row * inner;
        const size_t dst = ((size_t)page * pageSize + (size_t)off) * inner;
        const float* cr = cosT + (size_t)pos * half;
        const float* sr = sinT + (size_t)pos * half;
        for (uint32_t it = lane; it < kItems; it += 32) {
            const uint32_t h = it >> kShift, j = it & ((1u << kShift) - 1);
            const size_t hs = src + (size_t)h * headDim, hd = dst + (size_t)h * headDim;
            const float scale = FP8 ? kScale[h] : 1.f;
            if (HALF) {
                const uint32_t p0 = j * 8;
                float c[8], sn[8], e[8], o[8], re[8], ro[8];
                *(float4*)c = __ldg((const float4*)(cr + p0));
                *(float4*)(c + 4) = __ldg((const float4*)(cr + p0 + 4));
                *(float4*)sn = __ldg((const float4*)(sr + p0));
                *(float4*)(sn + 4) = __ldg((const float4*)(sr + p0 + 4));
                unpack<DT>(ld_stream((const char*)k + (hs + p0) * 2), e);
                unpack<DT>(ld_stream((const char*)k + (hs + half + p0) * 2), o);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    re[i] = sub(mul(e[i], c[i]), mul(o[i], sn[i]));
                    ro[i] = add(mul(e[i], sn[i]), mul(o[i], c[i]));
                }
                if (FP8) {  // rounded to the storage type first, as the separate RoPE op would have stored it
#pragma unroll
                    for (int i = 0; i < 8; i += 2) { round_pair_arith<DT>(re[i], re[i + 1]); round_pair_arith<DT>(ro[i], ro[i + 1]); }
                }
                store8(kPages, hd + p0, re, scale);
                store8(kPages, hd + half + p0, ro, scale);
            } else {
                const uint32_t p0 = j * 4;
                float c[4], sn[4], f[8], r[8];
                *(float4*)c = __ldg((const float4*)(cr + p0));
                *(float4*)sn = __ldg((const float4*)(sr + p0));
                unpack<DT>(ld_stream((const char*)k + (hs + 2 * p0) * 2), f);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    r[2 * i] = sub(mul(f[2 * i], c[i]), mul(f[2 * i + 1], sn[i]));
                    r[2 * i + 1] = add(mul(f[2 * i], sn[i]), mul(f[2 * i + 1], c[i]));
                }
                if (FP8) {
#pragma unroll
                    for (int i = 0; i < 8; i += 2) round_pair_arith<DT>(r[i], r[i + 1]);
                }
                store8(kPages, hd + 2 * p0, r, scale);
            }
        }
        for (uint32_t it = lane; it < vItems; it += 32) {
            const uint32_t h = it >> vShift, j = it & ((1u << vShift) - 1);
            const size_t hs = src + (size_t)h * headDim + j * 8, hd = dst + (size_t)h * headDim + j * 8;
            const Vec16 raw = ld_stream((const char*)v + hs * 2);
            if (FP8) {
                float f[8];
                unpack<DT>(raw, f);
                store8(vPages, hd, f, vScale[h]);
            } else {
                *(Vec16*)((char*)vPages + hd * 2) = raw;
            }
        }
    }
}

// scalar path: one thread per pair
template <int DT>
__global__ void __launch_bounds__(256) rope_rotate_scalar_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                                const float* __restrict__ cosT, const float* __restrict__ sinT,
                                                                size_t seqLen, size_t heads, size_t headDim, int halfMode) {
    using T = typename Storage<DT>::type;
    const size_t half = headDim / 2;
    const size_t total = seqLen * heads * half;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += stride) {
        size_t p = it % half, sh = it / half, s = sh / heads, base = sh * headDim;
        size_t ei = halfMode ? base + p : base + 2 * p;
        size_t oi = halfMode ? base + half + p : ei + 1;
        float e = Storage<DT>::load((const T*)in, ei), o = Storage<DT>::load((const T*)in, oi);
        float c = cosT[s * half + p], sn = sinT[s * half + p];
        Storage<DT>::store((T*)out, ei, sub(mul(e, c), mul(o, sn)));
        Storage<DT>::store((T*)out, oi, add(mul(e, sn), mul(o, c)));
    }
}

__global__ void rope_pairs_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ cosB,
                                  const float* __restrict__ sinB, size_t half) {
    size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= half) return;
    float e = in[2 * p], o = in[2 * p + 1], c = cosB[p], s = sinB[p];
    out[2 * p] = sub(mul(e, c), mul(o, s));
    out[2 * p + 1] = add(mul(e, s), mul(o, c));
}

// host: inverse frequencies in float64, as ropeInverseFrequency / llama3ScaledInverseFrequency
// (device/cpu/rope/compute.go:98-126)
static void fill_inv_freq(InvFreq* inv, int half, int headDim, double base, int scaling, double factor, double low, double high,
                          int origCtx) {
    for (int p = 0; p < half; p++) {
        double exponent = -(double)(2 * p) / (double)headDim;
        double f = pow(base, exponent);
        if (scaling == 1) {
            double wavelength = (2.0 * M_PI) / f;
            double lowW = (double)origCtx / low;
            double highW = (double)origCtx / high;
            if (wavelength > lowW) f = f / factor;
            else if (!(wavelength < highW)) {
                double smooth = ((double)origCtx / wavelength - low) / (high - low);
                f = (1.0 - smooth) * (f / factor) + smooth * f;
            }
        }
        inv->v[p] = f;
    }
}

// Validates the config the way device.RoPEConfig.Validate does (device/config.go:215-258).
int validate_rope(CUDAStatus* status, double base, uint32_t halfMode, uint32_t scaling, double factor, double low, double high,
                  uint32_t origCtx) {
    if (!(base > 0)) return fail(status, -2, "rope: base frequency must be positive, got %g", base);
    if (halfMode > 1) return fail(status, -2, "rope: unsupported mode %u", halfMode);
    if (scaling > 1) return fail(status, -2, "rope: unsupported scaling %u", scaling);
    if (scaling == 1) {
        if (!(factor > 0)) return fail(status, -2, "rope: scaling factor must be positive, got %g", factor);
        if (!(low > 0)) return fail(status, -2, "rope: low frequency factor must be positive, got %g", low);
        if (!(high > low)) return fail(status, -2, "rope: high frequency factor %g must exceed low frequency factor %g", high, low);
        if (origCtx == 0) return fail(status, -2, "rope: original context must be positive, got 0");
    }
    return 0;
}

// Builds the cos/sin table for positions startPos .. startPos+seqLen-1 at `table` (cos then sin, seqLen*half floats each).
int build_rope_table(Context* ctx, float* table, size_t seqLen, int headDim, double base, long long startPos, int scaling,
                     double factor, double low, double high, int origCtx, CUDAStatus* status) {
    int half = headDim / 2;
    if (half > 128) return fail(status, -6, "rope: head dimension %d exceeds the supported maximum of 256", headDim);
    InvFreq inv;
    fill_inv_freq(&inv, half, headDim, base, scaling, factor, low, high, origCtx);
    size_t n = seqLen * (size_t)half;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(table, table + n, inv, half, (long long)seqLen, startPos);
    return check_launch(ctx, status, "rope table");
}

// Returns the cos/sin table for this configuration from the context's cache, rebuilding it only when the configuration
// (or the number of positions) changed.  A decoder applies the same RoPE to q and k of every layer, so the float64
// angle evaluation runs once per configuration instead of once per call.
const float* cached_rope_table(Context* ctx, size_t seqLen, int headDim, double base, long long startPos, int scaling, double factor,
                               double low, double high, int origCtx, CUDAStatus* status) {
    const double key[10] = {(double)seqLen, (double)headDim, base, (double)startPos, (double)scaling, scaling ? factor : 0.0,
                            scaling ? low : 0.0, scaling ? high : 0.0, scaling ? (double)origCtx : 0.0, 0.0};
    const size_t need = seqLen * (size_t)(headDim / 2) * 2 * sizeof(float);
    if (ctx->ropeKeyValid && memcmp(key, ctx->ropeKey, sizeof(key)) == 0 && ctx->ropeTable && ctx->ropeTableBytes >= need)
        return ctx->ropeTable;
    ctx->ropeKeyValid = 0;
    if (ctx->ropeTableBytes < need) {
        if (ctx->ropeTable) {
            cudaStreamSynchronize(ctx->stream);  // earlier launches may still read the old table
            cudaFree(ctx->ropeTable);
            ctx->ropeTable = nullptr;
            ctx->ropeTableBytes = 0;
        }
        if (cudaMalloc((void**)&ctx->ropeTable, need) != cudaSuccess) {
            cudaGetLastError();
            fail(status, -7, "rope: table allocation of %zu bytes failed", need);
            return nullptr;
        }
        ctx->ropeTableBytes = need;
    }
    if (build_rope_table(ctx, ctx->ropeTable, seqLen, headDim, base, startPos, scaling, factor, low, high, origCtx, status) != 0) return nullptr;
    memcpy(ctx->ropeKey, key, sizeof(key));
    ctx->ropeKeyValid = 1;
    return ctx->ropeTable;
}

}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_rope_f64(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef,
                                      uint32_t seqLen, uint32_t numHeads, uint32_t headDim, double baseFreq, int64_t startPosition,
                                      uint32_t halfMode, uint32_t scaling, double scalingFactor, double lowFreqFactor,
                                      double highFreqFactor, uint32_t originalContext, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    // device/cpu/rope/compute.go:17-19: empty or odd head dimension is a silent no-op
    if (seqLen == 0 || numHeads == 0 || headDim == 0 || headDim % 2 != 0) return ok(status);
    int rc = validate_rope(status, baseFreq, halfMode, scaling, scalingFactor, lowFreqFactor, highFreqFactor, originalContext);
    if (rc != 0) return rc;
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "rope: unsupported dtype %d", elementDType);
    size_t es = dtype_size(elementDType);
    size_t elems = (size_t)seqLen * numHeads * headDim;
    PUTER_REQUIRE(inputRef, "input", elems * es);
    PUTER_REQUIRE(outRef, "out", elems * es);
    size_t half = headDim / 2;
    if (half > 128) return fail(status, -6, "rope: head dimension %u exceeds the supported maximum of 256", headDim);
    const float* table = cached_rope_table(ctx, seqLen, (int)headDim, baseFreq, (long long)startPosition, (int)scaling, scalingFactor,
                                           lowFreqFactor, highFreqFactor, (int)originalContext, status);
    if (!table) return status ? status->code : -7;
    const float* cosT = table;
    const float* sinT = table + (size_t)seqLen * half;
    const void* in = dev_ptr(inputRef);
    void* out = dev_ptr(outRef);
    int per = elementDType == DT_F32 ? 4 : 8;
    bool vec = (((uintptr_t)in | (uintptr_t)out) & 15u) == 0 && (halfMode ? half % per == 0 : headDim % per == 0);
    size_t items = vec ? elems / per : elems / 2;
    size_t blocks = (items + 255) / 256, cap = (size_t)ctx->smCount * 16;
    int grid = (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
    // work items of a head (a vector in interleaved mode, a vector and its partner in half mode)
    const size_t itemsPerHead = halfMode ? half / per : headDim / per;
    int itemShift = -1;
    for (int sft = 0; sft <= 8; sft++)
        if (itemsPerHead == ((size_t)1 << sft)) itemShift = sft;
    // the 16-byte table loads need the row of a position (half floats) and the item's offset in it to be 16-byte multiples
    const size_t tableStep = halfMode ? (size_t)per : (size_t)per / 2;
    const bool pow2 = vec && itemShift >= 0 && (size_t)seqLen * numHeads < 0xFFFFFFFFull / 2 && (half * 4) % 16 == 0 &&
                      (tableStep * 4) % (per == 4 && !halfMode ? 8 : 16) == 0 && ((uintptr_t)table & 15u) == 0 && ((size_t)seqLen * half * 4) % 16 == 0;
    if (pow2) {
        const uint32_t rowsPerBlock = 256u >> itemShift;
        const size_t rowBlocks = ((size_t)seqLen * numHeads + rowsPerBlock - 1) / rowsPerBlock;
        grid = (int)(rowBlocks < cap ? (rowBlocks ? rowBlocks : 1) : cap);
    }
#define ROPE_LAUNCH(DT)                                                                                                  \
    do {                                                                                                                 \
        if (pow2 && halfMode) rope_rotate_pow2_kernel<DT, true><<<grid, 256, 0, ctx->stream>>>(in, out, cosT, sinT, seqLen * numHeads, numHeads, headDim, itemShift); \
        else if (pow2) rope_rotate_pow2_kernel<DT, false><<<grid, 256, 0, ctx->stream>>>(in, out, cosT, sinT, seqLen * numHeads, numHeads, headDim, itemShift); \
        else if (!vec) rope_rotate_scalar_kernel<DT><<<grid, 256, 0, ctx->stream>>>(in, out, cosT, sinT, seqLen, numHeads, headDim, (int)halfMode); \
        else if (halfMode) rope_rotate_kernel<DT, true><<<grid, 256, 0, ctx->stream>>>(in, out, cosT, sinT, seqLen, numHeads, headDim); \
        else rope_rotate_kernel<DT, false><<<grid, 256, 0, ctx->stream>>>(in, out, cosT, sinT, seqLen, numHeads, headDim); \
    } while (0)
    if (elementDType == DT_F32) ROPE_LAUNCH(DT_F32);
    else if (elementDType == DT_BF16) ROPE_LAUNCH(DT_BF16);
    else ROPE_LAUNCH(DT_F16);
#undef ROPE_LAUNCH
    return check_launch(ctx, status, "rope");
}

extern "C" int cuda_dispatch_rope(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef,
                                  uint32_t seqLen, uint32_t numHeads, uint32_t headDim, uint32_t pairCount, float theta, float ropeFactor,
                                  float lowFreqFactor, float highFreqFactor, uint32_t originalContext, uint32_t halfMode,
                                  uint32_t positionOffset, uint64_t completionToken, CUDAStatus* status) {
    (void)pairCount;
    uint32_t scaling = (ropeFactor > 0.0f && originalContext > 0 && ropeFactor != 1.0f) ? 1u : 0u;
    return cuda_dispatch_rope_f64(contextRef, elementDType, inputRef, outRef, seqLen, numHeads, headDim, (double)theta,
                                  (int64_t)positionOffset, halfMode, scaling, (double)ropeFactor, (double)lowFreqFactor,
                                  (double)highFreqFactor, originalContext, completionToken, status);
}

extern "C" int cuda_dispatch_rope_pairs(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef,
                                        CUDABufferRef cosRef, CUDABufferRef sinRef, uint32_t halfDim, uint64_t completionToken,
                                        CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (elementDType != DT_F32) return fail(status, -6, "rope: RoPEPairs unsupported dtype");  // device/cpu/rope/ops.go:10-14
    if (halfDim == 0) return ok(status);
    PUTER_REQUIRE(inputRef, "input", (size_t)halfDim * 8);
    PUTER_REQUIRE(outRef, "out", (size_t)halfDim * 8);
    PUTER_REQUIRE(cosRef, "cos", (size_t)halfDim * 4);
    PUTER_REQUIRE(sinRef, "sin", (size_t)halfDim * 4);
    rope_pairs_kernel<<<(halfDim + 255) / 256, 256, 0, ctx->stream>>>((const float*)dev_ptr(inputRef), (float*)dev_ptr(outRef),
                                                                      (const float*)dev_ptr(cosRef), (const float*)dev_ptr(sinRef), halfDim);
    return check_launch(ctx, status, "rope pairs");
}

extern "C" int cuda_dispatch_rope_kv_page_write(CUDADeviceRef contextRef, int elementDType, int kvDType, CUDABufferRef kRef, CUDABufferRef vRef,
                                                CUDABufferRef positionsRef, CUDABufferRef pageIDsRef, CUDABufferRef offsetsRef,
                                                CUDABufferRef kPagesRef, CUDABufferRef vPagesRef, CUDABufferRef kScaleRef,
                                                CUDABufferRef vScaleRef, uint32_t rows, uint32_t kvHeads, uint32_t headDim,
                                                uint32_t pageCount, uint32_t pageSize, uint32_t maxPositions, double baseFreq,
                                                uint32_t halfMode, uint32_t scaling, double scalingFactor, double lowFreqFactor,
                                                double highFreqFactor, uint32_t originalContext, uint64_t completionToken,
                                                CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (rows == 0 || kvHeads == 0 || pageCount == 0 || pageSize == 0) return ok(status);
    if (elementDType != DT_F16 && elementDType != DT_BF16) return fail(status, -6, "rope kv page write: unsupported dtype %d", elementDType);
    const bool fp8 = kvDType == DT_E4M3;
    if (!fp8 && kvDType != elementDType) return fail(status, -6, "rope kv page write: unsupported cache dtype %d", kvDType);
    if (headDim == 0 || headDim % 16 != 0 || headDim > 256) return fail(status, -6, "rope kv page write: unsupported head dimension %u", headDim);
    if (maxPositions == 0) return fail(status, -2, "rope kv page write: maxPositions must be positive");
    int rc = validate_rope(status, baseFreq, halfMode, scaling, scalingFactor, lowFreqFactor, highFreqFactor, originalContext);
    if (rc != 0) return rc;
    const size_t inner = (size_t)kvHeads * headDim, kvEs = fp8 ? 1 : 2;
    PUTER_REQUIRE(kRef, "k", (size_t)rows * inner * 2);
    PUTER_REQUIRE(vRef, "v", (size_t)rows * inner * 2);
    PUTER_REQUIRE(positionsRef, "positions", (size_t)rows * 4);
    PUTER_REQUIRE(pageIDsRef, "pageIDs", (size_t)rows * 4);
    PUTER_REQUIRE(offsetsRef, "offsets", (size_t)rows * 4);
    PUTER_REQUIRE(kPagesRef, "kPages", (size_t)pageCount * pageSize * inner * kvEs);
    PUTER_REQUIRE(vPagesRef, "vPages", (size_t)pageCount * pageSize * inner * kvEs);
    if (fp8) {
        PUTER_REQUIRE(kScaleRef, "kScale", (size_t)kvHeads * 4);
        PUTER_REQUIRE(vScaleRef, "vScale", (size_t)kvHeads * 4);
    }
    const void* kp = dev_ptr(kRef);
    const void* vp = dev_ptr(vRef);
    void* kPool = dev_ptr(kPagesRef);
    void* vPool = dev_ptr(vPagesRef);
    if ((((uintptr_t)kp | (uintptr_t)vp | (uintptr_t)kPool | (uintptr_t)vPool) & 15u) != 0)
        return fail(status, -2, "rope kv page write: buffers must be 16-byte aligned");
    const float* table = cached_rope_table(ctx, maxPositions, (int)headDim, baseFreq, 0, (int)scaling, scalingFactor, lowFreqFactor,
                                           highFreqFactor, (int)originalContext, status);
    if (!table) return status ? status->code : -7;
    const size_t half = headDim / 2;
    const float* cosT = table;
    const float* sinT = table + (size_t)maxPositions * half;
    const size_t items = (size_t)rows * kvHeads * ((halfMode ? half : headDim) / 8 + headDim / 8);
    size_t blocks = (items + 255) / 256, cap = (size_t)ctx->smCount * 16;
    const int grid = (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
    const float* ks = fp8 ? (const float*)dev_ptr(kScaleRef) : nullptr;
    const float* vs = fp8 ? (const float*)dev_ptr(vScaleRef) : nullptr;
    // one warp per row where the items of a head are a power of two and the table rows can be read as 16-byte vectors
    int kShift = -1, vShift = -1;
    for (int sft = 0; sft <= 5; sft++) {
        if ((halfMode ? half : headDim) / 8 == ((size_t)1 << sft)) kShift = sft;
        if (headDim / 8 == ((size_t)1 << sft)) vShift = sft;
    }
    const bool byRows = kShift >= 0 && vShift >= 0 && half % 4 == 0 && ((uintptr_t)table & 15u) == 0 && ((size_t)maxPositions * half) % 4 == 0;
    size_t rowBlocks = ((size_t)rows + 7) / 8;
    const int rowGrid = (int)(rowBlocks < cap ? (rowBlocks ? rowBlocks : 1) : cap);
#define PRODUCER_LAUNCH(DT, HALF, FP8)                                                                                              \
    do {                                                                                                                            \
        if (byRows)                                                                                                                 \
            rope_kv_page_write_rows_kernel<DT, HALF, FP8><<<rowGrid, 256, 0, ctx->stream>>>(                                        \
                (const uint16_t*)kp, (const uint16_t*)vp, (const int32_t*)dev_ptr(positionsRef), (const int32_t*)dev_ptr(pageIDsRef), \
                (const int32_t*)dev_ptr(offsetsRef), kPool, vPool, ks, vs, cosT, sinT, rows, kvHeads, headDim, pageCount, pageSize, \
                maxPositions, kShift, vShift, ctx->errorFlag);                                                                      \
        else                                                                                                                        \
            rope_kv_page_write_kernel<DT, HALF, FP8><<<grid, 256, 0, ctx->stream>>>(                                                \
                (const uint16_t*)kp, (const uint16_t*)vp, (const int32_t*)dev_ptr(positionsRef), (const int32_t*)dev_ptr(pageIDsRef), \
                (const int32_t*)dev_ptr(offsetsRef), kPool, vPool, ks, vs, cosT, sinT, rows, kvHeads, headDim, pageCount, pageSize, \
                maxPositions, ctx->errorFlag);                                                                                      \
    } while (0)
#define PRODUCER_PICK(DT)                                                  \
    do {                                                                   \
        if (halfMode) { if (fp8) PRODUCER_LAUNCH(DT, true, true); else PRODUCER_LAUNCH(DT, true, false); }   \
        else { if (fp8) PRODUCER_LAUNCH(DT, false, true); else PRODUCER_LAUNCH(DT, false, false); }          \
    } while (0)
    if (elementDType == DT_BF16) PRODUCER_PICK(DT_BF16);
    else PRODUCER_PICK(DT_F16);
#undef PRODUCER_PICK
#undef PRODUCER_LAUNCH
    return check_launch(ctx, status, "rope kv page write");
}
