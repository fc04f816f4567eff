// Sibling row normalisations of RMSNorm: device.LayerNorm.LayerNorm, AdaptiveRMSNorm and ModulatedLayerNorm
// (device/interface.go:355-379).
//
// Reference semantics (device/cpu/layernorm/compute.go):
//   LayerNorm          :109-127, 484-511   mean and variance per row, epsilon 1e-5,
//                                           out = ((x - mean) * inv) * scale + bias
//   AdaptiveRMSNorm    :209-264, 387-482   mean square of the row, out = (x * inv) * (1 + scale) + shift with the
//                                           modulation row [scale | shift] of the row's batch
//   ModulatedLayerNorm :266-333, 513-570   LayerNorm statistics with the configured epsilon,
//                                           out = ((x - mean) * inv) * (1 + scale) + shift with [shift | scale] at
//                                           offset set * 3 * cols of the batch's modulation row
// Float32 rows carry the statistics in float64 as the CPU code does (float32 row sum -> float64 mean; float32 sum of squared
// differences -> float64 variance; 1/sqrt in float64); 16-bit rows use float32 statistics, the bf16 row sum being rounded to
// bf16 first (reduction/bf16_kernels.go:41-51).  Products and sums of the apply step are rounded one by one (no fused
// multiply-add), results are rounded to the storage type once.
//
// Every row is read from HBM once and written once: 2 x the row in traffic, the HBM minimum.  Rows that can travel as bulk
// copies (16-byte aligned, a multiple of 16 bytes) go through the per-warp shared-memory row pipeline of row_pipeline.cuh;
// other rows take one CTA per row (grid-stride), the row widened into shared memory, reduced twice and written.
#include <math.h>

#include "common.cuh"
#include "row_pipeline.cuh"

namespace puter {

namespace {

enum : int { OP_LAYERNORM = 0, OP_ADAPTIVE_RMS = 1, OP_MODULATED_LN = 2 };

__device__ __forceinline__ float block_sum_f32(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();  // scratch may still be read from the previous reduction
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < nw ? scratch[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// 16 bytes of storage <-> PER floats (4 for f32, 8 for the 16-bit types)
template <int DT> struct Per { static constexpr int kPer = DT == DT_F32 ? 4 : 8; };
template <int DT> __device__ __forceinline__ void unpack_row(const Vec16& v, float* f) {
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
template <int DT> __device__ __forceinline__ Vec16 pack_row(const float* f) {
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

struct RowNormParams {
    const void* in;
    const void* p0;   // LayerNorm: scale; the other two: modulation
    const void* p1;   // LayerNorm: bias
    const void* res;  // LayerNorm only, optional: rows added to the rounded result (the fused layernorm + add)
    void* out;
    int* errorFlag;
    size_t rows, cols, rowsPerBatch, modCols, set;
    double eps;
};

// VEC: cols is a multiple of the vector width and every buffer is 16-byte aligned (rows then stay aligned too)
template <int DT, int OP, bool VEC>
__global__ void __launch_bounds__(256) row_norm_kernel(RowNormParams p) {
    using T = typename Storage<DT>::type;
    constexpr int PER = Per<DT>::kPer;
    extern __shared__ float rowBuf[];  // the widened row
    __shared__ float scratch[8];
    const size_t cols = p.cols;
    // Rows of up to kAhead vectors per thread are fetched one row ahead into registers, so the loads of the next row are in
    // flight while this row is reduced and written (a CTA otherwise alternates between waiting for memory and computing).
    constexpr int kAhead = 4;
    const size_t nvec = cols / PER;
    const bool ahead = VEC && nvec <= (size_t)kAhead * 256;
    Vec16 nxt[kAhead];
    auto fetch = [&](size_t row) {
        const char* src = (const char*)((const T*)p.in + row * cols);
#pragma unroll
        for (int k = 0; k < kAhead; k++) {
            const size_t v = threadIdx.x + (size_t)k * 256;
            if (v < nvec) nxt[k] = ld_stream(src + v * 16);
        }
    };
    if (ahead && blockIdx.x < p.rows) fetch(blockIdx.x);
    for (size_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T* x = (const T*)p.in + row * cols;
        T* o = (T*)p.out + row * cols;
        // ---- load once, first reduction ----
        float acc = 0.f;
        if (ahead) {
#pragma unroll
            for (int k = 0; k < kAhead; k++) {
                const size_t v = threadIdx.x + (size_t)k * 256;
                if (v < nvec) {
                    float f[PER];
                    unpack_row<DT>(nxt[k], f);
#pragma unroll
                    for (int i = 0; i < PER; i += 4) *(float4*)(rowBuf + v * PER + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
#pragma unroll
                    for (int i = 0; i < PER; i++) acc += OP == OP_ADAPTIVE_RMS ? f[i] * f[i] : f[i];
                }
            }
            if (row + gridDim.x < p.rows) fetch(row + gridDim.x);
        } else if (VEC) {
            for (size_t v = threadIdx.x; v < cols / PER; v += blockDim.x) {
                float f[PER];
                unpack_row<DT>(ld_stream((const char*)x + v * 16), f);
#pragma unroll
                for (int i = 0; i < PER; i += 4) *(float4*)(rowBuf + v * PER + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
#pragma unroll
                for (int i = 0; i < PER; i++) acc += OP == OP_ADAPTIVE_RMS ? f[i] * f[i] : f[i];
            }
        } else {
            for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
                const float v = Storage<DT>::load(x, i);
                rowBuf[i] = v;
                acc += OP == OP_ADAPTIVE_RMS ? v * v : v;
            }
        }
        float total = block_sum_f32(acc, scratch);
        float mean = 0.f, inv;
        if (OP == OP_ADAPTIVE_RMS) {
            const float ms = __fdiv_rn(total, (float)cols);
            inv = (float)(1.0 / sqrt((double)ms + p.eps));
        } else {
            double var64;
            if (DT == DT_F32) {
                mean = (float)((double)total / (double)cols);
            } else {
                if (DT == DT_BF16) total = Storage<DT>::widen(Storage<DT>::narrow(total));
                mean = __fdiv_rn(total, (float)cols);
            }
            float sq = 0.f;
            if (VEC) {
                for (size_t v = threadIdx.x; v < cols / 4; v += blockDim.x) {
                    const float4 f = *(const float4*)(rowBuf + v * 4);
                    const float d0 = sub(f.x, mean), d1 = sub(f.y, mean), d2 = sub(f.z, mean), d3 = sub(f.w, mean);
                    sq = add(add(add(add(sq, mul(d0, d0)), mul(d1, d1)), mul(d2, d2)), mul(d3, d3));
                }
            } else {
                for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
                    const float d = sub(rowBuf[i], mean);
                    sq = add(sq, mul(d, d));
                }
            }
            sq = block_sum_f32(sq, scratch);
            if (DT == DT_F32) {
                var64 = (double)sq / (double)cols;
                inv = (float)(1.0 / sqrt(var64 + p.eps));
            } else if (OP == OP_LAYERNORM) {
                inv = (float)(1.0 / sqrt((double)add(__fdiv_rn(sq, (float)cols), (float)p.eps)));  // epsilon added in float32
            } else {
                inv = (float)(1.0 / sqrt((double)__fdiv_rn(sq, (float)cols) + p.eps));
            }
        }
        // ---- apply ----
        if (OP == OP_LAYERNORM) {
            const T* g = (const T*)p.p0;
            const T* b = (const T*)p.p1;
            if (VEC) {
                for (size_t v = threadIdx.x; v < cols / PER; v += blockDim.x) {
                    float gs[PER], bs[PER], r[PER];
                    unpack_row<DT>(*(const Vec16*)((const char*)g + v * 16), gs);
                    unpack_row<DT>(*(const Vec16*)((const char*)b + v * 16), bs);
#pragma unroll
                    for (int i = 0; i < PER; i++) r[i] = add(mul(mul(sub(rowBuf[v * PER + i], mean), inv), gs[i]), bs[i]);
                    if (p.res) {  // the unfused Add reads the stored (rounded) LayerNorm result
                        float rs[PER];
                        unpack_row<DT>(ld_stream((const char*)((const T*)p.res + row * cols) + v * 16), rs);
#pragma unroll
                        for (int i = 0; i < PER; i++) r[i] = add(Storage<DT>::widen(Storage<DT>::narrow(r[i])), rs[i]);
                    }
                    st_stream((char*)o + v * 16, pack_row<DT>(r));
                }
            } else {
                for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
                    const float d = mul(mul(sub(rowBuf[i], mean), inv), Storage<DT>::load(g, i));
                    float r = add(d, Storage<DT>::load(b, i));
                    if (p.res) r = add(Storage<DT>::widen(Storage<DT>::narrow(r)), Storage<DT>::load((const T*)p.res, row * cols + i));
                    Storage<DT>::store(o, i, r);
                }
            }
        } else {
            const size_t batch = row / p.rowsPerBatch;
            const T* m = (const T*)p.p0 + batch * p.modCols + (OP == OP_MODULATED_LN ? p.set * cols * 3 : 0);
            // AdaptiveRMSNorm: [scale | shift]; ModulatedLayerNorm: [shift | scale]
            if (VEC) {
                for (size_t v = threadIdx.x; v < cols / PER; v += blockDim.x) {
                    float first[PER], second[PER], r[PER];
                    unpack_row<DT>(*(const Vec16*)((const char*)m + v * 16), first);
                    unpack_row<DT>(*(const Vec16*)((const char*)(m + cols) + v * 16), second);
#pragma unroll
                    for (int i = 0; i < PER; i++) {
                        const float scale = OP == OP_ADAPTIVE_RMS ? first[i] : second[i], shift = OP == OP_ADAPTIVE_RMS ? second[i] : first[i];
                        const float x0 = rowBuf[v * PER + i];
                        const float nrm = mul(OP == OP_ADAPTIVE_RMS ? x0 : sub(x0, mean), inv);
                        r[i] = add(mul(nrm, add(1.0f, scale)), shift);
                    }
                    st_stream((char*)o + v * 16, pack_row<DT>(r));
                }
            } else {
                for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
                    const float first = Storage<DT>::load(m, i), second = Storage<DT>::load(m, cols + i);
                    const float scale = OP == OP_ADAPTIVE_RMS ? first : second, shift = OP == OP_ADAPTIVE_RMS ? second : first;
                    const float nrm = mul(OP == OP_ADAPTIVE_RMS ? rowBuf[i] : sub(rowBuf[i], mean), inv);
                    Storage<DT>::store(o, i, add(mul(nrm, add(1.0f, scale)), shift));
                }
            }
        }
        __syncthreads();  // rowBuf is overwritten by the next row
    }
}

__device__ __forceinline__ float warp_sum_f32(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Vector rows through the shared-memory row pipeline (row_pipeline.cuh): one warp per row, the raw row in a ring stage,
// two or three passes over it (sum, squared differences, apply) while the next rows of the warp are being copied in.
__device__ __forceinline__ float fold_parts(const float* part) {
    float t = part[0];
#pragma unroll
    for (int u = 1; u < ROWPIPE_UN; u++) t += part[u];
    return t;
}

template <int DT, int OP>
__global__ void __launch_bounds__(ROWPIPE_MAX_WARPS * 32) row_norm_ring_kernel(RowNormParams p, int stages) {
    using T = typename Storage<DT>::type;
    constexpr int PER = Per<DT>::kPer;
    constexpr int UN = ROWPIPE_UN;  // vectors per lane handled together: their loads are issued back to back, their sums are independent
    extern __shared__ __align__(128) unsigned char ringSmem[];
    const size_t cols = p.cols, nvec = cols / PER, rowBytes = cols * sizeof(T);
    const int lane = threadIdx.x & 31;
    rowpipe::Ring ring(ringSmem, blockDim.x >> 5, stages, rowBytes, p.in, p.rows);
    for (size_t row = ring.first(); row < p.rows; row = ring.next_row(row)) {
        const unsigned char* x = ring.acquire(p.errorFlag);
        if (!x) return;
        char* o = (char*)((T*)p.out + row * cols);
        float part[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) part[u] = 0.f;
        for (size_t v0 = lane; v0 < nvec; v0 += 32 * UN) {
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const size_t v = v0 + 32 * (size_t)u;
                if (v < nvec) {
                    float f[PER];
                    unpack_row<DT>(*(const Vec16*)(x + v * 16), f);
#pragma unroll
                    for (int i = 0; i < PER; i++) part[u] += OP == OP_ADAPTIVE_RMS ? f[i] * f[i] : f[i];
                }
            }
        }
        float total = warp_sum_f32(fold_parts(part));
        float mean = 0.f, inv;
        if (OP == OP_ADAPTIVE_RMS) {
            inv = (float)(1.0 / sqrt((double)__fdiv_rn(total, (float)cols) + p.eps));
        } else {
            if (DT == DT_F32) {
                mean = (float)((double)total / (double)cols);
            } else {
                if (DT == DT_BF16) total = Storage<DT>::widen(Storage<DT>::narrow(total));
                mean = __fdiv_rn(total, (float)cols);
            }
#pragma unroll
            for (int u = 0; u < UN; u++) part[u] = 0.f;
            for (size_t v0 = lane; v0 < nvec; v0 += 32 * UN) {
#pragma unroll
                for (int u = 0; u < UN; u++) {
                    const size_t v = v0 + 32 * (size_t)u;
                    if (v < nvec) {
                        float f[PER];
                        unpack_row<DT>(*(const Vec16*)(x + v * 16), f);
#pragma unroll
                        for (int i = 0; i < PER; i++) {
                            const float d = sub(f[i], mean);
                            part[u] = add(part[u], mul(d, d));
                        }
                    }
                }
            }
            const float sq = warp_sum_f32(fold_parts(part));
            if (DT == DT_F32) inv = (float)(1.0 / sqrt((double)sq / (double)cols + p.eps));
            else if (OP == OP_LAYERNORM) inv = (float)(1.0 / sqrt((double)add(__fdiv_rn(sq, (float)cols), (float)p.eps)));
            else inv = (float)(1.0 / sqrt((double)__fdiv_rn(sq, (float)cols) + p.eps));
        }
        const char* a0;
        const char* a1;
        if (OP == OP_LAYERNORM) {
            a0 = (const char*)p.p0;  // scale
            a1 = (const char*)p.p1;  // bias
        } else {
            const T* m = (const T*)p.p0 + (row / p.rowsPerBatch) * p.modCols + (OP == OP_MODULATED_LN ? p.set * cols * 3 : 0);
            a0 = (const char*)m;            // AdaptiveRMSNorm: scale; ModulatedLayerNorm: shift
            a1 = (const char*)(m + cols);   // AdaptiveRMSNorm: shift; ModulatedLayerNorm: scale
        }
        const char* resRow = (OP == OP_LAYERNORM && p.res) ? (const char*)((const T*)p.res + row * cols) : nullptr;
        for (size_t v0 = lane; v0 < nvec; v0 += 32 * UN) {
            Vec16 xv[UN], c0v[UN], c1v[UN], rv[UN];
#pragma unroll
            for (int u = 0; u < UN; u++) {  // all loads of the batch first
                const size_t v = v0 + 32 * (size_t)u;
                if (v < nvec) {
                    xv[u] = *(const Vec16*)(x + v * 16);
                    c0v[u] = *(const Vec16*)(a0 + v * 16);
                    c1v[u] = *(const Vec16*)(a1 + v * 16);
                    if (resRow) rv[u] = ld_stream(resRow + v * 16);
                }
            }
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const size_t v = v0 + 32 * (size_t)u;
                if (v < nvec) {
                    float f[PER], c0[PER], c1[PER], r[PER];
                    unpack_row<DT>(xv[u], f);
                    unpack_row<DT>(c0v[u], c0);
                    unpack_row<DT>(c1v[u], c1);
#pragma unroll
                    for (int i = 0; i < PER; i++) {
                        if (OP == OP_LAYERNORM) {
                            r[i] = add(mul(mul(sub(f[i], mean), inv), c0[i]), c1[i]);
                        } else {
                            const float scale = OP == OP_ADAPTIVE_RMS ? c0[i] : c1[i], shift = OP == OP_ADAPTIVE_RMS ? c1[i] : c0[i];
                            const float nrm = mul(OP == OP_ADAPTIVE_RMS ? f[i] : sub(f[i], mean), inv);
                            r[i] = add(mul(nrm, add(1.0f, scale)), shift);
                        }
                    }
                    if (resRow) {  // the unfused Add reads the stored (rounded) LayerNorm result
                        float rs[PER];
                        unpack_row<DT>(rv[u], rs);
#pragma unroll
                        for (int i = 0; i < PER; i++) r[i] = add(Storage<DT>::widen(Storage<DT>::narrow(r[i])), rs[i]);
                    }
                    st_stream(o + v * 16, pack_row<DT>(r));
                }
            }
        }
        ring.release();
    }
}

template <int DT> __device__ __forceinline__ void unpack16_fast(const Vec16& v, float* f) {
#pragma unroll
    for (int i = 0; i < 4; i++) unpack16_arith<DT>(v.w[i], f[2 * i], f[2 * i + 1]);
}
template <int DT> __device__ __forceinline__ Vec16 pack16_fast(const float* f) {
    Vec16 v;
#pragma unroll
    for (int i = 0; i < 4; i++) v.w[i] = pack16_arith<DT>(f[2 * i], f[2 * i + 1]);
    return v;
}

// 16-bit rows of up to 32 * VPL vectors: one warp per row, the raw 16-byte vectors of the row held in registers (VPL per lane,
// lane l owns vectors l, l + 32, ...), reductions by shuffles: no CTA-wide barrier between the passes.  The kernel is bound by
// instruction issue (three passes over twice the elements per byte, every product and sum separately rounded), so it is built to
// spend few instructions per element: conversions by the hardware (pack16_arith), four independent partial sums per lane, and for LayerNorm
// the scale and bias rows widened to float32 ONCE per CTA into shared memory (as two float4 planes per vector, so that a
// warp's 16-byte reads are conflict-free) instead of being fetched and widened again for every row.
template <int DT, int OP, int VPL>
__global__ void __launch_bounds__(256) row_norm_warp_kernel(RowNormParams p) {
    using T = typename Storage<DT>::type;
    constexpr int PER = 8;
    extern __shared__ float4 sCoef[];  // LayerNorm: [scale lo | scale hi | bias lo | bias hi][nvec]
    const size_t cols = p.cols, nvec = cols / PER;
    const int lane = threadIdx.x & 31;
    if (OP == OP_LAYERNORM) {
        for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            float c0[PER], c1[PER];
            unpack16_fast<DT>(*(const Vec16*)((const char*)p.p0 + v * 16), c0);
            unpack16_fast<DT>(*(const Vec16*)((const char*)p.p1 + v * 16), c1);
            sCoef[v] = make_float4(c0[0], c0[1], c0[2], c0[3]);
            sCoef[nvec + v] = make_float4(c0[4], c0[5], c0[6], c0[7]);
            sCoef[2 * nvec + v] = make_float4(c1[0], c1[1], c1[2], c1[3]);
            sCoef[3 * nvec + v] = make_float4(c1[4], c1[5], c1[6], c1[7]);
        }
        __syncthreads();
    }
    const size_t warpsTotal = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < p.rows; row += warpsTotal) {
        const char* x = (const char*)((const T*)p.in + row * cols);
        char* o = (char*)((T*)p.out + row * cols);
        Vec16 raw[VPL];
#pragma unroll
        for (int k = 0; k < VPL; k++) {
            const size_t v = lane + (size_t)k * 32;
            if (v < nvec) raw[k] = ld_stream(x + v * 16);
        }
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < VPL; k++) {
            if (lane + (size_t)k * 32 < nvec) {
                float f[PER];
                unpack16_fast<DT>(raw[k], f);
#pragma unroll
                for (int i = 0; i < PER; i++) part[i & 3] += OP == OP_ADAPTIVE_RMS ? f[i] * f[i] : f[i];
            }
        }
        float total = warp_sum_f32((part[0] + part[1]) + (part[2] + part[3]));
        float mean = 0.f, inv;
        if (OP == OP_ADAPTIVE_RMS) {
            inv = (float)(1.0 / sqrt((double)__fdiv_rn(total, (float)cols) + p.eps));
        } else {
            if (DT == DT_BF16) total = Storage<DT>::widen(Storage<DT>::narrow(total));
            mean = __fdiv_rn(total, (float)cols);
            float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < VPL; k++) {
                if (lane + (size_t)k * 32 < nvec) {
                    float f[PER];
                    unpack16_fast<DT>(raw[k], f);
#pragma unroll
                    for (int i = 0; i < PER; i++) {
                        const float d = sub(f[i], mean);
                        sq[i & 3] = add(sq[i & 3], mul(d, d));
                    }
                }
            }
            const float sqt = warp_sum_f32((sq[0] + sq[1]) + (sq[2] + sq[3]));
            if (OP == OP_LAYERNORM) inv = (float)(1.0 / sqrt((double)add(__fdiv_rn(sqt, (float)cols), (float)p.eps)));
            else inv = (float)(1.0 / sqrt((double)__fdiv_rn(sqt, (float)cols) + p.eps));
        }
        const char* a0 = nullptr;
        const char* a1 = nullptr;
        if (OP != OP_LAYERNORM) {
            const T* m = (const T*)p.p0 + (row / p.rowsPerBatch) * p.modCols + (OP == OP_MODULATED_LN ? p.set * cols * 3 : 0);
            a0 = (const char*)m;            // AdaptiveRMSNorm: scale; ModulatedLayerNorm: shift
            a1 = (const char*)(m + cols);   // AdaptiveRMSNorm: shift; ModulatedLayerNorm: scale
        }
        const char* res = (OP == OP_LAYERNORM && p.res) ? (const char*)((const T*)p.res + row * cols) : nullptr;
        // four vectors per round: their residual / modulation loads are all issued before the first is used (the streaming
        // stores in between would otherwise keep every load behind the store before it)
        constexpr int kRound = 4;
#pragma unroll
        for (int k0 = 0; k0 < VPL; k0 += kRound) {
            Vec16 extra0[kRound], extra1[kRound];  // LayerNorm: residual (extra0); the other two: modulation halves
#pragma unroll
            for (int j = 0; j < kRound; j++) {
                const size_t v = lane + (size_t)(k0 + j) * 32;
                if (v < nvec) {
                    if (OP == OP_LAYERNORM) {
                        if (res) extra0[j] = ld_stream(res + v * 16);
                    } else {
                        extra0[j] = *(const Vec16*)(a0 + v * 16);
                        extra1[j] = *(const Vec16*)(a1 + v * 16);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < kRound; j++) {
                const int k = k0 + j;
                const size_t v = lane + (size_t)k * 32;
                if (v < nvec) {
                    float f[PER], c0[PER], c1[PER], r[PER];
                    unpack16_fast<DT>(raw[k], f);
                    if (OP == OP_LAYERNORM) {
                        *(float4*)(c0) = sCoef[v];
                        *(float4*)(c0 + 4) = sCoef[nvec + v];
                        *(float4*)(c1) = sCoef[2 * nvec + v];
                        *(float4*)(c1 + 4) = sCoef[3 * nvec + v];
                    } else {
                        unpack16_fast<DT>(extra0[j], c0);
                        unpack16_fast<DT>(extra1[j], c1);
                    }
#pragma unroll
                    for (int i = 0; i < PER; i++) {
                        if (OP == OP_LAYERNORM) {
                            r[i] = add(mul(mul(sub(f[i], mean), inv), c0[i]), c1[i]);
                        } else {
                            const float scale = OP == OP_ADAPTIVE_RMS ? c0[i] : c1[i], shift = OP == OP_ADAPTIVE_RMS ? c1[i] : c0[i];
                            const float nrm = mul(OP == OP_ADAPTIVE_RMS ? f[i] : sub(f[i], mean), inv);
                            r[i] = add(mul(nrm, add(1.0f, scale)), shift);
                        }
                    }
                    if (OP == OP_LAYERNORM && res) {  // the unfused Add reads the stored (rounded) LayerNorm result
                        float rs[PER];
                        unpack16_fast<DT>(extra0[j], rs);
#pragma unroll
                        for (int i = 0; i < PER; i += 2) {
                            round_pair_arith<DT>(r[i], r[i + 1]);
                            r[i] = add(r[i], rs[i]);
                            r[i + 1] = add(r[i + 1], rs[i + 1]);
                        }
                    }
                    st_stream(o + v * 16, pack16_fast<DT>(r));
                }
            }
        }
    }
}

// float32 rows of up to 256 * VPT vectors (4096 columns at VPT = 4): one 256-thread block per row, the row in registers
// and the NEXT row of the block already on its way while this one is reduced and written.  Three blocks per SM then keep six
// rows (96 KB at 4096 columns) in flight, which a row kernel needs against ~2 us of loaded HBM latency; the shared-memory ring
// of row_norm_ring_kernel holds as many rows but spends a second and third pass of shared-memory reads on each.
// Statistics as the CPU code: float32 sums (a tree here), mean and variance formed in float64.
template <int OP, int VPT, bool RES>
__global__ void __launch_bounds__(256, 3) row_norm_f32_kernel(RowNormParams p) {
    __shared__ float red[2][2][8];  // [row parity][sum | squared differences][warp]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t cols = p.cols, nvec = cols / 4;
    bool has[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) has[k] = (size_t)tid + 256 * (size_t)k < nvec;
    float4 cur[VPT], nxt[VPT];
    auto fetch = [&](size_t row, float4* dst) {
        const float4* x = (const float4*)((const float*)p.in + row * cols);
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                const Vec16 v = ld_stream(x + tid + 256 * k);
                dst[k] = make_float4(__uint_as_float(v.w[0]), __uint_as_float(v.w[1]), __uint_as_float(v.w[2]), __uint_as_float(v.w[3]));
            }
    };
    auto block_sum = [&](float v, float* slot) {  // one barrier; `slot` alternates between rows, so no second one is needed
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) slot[warp] = v;
        __syncthreads();
        return ((slot[0] + slot[4]) + (slot[2] + slot[6])) + ((slot[1] + slot[5]) + (slot[3] + slot[7]));
    };
    if (blockIdx.x < p.rows) fetch(blockIdx.x, cur);
    int par = 0;
    for (size_t row = blockIdx.x; row < p.rows; row += gridDim.x, par ^= 1) {
        if (row + gridDim.x < p.rows) fetch(row + gridDim.x, nxt);
        float4 resv[VPT];
        const float4* res = RES ? (const float4*)((const float*)p.res + row * cols) : nullptr;
        if (RES) {
#pragma unroll
            for (int k = 0; k < VPT; k++)
                if (has[k]) {
                    const Vec16 v = ld_stream(res + tid + 256 * k);
                    resv[k] = make_float4(__uint_as_float(v.w[0]), __uint_as_float(v.w[1]), __uint_as_float(v.w[2]), __uint_as_float(v.w[3]));
                }
        }
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                const float f[4] = {cur[k].x, cur[k].y, cur[k].z, cur[k].w};
#pragma unroll
                for (int i = 0; i < 4; i++) part[i] += OP == OP_ADAPTIVE_RMS ? f[i] * f[i] : f[i];
            }
        const float total = block_sum((part[0] + part[1]) + (part[2] + part[3]), red[par][0]);
        float mean = 0.f, inv;
        if (OP == OP_ADAPTIVE_RMS) {
            inv = (float)(1.0 / sqrt((double)__fdiv_rn(total, (float)cols) + p.eps));
        } else {
            mean = (float)((double)total / (double)cols);
            float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < VPT; k++)
                if (has[k]) {
                    const float f[4] = {cur[k].x, cur[k].y, cur[k].z, cur[k].w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float d = sub(f[i], mean);
                        sq[i] = add(sq[i], mul(d, d));
                    }
                }
            const float sqt = block_sum((sq[0] + sq[1]) + (sq[2] + sq[3]), red[par][1]);
            inv = (float)(1.0 / sqrt((double)sqt / (double)cols + p.eps));
        }
        const float4 *a0, *a1;
        if (OP == OP_LAYERNORM) {
            a0 = (const float4*)p.p0;  // scale
            a1 = (const float4*)p.p1;  // bias
        } else {
            const float* m = (const float*)p.p0 + (row / p.rowsPerBatch) * p.modCols + (OP == OP_MODULATED_LN ? p.set * cols * 3 : 0);
            a0 = (const float4*)m;           // AdaptiveRMSNorm: scale; ModulatedLayerNorm: shift
            a1 = (const float4*)(m + cols);  // AdaptiveRMSNorm: shift; ModulatedLayerNorm: scale
        }
        float4* o = (float4*)((float*)p.out + row * cols);
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                const float4 c0v = a0[tid + 256 * k], c1v = a1[tid + 256 * k];  // a few KB shared by every row: cache hits
                const float f[4] = {cur[k].x, cur[k].y, cur[k].z, cur[k].w};
                const float c0[4] = {c0v.x, c0v.y, c0v.z, c0v.w}, c1[4] = {c1v.x, c1v.y, c1v.z, c1v.w};
                float r[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (OP == OP_LAYERNORM) {
                        r[i] = add(mul(mul(sub(f[i], mean), inv), c0[i]), c1[i]);
                    } else {
                        const float scale = OP == OP_ADAPTIVE_RMS ? c0[i] : c1[i], shift = OP == OP_ADAPTIVE_RMS ? c1[i] : c0[i];
                        const float nrm = mul(OP == OP_ADAPTIVE_RMS ? f[i] : sub(f[i], mean), inv);
                        r[i] = add(mul(nrm, add(1.0f, scale)), shift);
                    }
                }
                if (RES) {
                    r[0] = add(r[0], resv[k].x); r[1] = add(r[1], resv[k].y); r[2] = add(r[2], resv[k].z); r[3] = add(r[3], resv[k].w);
                }
                Vec16 ov;
#pragma unroll
                for (int i = 0; i < 4; i++) ov.w[i] = __float_as_uint(r[i]);
                st_stream(o + tid + 256 * k, ov);
            }
#pragma unroll
        for (int k = 0; k < VPT; k++) cur[k] = nxt[k];
    }
}

// 16-bit rows of 257..512 vectors (up to 4096 columns): the same plan as row_norm_f32_kernel — one 256-thread block per row,
// two vectors per thread, the block's next row in flight — plus what a 16-bit row needs because it is bound by instruction
// issue: the thread's slices of the scale / bias (or modulation) rows are widened ONCE and stay in registers (a thread owns
// the same columns of every row; modulation is reloaded when the batch changes).  Statistics and rounding points of
// row_norm_warp_kernel; the sums are formed by another tree.
template <int DT, int OP, bool RES>
__global__ void __launch_bounds__(256, 3) row_norm_block16_kernel(RowNormParams p) {
    using T = typename Storage<DT>::type;
    constexpr int PER = 8, VPT = 2;
    __shared__ float red[2][2][8];  // [row parity][sum | squared differences][warp]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t cols = p.cols, nvec = cols / PER;
    const bool has1 = (size_t)tid + 256 < nvec;  // (the first vector always exists: nvec > 256)
    const size_t vo[VPT] = {(size_t)tid * 16, ((size_t)tid + 256) * 16};
    auto block_sum = [&](float v, float* slot) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) slot[warp] = v;
        __syncthreads();
        return ((slot[0] + slot[4]) + (slot[2] + slot[6])) + ((slot[1] + slot[5]) + (slot[3] + slot[7]));
    };
    float c0[VPT][PER], c1[VPT][PER];  // LayerNorm: scale, bias; AdaptiveRMSNorm: scale, shift; ModulatedLayerNorm: shift, scale
    size_t coefBatch = ~(size_t)0;
    if (OP == OP_LAYERNORM) {
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (k == 0 || has1) {
                unpack16_fast<DT>(*(const Vec16*)((const char*)p.p0 + vo[k]), c0[k]);
                unpack16_fast<DT>(*(const Vec16*)((const char*)p.p1 + vo[k]), c1[k]);
            }
    }
    Vec16 cur[VPT], nxt[VPT];
    auto fetch = [&](size_t row, Vec16* dst) {
        const char* x = (const char*)((const T*)p.in + row * cols);
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (k == 0 || has1) dst[k] = ld_stream(x + vo[k]);
    };
    if (blockIdx.x < p.rows) fetch(blockIdx.x, cur);
    int par = 0;
    for (size_t row = blockIdx.x; row < p.rows; row += gridDim.x, par ^= 1) {
        if (row + gridDim.x < p.rows) fetch(row + gridDim.x, nxt);
        Vec16 resv[VPT];
        if (RES) {
            const char* res = (const char*)((const T*)p.res + row * cols);
#pragma unroll
            for (int k = 0; k < VPT; k++)
                if (k == 0 || has1) resv[k] = ld_stream(res + vo[k]);
        }
        if (OP != OP_LAYERNORM) {
            const size_t batch = row / p.rowsPerBatch;
            if (batch != coefBatch) {
                coefBatch = batch;
                const T* m = (const T*)p.p0 + batch * p.modCols + (OP == OP_MODULATED_LN ? p.set * cols * 3 : 0);
#pragma unroll
                for (int k = 0; k < VPT; k++)
                    if (k == 0 || has1) {
                        unpack16_fast<DT>(*(const Vec16*)((const char*)m + vo[k]), c0[k]);
                        unpack16_fast<DT>(*(const Vec16*)((const char*)(m + cols) + vo[k]), c1[k]);
                    }
            }
        }
        float f[VPT][PER];
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (k == 0 || has1) {
                unpack16_fast<DT>(cur[k], f[k]);
#pragma unroll
                for (int i = 0; i < PER; i++) part[i & 3] += OP == OP_ADAPTIVE_RMS ? f[k][i] * f[k][i] : f[k][i];
            }
        float total = block_sum((part[0] + part[1]) + (part[2] + part[3]), red[par][0]);
        float mean = 0.f, inv;
        if (OP == OP_ADAPTIVE_RMS) {
            inv = (float)(1.0 / sqrt((double)__fdiv_rn(total, (float)cols) + p.eps));
        } else {
            if (DT == DT_BF16) total = Storage<DT>::widen(Storage<DT>::narrow(total));
            mean = __fdiv_rn(total, (float)cols);
            float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < VPT; k++)
                if (k == 0 || has1) {
#pragma unroll
                    for (int i = 0; i < PER; i++) {
                        const float d = sub(f[k][i], mean);
                        sq[i & 3] = add(sq[i & 3], mul(d, d));
                    }
                }
            const float sqt = block_sum((sq[0] + sq[1]) + (sq[2] + sq[3]), red[par][1]);
            if (OP == OP_LAYERNORM) inv = (float)(1.0 / sqrt((double)add(__fdiv_rn(sqt, (float)cols), (float)p.eps)));
            else inv = (float)(1.0 / sqrt((double)__fdiv_rn(sqt, (float)cols) + p.eps));
        }
        char* o = (char*)((T*)p.out + row * cols);
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (k == 0 || has1) {
                float r[PER];
#pragma unroll
                for (int i = 0; i < PER; i++) {
                    if (OP == OP_LAYERNORM) {
                        r[i] = add(mul(mul(sub(f[k][i], mean), inv), c0[k][i]), c1[k][i]);
                    } else {
                        const float scale = OP == OP_ADAPTIVE_RMS ? c0[k][i] : c1[k][i], shift = OP == OP_ADAPTIVE_RMS ? c1[k][i] : c0[k][i];
                        const float nrm = mul(OP == OP_ADAPTIVE_RMS ? f[k][i] : sub(f[k][i], mean), inv);
                        r[i] = add(mul(nrm, add(1.0f, scale)), shift);
                    }
                }
                if (RES) {  // the unfused Add reads the stored (rounded) LayerNorm result
                    float rs[PER];
                    unpack16_fast<DT>(resv[k], rs);
#pragma unroll
                    for (int i = 0; i < PER; i += 2) {
                        round_pair_arith<DT>(r[i], r[i + 1]);
                        r[i] = add(r[i], rs[i]);
                        r[i + 1] = add(r[i + 1], rs[i + 1]);
                    }
                }
                st_stream(o + vo[k], pack16_fast<DT>(r));
            }
#pragma unroll
        for (int k = 0; k < VPT; k++) cur[k] = nxt[k];
    }
}

constexpr size_t kMaxCols = 16384;  // 64 KB of shared memory for the widened row

template <int OP>
int launch_row_norm(Context* ctx, int dt, const RowNormParams& p, CUDAStatus* status, const char* what) {
    if (p.cols > kMaxCols) return fail(status, -6, "%s: last dimension %zu exceeds the supported maximum of %zu", what, p.cols, kMaxCols);
    const size_t smem = (p.cols * sizeof(float) + 15) & ~(size_t)15;
    size_t blocks = p.rows, cap = (size_t)ctx->smCount * 8;
    if (blocks > cap) blocks = cap;
    const size_t es = dt == DT_F32 ? 4 : 2, per = 16 / es;
    // the modulation row of a batch starts at batch * modCols (+ set * 3 * cols) elements and its second half cols further on
    const bool vec = p.cols % per == 0 && (((uintptr_t)p.in | (uintptr_t)p.out | (uintptr_t)p.p0 | (uintptr_t)p.p1 | (uintptr_t)p.res) & 15u) == 0 &&
                     (OP == OP_LAYERNORM || p.modCols % per == 0);
    // Measured at 16384 x 4096: 16-bit rows are bound by instruction latency, not by memory, and run fastest with the row in
    // registers (one warp per row, 3.4-3.8 TB/s against 3.0-3.6 through shared memory); float32 rows run fastest through the
    // shared-memory row pipeline (4.3-5.0 TB/s against 3.8-4.3).  Rows that fit neither take one CTA per row.
    const size_t nvec = vec ? p.cols / per : 0;
    const int vpl = (es == 4 || nvec == 0 || nvec > 512) ? 0 : nvec <= 128 ? 4 : nvec <= 256 ? 8 : 16;
    size_t warpBlocks = (p.rows + 7) / 8;
    if (warpBlocks > cap) warpBlocks = cap;
    const rowpipe::Plan plan = (vec && !vpl) ? rowpipe::plan(p.cols * es) : rowpipe::Plan{0, 0, 0};
    size_t ringBlocks = 1;
    if (plan.warps) {
        size_t perSm = (220 * 1024) / (plan.smem + 1024);
        if (perSm < 1) perSm = 1;
        if (perSm > 4) perSm = 4;
        ringBlocks = (p.rows + plan.warps - 1) / plan.warps;
        if (ringBlocks > (size_t)ctx->smCount * perSm) ringBlocks = (size_t)ctx->smCount * perSm;
    }
#define ROWNORM_WARP(DT, VPL)                                                                                       \
    do {                                                                                                            \
        if (coefSmem > 48 * 1024) cudaFuncSetAttribute(row_norm_warp_kernel<DT, OP, VPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)coefSmem); \
        row_norm_warp_kernel<DT, OP, VPL><<<(unsigned)warpBlocks, 256, coefSmem, ctx->stream>>>(p);                 \
    } while (0)
#define ROWNORM_LAUNCH(DT)                                                                                          \
    do {                                                                                                            \
        if (plan.warps) {                                                                                           \
            cudaFuncSetAttribute(row_norm_ring_kernel<DT, OP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem); \
            row_norm_ring_kernel<DT, OP><<<(unsigned)ringBlocks, plan.warps * 32, plan.smem, ctx->stream>>>(p, plan.stages); \
        } else if (vec) {                                                                                           \
            if (smem > 48 * 1024) cudaFuncSetAttribute(row_norm_kernel<DT, OP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            row_norm_kernel<DT, OP, true><<<(unsigned)blocks, 256, smem, ctx->stream>>>(p);                          \
        } else {                                                                                                    \
            if (smem > 48 * 1024) cudaFuncSetAttribute(row_norm_kernel<DT, OP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            row_norm_kernel<DT, OP, false><<<(unsigned)blocks, 256, smem, ctx->stream>>>(p);                         \
        }                                                                                                           \
    } while (0)
#define ROWNORM_LAUNCH16(DT)                                                                                        \
    do {                                                                                                            \
        if (OP == OP_LAYERNORM && vec && nvec > 256 && nvec <= 512) {                                               \
            const size_t resident = (size_t)ctx->smCount * 3;                                                      \
            const unsigned g16 = (unsigned)(p.rows < resident ? p.rows : resident);                                \
            if (OP == OP_LAYERNORM && p.res) row_norm_block16_kernel<DT, OP, OP == OP_LAYERNORM><<<g16, 256, 0, ctx->stream>>>(p); \
            else row_norm_block16_kernel<DT, OP, false><<<g16, 256, 0, ctx->stream>>>(p);                           \
        } else if (vpl == 4) ROWNORM_WARP(DT, 4);                                                                          \
        else if (vpl == 8) ROWNORM_WARP(DT, 8);                                                                     \
        else if (vpl == 16) ROWNORM_WARP(DT, 16);                                                                   \
        else ROWNORM_LAUNCH(DT);                                                                                    \
    } while (0)
    // 16-bit rows, measured at 16384 x 4096 bf16 (block per row with the next row in flight / warp per row): LayerNorm 4.91 / 4.60
    // TB/s, with the fused residual 5.76 / 5.03; AdaptiveRMSNorm 4.15 / 5.40, ModulatedLayerNorm 3.51 / 4.63: LayerNorm takes the
    // block kernel, the two modulated norms the warp kernel.
    // LayerNorm's scale and bias rows, widened once per CTA: 2 * cols floats
    const size_t coefSmem = OP == OP_LAYERNORM ? p.cols * 2 * sizeof(float) : 0;
    if (dt == DT_F32 && vec && nvec > 256 && nvec <= 1024) {
        // measured at 16384 x 4096: the register kernel with the next row in flight against the shared-memory ring
        const size_t resident = (size_t)ctx->smCount * 3;
        const unsigned g32 = (unsigned)(p.rows < resident ? p.rows : resident);
        if (OP == OP_LAYERNORM && p.res) {
            if (nvec <= 512) row_norm_f32_kernel<OP, 2, OP == OP_LAYERNORM><<<g32, 256, 0, ctx->stream>>>(p);
            else row_norm_f32_kernel<OP, 4, OP == OP_LAYERNORM><<<g32, 256, 0, ctx->stream>>>(p);
        } else {
            if (nvec <= 512) row_norm_f32_kernel<OP, 2, false><<<g32, 256, 0, ctx->stream>>>(p);
            else row_norm_f32_kernel<OP, 4, false><<<g32, 256, 0, ctx->stream>>>(p);
        }
    } else if (dt == DT_F32) ROWNORM_LAUNCH(DT_F32);
    else if (dt == DT_BF16) ROWNORM_LAUNCH16(DT_BF16);
    else if (dt == DT_F16) ROWNORM_LAUNCH16(DT_F16);
    else return fail(status, -6, "%s: unsupported dtype %d", what, dt);
#undef ROWNORM_LAUNCH16
#undef ROWNORM_LAUNCH
#undef ROWNORM_WARP
    return check_launch(ctx, status, what);
}

}  // namespace

}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_layernorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                                       CUDABufferRef biasRef, CUDABufferRef outputRef, uint32_t rows, uint32_t cols, float epsilon,
                                       uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (rows == 0 || cols == 0) return ok(status);
    const size_t es = dtype_size(elementDType);
    if (es == 0) return fail(status, -6, "layernorm: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(inputRef, "input", (size_t)rows * cols * es);
    PUTER_REQUIRE(outputRef, "output", (size_t)rows * cols * es);
    PUTER_REQUIRE(scaleRef, "scale", (size_t)cols * es);
    PUTER_REQUIRE(biasRef, "bias", (size_t)cols * es);
    RowNormParams p = {};
    p.in = dev_ptr(inputRef); p.p0 = dev_ptr(scaleRef); p.p1 = dev_ptr(biasRef); p.out = dev_ptr(outputRef);
    p.rows = rows; p.cols = cols; p.rowsPerBatch = 1; p.errorFlag = ctx->errorFlag;
    p.eps = epsilon > 0.f ? (double)epsilon : 1e-5;  // the CPU op has no epsilon argument: 1e-5 (compute.go:11)
    return launch_row_norm<OP_LAYERNORM>(ctx, elementDType, p, status, "layernorm");
}

// The catalog's fused entry layernorm + add -> layernorm_residual (fusion/catalog.go:183-205, four inputs, ULP bound 2):
// out = LayerNorm(x, scale, bias) + residual, the LayerNorm result rounded to the storage type before the add exactly as the
// two separate ops would (so the fused result equals the unfused one bit for bit, inside the catalog's bound).
extern "C" int cuda_dispatch_layernorm_residual(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                                                CUDABufferRef biasRef, CUDABufferRef residualRef, CUDABufferRef outputRef, uint32_t rows,
                                                uint32_t cols, float epsilon, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (rows == 0 || cols == 0) return ok(status);
    const size_t es = dtype_size(elementDType);
    if (es == 0) return fail(status, -6, "layernorm_residual: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(inputRef, "input", (size_t)rows * cols * es);
    PUTER_REQUIRE(residualRef, "residual", (size_t)rows * cols * es);
    PUTER_REQUIRE(outputRef, "output", (size_t)rows * cols * es);
    PUTER_REQUIRE(scaleRef, "scale", (size_t)cols * es);
    PUTER_REQUIRE(biasRef, "bias", (size_t)cols * es);
    RowNormParams p = {};
    p.in = dev_ptr(inputRef); p.p0 = dev_ptr(scaleRef); p.p1 = dev_ptr(biasRef); p.res = dev_ptr(residualRef); p.out = dev_ptr(outputRef);
    p.rows = rows; p.cols = cols; p.rowsPerBatch = 1; p.errorFlag = ctx->errorFlag;
    p.eps = epsilon > 0.f ? (double)epsilon : 1e-5;
    return launch_row_norm<OP_LAYERNORM>(ctx, elementDType, p, status, "layernorm_residual");
}

static int check_modulated(CUDAStatus* status, const char* what, double eps, uint32_t rows, uint32_t rowsPerBatch, uint64_t modCols,
                           uint64_t needCols) {
    if (!(eps > 0)) return fail(status, -2, "%s: epsilon must be positive, got %g", what, eps);
    if (rowsPerBatch == 0) return fail(status, -2, "%s: rowsPerBatch must be positive", what);
    if (rows % rowsPerBatch != 0) return fail(status, -2, "%s: rows must be divisible by rowsPerBatch", what);
    if (modCols < needCols) return fail(status, -2, "%s: modulation width too small", what);
    return 0;
}

extern "C" int cuda_dispatch_adaptive_rmsnorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef modulationRef,
                                              CUDABufferRef outputRef, uint32_t rows, uint32_t cols, uint32_t rowsPerBatch,
                                              uint32_t modulationCols, double epsilon, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    int rc = check_modulated(status, "adaptive rmsnorm", epsilon, rows, rowsPerBatch, modulationCols, 2ull * cols);
    if (rc != 0) return rc;
    if (rows == 0 || cols == 0) return ok(status);
    const size_t es = dtype_size(elementDType);
    if (es == 0) return fail(status, -6, "adaptive rmsnorm: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(inputRef, "input", (size_t)rows * cols * es);
    PUTER_REQUIRE(outputRef, "output", (size_t)rows * cols * es);
    PUTER_REQUIRE(modulationRef, "modulation", (size_t)(rows / rowsPerBatch) * modulationCols * es);
    RowNormParams p = {};
    p.in = dev_ptr(inputRef); p.p0 = dev_ptr(modulationRef); p.out = dev_ptr(outputRef);
    p.rows = rows; p.cols = cols; p.rowsPerBatch = rowsPerBatch; p.modCols = modulationCols; p.eps = epsilon; p.errorFlag = ctx->errorFlag;
    return launch_row_norm<OP_ADAPTIVE_RMS>(ctx, elementDType, p, status, "adaptive rmsnorm");
}

extern "C" int cuda_dispatch_modulated_layernorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef,
                                                 CUDABufferRef modulationRef, CUDABufferRef outputRef, uint32_t rows, uint32_t cols,
                                                 uint32_t rowsPerBatch, uint32_t modulationCols, uint32_t set, double epsilon,
                                                 uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    int rc = check_modulated(status, "modulated layernorm", epsilon, rows, rowsPerBatch, modulationCols, ((uint64_t)set * 3 + 2) * cols);
    if (rc != 0) return rc;
    if (rows == 0 || cols == 0) return ok(status);
    const size_t es = dtype_size(elementDType);
    if (es == 0) return fail(status, -6, "modulated layernorm: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(inputRef, "input", (size_t)rows * cols * es);
    PUTER_REQUIRE(outputRef, "output", (size_t)rows * cols * es);
    PUTER_REQUIRE(modulationRef, "modulation", (size_t)(rows / rowsPerBatch) * modulationCols * es);
    RowNormParams p = {};
    p.in = dev_ptr(inputRef); p.p0 = dev_ptr(modulationRef); p.out = dev_ptr(outputRef);
    p.rows = rows; p.cols = cols; p.rowsPerBatch = rowsPerBatch; p.modCols = modulationCols; p.set = set; p.eps = epsilon;
    p.errorFlag = ctx->errorFlag;
    return launch_row_norm<OP_MODULATED_LN>(ctx, elementDType, p, status, "modulated layernorm");
}
