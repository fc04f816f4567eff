// RMSNorm and the fused residual-add + RMSNorm + gated-residual row kernel.
//
// Reference semantics (device/cpu/layernorm/compute.go:35-59,129-143,177-207,350-385):
//   f32     ss = float32(sum in float64 of x^2);  inv = float32(1/sqrt(float64(ss)/n + eps));  out = x * (inv * gamma)
//   16-bit  ss = storage-rounded(sum in float32 of x^2) — the dot product result is rounded to bf16/f16
//           (device/cpu/dot/bf16_generic.go:9-21);  ms = ss / n;  inv = float32(1/sqrt(float64(ms) + eps));
//           out = narrow((x * inv) * gamma)
// The row sum is formed by a tree reduction here instead of a sequential loop; for f32 it is carried in
// float64 so the float32 result is the same, for 16-bit types the float32 sum can differ in the last bits,
// which only matters when it falls within ~1e-6 of a bf16/f16 rounding boundary.
//
// Layout: one 256-thread block per row (grid-stride over rows, grid = multiple of the SM count); a row is
// read once with 16-byte loads and kept in registers between the reduction and the scaling pass.
#include "common.cuh"

namespace puter {

template <int DT> struct Lanes { static constexpr int kPer = DT == DT_F32 ? 4 : 8; };

// (16-bit data here always goes through arithmetic before it is stored: the hardware conversions of pack16_arith apply)
template <int DT> __device__ __forceinline__ void unpack(const Vec16& v, float* f) {
    if (DT == DT_F32) {
#pragma unroll
        for (int i = 0; i < 4; i++) f[i] = __uint_as_float(v.w[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) unpack16_arith<DT>(v.w[i], f[2 * i], f[2 * i + 1]);
    }
}
template <int DT> __device__ __forceinline__ Vec16 pack(const float* f) {
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
// rounds to the storage dtype and back (identity for f32)
template <int DT> __device__ __forceinline__ float round_storage(float v) {
    if (DT == DT_F32) return v;
    return Storage<DT>::widen(Storage<DT>::narrow(v));
}

template <typename T> __device__ __forceinline__ T block_sum(T v, T* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();  // smem may still be read from the previous row
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    T t = lane < nw ? smem[lane] : T(0);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

template <int DT> __device__ __forceinline__ float inv_rms(double sumsq, size_t cols, double eps) {
    if (DT == DT_F32) {
        float ss = (float)sumsq;
        return (float)(1.0 / sqrt((double)ss / (double)cols + eps));
    }
    float ss = round_storage<DT>((float)sumsq);
    float ms = __fdiv_rn(ss, (float)cols);
    return (float)(1.0 / sqrt((double)ms + eps));
}

struct RowArgs {
    const void* x;         // input rows
    const void* residual;  // FUSED: added to x first
    const void* scale;     // gamma [cols]
    const void* branch;    // FUSED + gated: branch rows
    const void* mod;       // FUSED + gated: modulation [batches, modCols]
    void* hOut;            // FUSED: x + residual (optional)
    void* normOut;         // RMSNorm result
    void* gatedOut;        // FUSED + gated
    size_t rows, cols, rowsPerBatch, modCols, set;
    double eps;
    // all-gather fused into the stores: every finished vector of normOut / gatedOut is also written to the same place of up
    // to 7 peers' gathered tensors (plain stores over NVLink); peer pointers address row 0 of the rank's slice
    char* normPeer[7];
    char* gatedPeer[7];
    int nPeer;
};

// read-once input: through the non-coherent path, unless an output of the same launch aliases an input (in-place use)
template <bool INPLACE> __device__ __forceinline__ Vec16 ld_in(const void* p) { return INPLACE ? *(const Vec16*)p : ld_stream(p); }

// MAXV 16-byte vectors per thread are cached in registers; rows longer than MAXV*blockDim vectors re-read.
// INPLACE: an output is the same buffer as x or residual (an in-place residual stream).  Every element is then read by
// the one thread that later writes it, before it writes it; inputs are read with plain loads, and the second pass over
// the vectors beyond the register cache takes x + residual from hOut (already stored) instead of adding again.
template <int DT, int MAXV, bool FUSED, bool INPLACE>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(RowArgs a) {
    constexpr int PER = Lanes<DT>::kPer;
    constexpr size_t ES = DT == DT_F32 ? 4 : 2;
    __shared__ double smemD[32];
    __shared__ float smemF[32];
    const size_t nvec = a.cols / PER;
    const bool gated = FUSED && a.branch != nullptr;
    for (size_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const char* xr = (const char*)a.x + row * a.cols * ES;
        const char* rr = FUSED ? (const char*)a.residual + row * a.cols * ES : nullptr;
        Vec16 cache[MAXV];
        Vec16 cacheB[MAXV];  // branch rows, fetched before the reduction so their latency overlaps it
        double accD = 0.0;
        float accF = 0.f;
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            size_t v = threadIdx.x + (size_t)i * blockDim.x;
            if (v < nvec) {
                Vec16 in = ld_in<INPLACE>(xr + v * 16);
                if (gated) cacheB[i] = ld_stream((const char*)a.branch + row * a.cols * ES + v * 16);  // never aliased (checked by the host)
                float f[PER];
                unpack<DT>(in, f);
                if (FUSED) {
                    Vec16 rin = ld_in<INPLACE>(rr + v * 16);
                    float g[PER];
                    unpack<DT>(rin, g);
                    if (DT == DT_F32) {
#pragma unroll
                        for (int j = 0; j < PER; j++) f[j] = add(f[j], g[j]);
                        in = pack<DT>(f);
                    } else {
                        // the unfused Add would store its result in the 16-bit type: round here, once, pair by pair
#pragma unroll
                        for (int j = 0; j < PER; j += 2) {
                            f[j] = add(f[j], g[j]);
                            f[j + 1] = add(f[j + 1], g[j + 1]);
                            in.w[j / 2] = round_pair_arith<DT>(f[j], f[j + 1]);
                        }
                    }
                    if (a.hOut) st_stream((char*)a.hOut + row * a.cols * ES + v * 16, in);
                }
                cache[i] = in;
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    if (DT == DT_F32) accD += (double)f[j] * (double)f[j];
                    else accF = fmaf(f[j], f[j], accF);
                }
            }
        }
        // rows that do not fit the register cache: keep summing from memory
        for (size_t v = threadIdx.x + (size_t)MAXV * blockDim.x; v < nvec; v += blockDim.x) {
            Vec16 in = *(const Vec16*)(xr + v * 16);
            float f[PER];
            unpack<DT>(in, f);
            if (FUSED) {
                Vec16 rin = *(const Vec16*)(rr + v * 16);
                float g[PER];
                unpack<DT>(rin, g);
#pragma unroll
                for (int j = 0; j < PER; j++) f[j] = round_storage<DT>(add(f[j], g[j]));
                if (a.hOut) *(Vec16*)((char*)a.hOut + row * a.cols * ES + v * 16) = pack<DT>(f);
            }
#pragma unroll
            for (int j = 0; j < PER; j++) {
                if (DT == DT_F32) accD += (double)f[j] * (double)f[j];
                else accF = fmaf(f[j], f[j], accF);
            }
        }
        double total = DT == DT_F32 ? block_sum<double>(accD, smemD) : (double)block_sum<float>(accF, smemF);
        const float inv = inv_rms<DT>(total, a.cols, a.eps);
        const size_t mo = gated ? (row / a.rowsPerBatch) * a.modCols + a.set * a.cols * 3 + a.cols * 2 : 0;

        auto finish = [&](size_t v, const Vec16& hv, const Vec16* bv) {
            float h[PER], g[PER], o[PER];
            unpack<DT>(hv, h);
            unpack<DT>(*(const Vec16*)((const char*)a.scale + v * 16), g);
#pragma unroll
            for (int j = 0; j < PER; j++) {
                if (DT == DT_F32) o[j] = mul(h[j], mul(inv, g[j]));   // x * (inv * gamma), compute.go:358-362
                else o[j] = mul(mul(h[j], inv), g[j]);                // (x * inv) * gamma, compute.go:370-373
            }
            const Vec16 nv = pack<DT>(o);
            st_stream((char*)a.normOut + row * a.cols * ES + v * 16, nv);
            for (int r = 0; r < a.nPeer; r++) st_stream(a.normPeer[r] + row * a.cols * ES + v * 16, nv);
            if (gated) {
                float b[PER], m[PER];
                unpack<DT>(bv ? *bv : ld_stream((const char*)a.branch + row * a.cols * ES + v * 16), b);
                unpack<DT>(*(const Vec16*)((const char*)a.mod + (mo + v * PER) * ES), m);
#pragma unroll
                for (int j = 0; j < PER; j++) o[j] = add(h[j], mul(m[j], b[j]));
                const Vec16 gv = pack<DT>(o);
                st_stream((char*)a.gatedOut + row * a.cols * ES + v * 16, gv);
                for (int r = 0; r < a.nPeer; r++) st_stream(a.gatedPeer[r] + row * a.cols * ES + v * 16, gv);
            }
        };
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            size_t v = threadIdx.x + (size_t)i * blockDim.x;
            if (v < nvec) finish(v, cache[i], &cacheB[i]);
        }
        for (size_t v = threadIdx.x + (size_t)MAXV * blockDim.x; v < nvec; v += blockDim.x) {
            Vec16 hv;
            if (FUSED && INPLACE && a.hOut) {
                hv = *(const Vec16*)((const char*)a.hOut + row * a.cols * ES + v * 16);  // stored by this thread in the first pass
            } else if (FUSED) {
                float f[PER], g[PER];
                unpack<DT>(*(const Vec16*)(xr + v * 16), f);
                unpack<DT>(*(const Vec16*)(rr + v * 16), g);
#pragma unroll
                for (int j = 0; j < PER; j++) f[j] = round_storage<DT>(add(f[j], g[j]));
                hv = pack<DT>(f);
            } else {
                hv = *(const Vec16*)(xr + v * 16);
            }
            finish(v, hv, nullptr);
        }
    }
}

// Plain RMSNorm of rows of up to 256 * VPT vectors: one 256-thread block per row, the row in registers, the thread's slice of
// the scale row widened once, and the NEXT row of the block already on its way while this one is reduced and written (a row
// kernel needs several rows per SM in flight against ~2 us of loaded HBM latency).  Arithmetic, rounding points and summation
// tree of rmsnorm_rows_kernel: bit-identical results.
template <int DT, int VPT>
__global__ void __launch_bounds__(256, DT == DT_F32 ? 3 : 4) rmsnorm_ahead_kernel(RowArgs a) {
    constexpr int PER = Lanes<DT>::kPer;
    constexpr size_t ES = DT == DT_F32 ? 4 : 2;
    __shared__ double redD[2][8];
    __shared__ float redF[2][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t nvec = a.cols / PER, rowBytes = a.cols * ES;
    bool has[VPT];
    float sc[VPT][PER];
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        has[k] = (size_t)tid + 256 * (size_t)k < nvec;
        if (has[k]) unpack<DT>(*(const Vec16*)((const char*)a.scale + ((size_t)tid + 256 * k) * 16), sc[k]);
    }
    Vec16 cur[VPT], nxt[VPT];
    auto fetch = [&](size_t row, Vec16* dst) {
        const char* x = (const char*)a.x + row * rowBytes;
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) dst[k] = ld_stream(x + ((size_t)tid + 256 * k) * 16);
    };
    if (blockIdx.x < a.rows) fetch(blockIdx.x, cur);
    int par = 0;
    for (size_t row = blockIdx.x; row < a.rows; row += gridDim.x, par ^= 1) {
        if (row + gridDim.x < a.rows) fetch(row + gridDim.x, nxt);
        double accD = 0.0;
        float accF = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                float f[PER];
                unpack<DT>(cur[k], f);
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    if (DT == DT_F32) accD += (double)f[j] * (double)f[j];
                    else accF = fmaf(f[j], f[j], accF);
                }
            }
        double total;
        if (DT == DT_F32) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) accD += __shfl_xor_sync(0xffffffffu, accD, o);
            if (lane == 0) redD[par][warp] = accD;
            __syncthreads();
            const double* r = redD[par];
            total = ((r[0] + r[4]) + (r[2] + r[6])) + ((r[1] + r[5]) + (r[3] + r[7]));
        } else {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) accF += __shfl_xor_sync(0xffffffffu, accF, o);
            if (lane == 0) redF[par][warp] = accF;
            __syncthreads();
            const float* r = redF[par];
            total = (double)(((r[0] + r[4]) + (r[2] + r[6])) + ((r[1] + r[5]) + (r[3] + r[7])));
        }
        const float inv = inv_rms<DT>(total, a.cols, a.eps);
        char* o = (char*)a.normOut + row * rowBytes;
#pragma unroll
        for (int k = 0; k < VPT; k++)
            if (has[k]) {
                float h[PER], r[PER];
                unpack<DT>(cur[k], h);
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    if (DT == DT_F32) r[j] = mul(h[j], mul(inv, sc[k][j]));   // x * (inv * gamma), compute.go:358-362
                    else r[j] = mul(mul(h[j], inv), sc[k][j]);                // (x * inv) * gamma, compute.go:370-373
                }
                st_stream(o + ((size_t)tid + 256 * k) * 16, pack<DT>(r));
            }
#pragma unroll
        for (int k = 0; k < VPT; k++) cur[k] = nxt[k];
    }
}

// The fused row of the transformer block at its usual width: 16-bit rows of 257..512 vectors (2056..4096 columns), one
// 256-thread block per row, two vectors per thread.  The generic kernel above spends ~48 instructions per element on this
// shape and is bound by instruction issue; this one spends about a third of that:
//   * a thread owns the same two vector positions of every row, so its slice of the scale row (and of the batch's modulation
//     row, reloaded when the batch changes) is widened to float32 ONCE and stays in registers;
//   * all six loads of a row (x, residual, branch) are issued before the first is used;
//   * x + residual stays in float32 registers between the reduction and the outputs; conversions by the hardware;
//   * one barrier per row: the per-warp partial sums alternate between two shared arrays.
// Same arithmetic, rounding points and summation tree as the generic kernel: the results are bit-identical.
template <int DT, bool GATED, bool INPLACE>
__global__ void __launch_bounds__(256, 3) add_rmsnorm16_kernel(RowArgs a) {
    constexpr int PER = 8;
    __shared__ float red[2][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t nvec = a.cols / PER, rowBytes = a.cols * 2;
    const size_t vo[2] = {(size_t)tid * 16, (size_t)(tid + 256) * 16};  // byte offsets of this thread's vectors in a row
    const bool has1 = (size_t)tid + 256 < nvec;                           // (the first always exists: nvec > 256)
    float sc[2][PER];
    unpack<DT>(*(const Vec16*)((const char*)a.scale + vo[0]), sc[0]);
    if (has1) unpack<DT>(*(const Vec16*)((const char*)a.scale + vo[1]), sc[1]);
    float md[2][PER];
    size_t mdBatch = ~(size_t)0;
    int par = 0;
    for (size_t row = blockIdx.x; row < a.rows; row += gridDim.x, par ^= 1) {
        const size_t ro = row * rowBytes;
        Vec16 xin[2], rin[2], bin[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (i == 0 || has1) {
                xin[i] = ld_in<INPLACE>((const char*)a.x + ro + vo[i]);
                rin[i] = ld_in<INPLACE>((const char*)a.residual + ro + vo[i]);
                if (GATED) bin[i] = ld_stream((const char*)a.branch + ro + vo[i]);  // never aliased (checked by the host)
            }
        }
        if (GATED) {
            const size_t batch = row / a.rowsPerBatch;
            if (batch != mdBatch) {
                mdBatch = batch;
                const char* m = (const char*)a.mod + (batch * a.modCols + a.set * a.cols * 3 + a.cols * 2) * 2;
                unpack<DT>(*(const Vec16*)(m + vo[0]), md[0]);
                if (has1) unpack<DT>(*(const Vec16*)(m + vo[1]), md[1]);
            }
        }
        float h[2][PER];
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (i == 0 || has1) {
                float g[PER];
                unpack<DT>(xin[i], h[i]);
                unpack<DT>(rin[i], g);
                Vec16 hv;
                // the unfused Add would store its result in the 16-bit type: round here, once, pair by pair
#pragma unroll
                for (int j = 0; j < PER; j += 2) {
                    h[i][j] = add(h[i][j], g[j]);
                    h[i][j + 1] = add(h[i][j + 1], g[j + 1]);
                    hv.w[j / 2] = round_pair_arith<DT>(h[i][j], h[i][j + 1]);
                }
                if (a.hOut) st_stream((char*)a.hOut + ro + vo[i], hv);
#pragma unroll
                for (int j = 0; j < PER; j++) acc = fmaf(h[i][j], h[i][j], acc);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) red[par][warp] = acc;
        __syncthreads();
        // the order of the generic kernel's two-level shuffle tree
        const float* r = red[par];
        const float total = ((r[0] + r[4]) + (r[2] + r[6])) + ((r[1] + r[5]) + (r[3] + r[7]));
        const float inv = inv_rms<DT>((double)total, a.cols, a.eps);
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (i == 0 || has1) {
                float o[PER];
#pragma unroll
                for (int j = 0; j < PER; j++) o[j] = mul(mul(h[i][j], inv), sc[i][j]);  // (x * inv) * gamma, compute.go:370-373
                const Vec16 nv = pack<DT>(o);
                st_stream((char*)a.normOut + ro + vo[i], nv);
                for (int p = 0; p < a.nPeer; p++) st_stream(a.normPeer[p] + ro + vo[i], nv);
                if (GATED) {
                    float b[PER];
                    unpack<DT>(bin[i], b);
#pragma unroll
                    for (int j = 0; j < PER; j++) o[j] = add(h[i][j], mul(md[i][j], b[j]));
                    const Vec16 gv = pack<DT>(o);
                    st_stream((char*)a.gatedOut + ro + vo[i], gv);
                    for (int p = 0; p < a.nPeer; p++) st_stream(a.gatedPeer[p] + ro + vo[i], gv);
                }
            }
        }
    }
}

// Rows of up to 16 vectors per lane (4096 16-bit / 2048 float32 columns): one WARP per row.  No block barrier, the
// reduction is five shuffles, and every lane has up to 16 independent 16-byte loads in flight per stream, which is what
// a latency-bound 8 KB row needs to keep HBM busy.  Same arithmetic and rounding points as the block-per-row kernel.
template <int DT, bool FUSED>
__global__ void __launch_bounds__(256) rmsnorm_warp_rows_kernel(RowArgs a) {
    constexpr int PER = Lanes<DT>::kPer;
    constexpr size_t ES = DT == DT_F32 ? 4 : 2;
    constexpr int WV = 16;
    const size_t nvec = a.cols / PER;
    const bool gated = FUSED && a.branch != nullptr;
    const int lane = threadIdx.x & 31;
    const size_t warpsTotal = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < a.rows; row += warpsTotal) {
        const char* xr = (const char*)a.x + row * a.cols * ES;
        const char* rr = FUSED ? (const char*)a.residual + row * a.cols * ES : nullptr;
        Vec16 cache[WV];
        Vec16 res[WV];
#pragma unroll
        for (int i = 0; i < WV; i++) {
            const size_t v = lane + 32 * (size_t)i;
            if (v < nvec) {
                cache[i] = ld_stream(xr + v * 16);
                if (FUSED) res[i] = ld_stream(rr + v * 16);
            }
        }
        double accD = 0.0;
        float accF = 0.f;
#pragma unroll
        for (int i = 0; i < WV; i++) {
            const size_t v = lane + 32 * (size_t)i;
            if (v < nvec) {
                float f[PER];
                unpack<DT>(cache[i], f);
                if (FUSED) {
                    float g[PER];
                    unpack<DT>(res[i], g);
#pragma unroll
                    for (int j = 0; j < PER; j++) f[j] = round_storage<DT>(add(f[j], g[j]));
                    cache[i] = pack<DT>(f);
                    if (a.hOut) st_stream((char*)a.hOut + row * a.cols * ES + v * 16, cache[i]);
                }
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    if (DT == DT_F32) accD += (double)f[j] * (double)f[j];
                    else accF = fmaf(f[j], f[j], accF);
                }
            }
        }
        if (gated) {
            // the branch rows reuse the residual registers; their loads fly during the reduction
#pragma unroll
            for (int i = 0; i < WV; i++) {
                const size_t v = lane + 32 * (size_t)i;
                if (v < nvec) res[i] = ld_stream((const char*)a.branch + row * a.cols * ES + v * 16);
            }
        }
        double total;
        if (DT == DT_F32) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) accD += __shfl_xor_sync(0xffffffffu, accD, o);
            total = accD;
        } else {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) accF += __shfl_xor_sync(0xffffffffu, accF, o);
            total = (double)accF;
        }
        const float inv = inv_rms<DT>(total, a.cols, a.eps);
        const size_t mo = gated ? (row / a.rowsPerBatch) * a.modCols + a.set * a.cols * 3 + a.cols * 2 : 0;
#pragma unroll
        for (int i = 0; i < WV; i++) {
            const size_t v = lane + 32 * (size_t)i;
            if (v < nvec) {
                float h[PER], g[PER], o[PER];
                unpack<DT>(cache[i], h);
                unpack<DT>(*(const Vec16*)((const char*)a.scale + v * 16), g);
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    if (DT == DT_F32) o[j] = mul(h[j], mul(inv, g[j]));
                    else o[j] = mul(mul(h[j], inv), g[j]);
                }
                st_stream((char*)a.normOut + row * a.cols * ES + v * 16, pack<DT>(o));
                if (gated) {
                    float b[PER], m[PER];
                    unpack<DT>(res[i], b);
                    unpack<DT>(*(const Vec16*)((const char*)a.mod + (mo + v * PER) * ES), m);
#pragma unroll
                    for (int j = 0; j < PER; j++) o[j] = add(h[j], mul(m[j], b[j]));
                    st_stream((char*)a.gatedOut + row * a.cols * ES + v * 16, pack<DT>(o));
                }
            }
        }
    }
}

// any alignment, any column count: scalar loads, same arithmetic
template <int DT, bool FUSED>
__global__ void __launch_bounds__(256) rmsnorm_rows_scalar_kernel(RowArgs a) {
    using T = typename Storage<DT>::type;
    __shared__ double smemD[32];
    __shared__ float smemF[32];
    const bool gated = FUSED && a.branch != nullptr;
    for (size_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const T* xr = (const T*)a.x + row * a.cols;
        const T* rr = FUSED ? (const T*)a.residual + row * a.cols : nullptr;
        double accD = 0.0;
        float accF = 0.f;
        for (size_t c = threadIdx.x; c < a.cols; c += blockDim.x) {
            float h = Storage<DT>::load(xr, c);
            if (FUSED) h = round_storage<DT>(add(h, Storage<DT>::load(rr, c)));
            if (DT == DT_F32) accD += (double)h * (double)h;
            else accF = fmaf(h, h, accF);
        }
        double total = DT == DT_F32 ? block_sum<double>(accD, smemD) : (double)block_sum<float>(accF, smemF);
        const float inv = inv_rms<DT>(total, a.cols, a.eps);
        const size_t mo = gated ? (row / a.rowsPerBatch) * a.modCols + a.set * a.cols * 3 + a.cols * 2 : 0;
        for (size_t c = threadIdx.x; c < a.cols; c += blockDim.x) {
            float h = Storage<DT>::load(xr, c);
            if (FUSED) {
                h = round_storage<DT>(add(h, Storage<DT>::load(rr, c)));
                if (a.hOut) Storage<DT>::store((T*)a.hOut, row * a.cols + c, h);
            }
            float g = Storage<DT>::load((const T*)a.scale, c);
            float o = DT == DT_F32 ? mul(h, mul(inv, g)) : mul(mul(h, inv), g);
            Storage<DT>::store((T*)a.normOut, row * a.cols + c, o);
            if (gated) {
                float b = Storage<DT>::load((const T*)a.branch, row * a.cols + c);
                float m = Storage<DT>::load((const T*)a.mod, mo + c);
                Storage<DT>::store((T*)a.gatedOut, row * a.cols + c, add(h, mul(m, b)));
            }
        }
    }
}

template <int DT, bool FUSED>
static int launch_rows(Context* ctx, const RowArgs& a, CUDAStatus* status) {
    constexpr int PER = Lanes<DT>::kPer;
    uintptr_t bits = (uintptr_t)a.x | (uintptr_t)a.residual | (uintptr_t)a.scale | (uintptr_t)a.branch | (uintptr_t)a.mod |
                     (uintptr_t)a.hOut | (uintptr_t)a.normOut | (uintptr_t)a.gatedOut;
    bool vec = (bits & 15u) == 0 && a.cols % PER == 0 && (a.branch == nullptr || a.modCols % PER == 0);
    size_t cap = (size_t)ctx->smCount * 16;
    int grid = (int)(a.rows < cap ? a.rows : cap);
    const size_t nvec = a.cols / PER;
    const void* outs[3] = {a.hOut, a.normOut, a.gatedOut};
    bool inplace = false;
    for (const void* o : outs) inplace |= o && (o == a.x || o == a.residual);
    // measured at 16384 x 4096 bf16: plain RMSNorm 4.49 TB/s warp-per-row vs 4.05 block-per-row; the fused form needs twice the
    // registers per lane, fits one block per SM and is faster block-per-row (4.49 vs 3.27 TB/s)
    if (a.nPeer > 0 && !vec) return fail(status, -2, "rmsnorm: the gathered form needs 16-byte aligned rows");
    if (FUSED && DT != DT_F32 && vec && nvec > 256 && nvec <= 512) {
        const bool gated = a.branch != nullptr;
        constexpr int D16 = DT == DT_F32 ? DT_BF16 : DT;  // (never instantiated for float32 rows)
        const size_t resident = (size_t)ctx->smCount * 3;  // three blocks per SM fit: every block keeps its scale slice for ~rows/444 rows
        const int g16 = (int)(a.rows < resident ? a.rows : resident);
        if (gated && inplace) add_rmsnorm16_kernel<D16, true, true><<<g16, 256, 0, ctx->stream>>>(a);
        else if (gated) add_rmsnorm16_kernel<D16, true, false><<<g16, 256, 0, ctx->stream>>>(a);
        else if (inplace) add_rmsnorm16_kernel<D16, false, true><<<g16, 256, 0, ctx->stream>>>(a);
        else add_rmsnorm16_kernel<D16, false, false><<<g16, 256, 0, ctx->stream>>>(a);
        return check_launch(ctx, status, "add+rmsnorm+gated residual");
    }
    if (a.nPeer > 0 && !inplace) {
        if (nvec <= 2 * 256) rmsnorm_rows_kernel<DT, 2, FUSED, false><<<grid, 256, 0, ctx->stream>>>(a);
        else rmsnorm_rows_kernel<DT, 4, FUSED, false><<<grid, 256, 0, ctx->stream>>>(a);
    } else if (!FUSED && vec && !inplace && nvec > 256 && nvec <= (DT == DT_F32 ? 1024u : 512u)) {
        const size_t resident = (size_t)ctx->smCount * (DT == DT_F32 ? 3 : 4);
        const int ga = (int)(a.rows < resident ? a.rows : resident);
        if (nvec <= 512) rmsnorm_ahead_kernel<DT, 2><<<ga, 256, 0, ctx->stream>>>(a);
        else rmsnorm_ahead_kernel<DT, DT == DT_F32 ? 4 : 2><<<ga, 256, 0, ctx->stream>>>(a);  // (16-bit rows never get here)
    } else if (inplace && vec) rmsnorm_rows_kernel<DT, 4, FUSED, true><<<grid, 256, 0, ctx->stream>>>(a);
    else if (!FUSED && vec && nvec <= 512 && nvec >= 128 && a.rows >= 64) {
        size_t blocks = (a.rows + 7) / 8, capW = (size_t)ctx->smCount * 4;
        rmsnorm_warp_rows_kernel<DT, FUSED><<<(unsigned)(blocks < capW ? blocks : capW), 256, 0, ctx->stream>>>(a);
    } else if (vec && nvec <= 2 * 256) rmsnorm_rows_kernel<DT, 2, FUSED, false><<<grid, 256, 0, ctx->stream>>>(a);  // fewer registers, more rows in flight
    else if (vec) rmsnorm_rows_kernel<DT, 4, FUSED, false><<<grid, 256, 0, ctx->stream>>>(a);
    else rmsnorm_rows_scalar_kernel<DT, FUSED><<<grid, 256, 0, ctx->stream>>>(a);  // plain loads, element by element: in-place safe
    return check_launch(ctx, status, FUSED ? "add+rmsnorm+gated residual" : "rmsnorm");
}

// Aliasing rules of the row kernels: an output may be exactly the buffer of x or of residual (in-place); it may not
// overlap them partially, may not overlap scale, branch or modulation at all, and two outputs may not overlap each other.
static int check_row_aliasing(CUDAStatus* status, const RowArgs& a, size_t es) {
    const size_t bytes = a.rows * a.cols * es;
    auto overlap = [](const void* p, size_t pn, const void* q, size_t qn) {
        return p && q && (const char*)p < (const char*)q + qn && (const char*)q < (const char*)p + pn;
    };
    const void* outs[3] = {a.hOut, a.normOut, a.gatedOut};
    const char* names[3] = {"hOut", "normOut", "gatedOut"};
    const size_t batches = a.rowsPerBatch ? (a.rows + a.rowsPerBatch - 1) / a.rowsPerBatch : 0;
    for (int i = 0; i < 3; i++) {
        if (!outs[i]) continue;
        for (const void* in : {a.x, a.residual})
            if (in != outs[i] && overlap(outs[i], bytes, in, bytes))
                return fail(status, -2, "rmsnorm: %s partially overlaps an input (only the exact same buffer may be reused in place)", names[i]);
        if (overlap(outs[i], bytes, a.scale, a.cols * es) || overlap(outs[i], bytes, a.branch, bytes) ||
            overlap(outs[i], bytes, a.mod, batches * a.modCols * es))
            return fail(status, -2, "rmsnorm: %s overlaps scale, branch or modulation", names[i]);
        for (int j = i + 1; j < 3; j++)
            if (overlap(outs[i], bytes, outs[j], bytes)) return fail(status, -2, "rmsnorm: %s and %s overlap", names[i], names[j]);
    }
    return 0;
}

template <bool FUSED>
static int dispatch_rows(Context* ctx, int dt, const RowArgs& a, CUDAStatus* status) {
    int rc = check_row_aliasing(status, a, dtype_size(dt));
    if (rc != 0) return rc;
    if (dt == DT_F32) return launch_rows<DT_F32, FUSED>(ctx, a, status);
    if (dt == DT_BF16) return launch_rows<DT_BF16, FUSED>(ctx, a, status);
    if (dt == DT_F16) return launch_rows<DT_F16, FUSED>(ctx, a, status);
    return fail(status, -6, "layernorm: unsupported dtype %d", dt);
}

}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_rmsnorm_f64(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                                         CUDABufferRef outputRef, uint32_t rows, uint32_t cols, double epsilon, uint64_t completionToken,
                                         CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (rows == 0 || cols == 0) return ok(status);
    if (!(epsilon > 0)) return fail(status, -2, "rmsnorm: epsilon must be positive, got %g", epsilon);
    size_t es = dtype_size(elementDType);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "layernorm: unsupported dtype %d", elementDType);
    PUTER_REQUIRE(inputRef, "input", (size_t)rows * cols * es);
    PUTER_REQUIRE(scaleRef, "scale", (size_t)cols * es);
    PUTER_REQUIRE(outputRef, "output", (size_t)rows * cols * es);
    RowArgs a{};
    a.x = dev_ptr(inputRef);
    a.scale = dev_ptr(scaleRef);
    a.normOut = dev_ptr(outputRef);
    a.rows = rows;
    a.cols = cols;
    a.eps = epsilon;
    return dispatch_rows<false>(ctx, elementDType, a, status);
}

extern "C" int cuda_dispatch_rmsnorm(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef scaleRef,
                                     CUDABufferRef outputRef, uint32_t rows, uint32_t cols, float epsilon, uint64_t completionToken,
                                     CUDAStatus* status) {
    return cuda_dispatch_rmsnorm_f64(contextRef, elementDType, inputRef, scaleRef, outputRef, rows, cols, (double)epsilon,
                                     completionToken, status);
}

extern "C" int cuda_dispatch_add_rmsnorm_gated_residual(CUDADeviceRef contextRef, int elementDType, CUDABufferRef xRef,
                                                        CUDABufferRef residualRef, CUDABufferRef scaleRef, CUDABufferRef branchRef,
                                                        CUDABufferRef modulationRef, CUDABufferRef hOutRef, CUDABufferRef normOutRef,
                                                        CUDABufferRef gatedOutRef, uint32_t rows, uint32_t cols, double epsilon,
                                                        uint32_t rowsPerBatch, uint32_t modulationCols, uint32_t set,
                                                        uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (rows == 0 || cols == 0) return ok(status);
    if (!(epsilon > 0)) return fail(status, -2, "rmsnorm: epsilon must be positive, got %g", epsilon);
    size_t es = dtype_size(elementDType);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "layernorm: unsupported dtype %d", elementDType);
    size_t bytes = (size_t)rows * cols * es;
    PUTER_REQUIRE(xRef, "x", bytes);
    PUTER_REQUIRE(residualRef, "residual", bytes);
    PUTER_REQUIRE(scaleRef, "scale", (size_t)cols * es);
    PUTER_REQUIRE(normOutRef, "normOut", bytes);
    RowArgs a{};
    a.x = dev_ptr(xRef);
    a.residual = dev_ptr(residualRef);
    a.scale = dev_ptr(scaleRef);
    a.normOut = dev_ptr(normOutRef);
    a.hOut = hOutRef ? dev_ptr(hOutRef) : nullptr;
    a.rows = rows;
    a.cols = cols;
    a.eps = epsilon;
    if (branchRef) {
        if (rowsPerBatch == 0) return fail(status, -2, "gated residual: rows per batch must be positive");
        if ((uint64_t)modulationCols < ((uint64_t)set * 3 + 3) * cols)
            return fail(status, -2, "gated residual: modulation has %u columns, set %u needs %llu", modulationCols, set,
                        (unsigned long long)(((uint64_t)set * 3 + 3) * cols));
        size_t batches = ((size_t)rows + rowsPerBatch - 1) / rowsPerBatch;
        PUTER_REQUIRE(branchRef, "branch", bytes);
        PUTER_REQUIRE(modulationRef, "modulation", batches * modulationCols * es);
        PUTER_REQUIRE(gatedOutRef, "gatedOut", bytes);
        a.branch = dev_ptr(branchRef);
        a.mod = dev_ptr(modulationRef);
        a.gatedOut = dev_ptr(gatedOutRef);
        a.rowsPerBatch = rowsPerBatch;
        a.modCols = modulationCols;
        a.set = set;
    }
    return dispatch_rows<true>(ctx, elementDType, a, status);
}

// The fused kernel with the all-gather of its two outputs folded into its stores.  normAll / gatedAll are arrays of `world`
// buffer handles: entry r is rank r's gathered tensor [world * rows, cols] as mapped into this process (its own for
// r == rank, cuda_buffer_ipc_import of the peers' otherwise).  This rank's rows land at row offset rank * rows of every one of
// them.  Completion is stream-ordered for the local copy only: a consumer on another GPU needs a cross-rank barrier after the
// call (the caller's collective library provides it).  No TMA, no multicast: plain 16-byte stores over NVLink.
extern "C" int cuda_dispatch_add_rmsnorm_gated_residual_gather(CUDADeviceRef contextRef, int elementDType, CUDABufferRef xRef,
                                                               CUDABufferRef residualRef, CUDABufferRef scaleRef, CUDABufferRef branchRef,
                                                               CUDABufferRef modulationRef, const CUDABufferRef* normAll,
                                                               const CUDABufferRef* gatedAll, uint32_t world, uint32_t rank, uint32_t rows,
                                                               uint32_t cols, double epsilon, uint32_t rowsPerBatch, uint32_t modulationCols,
                                                               uint32_t set, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    if (rows == 0 || cols == 0) return ok(status);
    if (world == 0 || world > 8 || rank >= world) return fail(status, -2, "gathered rmsnorm: rank %u of %u (at most 8 ranks)", rank, world);
    if (!normAll || !gatedAll || !branchRef) return fail(status, -2, "gathered rmsnorm: nil output table or branch");
    if (!(epsilon > 0)) return fail(status, -2, "rmsnorm: epsilon must be positive, got %g", epsilon);
    size_t es = dtype_size(elementDType);
    if (elementDType != DT_F32 && elementDType != DT_F16 && elementDType != DT_BF16)
        return fail(status, -6, "layernorm: unsupported dtype %d", elementDType);
    const size_t bytes = (size_t)rows * cols * es;
    PUTER_REQUIRE(xRef, "x", bytes);
    PUTER_REQUIRE(residualRef, "residual", bytes);
    PUTER_REQUIRE(scaleRef, "scale", (size_t)cols * es);
    PUTER_REQUIRE(branchRef, "branch", bytes);
    if (rowsPerBatch == 0) return fail(status, -2, "gated residual: rows per batch must be positive");
    if ((uint64_t)modulationCols < ((uint64_t)set * 3 + 3) * cols) return fail(status, -2, "gated residual: modulation too narrow for the set");
    const size_t batches = ((size_t)rows + rowsPerBatch - 1) / rowsPerBatch;
    PUTER_REQUIRE(modulationRef, "modulation", batches * modulationCols * es);
    RowArgs a{};
    a.x = dev_ptr(xRef); a.residual = dev_ptr(residualRef); a.scale = dev_ptr(scaleRef); a.branch = dev_ptr(branchRef);
    a.mod = dev_ptr(modulationRef);
    a.rows = rows; a.cols = cols; a.eps = epsilon; a.rowsPerBatch = rowsPerBatch; a.modCols = modulationCols; a.set = set;
    for (uint32_t r = 0; r < world; r++) {
        PUTER_REQUIRE(normAll[r], "normAll[r]", (size_t)world * bytes);
        PUTER_REQUIRE(gatedAll[r], "gatedAll[r]", (size_t)world * bytes);
        char* n = (char*)dev_ptr(normAll[r]) + (size_t)rank * bytes;
        char* g = (char*)dev_ptr(gatedAll[r]) + (size_t)rank * bytes;
        if (r == rank) { a.normOut = n; a.gatedOut = g; }
        else { a.normPeer[a.nPeer] = n; a.gatedPeer[a.nPeer] = g; a.nPeer++; }
    }
    return dispatch_rows<true>(ctx, elementDType, a, status);
}
