// Paged decode attention: one new token per sequence, K/V read in place from the page pool.
//
// Equivalent, per sequence, to the reference composition page_gather(K), page_gather(V)
// (execution/page_intrinsic.go:217-352, device/cpu/shape/page_generic.go:30-50) followed by
// MultiHeadAttention with seqQ = 1, seqK = ctx and the bottom-right causal mask, under which every
// live key is visible (device/cpu/attention/typed_compute.go:142-237).  The 16-bit reference rounds
// each q.k dot product to the storage type before scaling (device/cpu/dot/bf16_generic.go:9-21);
// this kernel reproduces that rounding.  Softmax weights are kept in float32 (split into a high and a
// low 16-bit part for the tensor-core product), so results differ from the sequential CPU sums only by
// accumulation order.
//
// The kernel is HBM-bound (every K/V byte is read exactly once), so it is organised around the memory
// system rather than the math:
//   * the pool layout is [page, token, kvHead, headDim]; the eight warps of a CTA walk the same tokens,
//     one KV head each, so a CTA consumes whole 2 KB token rows / 32 KB pages while every warp owns a
//     private cp.async pipeline (no block-wide barrier anywhere in the main loop);
//   * work is split "stream-K" style: the global list of 16-token tiles of all sequences is cut into equal
//     contiguous ranges, one per worker (a CTA, or a fraction of one when there are fewer than 8 KV
//     heads), so every SM reads the same number of bytes whatever the context-length mix; a range may
//     span several sequences and a sequence several ranges;
//   * each (worker, sequence, KV head) triple leaves an un-normalised partial (max, sum, accumulator) in scratch
//     memory and bumps a counter, so a decode step is ONE launch: the tile prefix sums are recomputed by every CTA in
//     shared memory (a separate one-block kernel only beyond 1024 sequences).  The grid is launched cooperatively (one
//     CTA per SM, all resident), and the workers that share a sequence merge it TOGETHER once their own ranges are done:
//     each waits, bounded, for the sequence's counter, then normalises and writes its own share of the output rows from
//     one round of loads.  (One warp pulling 30 workers' partials through its SM's L2 port took ~19 us at the end of the
//     kernel; 30 warps on 30 SMs take ~3.)  Where a cooperative launch is refused, the warp that arrives last for a
//     (sequence, KV head) merges all of it in worker order;
//   * every warp's copies run two tiles ahead of its compute through the whole range, across sequence boundaries, and
//     carry an L2 evict-first hint: K/V bytes are read once and must not push out what is read again (page tables,
//     query rows, the partials, the kernel's instructions);
//   * the 16 TOKENS of a tile are the M = 16 rows of mma.sync m16n8k16 and the (<= 8, or 2 x 8) query heads of the KV
//     head's GQA group its N columns, fed by ldmatrix from XOR-swizzled shared memory; tensor-core throughput is
//     irrelevant here, the point is to keep the instruction count per byte far below the issue limit;
//   * fp8-e4m3 KV pages stay bytes in shared memory and are widened to f16 (exact) in registers, straight out of
//     ldmatrix; the per-KV-head scales are applied to the scores and to the output.
#include <math.h>
#include <stdlib.h>
#include <mutex>

#include "common.cuh"

namespace puter {

static constexpr int kHeadDim = 128;
static constexpr int kTile = 16;       // tokens per tile
static constexpr int kWarps = 8;
static constexpr int kThreads = kWarps * 32;

static constexpr int kPrefixSmem = 1024;  // sequences whose tile prefix sums fit the in-kernel scan

struct DecodeParams {
    const void* q;            // [batch, numHeads*128]
    const void* kPages;       // [pageCount, pageSize, kvHeads*128]
    const void* vPages;
    const int32_t* pageTable; // [batch, maxPages] or nullptr: pages are consecutive (contiguous K/V per sequence)
    const int32_t* ctxLens;   // [batch], or nullptr: every sequence has uniformCtx tokens
    const float* kScale;      // [kvHeads] or nullptr (fp8 only)
    const float* vScale;
    const int* tileStart;     // [batch+1] exclusive prefix of tiles per sequence, or nullptr: scanned in shared memory
    float* partAcc;           // [slots, numHeads, 128]
    float2* partML;           // [slots, numHeads]  (max in log2 domain, sum)
    int* counters;            // [batch, kvHeads] arrivals (then departures) per (sequence, KV head); zero on entry, zero again on exit
    void* out;                // [batch, numHeads*128]
    int* errorFlag;
    long long seqStrideKV;    // contiguous mode: elements between consecutive sequences' K (and V)
    int batch, maxPages, pageCount, pageSize, numHeads, kvHeads, group, uniformCtx;
    int headsPerPass, groups, workers;  // warps-as-heads per pass, sub-ranges per CTA, total workers
    int distributed;          // all CTAs of the grid run at the same time (cooperative launch): owners merge together
    float scaleLog2;          // (1/sqrt(headDim)) * log2(e)
    float scale;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// K/V bytes are read once: marked evict-first in L2 so that they do not push out what is read again (page tables, query rows,
// the partials of the merge, the kernel's own instructions)
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void cp_async16_kv(uint64_t pol, uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst), "l"(src), "r"(bytes), "l"(pol) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <bool BF16>
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    if (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// packs two f32 into the 16-bit MMA operand type (truncation-free: RNE)
template <bool BF16> __device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *(uint32_t*)&v;
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *(uint32_t*)&v;
}
template <bool BF16> __device__ __forceinline__ float unpack16_lo(uint32_t w) {
    if (BF16) return __uint_as_float(w << 16);
    return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu)));
}
template <bool BF16> __device__ __forceinline__ float unpack16_hi(uint32_t w) {
    if (BF16) return __uint_as_float(w & 0xFFFF0000u);
    return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
}
// rounds an f32 to the 16-bit storage type and back (the reference's rounded dot product)
template <bool BF16> __device__ __forceinline__ float round16(float v) {
    if (BF16) return __uint_as_float(f32_to_bf16_bits(v) << 16);
    return __half2float(__float2half_rn(v));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// tiles of sequence b; clamps negative and over-long contexts and flags them
__device__ __forceinline__ int seq_tiles(const DecodeParams& p, int b) {
    long long ctx = p.ctxLens ? (long long)p.ctxLens[b] : (long long)p.uniformCtx;
    if (ctx < 0) { ctx = 0; atomicExch(p.errorFlag, 1); }
    if (p.pageTable) {
        const long long cap = (long long)p.maxPages * p.pageSize;
        if (ctx > cap) { ctx = cap; atomicExch(p.errorFlag, 1); }
    }
    return (int)((ctx + kTile - 1) / kTile);
}

// context length of sequence b as the kernels use it: never beyond the tiles counted for it
__device__ __forceinline__ int seq_ctx(const DecodeParams& p, int b, int tiles) {
    const long long ctx = p.ctxLens ? (long long)p.ctxLens[b] : (long long)p.uniformCtx;
    const long long cap = (long long)tiles * kTile;
    return (int)(ctx < cap ? ctx : cap);
}

// Exclusive prefix sum of tiles per sequence over the whole block: out[0..batch].  Every thread of the block must call it.
__device__ void block_tile_prefix(const DecodeParams& p, int* out) {
    __shared__ int warpSums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nWarps = (blockDim.x + 31) >> 5;
    for (int base = 0; base < p.batch; base += blockDim.x) {
        const int b = base + threadIdx.x;
        const int tiles = b < p.batch ? seq_tiles(p, b) : 0;
        int incl = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        if (lane == 31) warpSums[warp] = incl;
        __syncthreads();
        int before = carry;
        for (int w = 0; w < warp; w++) before += warpSums[w];
        if (b < p.batch) out[b] = before + incl - tiles;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + incl;
        __syncthreads();
        (void)nWarps;
    }
    if (threadIdx.x == 0) out[p.batch] = carry;
    __syncthreads();
}

// the same scan as a kernel of its own, for batches beyond the in-kernel limit
__global__ void __launch_bounds__(1024) decode_prefix_kernel(DecodeParams p, int* __restrict__ tileStart) { block_tile_prefix(p, tileStart); }

// worker index that owns global tile g when T tiles are cut into NV equal contiguous ranges [v*T/NV, (v+1)*T/NV)
__device__ __forceinline__ long long worker_of_tile(long long g, long long T, long long NV) { return ((g + 1) * NV - 1) / T; }

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg((const float4*)p); }

// Workers that own tiles of sequence b, in worker order: [v0, v1], of which n have a non-empty range.
struct SeqOwners {
    long long T, W, v0, v1;
    int n;
    bool allOwn;  // every worker of the grid has a non-empty range (at least as many tiles as workers)
    // workers whose own range is empty (fewer tiles than workers) never write a partial
    __device__ __forceinline__ bool owns(long long v) const { return allOwn || (v + 1) * T / W > v * T / W; }
};
__device__ __forceinline__ SeqOwners seq_owners(const DecodeParams& p, const int* ts, int b) {
    SeqOwners so;
    so.T = ts[p.batch];
    so.W = p.workers;
    so.v0 = worker_of_tile(ts[b], so.T, so.W);
    so.v1 = worker_of_tile((long long)ts[b + 1] - 1, so.T, so.W);
    so.allOwn = so.T >= so.W;
    so.n = (int)(so.v1 - so.v0 + 1);
    if (!so.allOwn) {
        so.n = 0;
        for (long long v = so.v0; v <= so.v1; v++) so.n += so.owns(v) ? 1 : 0;
    }
    return so;
}

template <bool BF16>
__device__ __forceinline__ void store_out16(uint16_t* dst, const float* num, float den) {
    uint32_t w2[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float a = den > 0.f ? num[2 * i] / den : 0.f, c = den > 0.f ? num[2 * i + 1] / den : 0.f;
        const uint32_t lo = BF16 ? f32_to_bf16_bits(a) : f32_to_f16_bits(a), hi = BF16 ? f32_to_bf16_bits(c) : f32_to_f16_bits(c);
        w2[i] = lo | (hi << 16);
    }
    ((uint4*)dst)[0] = make_uint4(w2[0], w2[1], w2[2], w2[3]);
    ((uint4*)dst)[1] = make_uint4(w2[4], w2[5], w2[6], w2[7]);
}

// Merge of (sequence b, KV head kvh) with a lane per 16-dimension slice of a head (four heads per pass) and a loop over the
// owning workers in worker order.  Of the slices, numbered through the group's heads, this call handles those with
// slice % split == share: split = 1 merges everything, split = n with share = the caller's rank among the owners is one
// owner's part of a merge that all owners do together.  The whole warp must call it.
// The loads of eight owners (their (max, sum) pairs and accumulator slices) are all issued before the first is used, and
// the running maximum is updated per round, so a round costs ONE L2 round trip (about a microsecond on this part).
template <bool BF16>
__device__ __forceinline__ void merge_slices(const DecodeParams& p, const SeqOwners& so, int b, int kvh, int lane, int split, int share) {
    uint16_t* orow = (uint16_t*)p.out + (size_t)b * p.numHeads * kHeadDim;
    const long long v0 = so.v0, v1 = so.v1;
    const int hl = lane >> 3, d0 = (lane & 7) * 16;
    for (int hBase = 0; hBase < p.group; hBase += 4) {
        const bool valid = hBase + hl < p.group && (hBase * 8 + lane) % split == share;
        const int head = kvh * p.group + (hBase + hl < p.group ? hBase + hl : 0);
        const float2* mlBase = p.partML + (size_t)b * p.numHeads + head;                      // + v * numHeads
        const float* accBase = p.partAcc + ((size_t)b * p.numHeads + head) * kHeadDim + d0;  // + v * numHeads * 128
        float M = -INFINITY, den = 0.f;
        float num[16];
#pragma unroll
        for (int i = 0; i < 16; i++) num[i] = 0.f;
        constexpr int kBatch = 8;
        for (long long base = v0; base <= v1; base += kBatch) {
            float2 ml[kBatch];
            float4 acc[kBatch][4];
#pragma unroll
            for (int k = 0; k < kBatch; k++) {
                const long long v = base + k;
                if (valid && v <= v1 && so.owns(v)) {
                    ml[k] = __ldcg(mlBase + (size_t)v * p.numHeads);
                    const float* a = accBase + (size_t)v * p.numHeads * kHeadDim;
                    acc[k][0] = ldcg4(a);
                    acc[k][1] = ldcg4(a + 4);
                    acc[k][2] = ldcg4(a + 8);
                    acc[k][3] = ldcg4(a + 12);
                } else {
                    ml[k] = make_float2(-INFINITY, 0.f);
                    acc[k][0] = acc[k][1] = acc[k][2] = acc[k][3] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            float Mn = M;
#pragma unroll
            for (int k = 0; k < kBatch; k++) Mn = fmaxf(Mn, ml[k].x);
            if (Mn != M) {  // also the first round with any live owner: M = -inf scales the (zero) sums by zero
                const float s = (M == -INFINITY) ? 0.f : exp2f(M - Mn);
                den *= s;
#pragma unroll
                for (int i = 0; i < 16; i++) num[i] *= s;
                M = Mn;
            }
#pragma unroll
            for (int k = 0; k < kBatch; k++) {
                const float w = (ml[k].x == -INFINITY) ? 0.f : exp2f(ml[k].x - M);
                den += ml[k].y * w;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    num[4 * i] += acc[k][i].x * w; num[4 * i + 1] += acc[k][i].y * w;
                    num[4 * i + 2] += acc[k][i].z * w; num[4 * i + 3] += acc[k][i].w * w;
                }
            }
        }
        if (valid) store_out16<BF16>(orow + (size_t)head * kHeadDim + d0, num, den);
    }
}

// One owner's part of the merge of (sequence b, KV head kvh) when the sequence is spread over many workers: the owner with
// rank `share` among the n owners takes the 16-dimension slices share, share + n, ...  For a slice, a LANE PER OWNER loads
// that owner's (max, sum) pair and 16 accumulator values; the warp reduces them with a fixed shuffle tree that halves the
// values a lane carries at every level, so lane l ends up with the sum of dimension (l >> 1) of the slice.  More than 32
// owners take several such units per slice, combined in order with a running maximum.  The loads of four units are issued
// together: the whole duty is normally one L2 round trip.  The whole warp must call it.
template <bool BF16>
__device__ __forceinline__ void merge_across_lanes(const DecodeParams& p, const SeqOwners& so, int b, int kvh, int lane, int share) {
    uint16_t* orow = (uint16_t*)p.out + (size_t)b * p.numHeads * kHeadDim;
    const int slices = p.group * 8;
    const int passes = (int)((so.v1 - so.v0 + 32) / 32);
    const int mine = share < slices ? (slices - share + so.n - 1) / so.n : 0;  // slices share, share + n, ...
    const int units = mine * passes;
    // reversed bit order: the element a lane keeps is picked by its bits 4 (x8), 3 (x4), 2 (x2), 1 (x1)
    const int elem = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
    float M = -INFINITY, den = 0.f, num = 0.f;  // running state of the current slice (num: dimension `elem`)
    constexpr int kUnits = 4;
    for (int u0 = 0; u0 < units; u0 += kUnits) {
        float2 ml[kUnits];
        float4 acc[kUnits][4];
#pragma unroll
        for (int k = 0; k < kUnits; k++) {
            const int u = u0 + k;
            const int c = share + (u / passes) * so.n;
            const long long v = so.v0 + (long long)(u % passes) * 32 + lane;
            if (u < units && v <= so.v1 && so.owns(v)) {
                const size_t row = (size_t)(v + b) * p.numHeads + kvh * p.group + (c >> 3);
                ml[k] = __ldcg(p.partML + row);
                const float* a = p.partAcc + row * kHeadDim + (c & 7) * 16;
                acc[k][0] = ldcg4(a);
                acc[k][1] = ldcg4(a + 4);
                acc[k][2] = ldcg4(a + 8);
                acc[k][3] = ldcg4(a + 12);
            } else {
                ml[k] = make_float2(-INFINITY, 0.f);
                acc[k][0] = acc[k][1] = acc[k][2] = acc[k][3] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int k = 0; k < kUnits; k++) {
            const int u = u0 + k;
            if (u >= units) break;  // uniform over the warp
            float Mu = ml[k].x;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) Mu = fmaxf(Mu, __shfl_xor_sync(0xffffffffu, Mu, o));
            const float w = (ml[k].x == -INFINITY) ? 0.f : exp2f(ml[k].x - Mu);
            float du = ml[k].y * w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) du += __shfl_xor_sync(0xffffffffu, du, o);
            float val[16] = {acc[k][0].x * w, acc[k][0].y * w, acc[k][0].z * w, acc[k][0].w * w, acc[k][1].x * w, acc[k][1].y * w,
                             acc[k][1].z * w, acc[k][1].w * w, acc[k][2].x * w, acc[k][2].y * w, acc[k][2].z * w, acc[k][2].w * w,
                             acc[k][3].x * w, acc[k][3].y * w, acc[k][3].z * w, acc[k][3].w * w};
            // reduce-scatter: at the level of lane bit o a lane keeps one half of its values and receives the partner's
#pragma unroll
            for (int half = 8, o = 16; half >= 1; half >>= 1, o >>= 1) {
                const bool upper = (lane & o) != 0;
#pragma unroll
                for (int i = 0; i < half; i++) {
                    const float send = upper ? val[i] : val[i + half];
                    const float keep = upper ? val[i + half] : val[i];
                    val[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            float nu = val[0] + __shfl_xor_sync(0xffffffffu, val[0], 1);
            // combine with the slice's earlier units (owners 32 and up)
            if (u % passes == 0) { M = -INFINITY; den = 0.f; num = 0.f; }
            const float Mn = fmaxf(M, Mu);
            const float sOld = (M == -INFINITY) ? 0.f : exp2f(M - Mn), sNew = (Mu == -INFINITY) ? 0.f : exp2f(Mu - Mn);
            den = den * sOld + du * sNew;
            num = num * sOld + nu * sNew;
            M = Mn;
            if (u % passes == passes - 1 && (lane & 1) == 0) {
                const int c = share + (u / passes) * so.n;
                const float o = den > 0.f ? num / den : 0.f;
                orow[(size_t)(kvh * p.group + (c >> 3)) * kHeadDim + (c & 7) * 16 + elem] = (uint16_t)(BF16 ? f32_to_bf16_bits(o) : f32_to_f16_bits(o));
            }
        }
    }
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

static constexpr int kMergeSplitMax = 8;          // up to this many owners, every owner loops over all owners for its slices
static constexpr unsigned kMergeSpinLimit = 1u << 21;  // polls of an arrival counter before a warp gives up (~1 s)

// Called by a whole warp once its partial of (worker, sequence b, KV head kvh) is in scratch.
//   * A sequence that lies inside one worker's range is normalised and written at once.
//   * Otherwise the arrival is counted.  Where all CTAs of the grid are known to run at the same time (p.distributed), the
//     sequence is noted in `duty` and the warp moves on: once its range is done it waits for the other owners and merges ITS
//     share of the output, so a sequence spread over 30 workers is merged by 30 warps on 30 SMs at once instead of one SM
//     pulling all of it through its L2 port.  A range has at most two such sequences (its first and its last).
//   * Without that guarantee the warp that arrives last merges everything, in worker order, and zeroes the counter.
template <bool BF16>
__device__ __forceinline__ void segment_done(const DecodeParams& p, const int* ts, int b, int kvh, int lane, int& duty0, int& duty1, int& nDuty) {
    const SeqOwners so = seq_owners(p, ts, b);
    __threadfence();  // this lane's partial stores are visible device-wide before the arrival is counted
    __syncwarp();
    if (so.n > 1) {
        int* c = p.counters + (size_t)b * p.kvHeads + kvh;
        if (p.distributed) {
            // only the first and the last sequence of a range can be shared with other workers: two notes suffice
            if (lane == 0) atomicAdd(c, 1);
            if (nDuty++ == 0) duty0 = b; else duty1 = b;
            return;
        }
        int last = 0;
        if (lane == 0) {
            last = atomicAdd(c, 1) == so.n - 1;
            if (last) *c = 0;  // nobody else touches this counter again in this launch
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) return;
        __threadfence();
    }
    merge_slices<BF16>(p, so, b, kvh, lane, 1, 0);
}

// The deferred part of segment_done, for the one or two sequences a range shares with other workers: waits (bounded) until all
// owners of each have arrived — lane 0 polls the first counter and lane 1 the second, at the same time — then merges this
// worker's share of each and counts the departures; the last to depart returns a counter to zero.
// The range's LAST sequence is merged first: its other owners met it at the start of their ranges and arrived long ago (unless
// it spans whole ranges), while the first sequence waits for a worker that is finishing its own range right now.
template <bool BF16>
__device__ __forceinline__ void finish_duties(const DecodeParams& p, const int* ts, long long worker, int nDuty, int duty0, int duty1,
                                              int kvh, int lane) {
    if (nDuty == 0) return;
    const int bA = nDuty > 1 ? duty1 : duty0, bB = duty0;  // order of the merges
    const SeqOwners soA = seq_owners(p, ts, bA), soB = seq_owners(p, ts, bB);
    int ok = 1;
    if (lane < nDuty) {
        const int* c = p.counters + (size_t)(lane == 0 ? bA : bB) * p.kvHeads + kvh;
        const int need = lane == 0 ? soA.n : soB.n;
        unsigned spins = 0;
        while (ld_acquire_gpu(c) < need) {
            if (++spins > kMergeSpinLimit) { ok = 0; break; }
            __nanosleep(40);
        }
    }
    const int okA = __shfl_sync(0xffffffffu, ok, 0), okB = __shfl_sync(0xffffffffu, ok, 1);
    __syncwarp();  // the polling lanes' acquire loads, then this barrier: every lane's loads below see the owners' partials
    // one copy of the merge code, run once or twice (the second run finds it in the instruction cache)
#pragma unroll 1
    for (int d = 0; d < nDuty; d++) {
        const SeqOwners so = d == 0 ? soA : soB;
        const int b = d == 0 ? bA : bB, okay = d == 0 ? okA : okB;
        int* c = p.counters + (size_t)b * p.kvHeads + kvh;
        if (okay) {
            int share = (int)(worker - so.v0);
            if (!so.allOwn) {
                share = 0;
                for (long long v = so.v0; v < worker; v++) share += so.owns(v) ? 1 : 0;
            }
            if (so.n <= kMergeSplitMax) merge_slices<BF16>(p, so, b, kvh, lane, so.n, share);
            else merge_across_lanes<BF16>(p, so, b, kvh, lane, share);
        } else if (lane == 0) {
            atomicExch(p.errorFlag, 4);  // an owner never arrived: the rows of this sequence are not written
        }
        __syncwarp();
        if (lane == 0 && atomicAdd(c, 1) == 2 * so.n - 1) *c = 0;
    }
}

// ---------------------------------------------------------------------------------------------------------
// 16-bit (bf16 / f16) KV pages.  The TOKENS of a 16-token tile are the M = 16 rows of every m16n8k16 MMA and the (<= 8)
// query heads of the KV head's group its N = 8 columns: S^T = K Q^T and O^T += V^T P^T.  (With the heads as rows, 12 of
// 16 rows multiply zeros for a group of 4: twice the MMAs and twice the accumulator registers.)
//   * K tile rows feed the A operand through a plain ldmatrix, V^T through ldmatrix.trans, both from XOR-swizzled tiles;
//   * the score accumulator holds (token g, heads 2t, 2t+1); each score is rounded to the storage type before scaling,
//     as the reference's rounded dot product; the softmax weights stay float32 and enter the P V product as a high and a
//     low 16-bit part, each turned into the B-operand layout (head g, tokens 2t, 2t+1) by movmatrix;
//   * the maximum is reduced over the 8 lanes that share a head column; the row sums stay per lane until the end.
// ---------------------------------------------------------------------------------------------------------
static constexpr int kStages16 = 3;
static constexpr int kStage16 = 2 * kTile * kHeadDim * 2;          // K + V bytes of one tile for one head: 8 KB
static constexpr int kSmem16 = kStages16 * kStage16 * kWarps;      // 192 KB

// NT = n-tiles of 8 query heads per KV head (1: group <= 8, 2: group <= 16)
template <bool BF16, int NT>
__global__ void __launch_bounds__(kThreads, 1) paged_decode16_kernel(DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smemRaw[];
    __shared__ int sTileStart[kPrefixSmem + 1];
    const int* ts = p.tileStart;
    if (!ts) {
        block_tile_prefix(p, sTileStart);
        ts = sTileStart;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    if (warp >= p.groups * p.headsPerPass) return;
    const int sub = warp / p.headsPerPass;
    const int head0 = warp % p.headsPerPass;
    const long long worker = (long long)blockIdx.x * p.groups + sub;
    const long long T = ts[p.batch];
    if (T == 0) return;
    const long long lo = worker * T / p.workers, hi = (worker + 1) * T / p.workers;
    if (lo >= hi) return;
    unsigned char* wsm = smemRaw + (size_t)warp * (kStages16 * kStage16);
    const uint32_t wsmAddr = smem_u32(wsm);
    const uint64_t kvPolicy = l2_evict_first_policy();
    const size_t tokenStride = (size_t)p.kvHeads * kHeadDim * 2;  // bytes between tokens of a page
    const bool page16 = (p.pageSize % kTile) == 0;
    int seq;
    {
        int a = 0, z = p.batch;
        while (z - a > 1) {
            int m = (a + z) >> 1;
            if (ts[m] <= lo) a = m; else z = m;
        }
        seq = a;
    }
    // per-lane constants of the copy pattern: lane = (row in a group of 2 tokens, 16-byte chunk of the 256-byte row)
    const int cpRow = lane >> 4, cpChunk = lane & 15;
    const size_t cpSrc = (size_t)cpRow * tokenStride + (size_t)cpChunk * 16;
    // per-lane ldmatrix addresses inside a tile (swizzle: 16-byte chunk ^ (token & 7))
    const int lmRow = lane & 7, lmMat = lane >> 3;
    const uint32_t kLm = (uint32_t)(((lmMat & 1) * 8 + lmRow) * 256);   // K: matrices (tok 0-7 | 8-15) x (chunk 2kk | 2kk+1)
    const int kLmChunk = lmMat >> 1;
    const uint32_t vLm = (uint32_t)(((lmMat >> 1) * 8 + lmRow) * 256);  // V: matrices (chunk 2dt | 2dt+1) x (tok 0-7 | 8-15)
    const int vLmChunk = lmMat & 1;

    for (int kvh = head0; kvh < p.kvHeads; kvh += p.headsPerPass) {
        int b = seq;
        long long cur = lo;
        int duty0 = 0, duty1 = 0, nDuty = 0;  // sequences shared with other workers whose merge waits for the end of the range
        // ---- issue cursor: the copies run kStages16 - 1 tiles ahead of the compute and do not stop at a sequence boundary, so
        // the first tiles of the next sequence are on their way while this one's partial is stored and its arrival counted ----
        long long ig = lo;                      // next global tile to copy
        int ib = seq, istage = 0;
        long long iSegStart = 0, iSegEnd = lo;  // global tiles of sequence ib: [iSegStart, iSegEnd); empty = not set up yet
        int iCtx = 0;
        const int32_t* table = nullptr;
        const unsigned char *kBase = nullptr, *vBase = nullptr;
        int cbase = -0x40000000, cval = 0;
        auto page_of = [&](int entry) -> int {
            if (!table) return entry;
            if (entry - cbase >= 32 || entry < cbase) {
                cbase = entry;
                int idx = entry + lane;
                cval = idx < p.maxPages ? table[idx] : 0;
            }
            int pg = __shfl_sync(0xffffffffu, cval, entry - cbase);
            if (pg < 0 || pg >= p.pageCount) {
                if (lane == 0) atomicExch(p.errorFlag, 1);
                pg = 0;  // never dereference an out-of-range page
            }
            return pg;
        };
        // async copies of local tile `lt` (16 tokens) of sequence ib into stage `st`; rows past the context are zero-filled, never read
        auto issue = [&](int lt, int st) {
            const int ctx = iCtx;
            const int tok0 = lt * kTile;
            const uint32_t dstK = wsmAddr + st * kStage16, dstV = dstK + kTile * kHeadDim * 2;
            if (page16 || !table) {
                const int ps = table ? p.pageSize : kTile;
                const size_t pageOff = ((size_t)page_of(tok0 / ps) * ps + (size_t)(tok0 % ps)) * tokenStride;
                const unsigned char* ks = kBase + pageOff + cpSrc;
                const unsigned char* vs = vBase + pageOff + cpSrc;
                const bool full = tok0 + kTile <= ctx;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = 2 * i + cpRow;
                    const uint32_t so = (uint32_t)(r * 256) + (uint32_t)((cpChunk ^ (r & 7)) * 16);
                    const size_t rowOff = (size_t)(2 * i) * tokenStride;
                    if (full) {
                        cp_async16_kv(kvPolicy, dstK + so, ks + rowOff, 16);
                        cp_async16_kv(kvPolicy, dstV + so, vs + rowOff, 16);
                    } else {
                        const bool live = tok0 + r < ctx;
                        cp_async16_kv(kvPolicy, dstK + so, live ? ks + rowOff : kBase, live ? 16 : 0);
                        cp_async16_kv(kvPolicy, dstV + so, live ? vs + rowOff : vBase, live ? 16 : 0);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = 2 * i + cpRow;
                    const int tok = tok0 + r;
                    int pg = 0;
                    const int entry = tok / p.pageSize;
                    if (tok < ctx && entry < p.maxPages) {
                        pg = table[entry];
                        if (pg < 0 || pg >= p.pageCount) { atomicExch(p.errorFlag, 1); pg = 0; }
                    }
                    size_t off = ((size_t)pg * p.pageSize + tok % p.pageSize) * tokenStride;
                    const int bytes = tok < ctx ? 16 : 0;
                    if (bytes == 0) off = 0;
                    const uint32_t so = (uint32_t)(r * 256) + (uint32_t)((cpChunk ^ (r & 7)) * 16);
                    cp_async16_kv(kvPolicy, dstK + so, kBase + off + cpChunk * 16, bytes);
                    cp_async16_kv(kvPolicy, dstV + so, vBase + off + cpChunk * 16, bytes);
                }
            }
        };
        // copies the next tile of the range, if there is one, and closes a copy group either way
        auto issue_next = [&]() {
            if (ig < hi) {
                if (ig >= iSegEnd) {
                    while (ts[ib + 1] <= ig) ib++;  // skip empty sequences
                    iSegStart = ts[ib];
                    iSegEnd = ts[ib + 1];
                    iCtx = seq_ctx(p, ib, (int)(iSegEnd - iSegStart));
                    table = p.pageTable ? p.pageTable + (size_t)ib * p.maxPages : nullptr;
                    kBase = (const unsigned char*)p.kPages + (size_t)kvh * kHeadDim * 2;
                    vBase = (const unsigned char*)p.vPages + (size_t)kvh * kHeadDim * 2;
                    if (!table) {
                        kBase += (size_t)ib * p.seqStrideKV * 2;
                        vBase += (size_t)ib * p.seqStrideKV * 2;
                    }
                    cbase = -0x40000000;
                }
                issue((int)(ig - iSegStart), istage);
            }
            ig++;
            if (++istage == kStages16) istage = 0;
            cp_async_commit();
        };
#pragma unroll
        for (int s = 0; s < kStages16 - 1; s++) issue_next();
        int stage = 0;
        while (cur < hi) {
            while (ts[b + 1] <= cur) b++;  // skip empty sequences
            const long long segStart = ts[b], segEndAll = ts[b + 1];
            const long long segEnd = segEndAll < hi ? segEndAll : hi;
            const int tile0 = (int)(cur - segStart), tile1 = (int)(segEnd - segStart);  // local tile range [tile0, tile1)
            const int ctx = seq_ctx(p, b, (int)(segEndAll - segStart));
            // O^T: tile dt = dims 16dt .. 16dt+15; [0],[1] = (dim 16dt+g, heads 2t, 2t+1), [2],[3] = (dim 16dt+g+8, heads 2t, 2t+1)
            float oacc[8][NT][4];
#pragma unroll
            for (int dt = 0; dt < 8; dt++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) oacc[dt][nt][0] = oacc[dt][nt][1] = oacc[dt][nt][2] = oacc[dt][nt][3] = 0.f;
            float mcol[NT][2], lcol[NT][2];  // per head column (heads 8nt + 2t, + 1): running maximum (shared by the warp), this lane's sum
#pragma unroll
            for (int nt = 0; nt < NT; nt++) { mcol[nt][0] = mcol[nt][1] = -INFINITY; lcol[nt][0] = lcol[nt][1] = 0.f; }

            const int nTiles = tile1 - tile0;
            // (the query rows are fetched after the first K/V copies are on their way: they are not needed before the first MMA)
            // ---- Q as the B operand: k16 step kk: b0 = dims 16kk + 2t, +1 of head g; b1 = dims 16kk + 8 + 2t, +1 ----
            uint32_t qb[8][NT][2];
            {
                const uint16_t* qRow = (const uint16_t*)p.q + (size_t)b * p.numHeads * kHeadDim;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int gi = nt * 8 + g;
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) {
                        uint32_t w0 = 0, w1 = 0;
                        if (gi < p.group) {
                            const uint16_t* src = qRow + (size_t)(kvh * p.group + gi) * kHeadDim + kk * 16 + 2 * t;
                            w0 = *(const uint32_t*)src;
                            w1 = *(const uint32_t*)(src + 8);
                        }
                        qb[kk][nt][0] = w0;
                        qb[kk][nt][1] = w1;
                    }
                }
            }
            for (int it = 0; it < nTiles; it++) {
                cp_async_wait<kStages16 - 2>();
                __syncwarp();
                issue_next();
                const uint32_t tileK = wsmAddr + stage * kStage16, tileV = tileK + kTile * kHeadDim * 2;
                if (++stage == kStages16) stage = 0;
                // ---- S^T = K Q^T : 16 tokens x 8 heads per n-tile ----
                float sacc[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < 8; kk++) {
                    uint32_t a[4];
                    ldmatrix_x4(tileK + kLm + (((2 * kk + kLmChunk) ^ lmRow) * 16), a[0], a[1], a[2], a[3]);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) mma16816<BF16>(sacc[nt], a, qb[kk][nt][0], qb[kk][nt][1]);
                }
                // ---- round, scale, mask, online softmax (log2 domain); sacc[nt] = (token g, heads 2t, 2t+1), (token g+8, ...) ----
                const int tokBase = (tile0 + it) * kTile;
                const bool tail = tokBase + kTile > ctx;
                bool rescale = false;
                float alpha[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float x[2];
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            float sc = round16<BF16>(sacc[nt][2 * r + j]) * p.scaleLog2;  // the reference rounds the dot to storage first
                            if (tail && tokBase + 8 * r + g >= ctx) sc = -INFINITY;
                            x[r] = sc;
                        }
                        float mx = fmaxf(x[0], x[1]);
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                        const float mNew = fmaxf(mcol[nt][j], mx);
                        const float a = (mNew == -INFINITY) ? 1.0f : exp2f(mcol[nt][j] - mNew);
                        const float e0 = (x[0] == -INFINITY) ? 0.f : exp2f(x[0] - mNew);
                        const float e1 = (x[1] == -INFINITY) ? 0.f : exp2f(x[1] - mNew);
                        sacc[nt][j] = e0;
                        sacc[nt][2 + j] = e1;
                        lcol[nt][j] = lcol[nt][j] * a + (e0 + e1);
                        mcol[nt][j] = mNew;
                        alpha[nt][j] = a;
                        rescale |= a != 1.0f;
                    }
                }
                if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                    for (int dt = 0; dt < 8; dt++)
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            oacc[dt][nt][0] *= alpha[nt][0];
                            oacc[dt][nt][1] *= alpha[nt][1];
                            oacc[dt][nt][2] *= alpha[nt][0];
                            oacc[dt][nt][3] *= alpha[nt][1];
                        }
                }
                // ---- P^T as B operands, high and low 16-bit parts: (token g, heads 2t, 2t+1) -> movmatrix -> (head g, tokens 2t, 2t+1) ----
                uint32_t ph[NT][2], pl[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const float p0 = sacc[nt][2 * r], p1 = sacc[nt][2 * r + 1];
                        const uint32_t h = pack16<BF16>(p0, p1);
                        const uint32_t l = pack16<BF16>(p0 - unpack16_lo<BF16>(h), p1 - unpack16_hi<BF16>(h));  // what the rounding of P dropped
                        ph[nt][r] = movmatrix_trans(h);
                        pl[nt][r] = movmatrix_trans(l);
                    }
                }
                // ---- O^T += V^T P^T ----
#pragma unroll
                for (int dt = 0; dt < 8; dt++) {
                    uint32_t a[4];  // (dims 16dt+g, tok 2t..), (dims 16dt+8+g, tok 2t..), (dims 16dt+g, tok 8+2t..), (dims 16dt+8+g, tok 8+2t..)
                    ldmatrix_x4_trans(tileV + vLm + (((2 * dt + vLmChunk) ^ lmRow) * 16), a[0], a[1], a[2], a[3]);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        mma16816<BF16>(oacc[dt][nt], a, ph[nt][0], ph[nt][1]);
                        mma16816<BF16>(oacc[dt][nt], a, pl[nt][0], pl[nt][1]);
                    }
                }
            }
            // ---- end of this worker's part of sequence b: row sums reduced over the lanes of a head column, then either the
            // finished rows (the whole sequence lay inside this range: nothing to merge, no trip through scratch) or the
            // partial of (worker, sequence, KV head) ----
            const bool whole = cur == segStart && segEnd == segEndAll;
            {
                const long long slot = worker + b;
                uint16_t* orow = (uint16_t*)p.out + (size_t)b * p.numHeads * kHeadDim;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float l = lcol[nt][j];
                        l += __shfl_xor_sync(0xffffffffu, l, 4);
                        l += __shfl_xor_sync(0xffffffffu, l, 8);
                        l += __shfl_xor_sync(0xffffffffu, l, 16);
                        const int gi = nt * 8 + 2 * t + j;
                        if (gi < p.group) {
                            const int head = kvh * p.group + gi;
                            if (whole) {
                                uint16_t* o = orow + (size_t)head * kHeadDim;
#pragma unroll
                                for (int dt = 0; dt < 8; dt++) {
                                    const float x0 = l > 0.f ? oacc[dt][nt][j] / l : 0.f, x1 = l > 0.f ? oacc[dt][nt][2 + j] / l : 0.f;
                                    o[16 * dt + g] = (uint16_t)(BF16 ? f32_to_bf16_bits(x0) : f32_to_f16_bits(x0));
                                    o[16 * dt + g + 8] = (uint16_t)(BF16 ? f32_to_bf16_bits(x1) : f32_to_f16_bits(x1));
                                }
                            } else {
                                float* acc = p.partAcc + ((size_t)slot * p.numHeads + head) * kHeadDim;
#pragma unroll
                                for (int dt = 0; dt < 8; dt++) {
                                    acc[16 * dt + g] = oacc[dt][nt][j];
                                    acc[16 * dt + g + 8] = oacc[dt][nt][2 + j];
                                }
                                if (g == 0) p.partML[(size_t)slot * p.numHeads + head] = make_float2(mcol[nt][j], l);
                            }
                        }
                    }
                }
            }
            if (!whole) segment_done<BF16>(p, ts, b, kvh, lane, duty0, duty1, nDuty);
            cur = segEnd;
            if (cur >= segEndAll) b++;
        }
        cp_async_wait<0>();  // only empty groups are left
        __syncwarp();
        finish_duties<BF16>(p, ts, worker, nDuty, duty0, duty1, kvh, lane);
    }
}

// ---------------------------------------------------------------------------------------------------------
// fp8-e4m3 KV pages.  sm_100a has no native fp8 mma.sync (the assembler expands it into conversions plus f16 MMAs, ~20
// instructions each), so the bytes are widened to f16 (exact) in registers, straight out of ldmatrix, and the kernel is
// built to spend as few instructions per byte as it can:
//   * the TOKENS are the M = 16 rows of every m16n8k16 MMA and the (<= 8) query heads of the KV head's group its N = 8
//     columns: S^T = K Q^T and O^T += V^T P^T.  With the heads as rows (as in the 16-bit kernel) 12 of 16 rows would
//     multiply zeros for a group of 4; this way a 32-token step costs 16 + 16 MMAs and the output accumulator 32 registers;
//   * K: a non-transposed ldmatrix of the raw rows hands every lane 4 consecutive head dimensions of one token; two
//     cvt.f16x2.e4m3x2 turn them into A registers of an MMA whose K index runs over the dimensions
//     {4t, 4t+1 | 4t+2, 4t+3} of a 16-dimension chunk — the query fragments (B operand) are loaded in the same order;
//   * V: ldmatrix.trans on byte pairs + one byte permute per register gives, per lane, the tokens {2t, 2t+1} of the
//     dimensions 2g and 2g+1: the A registers of V^T with the rows of a 16-dimension tile ordered {0,2,..,14,1,3,..,15};
//   * P^T: the score accumulator holds (token g, heads 2t, 2t+1); movmatrix transposes the packed f16 pairs into the
//     B-operand layout (head g, tokens 2t, 2t+1);
//   * the softmax maximum is reduced over the 8 lanes that share a head column; the row sums stay per lane until the end.
// The bf16 query is multiplied in f16 (values beyond the f16 range would overflow), P in f16 (11 significant bits),
// accumulation in f32; the per-KV-head scales multiply the scores and the output.
// ---------------------------------------------------------------------------------------------------------
static constexpr int kTile8 = 32;                                  // tokens per fp8 step
static constexpr int kStage8 = 2 * kTile8 * kHeadDim;              // K + V bytes of one step for one head: 8 KB
static constexpr int kStages8 = 3;
static constexpr int kSmem8 = kStages8 * kStage8 * kWarps;         // 192 KB

// two e4m3 bytes (low / high 16 bits of `w`) -> f16x2, exact
__device__ __forceinline__ uint32_t e4m3x2_lo(uint32_t w) {
    uint32_t d;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(d) : "r"(w));
    return d;
}
__device__ __forceinline__ uint32_t e4m3x2_hi(uint32_t w) {
    uint32_t d;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, hi; }" : "=r"(d) : "r"(w));
    return d;
}
__device__ __forceinline__ float ex2_approx(float x) {  // 2^x, flush-to-zero, 2 ulp: ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma16816_f16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT = n-tiles of 8 query heads per KV head (1: group <= 8, 2: group <= 16)
template <bool BF16, int NT>
__global__ void __launch_bounds__(kThreads, 1) paged_decode_fp8_kernel(DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smemRaw[];
    __shared__ int sTileStart[kPrefixSmem + 1];
    const int* ts = p.tileStart;
    if (!ts) {
        block_tile_prefix(p, sTileStart);
        ts = sTileStart;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    if (warp >= p.groups * p.headsPerPass) return;
    const int sub = warp / p.headsPerPass;
    const int head0 = warp % p.headsPerPass;
    const long long worker = (long long)blockIdx.x * p.groups + sub;
    const long long T = ts[p.batch];
    if (T == 0) return;
    const long long lo = worker * T / p.workers, hi = (worker + 1) * T / p.workers;
    if (lo >= hi) return;
    unsigned char* wsm = smemRaw + (size_t)warp * (kStages8 * kStage8);
    const uint32_t wsmAddr = smem_u32(wsm);
    const uint64_t kvPolicy = l2_evict_first_policy();
    const size_t tokenStride = (size_t)p.kvHeads * kHeadDim;  // bytes between tokens of a page
    const bool page16 = (p.pageSize % kTile) == 0;
    int seq;
    {
        int a = 0, z = p.batch;
        while (z - a > 1) {
            int m = (a + z) >> 1;
            if (ts[m] <= lo) a = m; else z = m;
        }
        seq = a;
    }
    // per-lane constants of the copy pattern: lane = (row in a group of 4 tokens, 16-byte chunk of the 128-byte row)
    const int cpRow = lane >> 3, cpChunk = lane & 7;
    const size_t cpSrc = (size_t)cpRow * tokenStride + (size_t)cpChunk * 16;
    const uint32_t cpDstEven = (uint32_t)(cpRow * 128 + ((cpChunk ^ cpRow) * 16));        // rows 8j + cpRow
    const uint32_t cpDstOdd = (uint32_t)((cpRow + 4) * 128 + ((cpChunk ^ (cpRow + 4)) * 16));  // rows 8j + 4 + cpRow
    // per-lane ldmatrix addresses inside a stage (swizzle: 16-byte chunk ^ (token & 7))
    const int lmRow = lane & 7, lmMat = lane >> 3;
    const uint32_t kLm = (uint32_t)(((lmMat & 1) * 8 + lmRow) * 128);  // + 16*mt*128, chunk (2cp + (lmMat >> 1)) ^ lmRow
    const uint32_t vLm = (uint32_t)(lane * 128);                       // matrix j = tokens 8j..8j+7, chunk dt ^ lmRow

    for (int kvh = head0; kvh < p.kvHeads; kvh += p.headsPerPass) {
        int b = seq;
        long long cur = lo;
        int duty0 = 0, duty1 = 0, nDuty = 0;  // sequences shared with other workers whose merge waits for the end of the range
        // ---- issue cursor: the copies run kStages8 - 1 steps ahead of the compute and do not stop at a sequence boundary, so
        // the first steps of the next sequence are on their way while this one's partial is stored and its arrival counted ----
        long long icur = lo;         // global tile at which the next sequence's share of this range starts
        int ib = seq, istage = 0;
        int iTok = 0, iTokEnd = 0;   // tokens of sequence ib still to copy: [iTok, iTokEnd)
        const int32_t* table = nullptr;
        const unsigned char *kBase = nullptr, *vBase = nullptr;
        int cbase = -0x40000000, cval = 0;
        auto page_of = [&](int entry) -> int {
            if (!table) return entry;
            if (entry - cbase >= 32 || entry < cbase) {
                cbase = entry;
                int idx = entry + lane;
                cval = idx < p.maxPages ? table[idx] : 0;
            }
            int pg = __shfl_sync(0xffffffffu, cval, entry - cbase);
            if (pg < 0 || pg >= p.pageCount) {
                if (lane == 0) atomicExch(p.errorFlag, 1);
                pg = 0;  // never dereference an out-of-range page
            }
            return pg;
        };
        // async copies of the 32 tokens starting at `tsk` of sequence ib into stage `st` (rows past the share's end are zero-filled)
        auto issue = [&](int tsk, int st) {
            const int tokEnd = iTokEnd;
            const uint32_t dstK = wsmAddr + st * kStage8, dstV = dstK + kTile8 * kHeadDim;
            if (page16 || !table) {
                const int ps = table ? p.pageSize : kTile;
                const bool full = tsk + kTile8 <= tokEnd;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int tk = tsk + h * kTile;
                    size_t halfOff = 0;
                    if (tk < tokEnd) halfOff = ((size_t)page_of(tk / ps) * ps + (size_t)(tk % ps)) * tokenStride;
                    const unsigned char* ks = kBase + halfOff + cpSrc;
                    const unsigned char* vs = vBase + halfOff + cpSrc;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t so = (uint32_t)((h * 16 + (i >> 1) * 8) * 128) + ((i & 1) ? cpDstOdd : cpDstEven);
                        const size_t rowOff = (size_t)(4 * i) * tokenStride;
                        if (full) {
                            cp_async16_kv(kvPolicy, dstK + so, ks + rowOff, 16);
                            cp_async16_kv(kvPolicy, dstV + so, vs + rowOff, 16);
                        } else {
                            const bool live = tk + 4 * i + cpRow < tokEnd;
                            cp_async16_kv(kvPolicy, dstK + so, live ? ks + rowOff : kBase, live ? 16 : 0);
                            cp_async16_kv(kvPolicy, dstV + so, live ? vs + rowOff : vBase, live ? 16 : 0);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = i * 4 + cpRow;
                    const int tok = tsk + r;
                    int pg = 0;
                    const int entry = tok / p.pageSize;
                    if (tok < tokEnd && entry < p.maxPages) {
                        pg = table[entry];
                        if (pg < 0 || pg >= p.pageCount) { atomicExch(p.errorFlag, 1); pg = 0; }
                    }
                    size_t off = ((size_t)pg * p.pageSize + tok % p.pageSize) * tokenStride;
                    const int bytes = tok < tokEnd ? 16 : 0;
                    if (bytes == 0) off = 0;
                    const uint32_t so = r * 128 + ((cpChunk ^ (r & 7)) * 16);
                    cp_async16_kv(kvPolicy, dstK + so, kBase + off + cpChunk * 16, bytes);
                    cp_async16_kv(kvPolicy, dstV + so, vBase + off + cpChunk * 16, bytes);
                }
            }
        };
        // copies the next 32-token step of the range, if there is one, and closes a copy group either way.  A sequence's share
        // is cut into steps from its own first token, exactly as the compute loop below counts them.
        auto issue_next = [&]() {
            if (iTok >= iTokEnd && icur < hi) {
                while (ts[ib + 1] <= icur) ib++;  // skip empty sequences
                const long long s0 = ts[ib], s1 = ts[ib + 1];
                const long long e = s1 < hi ? s1 : hi;
                const int ctx = seq_ctx(p, ib, (int)(s1 - s0));
                const long long endTokL = (e - s0) * kTile;
                iTok = (int)(icur - s0) * kTile;
                iTokEnd = (int)(endTokL < ctx ? endTokL : ctx);
                icur = e;
                table = p.pageTable ? p.pageTable + (size_t)ib * p.maxPages : nullptr;
                kBase = (const unsigned char*)p.kPages + (size_t)kvh * kHeadDim;
                vBase = (const unsigned char*)p.vPages + (size_t)kvh * kHeadDim;
                if (!table) {
                    kBase += (size_t)ib * p.seqStrideKV;
                    vBase += (size_t)ib * p.seqStrideKV;
                }
                cbase = -0x40000000;
            }
            if (iTok < iTokEnd) {
                issue(iTok, istage);
                iTok += kTile8;
            }
            if (++istage == kStages8) istage = 0;
            cp_async_commit();
        };
#pragma unroll
        for (int s = 0; s < kStages8 - 1; s++) issue_next();
        int stage = 0;
        while (cur < hi) {
            while (ts[b + 1] <= cur) b++;
            const long long segStart = ts[b], segEndAll = ts[b + 1];
            const long long segEnd = segEndAll < hi ? segEndAll : hi;
            const int tok0 = (int)(cur - segStart) * kTile;
            const int ctx = seq_ctx(p, b, (int)(segEndAll - segStart));
            const long long endTokL = (segEnd - segStart) * kTile;
            const int tokEnd = (int)(endTokL < ctx ? endTokL : ctx);  // this worker's share of the sequence: [tok0, tokEnd)
            // O^T: tile dt = dims 16dt .. 16dt+15 in the row order {0,2,..,14,1,3,..,15}; [0],[1] = (dim 16dt+2g, heads 2t, 2t+1),
            // [2],[3] = (dim 16dt+2g+1, heads 2t, 2t+1)
            float oacc[8][NT][4];
#pragma unroll
            for (int dt = 0; dt < 8; dt++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) oacc[dt][nt][0] = oacc[dt][nt][1] = oacc[dt][nt][2] = oacc[dt][nt][3] = 0.f;
            float mcol[NT][2], lcol[NT][2];  // per head column (heads 8nt + 2t, + 1): running maximum (shared by the warp), this lane's sum
#pragma unroll
            for (int nt = 0; nt < NT; nt++) { mcol[nt][0] = mcol[nt][1] = -INFINITY; lcol[nt][0] = lcol[nt][1] = 0.f; }
            const float sScale = (p.kScale ? p.kScale[kvh] : 1.0f) * p.scaleLog2;

            const int nSteps = (tokEnd - tok0 + kTile8 - 1) / kTile8;
            // (the query rows are fetched after the first K/V copies are on their way: they are not needed before the first MMA)
            // ---- Q as the B operand, f16: chunk c (16 head dimensions): b0 = dims 16c+4t, +1 of head g; b1 = dims +2, +3 ----
            uint32_t qb[8][NT][2];
            {
                const uint16_t* qRow = (const uint16_t*)p.q + (size_t)b * p.numHeads * kHeadDim;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int gi = nt * 8 + g;
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        uint32_t w0 = 0, w1 = 0;
                        if (gi < p.group) {
                            const uint2 raw = *(const uint2*)(qRow + (size_t)(kvh * p.group + gi) * kHeadDim + c * 16 + 4 * t);
                            if (BF16) {
                                w0 = pack16<false>(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u));
                                w1 = pack16<false>(__uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u));
                            } else {
                                w0 = raw.x;
                                w1 = raw.y;
                            }
                        }
                        qb[c][nt][0] = w0;
                        qb[c][nt][1] = w1;
                    }
                }
            }
            for (int it = 0; it < nSteps; it++) {
                cp_async_wait<kStages8 - 2>();
                __syncwarp();
                issue_next();
                const uint32_t tileK = wsmAddr + stage * kStage8, tileV = tileK + kTile8 * kHeadDim;
                if (++stage == kStages8) stage = 0;
                // ---- S^T = K Q^T : 32 tokens x 8 heads per n-tile; two m-tiles of 16 tokens ----
                float sacc[2][NT][4];
#pragma unroll
                for (int mt = 0; mt < 2; mt++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) sacc[mt][nt][0] = sacc[mt][nt][1] = sacc[mt][nt][2] = sacc[mt][nt][3] = 0.f;
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
#pragma unroll
                    for (int cp = 0; cp < 4; cp++) {
                        uint32_t r0, r1, r2, r3;  // (tokens 0-7, chunk 2cp), (8-15, 2cp), (0-7, 2cp+1), (8-15, 2cp+1) of m-tile mt
                        ldmatrix_x4(tileK + kLm + mt * (16 * 128) + (((2 * cp + (lmMat >> 1)) ^ lmRow) * 16), r0, r1, r2, r3);
                        const uint32_t a0 = e4m3x2_lo(r0), a1 = e4m3x2_lo(r1), a2 = e4m3x2_hi(r0), a3 = e4m3x2_hi(r1);
                        const uint32_t c0 = e4m3x2_lo(r2), c1 = e4m3x2_lo(r3), c2 = e4m3x2_hi(r2), c3 = e4m3x2_hi(r3);
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            mma16816_f16(sacc[mt][nt], a0, a1, a2, a3, qb[2 * cp][nt][0], qb[2 * cp][nt][1]);
                            mma16816_f16(sacc[mt][nt], c0, c1, c2, c3, qb[2 * cp + 1][nt][0], qb[2 * cp + 1][nt][1]);
                        }
                    }
                }
                // ---- scale, mask, online softmax (log2 domain); sacc[mt][nt] = (token 16mt+g, heads 2t, 2t+1), (token 16mt+g+8, ...) ----
                const int tokBase = tok0 + it * kTile8;
                const bool tail = tokBase + kTile8 > tokEnd;
                bool rescale = false;
                float alpha[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float x[4];
#pragma unroll
                        for (int mt = 0; mt < 2; mt++) {
#pragma unroll
                            for (int r = 0; r < 2; r++) {
                                float sc = sacc[mt][nt][2 * r + j] * sScale;
                                if (tail && tokBase + 16 * mt + 8 * r + g >= tokEnd) sc = -INFINITY;
                                x[2 * mt + r] = sc;
                            }
                        }
                        float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                        const float mNew = fmaxf(mcol[nt][j], mx);
                        const float a = (mNew == -INFINITY) ? 1.0f : ex2_approx(mcol[nt][j] - mNew);
                        const float base = (mNew == -INFINITY) ? 0.f : mNew;
                        float sum = 0.f;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const float e = ex2_approx(x[i] - base);  // 2^-inf = 0 for masked tokens
                            sum += e;
                            sacc[i >> 1][nt][2 * (i & 1) + j] = e;
                        }
                        lcol[nt][j] = lcol[nt][j] * a + sum;
                        mcol[nt][j] = mNew;
                        alpha[nt][j] = a;
                        rescale |= a != 1.0f;
                    }
                }
                if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                    for (int dt = 0; dt < 8; dt++)
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            oacc[dt][nt][0] *= alpha[nt][0];
                            oacc[dt][nt][1] *= alpha[nt][1];
                            oacc[dt][nt][2] *= alpha[nt][0];
                            oacc[dt][nt][3] *= alpha[nt][1];
                        }
                }
                // ---- P^T as the f16 B operand: (token g, heads 2t, 2t+1) -> movmatrix -> (head g, tokens 2t, 2t+1) ----
                uint32_t pb[2][NT][2];
#pragma unroll
                for (int mt = 0; mt < 2; mt++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        pb[mt][nt][0] = movmatrix_trans(pack16<false>(sacc[mt][nt][0], sacc[mt][nt][1]));  // tokens 16mt + 0..7
                        pb[mt][nt][1] = movmatrix_trans(pack16<false>(sacc[mt][nt][2], sacc[mt][nt][3]));  // tokens 16mt + 8..15
                    }
                // ---- O^T += V^T P^T ----
#pragma unroll
                for (int dt = 0; dt < 8; dt++) {
                    uint32_t r0, r1, r2, r3;  // byte pairs (dims 16dt + 2g, +1) of tokens 8j + 2t (low half) and 8j + 2t + 1 (high half)
                    ldmatrix_x4_trans(tileV + vLm + ((dt ^ lmRow) * 16), r0, r1, r2, r3);
                    {
                        const uint32_t ev = __byte_perm(r0, r1, 0x6420), od = __byte_perm(r0, r1, 0x7531);
                        const uint32_t a0 = e4m3x2_lo(ev), a1 = e4m3x2_lo(od), a2 = e4m3x2_hi(ev), a3 = e4m3x2_hi(od);
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) mma16816_f16(oacc[dt][nt], a0, a1, a2, a3, pb[0][nt][0], pb[0][nt][1]);
                    }
                    {
                        const uint32_t ev = __byte_perm(r2, r3, 0x6420), od = __byte_perm(r2, r3, 0x7531);
                        const uint32_t a0 = e4m3x2_lo(ev), a1 = e4m3x2_lo(od), a2 = e4m3x2_hi(ev), a3 = e4m3x2_hi(od);
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) mma16816_f16(oacc[dt][nt], a0, a1, a2, a3, pb[1][nt][0], pb[1][nt][1]);
                    }
                }
            }
            // ---- end of this worker's part of sequence b: row sums reduced over the lanes of a head column, then either the
            // finished rows (the whole sequence lay inside this range: nothing to merge, no trip through scratch) or the
            // partial of (worker, sequence, KV head) ----
            const bool whole = cur == segStart && segEnd == segEndAll;
            {
                const long long slot = worker + b;
                const float vS = p.vScale ? p.vScale[kvh] : 1.0f;
                uint16_t* orow = (uint16_t*)p.out + (size_t)b * p.numHeads * kHeadDim;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float l = lcol[nt][j];
                        l += __shfl_xor_sync(0xffffffffu, l, 4);
                        l += __shfl_xor_sync(0xffffffffu, l, 8);
                        l += __shfl_xor_sync(0xffffffffu, l, 16);
                        const int gi = nt * 8 + 2 * t + j;
                        if (gi < p.group) {
                            const int head = kvh * p.group + gi;
                            if (whole) {
                                uint16_t* o = orow + (size_t)head * kHeadDim;
#pragma unroll
                                for (int dt = 0; dt < 8; dt++) {
                                    const float x0 = l > 0.f ? (oacc[dt][nt][j] * vS) / l : 0.f, x1 = l > 0.f ? (oacc[dt][nt][2 + j] * vS) / l : 0.f;
                                    const uint32_t lo = BF16 ? f32_to_bf16_bits(x0) : f32_to_f16_bits(x0), hi = BF16 ? f32_to_bf16_bits(x1) : f32_to_f16_bits(x1);
                                    *(uint32_t*)(o + 16 * dt + 2 * g) = lo | (hi << 16);
                                }
                            } else {
                                float* acc = p.partAcc + ((size_t)slot * p.numHeads + head) * kHeadDim;
#pragma unroll
                                for (int dt = 0; dt < 8; dt++)
                                    *(float2*)(acc + 16 * dt + 2 * g) = make_float2(oacc[dt][nt][j] * vS, oacc[dt][nt][2 + j] * vS);
                                if (g == 0) p.partML[(size_t)slot * p.numHeads + head] = make_float2(mcol[nt][j], l);
                            }
                        }
                    }
                }
            }
            if (!whole) segment_done<BF16>(p, ts, b, kvh, lane, duty0, duty1, nDuty);
            cur = segEnd;
            if (cur >= segEndAll) b++;
        }
        cp_async_wait<0>();  // only empty groups are left
        __syncwarp();
        finish_duties<BF16>(p, ts, worker, nDuty, duty0, duty1, kvh, lane);
    }
}

struct DecodeScratch {
    char* base;        // partial accumulators, (max, sum) pairs [, tile prefix sums for large batches]
    size_t bytes;      // capacity of `base`
    int* counters;     // arrival counters
    size_t counterBytes;
    bool clearCounters;  // the counters are not known to be zero: clear them on the stream first
};

size_t decode_scratch_bytes(uint32_t batch, uint32_t numHeads, int workers) {
    const size_t slots = (size_t)workers + batch;
    const size_t accBytes = slots * numHeads * kHeadDim * sizeof(float);
    const size_t mlBytes = ((slots * numHeads * sizeof(float2)) + 255) & ~(size_t)255;
    const size_t prefBytes = batch > (uint32_t)kPrefixSmem ? (((size_t)batch + 1) * sizeof(int) + 255) & ~(size_t)255 : 0;
    return accBytes + mlBytes + prefBytes;
}

// Host launcher shared by both paged entry points and the seqQ == 1 fast path of MultiHeadAttention.
// pageTable == nullptr selects contiguous K/V ([ctx, kvHeads*128] per sequence, sequences seqStrideKV apart);
// ctxLens == nullptr gives every sequence uniformCtx tokens.  `fixed` != nullptr supplies the scratch (nothing is
// allocated); otherwise it comes from the context's grow-only workspace and counter block.
int launch_paged_decode(Context* ctx, int dt, int kvDT, const void* q, const void* kPages, const void* vPages, const int32_t* pageTable,
                        const int32_t* ctxLens, int uniformCtx, const float* kScale, const float* vScale, void* out, int* errorFlag,
                        uint32_t batch, uint32_t maxPages, uint32_t pageCount, uint32_t pageSize, uint32_t numHeads, uint32_t kvHeads,
                        long long seqStrideKV, long long totalTilesHint, const DecodeScratch* fixed, CUDAStatus* status) {
    const int group = (int)(numHeads / kvHeads);
    DecodeParams p{};
    p.q = q; p.kPages = kPages; p.vPages = vPages; p.pageTable = pageTable; p.ctxLens = ctxLens; p.uniformCtx = uniformCtx;
    p.kScale = kScale; p.vScale = vScale; p.out = out;
    p.errorFlag = errorFlag ? errorFlag : ctx->errorFlag;
    p.seqStrideKV = seqStrideKV;
    p.batch = (int)batch; p.maxPages = (int)maxPages; p.pageCount = (int)pageCount; p.pageSize = (int)pageSize;
    p.numHeads = (int)numHeads; p.kvHeads = (int)kvHeads; p.group = group;
    p.headsPerPass = kvHeads < (uint32_t)kWarps ? (int)kvHeads : kWarps;
    p.groups = kWarps / p.headsPerPass;
    // grid: one CTA per SM, fewer when the problem is tiny (a worker should own at least ~4 tiles)
    long long ctas = ctx->smCount;
    if (totalTilesHint >= 0) {
        long long want = (totalTilesHint + 4LL * p.groups - 1) / (4LL * p.groups);
        if (want < 1) want = 1;
        if (want < ctas) ctas = want;
    }
    p.workers = (int)(ctas * p.groups);
    p.scale = (float)(1.0 / sqrt((double)kHeadDim));
    p.scaleLog2 = p.scale * 1.4426950408889634f;

    const size_t slots = (size_t)p.workers + batch;
    const size_t accBytes = slots * numHeads * kHeadDim * sizeof(float);
    const size_t mlBytes = ((slots * numHeads * sizeof(float2)) + 255) & ~(size_t)255;
    const size_t need = decode_scratch_bytes(batch, numHeads, p.workers);
    const size_t counterBytes = (size_t)batch * kvHeads * sizeof(int);
    char* ws;
    bool clear;
    if (fixed) {
        if (need > fixed->bytes || counterBytes > fixed->counterBytes)
            return fail(status, -2, "paged decode attention: scratch of %zu + %zu bytes exceeds the %zu + %zu supplied", need, counterBytes,
                        fixed->bytes, fixed->counterBytes);
        ws = fixed->base;
        p.counters = fixed->counters;
        clear = fixed->clearCounters;
    } else if (counterBytes <= ctx->decodeCounterBytes) {
        ws = (char*)ensure_workspace(ctx, need + 512, status);
        if (!ws) return status ? status->code : -7;
        p.counters = ctx->decodeCounters;  // zero since the context was opened; every launch leaves them zero
        clear = false;
    } else {
        const size_t cOff = (need + 255) & ~(size_t)255;
        ws = (char*)ensure_workspace(ctx, cOff + counterBytes + 512, status);
        if (!ws) return status ? status->code : -7;
        p.counters = (int*)(ws + cOff);  // the workspace is shared with other ops: not known to be zero
        clear = true;
    }
    p.partAcc = (float*)ws;
    p.partML = (float2*)(ws + accBytes);
    if (clear && cudaMemsetAsync(p.counters, 0, counterBytes, ctx->stream) != cudaSuccess)
        return fail(status, -7, "paged decode attention: clearing the arrival counters failed");
    if (batch > (uint32_t)kPrefixSmem) {
        int* tsG = (int*)(ws + accBytes + mlBytes);
        decode_prefix_kernel<<<1, 1024, 0, ctx->stream>>>(p, tsG);
        int rc = check_launch(ctx, status, "decode prefix");
        if (rc != 0) return rc;
        p.tileStart = tsG;
    }

    const bool bf16 = dt == DT_BF16;
    const bool fp8 = kvDT == DT_E4M3;
    // PUTER_DECODE_NO_COOPERATIVE (any value) forces the plain launch, in which the last warp to arrive merges a sequence alone:
    // the path a refused cooperative launch takes, reachable this way for tests
    const bool cooperative = getenv("PUTER_DECODE_NO_COOPERATIVE") == nullptr;
#define DECODE_LAUNCH(KERNEL, SMEM)                                                             \
    do {                                                                                        \
        cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM)); \
        p.distributed = cooperative ? 1 : 0;                                                    \
        void* args[] = {&p};                                                                    \
        if (!cooperative ||                                                                     \
            cudaLaunchCooperativeKernel((const void*)KERNEL, dim3((unsigned)ctas), dim3(kThreads), args, SMEM, ctx->stream) != cudaSuccess) { \
            cudaGetLastError();                                                                 \
            p.distributed = 0;                                                                  \
            KERNEL<<<(unsigned)ctas, kThreads, SMEM, ctx->stream>>>(p);                         \
        }                                                                                       \
    } while (0)
    if (fp8) {
        if (group <= 8) {
            if (bf16) DECODE_LAUNCH((paged_decode_fp8_kernel<true, 1>), kSmem8);
            else DECODE_LAUNCH((paged_decode_fp8_kernel<false, 1>), kSmem8);
        } else {
            if (bf16) DECODE_LAUNCH((paged_decode_fp8_kernel<true, 2>), kSmem8);
            else DECODE_LAUNCH((paged_decode_fp8_kernel<false, 2>), kSmem8);
        }
    } else {
        if (group <= 8) {
            if (bf16) DECODE_LAUNCH((paged_decode16_kernel<true, 1>), kSmem16);
            else DECODE_LAUNCH((paged_decode16_kernel<false, 1>), kSmem16);
        } else {
            if (bf16) DECODE_LAUNCH((paged_decode16_kernel<true, 2>), kSmem16);
            else DECODE_LAUNCH((paged_decode16_kernel<false, 2>), kSmem16);
        }
    }
#undef DECODE_LAUNCH
    return check_launch(ctx, status, "paged decode attention");
}

bool decode_supported(int dt, int kvDT, uint32_t numHeads, uint32_t kvHeads, uint32_t headDim) {
    if (dt != DT_BF16 && dt != DT_F16) return false;
    if (kvDT != dt && kvDT != DT_E4M3) return false;
    if (headDim != (uint32_t)kHeadDim || kvHeads == 0 || numHeads % kvHeads != 0) return false;
    return numHeads / kvHeads <= 16;
}

// ---------------------------------------------------------------------------------------------------------
// Fixed scratch of the allocation-free entry point.
//
// Some hosts may not allocate device memory at the moment they need to run a decode step: a serving loop
// whose memory is fully pre-planned and handed out by its own arena (so a hidden cudaMalloc would either
// fail or fragment the plan), a caller inside a latency-critical section where the implicit device
// synchronisation of cudaMalloc/cudaFree is not acceptable, or an embedding runtime that forbids driver
// allocations after start-up.  The regular entry point keeps its split-KV partials in a grow-only workspace
// that it allocates on demand; the allocation-free one keeps them in a fixed array that is part of the
// library image.
//
// The array lives in device memory of every GPU that loads the library, for the life of the process
// (kStaticScratchBytes per GPU).  In host code the symbol below is only a stand-in: its device address is
// obtained once per device with cudaGetSymbolAddress, with that device current, and that pointer is what
// the kernels receive.
// ---------------------------------------------------------------------------------------------------------
static constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB per GPU
static __device__ __align__(256) unsigned char g_decodeStaticScratch[kStaticScratchBytes];

static constexpr int kMaxDevices = 64;
static void* g_staticScratchPtr[kMaxDevices];  // per-device address of the array, resolved on first use
static std::mutex g_staticScratchMu;

// Resolves (once per device, with that device current) the device address of the scratch array.
static void* static_scratch_for(Context* ctx, CUDAStatus* status) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices) {
        fail(status, -2, "paged decode attention (no-alloc): device ordinal %d outside the supported 0..%d", ctx->device, kMaxDevices - 1);
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_staticScratchMu);
    if (!g_staticScratchPtr[ctx->device]) {
        void* p = nullptr;
        cudaError_t err = cudaSetDevice(ctx->device);
        if (err == cudaSuccess) err = cudaGetSymbolAddress(&p, g_decodeStaticScratch);
        if (err != cudaSuccess || !p) {
            fail(status, -7, "paged decode attention (no-alloc): cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
            return nullptr;
        }
        g_staticScratchPtr[ctx->device] = p;
    }
    return g_staticScratchPtr[ctx->device];
}

// Both paged entry points: validation, then the shared launcher (with the fixed array when noalloc).
static int paged_decode_entry(bool noalloc, CUDADeviceRef contextRef, int elementDType, int kvDType, CUDABufferRef queryRef,
                              CUDABufferRef kPagesRef, CUDABufferRef vPagesRef, CUDABufferRef pageTableRef, CUDABufferRef ctxLensRef,
                              CUDABufferRef kScaleRef, CUDABufferRef vScaleRef, CUDABufferRef outRef, CUDABufferRef errorFlagRef,
                              uint32_t batch, uint32_t maxPagesPerSeq, uint32_t pageCount, uint32_t pageSize, uint32_t numHeads,
                              uint32_t kvHeads, uint32_t headDim, CUDAStatus* status) {
    PUTER_ENTER(ctx);
    const char* what = noalloc ? "paged decode attention (no-alloc)" : "paged decode attention";
    if (batch == 0 || numHeads == 0) return ok(status);
    if (kvHeads == 0) kvHeads = numHeads;
    if (!decode_supported(elementDType, kvDType, numHeads, kvHeads, headDim))
        return fail(status, -6,
                    "%s: supported are bf16/f16 queries, KV pages of the same type or fp8-e4m3, head_dim 128, "
                    "<= 16 query heads per KV head (got dtype %d, kv dtype %d, heads %u/%u, head_dim %u)",
                    what, elementDType, kvDType, numHeads, kvHeads, headDim);
    if (pageSize == 0 || pageCount == 0 || maxPagesPerSeq == 0) return fail(status, -2, "%s: empty page geometry", what);
    const size_t kvEs = dtype_size(kvDType);
    const size_t poolBytes = (size_t)pageCount * pageSize * kvHeads * headDim * kvEs;
    PUTER_REQUIRE(queryRef, "query", (size_t)batch * numHeads * headDim * 2);
    PUTER_REQUIRE(outRef, "out", (size_t)batch * numHeads * headDim * 2);
    PUTER_REQUIRE(kPagesRef, "kPages", poolBytes);
    PUTER_REQUIRE(vPagesRef, "vPages", poolBytes);
    PUTER_REQUIRE(pageTableRef, "pageTable", (size_t)batch * maxPagesPerSeq * 4);
    PUTER_REQUIRE(ctxLensRef, "ctxLens", (size_t)batch * 4);
    const float* ks = nullptr;
    const float* vs = nullptr;
    if (kvDType == DT_E4M3 && kvDType != elementDType) {
        if (kScaleRef) { PUTER_REQUIRE(kScaleRef, "kScale", (size_t)kvHeads * 4); ks = (const float*)dev_ptr(kScaleRef); }
        if (vScaleRef) { PUTER_REQUIRE(vScaleRef, "vScale", (size_t)kvHeads * 4); vs = (const float*)dev_ptr(vScaleRef); }
    }
    int* flag = nullptr;
    if (errorFlagRef) { PUTER_REQUIRE(errorFlagRef, "errorFlag", 4); flag = (int*)dev_ptr(errorFlagRef); }
    if ((((uintptr_t)dev_ptr(kPagesRef) | (uintptr_t)dev_ptr(vPagesRef)) & 15u) != 0 || ((uintptr_t)dev_ptr(queryRef) & 7u) != 0 ||
        ((uintptr_t)dev_ptr(outRef) & 15u) != 0)
        return fail(status, -2, "%s: K/V pools and output must be 16-byte aligned, query rows 8-byte aligned", what);
    DecodeScratch fixed{};
    if (noalloc) {
        // carve the fixed array: arrival counters at its end (cleared on the stream before every launch: an earlier call with
        // another geometry may have left partials there), everything else from its start
        const int workers = ctx->smCount * (kWarps / (kvHeads < (uint32_t)kWarps ? (int)kvHeads : kWarps));
        const size_t need = decode_scratch_bytes(batch, numHeads, workers);
        const size_t counterBytes = (((size_t)batch * kvHeads * sizeof(int)) + 255) & ~(size_t)255;
        if (need + counterBytes > kStaticScratchBytes)
            return fail(status, -2,
                        "%s: batch %u with %u query heads needs %zu bytes of split-KV scratch, the fixed per-GPU array holds %zu; "
                        "use cuda_dispatch_paged_decode_attention or a smaller batch",
                        what, batch, numHeads, need + counterBytes, kStaticScratchBytes);
        char* base = (char*)static_scratch_for(ctx, status);
        if (!base) return status ? status->code : -7;
        fixed.base = base;
        fixed.bytes = kStaticScratchBytes - counterBytes;
        fixed.counters = (int*)(base + kStaticScratchBytes - counterBytes);
        fixed.counterBytes = counterBytes;
        fixed.clearCounters = true;
    }
    return launch_paged_decode(ctx, elementDType, kvDType, dev_ptr(queryRef), dev_ptr(kPagesRef), dev_ptr(vPagesRef),
                               (const int32_t*)dev_ptr(pageTableRef), (const int32_t*)dev_ptr(ctxLensRef), 0, ks, vs, dev_ptr(outRef), flag,
                               batch, maxPagesPerSeq, pageCount, pageSize, numHeads, kvHeads, 0, -1, noalloc ? &fixed : nullptr, status);
}

}  // namespace puter

using namespace puter;

extern "C" int cuda_dispatch_paged_decode_attention(CUDADeviceRef contextRef, int elementDType, int kvDType, CUDABufferRef queryRef,
                                                    CUDABufferRef kPagesRef, CUDABufferRef vPagesRef, CUDABufferRef pageTableRef,
                                                    CUDABufferRef ctxLensRef, CUDABufferRef kScaleRef, CUDABufferRef vScaleRef,
                                                    CUDABufferRef outRef, CUDABufferRef errorFlagRef, uint32_t batch, uint32_t maxPagesPerSeq,
                                                    uint32_t pageCount, uint32_t pageSize, uint32_t numHeads, uint32_t kvHeads,
                                                    uint32_t headDim, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    return paged_decode_entry(false, contextRef, elementDType, kvDType, queryRef, kPagesRef, vPagesRef, pageTableRef, ctxLensRef, kScaleRef,
                              vScaleRef, outRef, errorFlagRef, batch, maxPagesPerSeq, pageCount, pageSize, numHeads, kvHeads, headDim, status);
}

// Same operation and arguments as cuda_dispatch_paged_decode_attention, with the split-KV scratch in the
// library's fixed per-GPU array instead of an allocated workspace.  Calls no cudaMalloc / cudaFree and no
// allocating library routine.  Problems whose partials do not fit kStaticScratchBytes are refused with -2
// (with 32 query heads over 8 KV heads on a 148-SM GPU the limit is a batch of 355 sequences).
//
// The first call on a device resolves the array's device address (cudaGetSymbolAddress); make that first
// call outside of any stream capture.  Every call on a GPU shares the one array: two calls whose kernels
// can overlap on that GPU (different streams, or different contexts of the same device) race on it, so
// keep them stream-ordered.  The array keeps the previous call's contents; the only words that must start
// at zero, the arrival counters, are cleared on the stream at the start of every call, and every other
// scratch word a call reads is written earlier in the same call.
extern "C" int cuda_dispatch_paged_decode_attention_noalloc(CUDADeviceRef contextRef, int elementDType, int kvDType, CUDABufferRef queryRef,
                                                            CUDABufferRef kPagesRef, CUDABufferRef vPagesRef, CUDABufferRef pageTableRef,
                                                            CUDABufferRef ctxLensRef, CUDABufferRef kScaleRef, CUDABufferRef vScaleRef,
                                                            CUDABufferRef outRef, CUDABufferRef errorFlagRef, uint32_t batch,
                                                            uint32_t maxPagesPerSeq, uint32_t pageCount, uint32_t pageSize, uint32_t numHeads,
                                                            uint32_t kvHeads, uint32_t headDim, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    return paged_decode_entry(true, contextRef, elementDType, kvDType, queryRef, kPagesRef, vPagesRef, pageTableRef, ctxLensRef, kScaleRef,
                              vScaleRef, outRef, errorFlagRef, batch, maxPagesPerSeq, pageCount, pageSize, numHeads, kvHeads, headDim, status);
}
