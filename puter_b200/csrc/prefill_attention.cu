// Causal GQA prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Reference semantics: per batch item RoPE(q), RoPE(k) (device/cpu/rope/compute.go:55-193, results rounded to the
// 16-bit storage type) followed by MultiHeadAttention with the causal mask (device/cpu/attention/typed_compute.go:142-237):
// score = dot(q,k) * 1/sqrt(D), softmax over the visible keys, out = sum_k p[k] v[k], stored with round-to-nearest-even.
//
// Shape of the kernel (head_dim 128, 16-bit inputs):
//   * a work item is two tiles of 128 query rows of one (batch, query head); the grid is persistent (one CTA per SM), items
//     are numbered heavy (late rows) first and dealt to the CTAs in serpentine order, so a CTA pays launch, TMEM allocation
//     and barrier set-up once and the next item's Q tiles are loaded while the current item finishes;
//   * a TMA warp streams 128-key K and V tiles through a 2-stage shared-memory ring (SWIZZLE_128B boxes of 64 x 128) that
//     runs on across items, each tile serving both query tiles;
//   * one elected lane of the MMA warp issues tcgen05.mma (kind::f16, M=128, N=128, K=16):  S = Q K^T into TMEM,
//     then O += P V with P read back from TMEM as the A operand and V as an MN-major B operand; the two query tiles
//     take turns (a turn = the P V product of the tile's step and the score product of its next step, 16 MMAs back to
//     back), so the tensor core works on one tile while the other is in its softmax;
//   * two groups of four softmax warps own one S row per thread (TMEM lane = row): tcgen05.ld, online softmax in the
//     log2 domain, P packed to 16 bits and written over S with tcgen05.st; the O accumulator is rescaled lazily (only
//     when a row maximum grew by more than 2^8), so most iterations never touch it;
//   * RoPE is fused into the Q load: the raw Q tile lands by TMA and is rotated in shared memory (float32 math, unfused
//     multiplies, rounded to storage) before the first MMA.  K rows are each reused by 32 query tiles x 4 heads, so K is
//     rotated once by a streaming pre-pass into scratch, not once per tile.
//   * every wait on an mbarrier is bounded: on expiry the kernel raises the error flag, all roles drain and TMEM is freed.
#include <cuda.h>
#include <math.h>

#include "common.cuh"

namespace puter {

namespace pf {

constexpr int kD = 128;          // head dimension
constexpr int kBM = 128;         // query rows per CTA
constexpr int kBN = 128;         // keys per tile
constexpr int kStages = 2;
constexpr int kThreads = 384;     // warps 0-3 / 4-7 softmax of query tile 0 / 1, warp 8 MMA, warp 9 TMA loads, warps 10 / 11 output stores    // warps 0-3 / 4-7 softmax of query tile 0 / 1, warp 8 MMA, warp 9 TMA
constexpr uint32_t kTileBytes = kBN * kD * 2;          // one K or V tile: 32 KB
constexpr uint32_t kHalfTile = kTileBytes / 2;         // one 64-column swizzled block: 16 KB
constexpr uint32_t kSmemQ = 0;
constexpr uint32_t kSmemK = kSmemQ + 2 * kTileBytes;  // two query tiles
constexpr uint32_t kSmemV = kSmemK + kStages * kTileBytes;
constexpr uint32_t kSmemStage = kSmemV + kStages * kTileBytes;  // output staging tile (shared by the two query tiles in turn)
constexpr uint32_t kSmemBar = kSmemStage + kTileBytes;
constexpr uint32_t kSmemTotal = kSmemBar + 256 + 1024;  // + alignment slack
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;  // S0 S1 O0 O1, 128 columns each
constexpr long long kSpinLimit = 1ll << 24;

struct Params {
    CUtensorMap tmQ, tmK, tmV, tmO;
    void* out;               // [B, S, Hq*D]
    const float* ropeTable;  // cos [S, D/2] then sin [S, D/2], or nullptr
    int* errorFlag;
    int batch, seqLen, numHeads, kvHeads, causal, ropeMode;
    float scaleLog2;
    uint32_t vLBO, vSBO;
#ifdef PUTER_TRACE
    long long* trace;  // development builds only: per-phase clock64 stamps of one CTA
#endif
};

#ifdef PUTER_TRACE
#define PF_STAMP(slot)                                                                  \
    do {                                                                                \
        if (p.trace && blockIdx.x == gridDim.x / 2 && (slot) < 4096) p.trace[(slot)] = clock64(); \
    } while (0)
#else
#define PF_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait: returns false when the limit expired (the caller raises the abort flag)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abortFlag) {
    for (long long i = 0; i < kSpinLimit; i++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 1023) == 1023 && *abortFlag) return false;
    }
    return false;
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* tm, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(tm), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// shared-memory matrix descriptor (sm_100 format: version 1 in bits 46-47, swizzle mode in bits 61-63; 2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lboBytes, uint32_t sboBytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lboBytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sboBytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// instruction descriptor, kind::f16: D = f32, A/B = bf16 (1) or f16 (0), M = 128, N = 128; bMajorMN = B is MN-major
__device__ __forceinline__ uint32_t make_idesc(bool bf16, bool bMajorMN) {
    uint32_t d = 0;
    d |= 1u << 4;                      // accumulator format f32
    d |= (bf16 ? 1u : 0u) << 7;        // A format
    d |= (bf16 ? 1u : 0u) << 10;       // B format
    d |= (bMajorMN ? 1u : 0u) << 16;   // B major
    d |= (uint32_t)(kBN >> 3) << 17;   // N
    d |= (uint32_t)(kBM >> 4) << 24;   // M
    return d;
}

__device__ __forceinline__ void mma_ss(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *(uint32_t*)&v;
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *(uint32_t*)&v;
}
template <bool BF16> __device__ __forceinline__ float widen16(uint32_t b) {
    if (BF16) return __uint_as_float(b << 16);
    return __half2float(__ushort_as_half((unsigned short)b));
}
template <bool BF16> __device__ __forceinline__ uint32_t narrow16(float f) {
    if (BF16) return f32_to_bf16_bits(f);
    return f32_to_f16_bits(f);
}

// barrier slots (8 bytes each) inside the barrier area; [2] = one per query tile of the CTA
enum : uint32_t { BAR_Q = 0, BAR_QREADY = 2, BAR_K_FULL = 4, BAR_K_EMPTY = 6, BAR_V_FULL = 8, BAR_V_EMPTY = 10, BAR_S = 12, BAR_P = 14,
                  BAR_O = 16, BAR_P2 = 18, BAR_QFREE = 20, BAR_STAGED = 22, BAR_STGFREE = 24, BAR_COUNT = 25 };

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// rotate_q_fetch + rotate_q_tile: rotate the raw Q tile of one softmax group in shared memory (two swizzled 64-column blocks): the reference's RoPE on a
// 16-bit tensor (device/cpu/rope/compute.go:165-183), float32 math, results rounded to storage.  The 128 threads of the
// group walk the tile a few rows at a time with the lanes spread ALONG a row, so the cos/sin rows of the table (one per
// position) are read as contiguous 256-byte runs; a thread-per-row mapping made every table load touch 32 cache lines and
// cost ~5 us per CTA.  The products run two pairs at a time on the packed f32x2 pipe (second product fused into the sum).
// Fetches this lane's share of the cos/sin rows (32 independent 16-byte loads); issued before the Q tile has landed so the
// L2 round trips overlap the TMA load instead of queueing behind it.
__device__ __forceinline__ void rotate_q_fetch(float4* tab, int warpInGroup, int lane, int ropeMode, const float* table, int seqLen, int pos0) {
    const float* cosBase = table;
    const float* sinBase = table + (size_t)seqLen * (kD / 2);
    if (ropeMode == 1) {
        const int c = lane & 7;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int pos = min(pos0 + warpInGroup * 32 + it * 4 + (lane >> 3), seqLen - 1);
            tab[4 * it + 0] = __ldg((const float4*)(cosBase + (size_t)pos * 64 + c * 8));
            tab[4 * it + 1] = __ldg((const float4*)(cosBase + (size_t)pos * 64 + c * 8 + 4));
            tab[4 * it + 2] = __ldg((const float4*)(sinBase + (size_t)pos * 64 + c * 8));
            tab[4 * it + 3] = __ldg((const float4*)(sinBase + (size_t)pos * 64 + c * 8 + 4));
        }
    } else {
        const int cc = lane & 15;
#pragma unroll
        for (int it = 0; it < 16; it++) {
            const int pos = min(pos0 + warpInGroup * 32 + it * 2 + (lane >> 4), seqLen - 1);
            tab[2 * it + 0] = __ldg((const float4*)(cosBase + (size_t)pos * 64 + cc * 4));
            tab[2 * it + 1] = __ldg((const float4*)(sinBase + (size_t)pos * 64 + cc * 4));
        }
    }
}

template <bool BF16>
__device__ __forceinline__ void rotate_q_tile(unsigned char* tile, int warpInGroup, int lane, int ropeMode, const float4* tab, int seqLen, int pos0) {
    if (ropeMode == 1) {
        // half mode: 8 lanes per row; lane c owns pairs 8c .. 8c+7 = chunk c of block 0 with chunk c of block 1
        const int c = lane & 7;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int row = warpInGroup * 32 + it * 4 + (lane >> 3);
            if (pos0 + row >= seqLen) continue;
            const float4 c0 = tab[4 * it], c1 = tab[4 * it + 1], s0 = tab[4 * it + 2], s1 = tab[4 * it + 3];
            const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            unsigned char* p0 = tile + row * 128 + ((c ^ (row & 7)) * 16);
            Vec16 a = *(Vec16*)p0, bq = *(Vec16*)(p0 + kHalfTile);
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const uint64_t E = pk2(widen16<BF16>(a.w[w] & 0xFFFFu), widen16<BF16>(a.w[w] >> 16));
                const uint64_t O = pk2(widen16<BF16>(bq.w[w] & 0xFFFFu), widen16<BF16>(bq.w[w] >> 16));
                const uint64_t C = pk2(cs[2 * w], cs[2 * w + 1]), S = pk2(sn[2 * w], sn[2 * w + 1]), NS = pk2(-sn[2 * w], -sn[2 * w + 1]);
                float r0, r1, q0f, q1f;
                un2(fma2(O, NS, mul2(E, C)), r0, r1);   // e*c - o*s
                un2(fma2(E, S, mul2(O, C)), q0f, q1f);  // e*s + o*c
                a.w[w] = pack2<BF16>(r0, r1);
                bq.w[w] = pack2<BF16>(q0f, q1f);
            }
            *(Vec16*)p0 = a;
            *(Vec16*)(p0 + kHalfTile) = bq;
        }
    } else {
        // interleaved mode: 16 lanes per row; lane cc owns the 4 pairs of one 16-byte chunk (pairs 32*blk + 4c .. +3)
        const int cc = lane & 15, blk = cc >> 3, c = cc & 7;
#pragma unroll
        for (int it = 0; it < 16; it++) {
            const int row = warpInGroup * 32 + it * 2 + (lane >> 4);
            if (pos0 + row >= seqLen) continue;
            const float4 c4 = tab[2 * it], s4 = tab[2 * it + 1];
            unsigned char* ptr = tile + blk * kHalfTile + row * 128 + ((c ^ (row & 7)) * 16);
            Vec16 a = *(Vec16*)ptr;
            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float e = widen16<BF16>(a.w[w] & 0xFFFFu), o = widen16<BF16>(a.w[w] >> 16);
                a.w[w] = pack2<BF16>(sub(mul(e, cs[w]), mul(o, sn[w])), add(mul(e, sn[w]), mul(o, cs[w])));
            }
            *(Vec16*)ptr = a;
        }
    }
}

// Fetch the table rows, wait for the Q tile, rotate it.  Its own function (not inlined) so that the 128 table registers are
// allocated apart from the softmax loop of the caller (128 live scores per thread).
template <bool BF16>
__device__ __noinline__ bool rotate_q_when_loaded(unsigned char* tile, int warpInGroup, int lane, int ropeMode, const float* table, int seqLen,
                                                   int pos0, uint32_t barQ, uint32_t parity, volatile int* abortFlag) {
    float4 tab[32];
    rotate_q_fetch(tab, warpInGroup, lane, ropeMode, table, seqLen, pos0);
    const bool okay = __all_sync(0xffffffffu, mbar_wait(barQ, parity, abortFlag));
    if (okay) {
        rotate_q_tile<BF16>(tile, warpInGroup, lane, ropeMode, tab, seqLen, pos0);
        __syncwarp();
    }
    return okay;
}

// A work item = two 128-row query tiles (rows q0 .. q0+255) of one (batch, head); a CTA works through its share of the
// items.  Warps 0-3 / 4-7 are the softmax groups of tile 0 / 1, warp 8 issues the MMAs, warp 9 drives TMA.  TMEM columns: S0 0-127, S1 128-255, O0 256-383,
// O1 384-511; P_t overwrites the first 64 columns of S_t (each thread rewrites only the row it has already read).
// MMA order in steady state: PV0(j), QK0(j+1), PV1(j), QK1(j+1): each softmax group works while the tensor core
// runs the other tile's two products.
template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1) prefill_kernel(const __grid_constant__ Params p) {
    extern __shared__ unsigned char smemRaw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);  // swizzled boxes: 1024-byte aligned
    const uint32_t sBase = smem_u32(smem);
    const uint32_t barBase = sBase + kSmemBar;
    auto bar = [&](uint32_t i) { return barBase + i * 8; };
    __shared__ uint32_t tmemBaseShared;
    __shared__ int abortShared;
    volatile int* abortFlag = &abortShared;

    // warp index through a shuffle: the compiler then knows it is warp-uniform (and with it everything the MMA warp derives
    // from it), which lets the MMA descriptors live in uniform registers
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    // Work items (the two query tiles of one (batch, head, 256-row block)) are numbered heavy (late rows) first, consecutive
    // items sharing a KV head so K/V tiles hit in L2.  The grid is persistent: the resident CTAs are dealt items in serpentine
    // order (0..G-1, G-1..0, ...), which gives every CTA the same mix of long and short items; TMEM, the barriers and the K/V
    // ring live across items, and a CTA pays launch, allocation and barrier set-up once.
    struct Item { int head, b, kvHead, q0, nMax, nT0, nT1; };  // nT0 / nT1: key tiles query tile 0 / 1 needs
    // Decoded from the launch parameters on every call, behind an opaque copy of the item number: the softmax threads sit
    // at the register limit, and anything precomputed here would stay live across their main loop.
    auto get_item = [&](int it, Item& w) -> bool {
        asm volatile("" : "+r"(it));
        const int numPairs = (p.seqLen + 2 * kBM - 1) / (2 * kBM);
        const int perPair = p.numHeads * p.batch;
        const int G = (int)gridDim.x;
        const int idx = it * G + ((it & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
        if (idx >= numPairs * perPair) return false;
        const int rem = idx % perPair;
        w.head = rem % p.numHeads;
        w.b = rem / p.numHeads;
        w.kvHead = w.head / (p.numHeads / p.kvHeads);
        w.q0 = (numPairs - 1 - idx / perPair) * 2 * kBM;
        auto tiles_for = [&](int qs) {
            const int lastKey = p.causal ? min(p.seqLen, qs + kBM) : p.seqLen;
            return qs < p.seqLen ? (lastKey + kBN - 1) / kBN : 0;
        };
        w.nT0 = tiles_for(w.q0);
        w.nT1 = tiles_for(w.q0 + kBM);
        w.nMax = max(w.nT0, w.nT1);
        return true;
    };

    if (threadIdx.x == 0) {
        abortShared = 0;
        for (int t = 0; t < 2; t++) {
            mbar_init(bar(BAR_Q + t), 1);
            mbar_init(bar(BAR_QREADY + t), 128);
            mbar_init(bar(BAR_S + t), 1);
            mbar_init(bar(BAR_P + t), 128);
            mbar_init(bar(BAR_P2 + t), 128);
            mbar_init(bar(BAR_O + t), 1);
            mbar_init(bar(BAR_QFREE + t), 1);
            mbar_init(bar(BAR_STAGED + t), 128);
        }
        mbar_init(bar(BAR_STGFREE), 1);
        for (int s = 0; s < kStages; s++) {
            mbar_init(bar(BAR_K_FULL + s), 1);
            mbar_init(bar(BAR_K_EMPTY + s), 1);
            mbar_init(bar(BAR_V_FULL + s), 1);
            mbar_init(bar(BAR_V_EMPTY + s), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmemBaseShared)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, tmemBaseShared, 0);

    // Register reallocation between warpgroups (first thing inside each group's branch, so that the compiler sees which code
    // runs under which budget): a CTA of 3 warps per scheduler is limited to 168 registers per thread, which left the softmax
    // threads (128 scores live per thread) no room to overlap the FMA -> exp2 -> add chains of different elements.  The MMA /
    // TMA warpgroup (warps 8-11) drops to 96 registers, the two softmax warpgroups
    // rise to 200: 6 % more throughput and no spills.
    if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    if (warp >= 10) {
        // ------------------------------------------------ output stores -----------------------------------------------
        // Warp 10 / 11 writes the staged output tile of query tile 0 / 1 with TMA and, once the store has read shared memory,
        // passes the staging tile on.  A softmax thread doing this made its whole warp (and, through the QREADY barrier, its
        // whole group) wait ~1.5 us per item for the store before it could start on the next item.
        const int t = warp - 10;
        if (lane == 0) {
            uint32_t uc = 0;  // parity of the items this tile took part in so far
            bool okay = true;
            Item w = {};
            for (int it = 0; okay && get_item(it, w); it++) {
                if ((t == 0 ? w.nT0 : w.nT1) == 0) continue;
                okay = mbar_wait(bar(BAR_STAGED + t), uc & 1, abortFlag);  // every row staged, made visible to the async proxy
                if (!okay) break;
                const uint32_t src = sBase + kSmemStage;
                tma_store_4d(&p.tmO, src, 0, w.head, w.q0 + t * kBM, w.b);
                tma_store_4d(&p.tmO, src + kHalfTile, 64, w.head, w.q0 + t * kBM, w.b);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory must outlive the read
                mbar_arrive(bar(BAR_STGFREE));
                if (t == 0 && w.nT1 == 0) mbar_arrive(bar(BAR_STGFREE));  // no second tile in this item: its turn too
                uc ^= 1u;
            }
            if (!okay) *abortFlag = 1;
        }
    } else if (warp == 9) {
        // ------------------------------------------------ TMA producer ------------------------------------------------
        if (lane == 0) {
            uint32_t lc = 0;        // ring position of key tile 0 of the current item: the K/V ring runs on across items
            uint32_t uc[2] = {};    // items each query tile took part in so far
            bool okay = true;
            Item w = {};
            auto load_k = [&](int j) {
                const uint32_t ring = lc + (uint32_t)j;
                const int st = ring % kStages;
                if (ring >= kStages && !mbar_wait(bar(BAR_K_EMPTY + st), ((ring / kStages) - 1) & 1, abortFlag)) return false;
                mbar_expect_tx(bar(BAR_K_FULL + st), kTileBytes);
                const uint32_t kDst = sBase + kSmemK + st * kTileBytes;
                tma_load_4d(kDst, &p.tmK, bar(BAR_K_FULL + st), 0, w.kvHead, j * kBN, w.b);
                tma_load_4d(kDst + kHalfTile, &p.tmK, bar(BAR_K_FULL + st), 64, w.kvHead, j * kBN, w.b);
                return true;
            };
            auto load_v = [&](int j) {
                const uint32_t ring = lc + (uint32_t)j;
                const int st = ring % kStages;
                if (ring >= kStages && !mbar_wait(bar(BAR_V_EMPTY + st), ((ring / kStages) - 1) & 1, abortFlag)) return false;
                mbar_expect_tx(bar(BAR_V_FULL + st), kTileBytes);
                const uint32_t vDst = sBase + kSmemV + st * kTileBytes;
                tma_load_4d(vDst, &p.tmV, bar(BAR_V_FULL + st), 0, w.kvHead, j * kBN, w.b);
                tma_load_4d(vDst + kHalfTile, &p.tmV, bar(BAR_V_FULL + st), 64, w.kvHead, j * kBN, w.b);
                return true;
            };
            auto load_q = [&](int t) {
                if ((t == 0 ? w.nT0 : w.nT1) == 0) return true;
                // the buffer is free once the last score product of the tile's previous item has run
                if (uc[t] > 0 && !mbar_wait(bar(BAR_QFREE + t), (uc[t] - 1) & 1, abortFlag)) return false;
                uc[t]++;
                mbar_expect_tx(bar(BAR_Q + t), kTileBytes);
                tma_load_4d(sBase + kSmemQ + t * kTileBytes, &p.tmQ, bar(BAR_Q + t), 0, w.head, w.q0 + t * kBM, w.b);
                tma_load_4d(sBase + kSmemQ + t * kTileBytes + kHalfTile, &p.tmQ, bar(BAR_Q + t), 64, w.head, w.q0 + t * kBM, w.b);
                return true;
            };
            // K and V rings are released separately: a K stage is free as soon as both score products of its tile have run,
            // a V stage after both P V products, so the next K tile is in flight a whole period early.  One thread issues
            // every load and each wait blocks it, so the loads of an item are ordered by the time their buffers come free
            // at the end of the previous item: K stage of key tile 0, Q buffer 0 (after tile 0's last score product), V stage
            // of key tile 0, Q buffer 1, then the rest of the ring.  The very first item has nothing to wait for and starts
            // with Q.
            for (int it = 0; okay && get_item(it, w); it++) {
                if (it == 0) okay = load_q(0) && load_k(0) && load_q(1) && load_v(0);
                else okay = load_k(0) && load_q(0) && load_v(0) && load_q(1);
                for (int j = 1; j < w.nMax && okay; j++) okay = load_k(j) && load_v(j);
                lc += (uint32_t)w.nMax;
            }
            if (!okay) *abortFlag = 1;
        }
    } else if (warp == 8) {
        // ------------------------------------------------ MMA issuer --------------------------------------------------
        // One elected thread issues every MMA.  tcgen05.mma issue blocks at the tensor core's own pace (the queue behind it is
        // only a product or two deep), so the tensor core idles whenever this thread polls a barrier between products.  A
        // turn of a tile therefore first collects every input it needs (V tile, next K tile, P) and then issues the P V
        // product of the tile's current step and the score product of its next step as 16 MMAs back to back.  The tiles take
        // turns, which keeps them half a period apart: one is on the tensor core while the other is in its softmax.
        // The whole warp runs the loop converged and one elected lane issues: with a divergent "lane 0 only" branch the
        // compiler has to build every descriptor in vector registers and move it to the uniform registers the MMA reads,
        // ~10 instructions per product competing for issue slots with two softmax warps on the same scheduler.
        {
            const bool leader = elect_one();
            const uint32_t idescQK = make_idesc(BF16, false);
            const uint32_t idescPV = make_idesc(BF16, true);
            bool okay = true;
            // descriptors: a constant high word plus a low word whose address field (bytes >> 4) is advanced by
            // compile-time offsets and a per-stage delta
            const uint64_t kmajorHi = make_desc(0, 16, 1024) >> 32, vHi = make_desc(0, p.vLBO, p.vSBO) >> 32;
            const uint32_t qLo = (uint32_t)make_desc(sBase + kSmemQ, 16, 1024), kLo = (uint32_t)make_desc(sBase + kSmemK, 16, 1024);
            const uint32_t vLo = (uint32_t)make_desc(sBase + kSmemV, p.vLBO, p.vSBO);
            auto desc = [](uint64_t hi, uint32_t lo) { return (hi << 32) | (uint64_t)lo; };
            uint32_t lc = 0;        // ring position of key tile 0 of the current item
            uint32_t sc[2] = {};    // key-tile steps each query tile has run so far (parity of its S / P barriers)
            uint32_t uc[2] = {};    // items each query tile took part in so far (parity of its Q / O barriers)
            int nT[2] = {};
            auto issue_qk = [&](int t, int j) {
                const uint32_t kS = kLo + ((lc + (uint32_t)j) % kStages) * (kTileBytes >> 4);
                const uint32_t qS = qLo + (uint32_t)t * (kTileBytes >> 4);
                const uint32_t dS = tmem + kColS + t * 128;
#pragma unroll
                for (int kk = 0; kk < 8; kk++) {
                    const uint32_t off = ((kk >> 2) * kHalfTile + (kk & 3) * 32) >> 4;
                    if (leader) mma_ss(dS, desc(kmajorHi, qS + off), desc(kmajorHi, kS + off), idescQK, kk > 0);
                }
                if (leader) {
                    mma_commit(bar(BAR_S + t));
                    if (j + 1 == nT[t]) mma_commit(bar(BAR_QFREE + t));  // the Q tile is no longer read
                    // last score product that reads this K stage (tile 1 while it is still running, else tile 0)
                    if (t == 1 || j >= nT[1]) mma_commit(bar(BAR_K_EMPTY + (lc + (uint32_t)j) % kStages));
                }
                __syncwarp();
            };
            auto issue_pv = [&](int t, int j) {
                const uint32_t vS = vLo + ((lc + (uint32_t)j) % kStages) * (kTileBytes >> 4);
                const uint32_t dO = tmem + kColO + t * 128, aP = tmem + kColS + t * 128;
                if (leader) mma_ts(dO, aP, desc(vHi, vS), idescPV, j > 0);
#pragma unroll
                for (int kk = 1; kk < 4; kk++)
                    if (leader) mma_ts(dO, aP + kk * 8, desc(vHi, vS + ((kk * 16 * 128) >> 4)), idescPV, 1);
                if (!mbar_wait(bar(BAR_P2 + t), (sc[t] + (uint32_t)j) & 1, abortFlag)) return false;  // second half of P (keys 64..127)
                fence_after();
#pragma unroll
                for (int kk = 4; kk < 8; kk++)
                    if (leader) mma_ts(dO, aP + kk * 8, desc(vHi, vS + ((kk * 16 * 128) >> 4)), idescPV, 1);
                __syncwarp();
                return true;
            };
            Item w = {};
            for (int it = 0; okay && get_item(it, w); it++) {
                nT[0] = w.nT0;
                nT[1] = w.nT1;
                const int nMax = w.nMax;
                // first scores of both tiles (a tile's softmax group is past the previous item's epilogue when it hands
                // over the first P, which is what the first P V product waits for before it overwrites O)
                for (int t = 0; t < 2 && okay; t++) {
                    if (nT[t] == 0) continue;
                    okay = mbar_wait(bar(BAR_QREADY + t), uc[t] & 1, abortFlag);
                    if (okay) okay = mbar_wait(bar(BAR_K_FULL + lc % kStages), (lc / kStages) & 1, abortFlag);
                    if (!okay) break;
                    fence_after();
                    issue_qk(t, 0);
                }
                for (int j = 0; j < nMax && okay; j++) {
                    const uint32_t ring = lc + (uint32_t)j;
                    const int st = ring % kStages;
                    for (int t = 0; t < 2 && okay; t++) {
                        if (j >= nT[t]) continue;
                        PF_STAMP(2048 + 512 * t + j * 8 + 0);
                        if (t == 0 || j >= nT[0]) {  // (tile 1 finds the stages its neighbour has already waited for)
                            okay = mbar_wait(bar(BAR_V_FULL + st), (ring / kStages) & 1, abortFlag);
                            if (okay && j + 1 < nMax) okay = mbar_wait(bar(BAR_K_FULL + (ring + 1) % kStages), ((ring + 1) / kStages) & 1, abortFlag);
                        }
                        PF_STAMP(2048 + 512 * t + j * 8 + 1);
                        if (okay) okay = mbar_wait(bar(BAR_P + t), (sc[t] + (uint32_t)j) & 1, abortFlag);
                        if (!okay) break;
                        fence_after();
                        PF_STAMP(2048 + 512 * t + j * 8 + 2);
                        okay = issue_pv(t, j);
                        if (!okay) break;
                        PF_STAMP(2048 + 512 * t + j * 8 + 3);
                        if (j + 1 < nT[t]) issue_qk(t, j + 1);
                        else if (leader) mma_commit(bar(BAR_O + t));
                        // last product that reads this V stage (tile 1 while it is still running, else tile 0)
                        if (leader && (t == 1 || j >= nT[1])) mma_commit(bar(BAR_V_EMPTY + st));
                        __syncwarp();
                        PF_STAMP(2048 + 512 * t + j * 8 + 4);
                    }
                }
                lc += (uint32_t)nMax;
                for (int t = 0; t < 2; t++) {
                    sc[t] += (uint32_t)nT[t];
                    uc[t] += nT[t] > 0 ? 1u : 0u;
                }
            }
            if (!okay) *abortFlag = 1;
        }
    } else if (warp < 8) {
        // ------------------------------------------------ softmax / epilogue groups -----------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        const int t = warp >> 2;                  // query tile of this group
        const int row = threadIdx.x & 127;        // TMEM lane = query row within the tile
        const uint32_t laneBase = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t colS = kColS + t * 128, colO = kColO + t * 128;
        const float scale = p.scaleLog2;
        bool okay = true;
        uint32_t sc = 0, uc = 0;  // parities of the key-tile steps / items this group has run so far (barrier phases)
#pragma unroll 1
        for (int it = 0; okay; it++) {
        int n, q0;
        {
            Item w;
            if (!get_item(it, w)) break;
            n = t == 0 ? w.nT0 : w.nT1;
            q0 = w.q0;
        }
        if (n == 0) continue;
        const int qPos = q0 + t * kBM + row;
        {
            if (p.ropeMode != 2 && p.ropeTable != nullptr)
                okay = rotate_q_when_loaded<BF16>(smem + kSmemQ + t * kTileBytes, warp & 3, lane, p.ropeMode, p.ropeTable, p.seqLen,
                                                  q0 + t * kBM, bar(BAR_Q + t), uc & 1, abortFlag);
            else
                okay = __all_sync(0xffffffffu, mbar_wait(bar(BAR_Q + t), uc & 1, abortFlag));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
            mbar_arrive(bar(BAR_QREADY + t));
        }
        float mUsed = -INFINITY;   // the maximum the stored P and O are relative to (scaled, log2 domain)
        float lsum = 0.f;
        for (int j = 0; j < n && okay; j++) {
            if ((threadIdx.x & 127) == 0) PF_STAMP(1024 * t + j * 8 + 0);
            okay = __all_sync(0xffffffffu, mbar_wait(bar(BAR_S + t), (sc ^ (uint32_t)j) & 1, abortFlag));  // keeps the warp convergent
            if (!okay) break;
            fence_after();
            if ((threadIdx.x & 127) == 0) PF_STAMP(1024 * t + j * 8 + 1);
            uint32_t sreg[128];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_ld32(laneBase + colS + c * 32, sreg + c * 32);
            tmem_wait_ld();
            if ((threadIdx.x & 127) == 0) PF_STAMP(1024 * t + j * 8 + 2);
            const int key0 = j * kBN;
            if ((p.causal && key0 + kBN - 1 > q0 + t * kBM) || (key0 + kBN > p.seqLen)) {
                // diagonal or ragged tile: mask keys beyond the row position / the sequence end
#pragma unroll
                for (int i = 0; i < 128; i++) {
                    const int key = key0 + i;
                    if ((p.causal && key > qPos) || key >= p.seqLen) sreg[i] = 0xFF800000u;  // -inf
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
#pragma unroll
                for (int u = 0; u < 4; u++) mx4[u] = fmax3(mx4[u], __uint_as_float(sreg[i + 2 * u]), __uint_as_float(sreg[i + 2 * u + 1]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale;  // scale > 0
            // lazy rescale: keep the old reference maximum unless the row maximum grew by more than 8 (a factor 256)
            const bool first = mUsed == -INFINITY;
            const bool grow = first ? (mx > -INFINITY) : (mx > mUsed + 8.0f);
            const float mNew = grow ? mx : mUsed;
            const float alpha = (grow && !first) ? ex2_approx(mUsed - mNew) : 1.0f;
            if (j > 0 && __any_sync(0xffffffffu, grow && !first)) {
                // some row of this warp moved its maximum: rescale the O rows (alpha = 1 for the others)
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    uint32_t oreg[32];
                    tmem_ld32(laneBase + colO + c * 32, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                    tmem_st32(laneBase + colO + c * 32, oreg);
                }
            }
            if ((threadIdx.x & 127) == 0) PF_STAMP(1024 * t + j * 8 + 3);
            lsum *= alpha;
            mUsed = mNew;
            const float negM = first && !grow ? 0.f : -mUsed;  // fully masked so far: every score is -inf and exp gives 0
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            // scale-and-shift and the row sums run two elements at a time on the packed f32x2 pipe (same roundings as the
            // scalar fused multiply-add / add); every exponential runs on the special-function unit (moving a quarter of
            // them to a polynomial on the FMA pipe, packed or not, never paid, with 168 or with 200 registers per thread:
            // one warp per scheduler hides little latency, so the extra instructions cost more than the unit's queue).
            // P is packed in place (word i receives elements 2i and 2i+1, consumed by then) and written over the first 64
            // columns of S in two halves of 64 keys, each handed to the MMA warp as soon as it is stored, so the first half
            // of the P V product overlaps the second half of the exponentials.
            const uint64_t SC = pk2(scale, scale), NM = pk2(negM, negM);
            uint64_t sumA = pk2(0.f, 0.f), sumB = pk2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                const uint64_t X01 = fma2(pk2(__uint_as_float(sreg[2 * i]), __uint_as_float(sreg[2 * i + 1])), SC, NM);
                const uint64_t X23 = fma2(pk2(__uint_as_float(sreg[2 * i + 2]), __uint_as_float(sreg[2 * i + 3])), SC, NM);
                float x0, x1, x2, x3;
                un2(X01, x0, x1);
                un2(X23, x2, x3);
                const uint64_t E01 = pk2(ex2_approx(x0), ex2_approx(x1)), E23 = pk2(ex2_approx(x2), ex2_approx(x3));
                sumA = add2(sumA, E01);
                sumB = add2(sumB, E23);
                float e0, e1, e2, e3;
                un2(E01, e0, e1);
                un2(E23, e2, e3);
                sreg[i] = pack2<BF16>(e0, e1);
                sreg[i + 1] = pack2<BF16>(e2, e3);
                if (i == 30) {
                    tmem_st32(laneBase + colS, sreg);
                    tmem_wait_st();
                    fence_before();
                    mbar_arrive(bar(BAR_P + t));
                }
            }
            {
                float a0, a1, b0, b1;
                un2(sumA, a0, a1);
                un2(sumB, b0, b1);
                sum4[0] = a0; sum4[1] = a1; sum4[2] = b0; sum4[3] = b1;
            }
            tmem_st32(laneBase + colS + 32, sreg + 32);
            tmem_wait_st();
            fence_before();
            mbar_arrive(bar(BAR_P2 + t));
            if ((threadIdx.x & 127) == 0) PF_STAMP(1024 * t + j * 8 + 4);
            lsum += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if ((threadIdx.x & 127) == 0) PF_STAMP(1024 * t + j * 8 + 5);
        }
        // epilogue: wait for the last P V product of this tile, normalise and store
        {
            if (okay) okay = __all_sync(0xffffffffu, mbar_wait(bar(BAR_O + t), uc & 1, abortFlag));
            // Stage the normalised rows in the swizzled box layout and let TMA write them out as two 64-column boxes:
            // coalesced, asynchronous, and clipped at the end of the sequence by the tensor map.  The staging tile is shared
            // by the groups in turn (tile 0, tile 1, tile 0 of the next item, ...): STGFREE completes one phase per release,
            // so tile 0 waits for an odd phase (none before its first item) and tile 1 for an even one.
            if (okay && (t == 1 || it > 0)) okay = __all_sync(0xffffffffu, mbar_wait(bar(BAR_STGFREE), t == 0 ? 1u : 0u, abortFlag));
            if (okay) {
                fence_after();
                const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
                unsigned char* stage = smem + kSmemStage + row * 128;
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    uint32_t oreg[32];
                    tmem_ld32(laneBase + colO + c * 32, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int v4 = 0; v4 < 4; v4++) {
                        Vec16 o;
#pragma unroll
                        for (int w = 0; w < 4; w++)
                            o.w[w] = pack2<BF16>(__uint_as_float(oreg[v4 * 8 + 2 * w]) * inv, __uint_as_float(oreg[v4 * 8 + 2 * w + 1]) * inv);
                        const int chunk = c * 4 + v4;  // 16-byte chunk of the 256-byte row
                        *(Vec16*)(stage + (chunk >> 3) * kHalfTile + (((chunk & 7) ^ (row & 7)) * 16)) = o;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                // every row of the group is staged: the store warp of this tile (counted barrier, bounded wait) takes it from here
                mbar_arrive(bar(BAR_STAGED + t));
            } else {
                *abortFlag = 1;
            }
        }
        sc ^= (uint32_t)n;
        uc ^= 1u;
        }  // items
    }
    // ---------------------------------------------------- teardown ----------------------------------------------------
    fence_before();
    __syncthreads();
    if (abortShared && threadIdx.x == 0) atomicExch(p.errorFlag, 2);
    if (warp == 8) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

}  // namespace pf

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

// [B, S, H, 128] 16-bit tensor -> 4-D map (d, head, s, b) with a 64 x 1 x 128 x 1 box and 128-byte swizzle
static bool make_map(CUtensorMap* tm, const void* base, bool bf16, uint32_t batch, uint32_t seq, uint32_t heads) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {128, heads, seq, batch};
    cuuint64_t strides[3] = {256, (cuuint64_t)heads * 256, (cuuint64_t)seq * heads * 256};
    cuuint32_t box[4] = {64, 1, 128, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, (void*)base, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool prefill_supported(int dt, uint32_t seqQ, uint32_t seqK, uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal) {
    if (dt != DT_BF16 && dt != DT_F16) return false;
    if (headDim != 128 || seqQ != seqK || seqQ < 128) return false;  // square (self-attention) problems; short ones use the exact kernel
    if (kvHeads == 0 || numHeads % kvHeads != 0) return false;
    (void)causal;
    return encode_fn() != nullptr;
}

// K pre-pass: rotates [B, S, Hkv, 128] rows with the per-position table (positions restart for every batch item)
template <bool BF16>
__global__ void __launch_bounds__(256) rope_k_prepass_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out,
                                                            const float* __restrict__ table, size_t batch, size_t seqLen, size_t heads,
                                                            int halfMode) {
    const size_t half = 64;
    const float* cosT = table;
    const float* sinT = table + seqLen * half;
    const size_t itemsPerHead = halfMode ? 8 : 16;  // 16-byte work items per head row
    const size_t total = batch * seqLen * heads * itemsPerHead;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += stride) {
        const size_t j = it % itemsPerHead, row = it / itemsPerHead;  // row = (b*S + s)*heads + h
        const size_t s = (row / heads) % seqLen;
        const uint16_t* src = in + row * 128;
        uint16_t* dst = out + row * 128;
        if (halfMode) {
            Vec16 a = ld_stream(src + j * 8), bq = ld_stream(src + 64 + j * 8);
            const float4 c0 = __ldg((const float4*)(cosT + s * half + j * 8)), c1 = __ldg((const float4*)(cosT + s * half + j * 8 + 4));
            const float4 s0 = __ldg((const float4*)(sinT + s * half + j * 8)), s1 = __ldg((const float4*)(sinT + s * half + j * 8 + 4));
            const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                float re[2], ro[2];
#pragma unroll
                for (int hsel = 0; hsel < 2; hsel++) {
                    const int pi = w * 2 + hsel;
                    const float e = pf::widen16<BF16>((a.w[w] >> (16 * hsel)) & 0xFFFFu), o = pf::widen16<BF16>((bq.w[w] >> (16 * hsel)) & 0xFFFFu);
                    re[hsel] = sub(mul(e, cs[pi]), mul(o, sn[pi]));
                    ro[hsel] = add(mul(e, sn[pi]), mul(o, cs[pi]));
                }
                a.w[w] = pf::pack2<BF16>(re[0], re[1]);
                bq.w[w] = pf::pack2<BF16>(ro[0], ro[1]);
            }
            st_stream(dst + j * 8, a);
            st_stream(dst + 64 + j * 8, bq);
        } else {
            Vec16 a = ld_stream(src + j * 8);
            const float4 c4 = __ldg((const float4*)(cosT + s * half + j * 4)), s4 = __ldg((const float4*)(sinT + s * half + j * 4));
            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float e = pf::widen16<BF16>(a.w[w] & 0xFFFFu), o = pf::widen16<BF16>(a.w[w] >> 16);
                a.w[w] = pf::pack2<BF16>(sub(mul(e, cs[w]), mul(o, sn[w])), add(mul(e, sn[w]), mul(o, cs[w])));
            }
            st_stream(dst + j * 8, a);
        }
    }
}

int launch_prefill(Context* ctx, int dt, const void* q, const void* k, const void* v, void* out, uint32_t batch, uint32_t seqLen,
                   uint32_t numHeads, uint32_t kvHeads, uint32_t headDim, uint32_t causal, int ropeMode, const float* ropeTable,
                   CUDAStatus* status) {
    if (!prefill_supported(dt, seqLen, seqLen, numHeads, kvHeads, headDim, causal))
        return fail(status, -6, "prefill attention: tensor-core kernel not available for this shape");
    const bool bf16 = dt == DT_BF16;
    const void* kUse = k;
    if (ropeMode != 2) {
        if (!ropeTable) return fail(status, -2, "prefill attention: missing rope table");
        // rotated K lives in the workspace (the caller sized it)
        const size_t kBytes = (size_t)batch * seqLen * kvHeads * 128 * 2;
        if (ctx->workspaceBytes < kBytes) return fail(status, -7, "prefill attention: workspace not prepared");
        uint16_t* kRot = (uint16_t*)ctx->workspace;
        const size_t items = (size_t)batch * seqLen * kvHeads * (ropeMode == 1 ? 8 : 16);
        size_t blocks = (items + 255) / 256, cap = (size_t)ctx->smCount * 16;
        if (blocks > cap) blocks = cap;
        if (bf16) rope_k_prepass_kernel<true><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const uint16_t*)k, kRot, ropeTable, batch, seqLen, kvHeads, ropeMode);
        else rope_k_prepass_kernel<false><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const uint16_t*)k, kRot, ropeTable, batch, seqLen, kvHeads, ropeMode);
        int rc = check_launch(ctx, status, "rope K pre-pass");
        if (rc != 0) return rc;
        kUse = kRot;
    }
    pf::Params p;
    memset(&p, 0, sizeof(p));
    if (!make_map(&p.tmQ, q, bf16, batch, seqLen, numHeads) || !make_map(&p.tmK, kUse, bf16, batch, seqLen, kvHeads) ||
        !make_map(&p.tmV, v, bf16, batch, seqLen, kvHeads) || !make_map(&p.tmO, out, bf16, batch, seqLen, numHeads))
        return fail(status, -7, "prefill attention: tensor map encoding failed");
    p.out = out;
    p.ropeTable = ropeMode != 2 ? ropeTable : nullptr;
    p.errorFlag = ctx->errorFlag;
    p.batch = (int)batch; p.seqLen = (int)seqLen; p.numHeads = (int)numHeads; p.kvHeads = (int)kvHeads;
    p.causal = (int)causal; p.ropeMode = ropeMode;
    p.scaleLog2 = (float)(1.0 / sqrt(128.0)) * 1.4426950408889634f;
    p.vLBO = pf::kHalfTile;  // next 64 head dimensions (next swizzled block)
    p.vSBO = 1024;           // next 8 keys
#ifdef PUTER_TRACE
    p.trace = nullptr;
    if (const char* e = getenv("PUTER_TRACE_PTR")) p.trace = (long long*)strtoull(e, nullptr, 0);
#endif
    unsigned items = ((seqLen + 2 * pf::kBM - 1) / (2 * pf::kBM)) * numHeads * batch;
    dim3 grid(items < (unsigned)ctx->smCount ? items : (unsigned)ctx->smCount);  // persistent: one CTA per SM (shared memory allows no more)
#define PF_LAUNCH(B)                                                                                                           \
    do {                                                                                                                       \
        cudaFuncSetAttribute(pf::prefill_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf::kSmemTotal);      \
        pf::prefill_kernel<B><<<grid, pf::kThreads, pf::kSmemTotal, ctx->stream>>>(p);                                     \
    } while (0)
    // (scores are not re-rounded to the storage type before the softmax as the CPU path does: contexts in exact mode take the
    // scalar kernel, which does)
    if (bf16) PF_LAUNCH(true);
    else PF_LAUNCH(false);
#undef PF_LAUNCH
    return check_launch(ctx, status, "prefill attention");
}

}  // namespace puter
