// Row pipeline shared by the row-wise kernels that make several passes over a row (LayerNorm family, row softmax):
// every warp owns a private ring of whole rows in shared memory, filled by bulk asynchronous copies (cp.async.bulk,
// completion counted in bytes on an mbarrier) that one lane issues.  The warp reads its row from shared memory as often as
// the operation needs, and the row costs no registers.  No block-wide barrier, no interaction between warps.
//
// Measured on 16384 x 4096 rows: what pays is warps per SM, not ring depth (the passes over a row are bound by instruction
// latency): 16 warps with one stage each beat 8 warps with three stages by 25-30 %, and deeper rings at equal warp count
// changed nothing.  The defaults below are that configuration; the ring logic keeps the general form.
//
// A bulk copy needs 16-byte aligned addresses and a size that is a multiple of 16 bytes: callers take this path only for
// rows that satisfy both, everything else runs their scalar kernels.  Every wait is bounded; a wait that runs out raises the
// error flag and the warp leaves after giving its other copies the same bounded chance to land.
#pragma once

#include "common.cuh"

#ifndef ROWPIPE_MAX_WARPS
#define ROWPIPE_MAX_WARPS 16
#endif
#ifndef ROWPIPE_MAX_STAGES
#define ROWPIPE_MAX_STAGES 1
#endif
#ifndef ROWPIPE_UN
#define ROWPIPE_UN 4
#endif

namespace puter {
namespace rowpipe {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// waits until the phase with the given parity has completed; false when the poll limit ran out (~1 s)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 24); i++) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned), completion on `bar`
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

// State of one warp's ring.  Usage:
//     Ring ring(smem, warpsPerBlock, stages, rowBytes, src, rows);      // all lanes
//     for (size_t row = ring.first(); row < rows; row = ring.next_row(row)) {
//         const unsigned char* x = ring.acquire(errorFlag);              // nullptr: a wait ran out, leave
//         ... read x ...
//         ring.release();                                                // re-arms the stage with the warp's next row
//     }
struct Ring {
    unsigned char* base;   // this warp's stages
    uint32_t barBase;      // shared address of this warp's first mbarrier
    const char* src;
    size_t rows, rowBytes, stageBytes, landOffset, stride, nextIssue;
    int stages, stage;
    uint32_t phase;
    int lane;
    int armed;             // stages that have a copy outstanding or landed but not consumed

    // stageBytes_ > rowBytes_ gives every stage room beyond the row (for results kept in shared memory); the row then lands
    // landOffset_ bytes into its stage (both multiples of 16) and acquire() still returns the start of the stage
    __device__ __forceinline__ Ring(unsigned char* smem, int warpsPerBlock, int stages_, size_t rowBytes_, const void* src_, size_t rows_,
                                    size_t stageBytes_ = 0, size_t landOffset_ = 0)
        : src((const char*)src_), rows(rows_), rowBytes(rowBytes_), stageBytes(stageBytes_ ? stageBytes_ : rowBytes_), landOffset(landOffset_),
          stages(stages_), stage(0), phase(0), armed(0) {
        const int warp = threadIdx.x >> 5;
        lane = threadIdx.x & 31;
        base = smem + (size_t)warp * stages * stageBytes;
        unsigned char* bars = smem + (size_t)warpsPerBlock * stages * stageBytes + (size_t)warp * stages * 8;
        barBase = smem_addr(bars);
        stride = (size_t)gridDim.x * warpsPerBlock;
        nextIssue = (size_t)blockIdx.x * warpsPerBlock + warp;
        if (lane == 0) {
            for (int s = 0; s < stages; s++) mbar_init(barBase + 8 * s, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        for (int s = 0; s < stages; s++) issue(s);
    }
    __device__ __forceinline__ size_t first() const { return (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); }
    __device__ __forceinline__ size_t next_row(size_t row) const { return row + stride; }

    __device__ __forceinline__ void issue(int s) {
        if (nextIssue < rows) {
            if (lane == 0) {
                const uint32_t bar = barBase + 8 * s;
                mbar_expect_tx(bar, (uint32_t)rowBytes);
                bulk_load(smem_addr(base + (size_t)s * stageBytes + landOffset), src + nextIssue * rowBytes, (uint32_t)rowBytes, bar);
            }
            nextIssue += stride;
            armed++;
        }
    }
    __device__ __forceinline__ const unsigned char* acquire(int* errorFlag) {
        if (!mbar_wait(barBase + 8 * stage, phase)) {
            if (lane == 0) atomicExch(errorFlag, 3);
            // the other copies of this warp get the same bounded time to land before the warp leaves
            int s = stage;
            uint32_t ph = phase;
            for (int k = 1; k < armed; k++) {
                if (++s == stages) { s = 0; ph ^= 1; }
                mbar_wait(barBase + 8 * s, ph);
            }
            return nullptr;
        }
        return base + (size_t)stage * stageBytes;
    }
    __device__ __forceinline__ void release() {
        __syncwarp();  // every lane has finished reading the stage
        armed--;
        issue(stage);
        if (++stage == stages) { stage = 0; phase ^= 1; }
    }
};

// Host side: warps per block, stages per warp and dynamic shared memory for stages of `rowBytes` (0 warps: row too long).
struct Plan {
    int warps, stages;
    size_t smem;
};
inline Plan plan(size_t rowBytes) {
    const size_t budget = 200 * 1024;
    Plan p{0, 0, 0};
    if (rowBytes == 0 || rowBytes % 16 != 0) return p;
    for (int warps = ROWPIPE_MAX_WARPS; warps >= 1; warps--) {
        size_t stages = budget / ((size_t)warps * rowBytes);
        if (stages > ROWPIPE_MAX_STAGES) stages = ROWPIPE_MAX_STAGES;
        if (stages >= (ROWPIPE_MAX_STAGES > 1 ? 2 : 1) || (warps == 1 && stages >= 1)) {
            p.warps = warps;
            p.stages = (int)stages;
            p.smem = (size_t)warps * stages * rowBytes + (size_t)warps * stages * 8;
            return p;
        }
    }
    return p;
}

}  // namespace rowpipe
}  // namespace puter
