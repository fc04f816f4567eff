// Paged KV storage ops (device.Shape.PageWrite / PageGather, KVPageWrite / KVPageGather).
//
// Reference semantics (device/cpu/shape/page_generic.go:5-50, page.go:104-211,
// execution/page_intrinsic.go:361-438): storage is [pages, pageSize, inner] (optionally one layer of a
// rank-5 tensor selected by an element offset);
//   write : out[(pageID*pageSize + offset)*inner ...] = values[row]   (out is a copy of storage, or storage itself)
//   gather: out[row] = storage[(table[row / pageSize]*pageSize + row % pageSize)*inner ...]
// Page ids / offsets outside the valid range make the CPU op fail before touching memory; on the device such
// rows are never dereferenced: they are skipped and a device-side error flag is raised, which the host reads
// at the next synchronisation.  Pure byte movement: 16-byte vectors when rows allow, any dtype by element size.
// Two value rows aimed at the same (page, offset) in one write race with each other (the CPU loop keeps the
// last one); a KV cache never does that, and callers that might must split the write.
#include "common.cuh"

namespace puter {

__global__ void __launch_bounds__(256) page_write_kernel(char* __restrict__ out, const char* __restrict__ values,
                                                        const int32_t* __restrict__ pageIDs, const int32_t* __restrict__ offsets,
                                                        size_t pageCount, size_t pageSize, size_t rowBytes, size_t valueRows,
                                                        int vec, int* __restrict__ errorFlag) {
    const size_t unit = vec ? 16 : 1;
    const size_t perRow = rowBytes / unit;
    const size_t total = valueRows * perRow;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t row = i / perRow, c = i % perRow;
        long long page = pageIDs[row], off = offsets[row];
        if (page < 0 || page >= (long long)pageCount || off < 0 || off >= (long long)pageSize) {
            if (c == 0) atomicExch(errorFlag, 1);
            continue;
        }
        size_t dst = ((size_t)page * pageSize + (size_t)off) * rowBytes + c * unit;
        if (vec) *(Vec16*)(out + dst) = ld_stream(values + row * rowBytes + c * 16);
        else out[dst] = values[row * rowBytes + c];
    }
}

__global__ void __launch_bounds__(256) page_gather_kernel(const char* __restrict__ storage, const int32_t* __restrict__ pageTable,
                                                         char* __restrict__ out, size_t pageCount, size_t pageSize, size_t rowBytes,
                                                         size_t outRows, int vec, int* __restrict__ errorFlag) {
    const size_t unit = vec ? 16 : 1;
    const size_t perRow = rowBytes / unit;
    const size_t total = outRows * perRow;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t row = i / perRow, c = i % perRow;
        long long page = pageTable[row / pageSize];
        if (page < 0 || page >= (long long)pageCount) {
            if (c == 0) atomicExch(errorFlag, 1);
            continue;
        }
        size_t src = ((size_t)page * pageSize + row % pageSize) * rowBytes + c * unit;
        if (vec) st_stream(out + row * rowBytes + c * 16, ld_stream(storage + src));
        else out[row * rowBytes + c] = storage[src];
    }
}

// Rows of at least 16 vectors (256 bytes; a KV row of 8 heads x 128 bf16 is 2 KB): one WARP per row.  The page of a row is
// looked up once per row instead of once per 16-byte item, there is no division per item (the element-wise kernels above spend
// four 64-bit divisions on every item), and a lane has four independent copies in flight.
__global__ void __launch_bounds__(256) page_write_rows_kernel(char* __restrict__ out, const char* __restrict__ values,
                                                             const int32_t* __restrict__ pageIDs, const int32_t* __restrict__ offsets,
                                                             size_t pageCount, size_t pageSize, size_t rowBytes, size_t valueRows,
                                                             int* __restrict__ errorFlag) {
    const int lane = threadIdx.x & 31;
    const size_t perRow = rowBytes / 16;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < valueRows; row += warps) {
        const long long page = pageIDs[row], off = offsets[row];
        if (page < 0 || page >= (long long)pageCount || off < 0 || off >= (long long)pageSize) {
            if (lane == 0) atomicExch(errorFlag, 1);
            continue;
        }
        char* dst = out + ((size_t)page * pageSize + (size_t)off) * rowBytes;
        const char* src = values + row * rowBytes;
        for (size_t v0 = lane; v0 < perRow; v0 += 128) {
            Vec16 t[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (v0 + 32 * u < perRow) t[u] = ld_stream(src + (v0 + 32 * u) * 16);
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (v0 + 32 * u < perRow) *(Vec16*)(dst + (v0 + 32 * u) * 16) = t[u];
        }
    }
}

__global__ void __launch_bounds__(256) page_gather_rows_kernel(const char* __restrict__ storage, const int32_t* __restrict__ pageTable,
                                                              char* __restrict__ out, size_t pageCount, size_t pageSize, size_t rowBytes,
                                                              size_t outRows, int* __restrict__ errorFlag) {
    const int lane = threadIdx.x & 31;
    const size_t perRow = rowBytes / 16;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < outRows; row += warps) {
        const size_t entry = row / pageSize;
        const long long page = pageTable[entry];
        if (page < 0 || page >= (long long)pageCount) {
            if (lane == 0) atomicExch(errorFlag, 1);
            continue;
        }
        const char* src = storage + ((size_t)page * pageSize + (row - entry * pageSize)) * rowBytes;
        char* dst = out + row * rowBytes;
        for (size_t v0 = lane; v0 < perRow; v0 += 128) {
            Vec16 t[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (v0 + 32 * u < perRow) t[u] = ld_stream(src + (v0 + 32 * u) * 16);
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (v0 + 32 * u < perRow) st_stream(dst + (v0 + 32 * u) * 16, t[u]);
        }
    }
}

// output[b] = input[b, seq - 1, :]: rows of rowBytes, one per batch item (device/cpu/shape/ops.go:133-160)
__global__ void __launch_bounds__(256) last_token_kernel(const char* __restrict__ in, char* __restrict__ out, size_t batch, size_t seq,
                                                        size_t rowBytes, int vec) {
    const size_t unit = vec ? 16 : 1;
    const size_t perRow = rowBytes / unit;
    const size_t total = batch * perRow;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t b = i / perRow, c = i % perRow;
        const size_t src = ((b * seq + seq - 1) * rowBytes) + c * unit;
        if (vec) st_stream(out + b * rowBytes + c * 16, ld_stream(in + src));
        else out[b * rowBytes + c] = in[src];
    }
}

}  // namespace puter

using namespace puter;

static int page_grid(Context* ctx, size_t items) {
    size_t blocks = (items + 255) / 256, cap = (size_t)ctx->smCount * 16;
    if (blocks > cap) blocks = cap;
    return blocks ? (int)blocks : 1;
}

extern "C" int cuda_dispatch_kv_page_write(CUDADeviceRef contextRef, int elementDType, CUDABufferRef storageRef, CUDABufferRef valuesRef,
                                           CUDABufferRef pageIDsRef, CUDABufferRef offsetsRef, CUDABufferRef outputRef, uint32_t pageCount,
                                           uint32_t pageSize, uint32_t inner, uint32_t valueRows, uint64_t storageOffset,
                                           uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    size_t es = dtype_size(elementDType);
    if (es == 0) return fail(status, -6, "page write: unsupported dtype %d", elementDType);
    if (pageCount == 0 || pageSize == 0 || inner == 0) return ok(status);
    size_t layerBytes = (size_t)pageCount * pageSize * inner * es;
    size_t offBytes = (size_t)storageOffset * es;
    PUTER_REQUIRE(storageRef, "storage", offBytes + layerBytes);
    PUTER_REQUIRE(outputRef, "output", offBytes + layerBytes);
    char* st = (char*)dev_ptr(storageRef) + offBytes;
    char* out = (char*)dev_ptr(outputRef) + offBytes;
    if (out != st) {
        // functional form of the CPU op: the result starts as a copy of the storage layer
        if (cudaMemcpyAsync(out, st, layerBytes, cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess)
            return fail(status, -7, "page write: storage copy failed");
    }
    if (valueRows == 0) return ok(status);
    size_t rowBytes = (size_t)inner * es;
    PUTER_REQUIRE(valuesRef, "values", (size_t)valueRows * rowBytes);
    PUTER_REQUIRE(pageIDsRef, "pageIDs", (size_t)valueRows * 4);
    PUTER_REQUIRE(offsetsRef, "offsets", (size_t)valueRows * 4);
    const char* vals = (const char*)dev_ptr(valuesRef);
    int vec = rowBytes % 16 == 0 && (((uintptr_t)out | (uintptr_t)vals) & 15u) == 0;
    size_t items = (size_t)valueRows * (vec ? rowBytes / 16 : rowBytes);
    if (vec && rowBytes >= 256)
        page_write_rows_kernel<<<page_grid(ctx, (size_t)valueRows * 32), 256, 0, ctx->stream>>>(
            out, vals, (const int32_t*)dev_ptr(pageIDsRef), (const int32_t*)dev_ptr(offsetsRef), pageCount, pageSize, rowBytes, valueRows,
            ctx->errorFlag);
    else
        page_write_kernel<<<page_grid(ctx, items), 256, 0, ctx->stream>>>(out, vals, (const int32_t*)dev_ptr(pageIDsRef),
                                                                          (const int32_t*)dev_ptr(offsetsRef), pageCount, pageSize, rowBytes,
                                                                          valueRows, vec, ctx->errorFlag);
    return check_launch(ctx, status, "kv page write");
}

extern "C" int cuda_dispatch_kv_page_gather(CUDADeviceRef contextRef, int elementDType, CUDABufferRef storageRef, CUDABufferRef pageTableRef,
                                            CUDABufferRef outputRef, uint32_t pageCount, uint32_t pageSize, uint32_t inner, uint32_t outRows,
                                            uint64_t storageOffset, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    size_t es = dtype_size(elementDType);
    if (es == 0) return fail(status, -6, "page gather: unsupported dtype %d", elementDType);
    if (pageCount == 0 || pageSize == 0 || inner == 0 || outRows == 0) return ok(status);
    size_t rowBytes = (size_t)inner * es;
    size_t offBytes = (size_t)storageOffset * es;
    PUTER_REQUIRE(storageRef, "storage", offBytes + (size_t)pageCount * pageSize * rowBytes);
    PUTER_REQUIRE(pageTableRef, "pageTable", (((size_t)outRows + pageSize - 1) / pageSize) * 4);
    PUTER_REQUIRE(outputRef, "output", (size_t)outRows * rowBytes);
    const char* st = (const char*)dev_ptr(storageRef) + offBytes;
    char* out = (char*)dev_ptr(outputRef);
    int vec = rowBytes % 16 == 0 && (((uintptr_t)out | (uintptr_t)st) & 15u) == 0;
    size_t items = (size_t)outRows * (vec ? rowBytes / 16 : rowBytes);
    if (vec && rowBytes >= 256)
        page_gather_rows_kernel<<<page_grid(ctx, (size_t)outRows * 32), 256, 0, ctx->stream>>>(st, (const int32_t*)dev_ptr(pageTableRef), out,
                                                                                              pageCount, pageSize, rowBytes, outRows, ctx->errorFlag);
    else
        page_gather_kernel<<<page_grid(ctx, items), 256, 0, ctx->stream>>>(st, (const int32_t*)dev_ptr(pageTableRef), out, pageCount, pageSize,
                                                                           rowBytes, outRows, vec, ctx->errorFlag);
    return check_launch(ctx, status, "kv page gather");
}

extern "C" int cuda_dispatch_last_token(CUDADeviceRef contextRef, int elementDType, CUDABufferRef inputRef, CUDABufferRef outRef, uint32_t batch,
                                        uint32_t seq, uint32_t hidden, uint64_t completionToken, CUDAStatus* status) {
    (void)completionToken;
    PUTER_ENTER(ctx);
    size_t es = dtype_size(elementDType);
    if (es == 0) return fail(status, -6, "last token: unsupported dtype %d", elementDType);
    if (batch == 0 || seq == 0 || hidden == 0) return ok(status);  // device/cpu/shape/ops.go:140-142
    const size_t rowBytes = (size_t)hidden * es;
    PUTER_REQUIRE(inputRef, "input", (size_t)batch * seq * rowBytes);
    PUTER_REQUIRE(outRef, "output", (size_t)batch * rowBytes);
    const char* in = (const char*)dev_ptr(inputRef);
    char* out = (char*)dev_ptr(outRef);
    int vec = rowBytes % 16 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15u) == 0;
    size_t items = (size_t)batch * (vec ? rowBytes / 16 : rowBytes);
    last_token_kernel<<<page_grid(ctx, items), 256, 0, ctx->stream>>>(in, out, batch, seq, rowBytes, vec);
    return check_launch(ctx, status, "last token");
}
