// Runtime half of the C ABI: contexts (one per GPU ordinal), buffer handles, streams, status.
// Mirrors the conventions of the reference bridge (device/cuda/internal/bridge/runtime.c,
// status.c) with precompiled sm_100a kernels in place of the NVRTC module cache.
#include <stdarg.h>
#include <mutex>

#include "common.cuh"

namespace puter {

int fail(CUDAStatus* status, int code, const char* fmt, ...) {
    if (status) {
        status->code = code;
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(status->message, CUDA_STATUS_MESSAGE_BYTES, fmt, ap);
        va_end(ap);
    }
    return code;
}

int ok(CUDAStatus* status) {
    if (status) {
        status->code = 0;
        status->message[0] = 0;
    }
    return 0;
}

Context* ctx_of(CUDADeviceRef ref, CUDAStatus* status) {
    if (!ref) {
        fail(status, -1, "cuda: nil device context");
        return nullptr;
    }
    return (Context*)ref;
}

void* dev_ptr(CUDABufferRef ref) { return ref ? ((Buffer*)ref)->ptr : nullptr; }

int check_buffer(CUDAStatus* status, CUDABufferRef ref, const char* name, size_t needBytes) {
    if (!ref || !((Buffer*)ref)->ptr) return fail(status, -2, "cuda: nil buffer '%s'", name);
    Buffer* b = (Buffer*)ref;
    if (b->bytes >= 0 && (size_t)b->bytes < needBytes)
        return fail(status, -2, "cuda: buffer '%s' holds %lld bytes, call needs %zu", name, b->bytes, needBytes);
    return 0;
}

int check_launch(Context* ctx, CUDAStatus* status, const char* what) {
    ctx->launches++;
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(status, -7, "cuda: launch of %s failed: %s", what, cudaGetErrorString(err));
    return ok(status);
}

void* ensure_workspace(Context* ctx, size_t bytes, CUDAStatus* status) {
    if (bytes <= ctx->workspaceBytes) return ctx->workspace;
    // grow-only; the old block may still be in use by work queued on the stream
    if (ctx->workspace) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->workspace);
        ctx->workspace = nullptr;
        ctx->workspaceBytes = 0;
    }
    size_t want = bytes + (bytes >> 2);
    if (cudaMalloc(&ctx->workspace, want) != cudaSuccess) {
        cudaGetLastError();
        fail(status, -7, "cuda: workspace allocation of %zu bytes failed", want);
        return nullptr;
    }
    ctx->workspaceBytes = want;
    return ctx->workspace;
}

static std::mutex g_mu;
static Context* g_default = nullptr;

}  // namespace puter

using namespace puter;

extern "C" {

void cuda_status_clear(CUDAStatus* status) {
    if (!status) return;
    status->code = 0;
    status->message[0] = 0;
}

void cuda_status_set(CUDAStatus* status, int code, const char* message) {
    if (!status) return;
    status->code = code;
    snprintf(status->message, CUDA_STATUS_MESSAGE_BYTES, "%s", message ? message : "");
}

int cuda_open_device_index(int ordinal, CUDADeviceRef* outDevice, CUDAStatus* status) {
    cuda_status_clear(status);
    if (!outDevice) return fail(status, -2, "cuda: nil outDevice");
    *outDevice = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return fail(status, -1, "cuda: no CUDA device available (this library has no CPU fallback)");
    }
    if (ordinal < 0 || ordinal >= count) return fail(status, -1, "cuda: device ordinal %d out of range (%d devices)", ordinal, count);
    if (cudaSetDevice(ordinal) != cudaSuccess) return fail(status, -1, "cuda: cudaSetDevice(%d) failed", ordinal);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess) return fail(status, -1, "cuda: device properties unavailable");
    if (prop.major < 10)
        return fail(status, -1, "cuda: device %d is sm_%d%d; this library ships sm_100a code only", ordinal, prop.major, prop.minor);
    Context* ctx = new Context();
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = ordinal;
    ctx->ccMajor = prop.major;
    ctx->smCount = prop.multiProcessorCount;
    ctx->totalMem = (long long)prop.totalGlobalMem;
    if (cudaStreamCreateWithFlags(&ctx->ownStream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&ctx->uploadStream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return fail(status, -7, "cuda: stream creation failed");
    }
    ctx->stream = ctx->ownStream;
    for (int i = 0; i < 4; i++) cudaEventCreateWithFlags(&ctx->stageEvents[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&ctx->streamSwitchEvent, cudaEventDisableTiming);
    if (cudaMalloc((void**)&ctx->errorFlag, 256) != cudaSuccess) {
        delete ctx;
        return fail(status, -7, "cuda: context allocation failed");
    }
    cudaMemset(ctx->errorFlag, 0, 256);
    ctx->decodeCounterBytes = 64 << 10;
    if (cudaMalloc((void**)&ctx->decodeCounters, ctx->decodeCounterBytes) != cudaSuccess) {
        cudaFree(ctx->errorFlag);
        delete ctx;
        return fail(status, -7, "cuda: context allocation failed");
    }
    cudaMemset(ctx->decodeCounters, 0, ctx->decodeCounterBytes);
    *outDevice = ctx;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_default) g_default = ctx;
    return ok(status);
}

int cuda_open_device(CUDADeviceRef* outDevice, CUDAStatus* status) { return cuda_open_device_index(0, outDevice, status); }

void cuda_close_device(CUDADeviceRef device) {
    if (!device) return;
    Context* ctx = (Context*)device;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamSynchronize(ctx->uploadStream);
    if (ctx->workspace) cudaFree(ctx->workspace);
    for (int i = 0; i < 2; i++)
        if (ctx->pinned[i]) cudaFreeHost(ctx->pinned[i]);
    if (ctx->errorFlag) cudaFree(ctx->errorFlag);
    if (ctx->decodeCounters) cudaFree(ctx->decodeCounters);
    if (ctx->ropeTable) cudaFree(ctx->ropeTable);
    for (int i = 0; i < 4; i++)
        if (ctx->stageEvents[i]) cudaEventDestroy(ctx->stageEvents[i]);
    if (ctx->streamSwitchEvent) cudaEventDestroy(ctx->streamSwitchEvent);
    cudaStreamDestroy(ctx->ownStream);
    cudaStreamDestroy(ctx->uploadStream);
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (g_default == ctx) g_default = nullptr;
    }
    delete ctx;
}

long long cuda_device_total_memory(CUDADeviceRef device) { return device ? ((Context*)device)->totalMem : 0; }
int cuda_device_capability_major(CUDADeviceRef device) { return device ? ((Context*)device)->ccMajor : 0; }

CUDABufferRef cuda_buffer_alloc(CUDADeviceRef device, long long bytes) {
    if (!device || bytes <= 0) return nullptr;
    Context* ctx = (Context*)device;
    cudaSetDevice(ctx->device);
    void* p = nullptr;
    if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    Buffer* b = new Buffer{p, bytes, 1, ctx->device};
    return b;
}

CUDABufferRef cuda_buffer_wrap(CUDADeviceRef device, void* devicePtr, long long bytes) {
    if (!device || !devicePtr) return nullptr;
    return new Buffer{devicePtr, bytes, 0, ((Context*)device)->device};
}

void cuda_buffer_release(CUDABufferRef buffer) {
    if (!buffer) return;
    Buffer* b = (Buffer*)buffer;
    if (b->owned == 1 && b->ptr) {
        cudaSetDevice(b->device);
        cudaFree(b->ptr);
    } else if (b->owned == 2 && b->ptr) {  // a peer's allocation mapped by cuda_buffer_ipc_import
        cudaSetDevice(b->device);
        cudaIpcCloseMemHandle(b->ptr);
    }
    delete b;
}

int cuda_buffer_ipc_export(CUDABufferRef buffer, void* outHandle64, CUDAStatus* status) {
    cuda_status_clear(status);
    if (!buffer || !outHandle64) return fail(status, -2, "cuda: nil argument in ipc export");
    Buffer* b = (Buffer*)buffer;
    if (b->owned != 1) return fail(status, -2, "cuda: only buffers allocated by cuda_buffer_alloc can be exported");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI fixes the handle at 64 bytes");
    cudaSetDevice(b->device);
    cudaIpcMemHandle_t h;
    cudaError_t err = cudaIpcGetMemHandle(&h, b->ptr);
    if (err != cudaSuccess) return fail(status, -7, "cuda: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(err));
    memcpy(outHandle64, &h, 64);
    return ok(status);
}

CUDABufferRef cuda_buffer_ipc_import(CUDADeviceRef device, const void* handle64, long long bytes, CUDAStatus* status) {
    cuda_status_clear(status);
    Context* ctx = ctx_of(device, status);
    if (!ctx) return nullptr;
    if (!handle64 || bytes <= 0) { fail(status, -2, "cuda: nil handle in ipc import"); return nullptr; }
    cudaSetDevice(ctx->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess || !p) {
        cudaGetLastError();
        fail(status, -7, "cuda: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(err));
        return nullptr;
    }
    ok(status);
    return new Buffer{p, bytes, 2, ctx->device};
}

void* cuda_buffer_device_ptr(CUDABufferRef buffer) { return dev_ptr(buffer); }

int cuda_memcpy_async_h2d(CUDABufferRef dst, const void* src, long long bytes, CUDAStreamRef stream, CUDAStatus* status) {
    cuda_status_clear(status);
    if (bytes == 0) return ok(status);
    if (!dst || !src) return fail(status, -2, "cuda: nil buffer in h2d copy");
    Buffer* b = (Buffer*)dst;
    if (b->bytes >= 0 && bytes > b->bytes) return fail(status, -2, "cuda: h2d copy of %lld bytes exceeds buffer (%lld)", bytes, b->bytes);
    cudaSetDevice(b->device);
    cudaError_t err = cudaMemcpyAsync(b->ptr, src, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream);
    if (err != cudaSuccess) return fail(status, -7, "cuda: h2d copy failed: %s", cudaGetErrorString(err));
    return ok(status);
}

int cuda_memcpy_async_d2h(void* dst, CUDABufferRef src, long long bytes, CUDAStreamRef stream, CUDAStatus* status) {
    cuda_status_clear(status);
    if (bytes == 0) return ok(status);
    if (!dst || !src) return fail(status, -2, "cuda: nil buffer in d2h copy");
    Buffer* b = (Buffer*)src;
    if (b->bytes >= 0 && bytes > b->bytes) return fail(status, -2, "cuda: d2h copy of %lld bytes exceeds buffer (%lld)", bytes, b->bytes);
    cudaSetDevice(b->device);
    cudaError_t err = cudaMemcpyAsync(dst, b->ptr, (size_t)bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (err != cudaSuccess) return fail(status, -7, "cuda: d2h copy failed: %s", cudaGetErrorString(err));
    return ok(status);
}

int cuda_memcpy_async_d2d(CUDABufferRef dst, CUDABufferRef src, long long bytes, CUDAStreamRef stream, CUDAStatus* status) {
    cuda_status_clear(status);
    if (bytes == 0) return ok(status);
    if (!dst || !src) return fail(status, -2, "cuda: nil buffer in d2d copy");
    Buffer* d = (Buffer*)dst;
    Buffer* s = (Buffer*)src;
    if (d->bytes >= 0 && bytes > d->bytes) return fail(status, -2, "cuda: d2d copy of %lld bytes exceeds the destination (%lld)", bytes, d->bytes);
    if (s->bytes >= 0 && bytes > s->bytes) return fail(status, -2, "cuda: d2d copy of %lld bytes exceeds the source (%lld)", bytes, s->bytes);
    cudaSetDevice(d->device);
    cudaError_t err = cudaMemcpyAsync(d->ptr, s->ptr, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
    if (err != cudaSuccess) return fail(status, -7, "cuda: d2d copy failed: %s", cudaGetErrorString(err));
    return ok(status);
}

int cuda_stream_synchronize(CUDAStreamRef stream, CUDAStatus* status) {
    cuda_status_clear(status);
    cudaError_t err = cudaStreamSynchronize((cudaStream_t)stream);
    if (err != cudaSuccess) return fail(status, -7, "cuda: stream synchronize failed: %s", cudaGetErrorString(err));
    return ok(status);
}

CUDADeviceRef cuda_default_context(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    return g_default;
}

CUDAStreamRef cuda_context_upload_stream(CUDADeviceRef device) { return device ? (CUDAStreamRef)((Context*)device)->uploadStream : nullptr; }
CUDAStreamRef cuda_context_default_stream(CUDADeviceRef device) { return device ? (CUDAStreamRef)((Context*)device)->stream : nullptr; }

int cuda_context_set_stream(CUDADeviceRef device, void* cudaStream, CUDAStatus* status) {
    cuda_status_clear(status);
    Context* ctx = ctx_of(device, status);
    if (!ctx) return -1;
    cudaStream_t next = (cudaStream_t)cudaStream;  // NULL = the legacy default stream
    if (next != ctx->stream) {
        // the context's scratch (workspace, RoPE table, decode counters) may still be read by kernels queued on the old stream:
        // whatever the new stream launches is ordered after them
        cudaSetDevice(ctx->device);
        if (cudaEventRecord(ctx->streamSwitchEvent, ctx->stream) == cudaSuccess) cudaStreamWaitEvent(next, ctx->streamSwitchEvent, 0);
        cudaGetLastError();
        ctx->stream = next;
    }
    return ok(status);
}

int cuda_context_reset_stream(CUDADeviceRef device, CUDAStatus* status) {
    cuda_status_clear(status);
    Context* ctx = ctx_of(device, status);
    if (!ctx) return -1;
    if (ctx->stream != ctx->ownStream) {
        cudaSetDevice(ctx->device);
        if (cudaEventRecord(ctx->streamSwitchEvent, ctx->stream) == cudaSuccess) cudaStreamWaitEvent(ctx->ownStream, ctx->streamSwitchEvent, 0);
        cudaGetLastError();
        ctx->stream = ctx->ownStream;
    }
    return ok(status);
}

int cuda_context_set_exact(CUDADeviceRef device, int exact, CUDAStatus* status) {
    cuda_status_clear(status);
    Context* ctx = ctx_of(device, status);
    if (!ctx) return -1;
    ctx->exact = exact ? 1 : 0;
    return ok(status);
}

int cuda_context_take_error(CUDADeviceRef device, int* outFlag, CUDAStatus* status) {
    cuda_status_clear(status);
    Context* ctx = ctx_of(device, status);
    if (!ctx) return -1;
    if (!outFlag) return fail(status, -2, "cuda: nil outFlag");
    cudaSetDevice(ctx->device);
    int flag = 0;
    cudaError_t err = cudaMemcpyAsync(&flag, ctx->errorFlag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
    if (err == cudaSuccess) err = cudaMemsetAsync(ctx->errorFlag, 0, sizeof(int), ctx->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(ctx->stream);
    if (err != cudaSuccess) return fail(status, -7, "cuda: reading the error flag failed: %s", cudaGetErrorString(err));
    *outFlag = flag;
    return ok(status);
}

unsigned long long cuda_context_launch_count(CUDADeviceRef device) { return device ? ((Context*)device)->launches : 0ull; }

void* cuda_host_alloc(long long bytes) {
    void* p = nullptr;
    if (bytes <= 0 || cudaMallocHost(&p, (size_t)bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

void cuda_host_free(void* ptr) {
    if (ptr) cudaFreeHost(ptr);
}

}  // extern "C"
