// runtime.cu -- device, memory, stream and graph entry points of libsmall_b200
// (the platform side of alloc_buffer/free_buffer and of Buffer::data(),
// include/small/platforms/reference/Buffer.hpp:36-61).
#include "common.cuh"

namespace sb
{
thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches{0};

int check_window_layer(const small_b200_layer *L, const char *name, bool dense, int max_stride)
{
    if (!L)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: null layer.");
    if (L->stride < 1 || L->stride > max_stride || L->stride_h < 0 || L->stride_h > max_stride)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: stride unsupported.");
    const bool first_layer = dense && (L->C == 1 || L->C == 2 || L->C == 3);
    if (L->C <= 0 || (L->C % CB != 0 && !first_layer))
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: in_channels unsupported.");
    if (dense && (L->K <= 0 || L->K % CB != 0))
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: out_channels unsupported.");
    if (L->N < 0 || L->H <= 0 || L->W <= 0 || L->Fh <= 0 || L->Fw <= 0 || L->pad_t < 0 ||
        L->pad_b < 0 || L->pad_l < 0 || L->pad_r < 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: bad shape.");
    return SMALL_B200_OK;
}
} // namespace sb

using namespace sb;

extern "C"
{
const char *small_b200_last_error(void) { return g_last_error.c_str(); }

int small_b200_device_count(int *count)
{
    SB_CUDA(cudaGetDeviceCount(count));
    return SMALL_B200_OK;
}

int small_b200_set_device(int device)
{
    SB_CUDA(cudaSetDevice(device));
    return SMALL_B200_OK;
}

uint64_t small_b200_launch_count(void) { return g_launches.load(); }

int small_b200_malloc(size_t bytes, void **ptr)
{
    SB_CUDA(cudaMalloc(ptr, bytes ? bytes : 1));
    return SMALL_B200_OK;
}

int small_b200_malloc_managed(size_t bytes, void **ptr)
{
    SB_CUDA(cudaMallocManaged(ptr, bytes ? bytes : 1));
    return SMALL_B200_OK;
}

int small_b200_malloc_host(size_t bytes, void **ptr)
{
    SB_CUDA(cudaMallocHost(ptr, bytes ? bytes : 1));
    return SMALL_B200_OK;
}

int small_b200_malloc_host_upload(size_t bytes, void **ptr)
{
    SB_CUDA(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocWriteCombined));
    return SMALL_B200_OK;
}

int small_b200_free(void *ptr)
{
    SB_CUDA(cudaFree(ptr));
    return SMALL_B200_OK;
}

int small_b200_free_host(void *ptr)
{
    SB_CUDA(cudaFreeHost(ptr));
    return SMALL_B200_OK;
}

int small_b200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream)
{
    SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return SMALL_B200_OK;
}

int small_b200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream)
{
    SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return SMALL_B200_OK;
}

int small_b200_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream)
{
    SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return SMALL_B200_OK;
}

int small_b200_prefetch(const void *managed_ptr, size_t bytes, void *stream)
{
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev));
    cudaMemLocation loc;
    loc.type = cudaMemLocationTypeDevice;
    loc.id = dev;
    SB_CUDA(cudaMemPrefetchAsync_v2(managed_ptr, bytes, loc, 0, as_stream(stream)));
    return SMALL_B200_OK;
}

int small_b200_stream_create(void **stream)
{
    cudaStream_t s;
    SB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return SMALL_B200_OK;
}

int small_b200_stream_destroy(void *stream)
{
    SB_CUDA(cudaStreamDestroy(as_stream(stream)));
    return SMALL_B200_OK;
}

int small_b200_stream_sync(void *stream)
{
    SB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return SMALL_B200_OK;
}

int small_b200_device_sync(void)
{
    SB_CUDA(cudaDeviceSynchronize());
    return SMALL_B200_OK;
}

int small_b200_graph_begin(void *stream)
{
    SB_CUDA(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeThreadLocal));
    return SMALL_B200_OK;
}

int small_b200_graph_end(void *stream, void **graph_exec)
{
    cudaGraph_t g = nullptr;
    SB_CUDA(cudaStreamEndCapture(as_stream(stream), &g));
    cudaGraphExec_t ge = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess)
        return cuda_fail(e, "cudaGraphInstantiate");
    *graph_exec = ge;
    return SMALL_B200_OK;
}

int small_b200_graph_launch(void *graph_exec, void *stream)
{
    SB_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph_exec), as_stream(stream)));
    return SMALL_B200_OK;
}

int small_b200_graph_destroy(void *graph_exec)
{
    SB_CUDA(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(graph_exec)));
    return SMALL_B200_OK;
}
} // extern "C"
