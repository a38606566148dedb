// peer.cu -- device buffers that the other GPUs of the box can write into.
//
// The reference project is single-GPU; nothing here has a counterpart in it.  A replicated
// multi-GPU result (every rank ends up with the whole C) is produced by letting each rank's
// GEMM store its column shard straight into every rank's copy of C (s24_spmm_scatter), so the
// copies of C must be mapped into every process.  These helpers wrap the CUDA IPC calls for
// that: one process allocates and exports, the others open the handle and get an address that
// their kernels can store to over NVLink.  They are the only entry points of the library that
// allocate or map memory; they synchronise like cudaMalloc / cudaFree and belong in set-up code.
#include "s24_common.cuh"

using namespace s24;

static_assert(sizeof(cudaIpcMemHandle_t) == S24_PEER_HANDLE_BYTES, "handle size");

extern "C" int s24_peer_alloc(size_t bytes, void** ptr)
{
    if (ptr == nullptr || bytes == 0) return fail(S24_ERR_INVALID_ARG, "peer_alloc: null result pointer or zero size");
    *ptr = nullptr;
    return check_cuda(cudaMalloc(ptr, bytes), "peer_alloc: cudaMalloc");
}

extern "C" int s24_peer_free(void* ptr)
{
    if (ptr == nullptr) return S24_OK;
    return check_cuda(cudaFree(ptr), "peer_free: cudaFree");
}

extern "C" int s24_peer_export(const void* ptr, void* handle)
{
    if (ptr == nullptr || handle == nullptr) return fail(S24_ERR_INVALID_ARG, "peer_export: null pointer");
    cudaIpcMemHandle_t h;
    int rc = check_cuda(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)), "peer_export: cudaIpcGetMemHandle");
    if (rc) return rc;
    memcpy(handle, &h, sizeof(h));
    return S24_OK;
}

extern "C" int s24_peer_open(const void* handle, void** ptr)
{
    if (ptr == nullptr || handle == nullptr) return fail(S24_ERR_INVALID_ARG, "peer_open: null pointer");
    *ptr = nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    // opened with the calling process's device current: peer access from that device to the
    // owner's is enabled as part of the call
    return check_cuda(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "peer_open: cudaIpcOpenMemHandle");
}

extern "C" int s24_peer_close(void* ptr)
{
    if (ptr == nullptr) return S24_OK;
    return check_cuda(cudaIpcCloseMemHandle(ptr), "peer_close: cudaIpcCloseMemHandle");
}

// A block of rows, `width_bytes` wide, from one pitched buffer to another: the transfer of a
// column shard of a row-major matrix into a peer's copy of that matrix.  Runs on the copy
// engines (cudaMemcpy2DAsync), so it needs no SM and overlaps a persistent GEMM; dst may be a
// peer mapping obtained from s24_peer_open.
extern "C" int s24_peer_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                                size_t rows, void* stream)
{
    if (dst == nullptr || src == nullptr) return fail(S24_ERR_INVALID_ARG, "peer_copy_2d: null pointer");
    if (width_bytes == 0 || rows == 0) return S24_OK;
    if (dst_pitch < width_bytes || src_pitch < width_bytes)
        return fail(S24_ERR_SHAPE, "peer_copy_2d: pitches (%zu, %zu) must be at least the width (%zu bytes)", dst_pitch, src_pitch,
                    width_bytes);
    return check_cuda(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault,
                                        static_cast<cudaStream_t>(stream)),
                      "peer_copy_2d: cudaMemcpy2DAsync");
}
