// s24_common.cuh -- status reporting shared by the translation units of libs24.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/s24.h"

namespace s24 {

// per-thread text of the last failure, read through s24_last_error()
char* last_error_buffer();

inline int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

inline int check_cuda(cudaError_t e, const char* what)
{
    if (e == cudaSuccess) return S24_OK;
    return fail(S24_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// number of SMs of the current device (cached per device)
int sm_count();

}  // namespace s24
