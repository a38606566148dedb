// spmm_shared.cuh -- pieces shared by the tcgen05 sparse GEMM kernels: tile geometry, the
// persistent tile walk, the timeout report and the host helpers that build TMA descriptors.
#pragma once

#include "s24_common.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace s24 {

constexpr int kBlockK = 128;        // logical K per pipeline stage
constexpr int kRowsPerCta = 128;
#ifndef S24_GROUP_M
#define S24_GROUP_M 8
#endif
constexpr int kGroupM = S24_GROUP_M;   // M-tiles per raster group (compression/common.py:155)
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
    void* C;
    int64_t ldc;
    int M, N, K;
    int bf16;
    int* status;
    // fused output prune (unused by the plain kernel)
    void* c_vals;
    uint32_t* c_meta_ref;
    uint32_t* c_meta_tc;
    // scatter epilogue: the C tile goes to each of these (this GPU's buffer and peers' mappings),
    // all with row stride ldc; unused by the other kernels
    void* dst[8];
    int n_dst;
    // limit of every barrier wait in nanoseconds, and (self-test only, 0 = off) the number of
    // k-blocks after which the producer stops loading so that the other roles' waits run out
    unsigned long long wait_limit_ns;
    int selftest_stop_after_kblocks;
};

__device__ __forceinline__ void report_timeout(int* status, volatile int* abort_flag, int code)
{
    atomicCAS(status, 0, code);
    *abort_flag = 1;
}

// tile t of the persistent walk: groups of kGroupM row tiles swept along N so that B tiles stay in L2
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& tm, int& tn)
{
    const int group_size = kGroupM * num_n;
    const int group_id = t / group_size;
    const int first_m = group_id * kGroupM;
    const int gm = min(num_m - first_m, kGroupM);
    const int in_group = t - group_id * group_size;
    tm = first_m + in_group % gm;
    tn = in_group / gm;
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int bf16)
{
    if (bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// host side (defined in spmm_tcgen05.cu)
int make_map_2d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t inner,
                uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                CUtensorMapSwizzle swz, const char* what);
int* status_word_address();   // device address of the status word on the current device, or null

}  // namespace s24
