// api.cu -- library-wide state behind the C ABI: version, last error, device properties.
#include "s24_common.cuh"

namespace s24 {

char* last_error_buffer()
{
    static thread_local char buf[512] = {0};
    return buf;
}

int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace s24

extern "C" int s24_version(void) { return S24_VERSION; }

extern "C" const char* s24_last_error(void) { return s24::last_error_buffer(); }
