/* A C caller of the library: compiled with gcc against include/s24.h and linked to libs24.so,
 * it exercises the part of the C ABI that needs no GPU (version, sizes, argument validation, the
 * per-thread error text).  Test infrastructure: shows that the boundary is plain C. */
#include <stdio.h>
#include <string.h>
#include "s24.h"

#define CHECK(cond)                                                            \
    do {                                                                       \
        if (!(cond)) {                                                         \
            printf("FAILED line %d: %s (last error: %s)\n", __LINE__, #cond, s24_last_error()); \
            return 1;                                                          \
        }                                                                      \
    } while (0)

int main(void)
{
    static char buf[4096] __attribute__((aligned(64)));
    s24_tile_cfg cfg = {256, 256, 0, 0};
    CHECK(s24_version() == S24_VERSION);
    CHECK(s24_meta_tc_bytes(8192, 8192) == (size_t)S24_STATIC_SCRATCH_BYTES);
    CHECK(s24_meta_tc_bytes(160, 192) == 4 * 2048);
    CHECK(s24_meta_tc_bytes(0, 128) == 0);
    CHECK(s24_prune(NULL, buf, 8, S24_FP16, S24_MODE_SIGNED, S24_TIE_REFERENCE, NULL) == S24_ERR_INVALID_ARG);
    CHECK(s24_prune(buf, buf, 6, S24_FP16, S24_MODE_SIGNED, S24_TIE_REFERENCE, NULL) == S24_ERR_SHAPE);
    CHECK(strstr(s24_last_error(), "divisible by 4") != NULL);
    CHECK(s24_prune(buf, buf, 0, S24_FP16, S24_MODE_SIGNED, S24_TIE_LOWER, NULL) == S24_OK);     /* nothing to do */
    CHECK(s24_compress(buf, 48, 64, 64, S24_BF16, buf, buf, NULL, NULL) == S24_ERR_SHAPE);
    CHECK(s24_prune_compress(buf, 0, 64, 64, S24_FP16, S24_MODE_MAGNITUDE, S24_TIE_HIGHER, buf, buf, NULL, NULL) == S24_OK);
    CHECK(s24_spmm(buf, buf, buf, buf, 128, 128, 96, 128, 128, S24_FP16, &cfg, NULL) == S24_ERR_SHAPE);
    CHECK(s24_spmm_bt(buf, buf, buf, buf, 128, 12, 128, 128, 128, S24_FP16, NULL, NULL) == S24_ERR_SHAPE);   /* N % 8 */
    CHECK(s24_spmm_prune_out(buf, buf, buf, buf, buf, NULL, 128, 64, 128, 64, S24_FP16, NULL, NULL) == S24_ERR_SHAPE); /* N % 128 */
    CHECK(s24_spmm_ref_meta_noalloc(buf, buf, buf, buf, 16384, 128, 16384, 128, 128, S24_FP16, NULL, NULL) == S24_ERR_SHAPE);
    CHECK(strstr(s24_last_error(), "built-in buffer") != NULL);
    CHECK(s24_peer_copy_2d(buf, 16, buf, 64, 32, 4, NULL) == S24_ERR_SHAPE);
    CHECK(s24_relayout_shards(buf, buf, 4, 2, 12, 24, NULL) == S24_ERR_SHAPE);
    printf("abi smoke ok\n");
    return 0;
}
