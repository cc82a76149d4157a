/* A plain C program against include/cachegen_b200.h and libcachegen_b200.so: what a binding written in
 * another language sees.  It makes no GPU work: version, status strings, and calls that must be refused
 * on their arguments before anything is launched. */
#include <stdio.h>
#include <string.h>

#include "cachegen_b200.h"

static int fails = 0;
#define EXPECT(cond)                                               \
    do {                                                           \
        if (!(cond)) {                                             \
            printf("FAILED line %d: %s\n", __LINE__, #cond);       \
            fails++;                                               \
        }                                                          \
    } while (0)

int main(void) {
    int64_t strides[3] = {1, 1, 1};
    cg_decode_job job;
    memset(&job, 0, sizeof job);
    printf("version %s\n", cg_version());
    EXPECT(strlen(cg_version()) > 0);
    EXPECT(strcmp(cg_status_string(CG_OK), cg_status_string(CG_E_NULL)) != 0);
    EXPECT(cg_calculate_cdf(NULL, strides, 1, 1, 1, 8, NULL, NULL) == CG_E_NULL);
    EXPECT(cg_decode_prefsum(NULL, NULL, 0, NULL, NULL, strides, 1, 1, 1, 9, NULL, NULL) == CG_E_NULL);
    EXPECT(cg_decode_offsets(&job, 1, 2, 128, NULL, NULL, NULL) == CG_E_NULL);
    EXPECT(cg_decode_offsets(&job, CG_MAX_DECODE_JOBS + 1, 2, 128, (int64_t *)&job, NULL, NULL) == CG_E_CAPACITY);
    EXPECT(cg_decode_dequant(&job, 1, 1, 1, 128, 9, NULL, CG_F16, CG_F16, 1, 1, 1, 1, NULL, NULL) < 0);
    EXPECT(sizeof(cg_decode_job) == 96);
    {
        cg_workspace_sizes ws;
        EXPECT(cg_workspace_bytes(64, 300, 4096, &ws) == CG_OK);
        EXPECT(ws.nsub == 2 && ws.scratch_stride == 520 && ws.encode_scratch == 2LL * 64 * 4096 * 520);
        EXPECT(ws.encode_lengths == 2LL * 64 * 4096 * 4 && ws.encode_group_off == 2LL * 64 * 32 * 8);
        EXPECT(ws.encode_sub_off == 24 && ws.decode_group_off == 64LL * 32 * 8 && ws.symbols == 64LL * 300 * 4096);
        EXPECT(cg_workspace_bytes(64, 100, 320, &ws) == CG_OK && ws.scratch_stride == 208 && ws.nsub == 1);
        EXPECT(ws.decode_group_off == 64LL * 3 * 8);
        EXPECT(cg_workspace_bytes(0, 1, 1, &ws) == CG_E_SHAPE && cg_workspace_bytes(1, 1, 1, NULL) == CG_E_NULL);
    }
    EXPECT(CG_STREAM_CAPACITY(256) == 520);
    printf(fails ? "%d checks failed\n" : "all checks passed\n", fails);
    return fails != 0;
}
