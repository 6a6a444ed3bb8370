/* A plain C99 consumer of the public headers: proves that hccl.h / hccl_types.h / hcom.h / hccl_b200.h compile as C and that
 * the library links and runs from C.  Four CPU ranks in one process (host-memory transport): AllReduce, AllGather, the
 * group-name front end and the topology description.  Prints "c consumer ok" and exits 0 on success. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "hccl/hccl.h"
#include "hccl/hccl_b200.h"
#include "hccl/hcom.h"

#define NR 4
#define N 1000

#define CHECK(call)                                                                                   \
    do {                                                                                              \
        HcclResult rc_ = (call);                                                                      \
        if (rc_ != HCCL_SUCCESS) {                                                                    \
            fprintf(stderr, "%s:%d: %s -> %d (%s)\n", __FILE__, __LINE__, #call, (int)rc_, HcclGetErrorString(rc_)); \
            return 1;                                                                                 \
        }                                                                                             \
    } while (0)

int main(void)
{
    HcclCommConfig cfg;
    HcclComm comm = NULL;
    HcclB200Op op;
    float *in[NR], *out[NR], *gat[NR];
    void *sends[NR], *recvs[NR];
    HcclTopoDescs topo[HCCL_TOPO_MAX];
    uint32_t size = 0, r, i;
    char name[COMM_NAME_MAX_LENGTH];

    HcclCommConfigInit(&cfg);
    cfg.hcclBufferSize = 4;
    CHECK(HcclB200CommInitLocal(NR, 0 /* host transport */, 0, &cfg, &comm));
    CHECK(HcclGetRankSize(comm, &size));
    if (size != NR) return 2;
    CHECK(HcclGetCommName(comm, name));

    for (r = 0; r < NR; ++r) {
        in[r] = (float *)malloc(sizeof(float) * N);
        out[r] = (float *)calloc(N, sizeof(float));
        gat[r] = (float *)calloc((size_t)N * NR, sizeof(float));
        for (i = 0; i < N; ++i) in[r][i] = (float)(r + 1) * 0.5f + (float)i;
    }
    memset(&op, 0, sizeof(op));
    op.coll = HCCL_B200_ALLREDUCE;
    op.dataType = HCCL_DATA_TYPE_FP32;
    op.op = HCCL_REDUCE_SUM;
    op.count = N;
    for (r = 0; r < NR; ++r) { sends[r] = in[r]; recvs[r] = out[r]; }
    CHECK(HcclB200Collective(comm, &op, sends, recvs, NULL));
    for (r = 0; r < NR; ++r)
        for (i = 0; i < N; ++i)
            if (out[r][i] != 0.5f * (1 + 2 + 3 + 4) + (float)NR * (float)i) { fprintf(stderr, "allreduce mismatch\n"); return 3; }

    op.coll = HCCL_B200_ALLGATHER;
    for (r = 0; r < NR; ++r) recvs[r] = gat[r];
    CHECK(HcclB200Collective(comm, &op, sends, recvs, NULL));
    for (r = 0; r < NR; ++r)
        for (i = 0; i < (uint32_t)N * NR; ++i)
            if (gat[r][i] != in[i / N][i % N]) { fprintf(stderr, "allgather mismatch\n"); return 4; }

    CHECK(HcclGetTopoDesc(comm, topo, HCCL_TOPO_MAX));
    if (topo[HCCL_TOPO_L0].rankSize != NR || !(topo[HCCL_TOPO_L0].algSets & HCCL_ALG_MESH) || topo[HCCL_TOPO_L1].rankSize != 0) return 5;

    CHECK(HcomInitByComm(comm));
    CHECK(HcomGetRankSize(NULL, &size));
    if (size != NR) return 6;
    {
        float shares[2] = {25.0f, 75.0f}, back[4];
        uint32_t nseg = 4;
        CHECK(HcomSetGradFusionBySize(HCCL_WORLD_GROUP, 2, shares));
        CHECK(HcomGetGradFusionBySize(NULL, &nseg, back));
        if (nseg != 2 || back[1] != 75.0f) return 7;
    }
    CHECK(HcomDestroy());

    if (HcclAllReduce(NULL, NULL, 1, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, NULL) != HCCL_E_PTR) return 8;
    CHECK(HcclCommDestroy(comm));
    for (r = 0; r < NR; ++r) { free(in[r]); free(out[r]); free(gat[r]); }
    printf("c consumer ok\n");
    return 0;
}
