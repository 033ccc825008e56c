/*
 * drone_pr_compat.h — the C interface DRONE's Go workers bind through cgo for the pr_cuda, cc_cuda and sssp_cuda
 * jobs, served by libdrone_b200.  libdrone_pr_compat.so exports exactly these symbols, so it can take the place of
 * libGRAPH_Lib + libPR_Lib + libCC_Lib + libSSSP_Lib + libALG_COMMON_Lib on the link line of
 * DRONE/src/tools/cuda_convert.go:6-12.
 *
 * The struct layouts repeat, field for field, DRONE/src/cuda/graph.h:16-43 (Graph, Comm),
 * DRONE/src/cuda/algorithm/pr.h:7-16 (PRValues), cc.h:18-22 (CCValues), sssp.h:8-12 (SSSPValues) and
 * DRONE/src/cuda/algorithm/common.h:23-27 (Response): Go
 * allocates Comm and PRValues itself and receives Response by value, so sizes and offsets are part of the ABI.
 */
#ifndef DRONE_PR_COMPAT_H
#define DRONE_PR_COMPAT_H

#include <cuda_runtime.h>
#include <nccl.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct Graph {
    int *Global2Local;       /* device, [globalVertexSize]; -1 where the vertex is not local */
    int *Local2Global;       /* device, [localVertexSize] */
    int *MasterWorkerIndex;  /* device, [localVertexSize+1]: CSR over Master2Workers */
    int *Master2Workers;     /* device: workers holding a mirror of each local master */
    int MasterSize, MirrorWorkerSize;
    int *Mirror2Worker;      /* device, [localVertexSize]: -1 or the worker owning the master copy */
    int MirrorSize;
    int *index;              /* device CSR by source vertex */
    int *dst;
    float *edgeLen;
    int *localVertexSize, *globalVertexSize, *edgeSize;   /* host-readable scalars */
    int gridSize, blockSize;
    int *active;             /* device, set by PR_PEVal */
    int *updateByMessage;    /* device, set by PR_PEVal */
    int GID;                 /* CUDA device ordinal of this worker */
} Graph;

typedef struct Comm {
    ncclComm_t comm;
    cudaStream_t s;
} Comm;

typedef struct PRValues {
    int *sendID, *recvID;          /* unused: the exchange is static, ids are never sent */
    float *sendDiff, *recvDiff;    /* unused */
    float *prValue, *accValue, *diffValue;
    float *globalAcc, *globalDiff; /* unused by callers */
    int *outDegree;
} PRValues;

typedef struct CCValues {
    int *sendID, *recvID;              /* unused: the exchange is static */
    int *sendCCValue, *recvCCValue;    /* unused */
    int *ccValue;                      /* device, [localVertexSize]: labels (GLOBAL vertex ids), set by CC_PEVal */
} CCValues;

typedef struct SSSPValues {
    int *sendID, *recvID;              /* unused */
    float *sendDis, *recvDis;          /* unused */
    float *distance;                   /* device, [localVertexSize]; 1e8 = not reached; set by SSSP_PEVal */
} SSSPValues;

typedef struct Response {
    int Mirror2MasterSendSize, Mirror2MasterRecvSize, Master2MirrorSendSize, Master2MirrorRecvSize;
    int VisitedSize, LocalVertexSize;
    float CalTime, SendTime;
} Response;

/* DRONE/src/cuda/graph.h:45-52.  build_graph also creates the NCCL communicator: worker 0 writes the unique id to
 * ./nccl.id, the others read it (DRONE/src/cuda/graph.cu:31-37,122-128). */
Graph *build_graph(int globalVertexSize, int edgeSize, int *u, int *v, int workerId, int workerNum, Comm *comm);
int getLocalVertexSize(Graph *g);
int getGlobalVertexSize(Graph *g);
void addMasterRoute(Graph *g, int *masterVertex, int *mirrorNumber, int *mirrorWorkers, int masterSize,
                    int mirrorWorkerSize);
void addMirrorRoute(Graph *g, int *mirrorVertex, int *masterWorker, int mirrorSize);

/* DRONE/src/cuda/algorithm/pr.h:18-21 */
void loadOutDegree(Graph *g, PRValues *values, int *globalOutDegree);
Response PR_PEVal(Graph *g, PRValues *values, int workerId, int workerNum, Comm *comm);
Response PR_IncEVal(Graph *g, PRValues *values, int workerId, int workerNum, Comm *comm);


/* DRONE/src/cuda/algorithm/cc.h:25-26 and sssp.h:15-16 */
Response CC_PEVal(Graph *g, CCValues *values, int workerId, int workerNum, Comm *comm);
Response CC_IncEVal(Graph *g, CCValues *values, int workerId, int workerNum, Comm *comm);
Response SSSP_PEVal(Graph *g, SSSPValues *values, int startId, int workerId, int workerNum, Comm *comm);
Response SSSP_IncEVal(Graph *g, SSSPValues *values, int workerId, int workerNum, Comm *comm);

#ifdef __cplusplus
}
#endif
#endif /* DRONE_PR_COMPAT_H */
