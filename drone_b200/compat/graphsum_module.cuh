// CUDAGraphSum with the reference's module interface, served by libdrone_b200.
//
// Same class name, base class, constructor arguments and forward(bool)/backward() as
// cuda_gcn/src/cuda/cuda_module.cuh:31-37,62-88, so CUDAGCN's module list (cuda_gcn/src/cuda/cuda_gcn.cu:56-57,
// 78-79,138-149) can hold it unchanged.  When this header is used inside the reference tree, include the
// reference's own declarations first and define DRONE_COMPAT_HAVE_REFERENCE_TYPES; otherwise the minimal
// declarations below (same field order as the reference: graph.h:17-46, cuda_variable.cuh:17-30, seq.h:73-75,
// cuda_communicate.cuh:34-46) stand in for them.
#pragma once

#include <cuda_runtime.h>
#include <nccl.h>
#include <string>

extern "C" {
#include "../../include/drone_b200.h"
}

#ifndef DRONE_COMPAT_HAVE_REFERENCE_TYPES
typedef struct Graph {          // cuda_gcn/src/cuda/graph.h:17-41 (has srcID/dstID, unlike DRONE's twin)
    int *Global2Local, *Local2Global;
    int *MasterWorkerIndex, *Master2Workers;
    int MasterSize, MirrorWorkerSize;
    int *Mirror2Worker;
    int MirrorSize;
    int *index, *dst, *srcID, *dstID;
    float *edgeLen;
    int *localVertexSize, *globalVertexSize, *edgeSize;
    int gridSize, blockSize;
    int *active, *updateByMessage;
    int GID;
} Graph;
typedef struct Comm { ncclComm_t comm; cudaStream_t s; } Comm;
struct Degree { int *inDegree, *outDegree; };
struct Buffer;                  // the reference's per-call exchange buffers; not used any more
struct CUDAVariable {
    float *data, *grad;
    bool requires_grad, is_weight;
    int size;
};
class CUDAModule {
public:
    virtual void forward(bool) = 0;
    virtual void backward() = 0;
    virtual ~CUDAModule() {}
    std::string ModuleName;
};
#endif

class CUDAGraphSum : public CUDAModule {
    CUDAVariable *in, *out;
    Graph *graph;
    Comm *comm;
    Degree *degree;
    Buffer *buffer;
    int dim, workerId, workerNum, layer;
    drone_plan *plan = nullptr;      // replaces the cuSPARSE handle, matA/matAT, the transposed arrays and descriptors
    drone_xplan *xplan = nullptr;    // replaces the per-call counts and ids of Buffer
    drone_comm *dcomm = nullptr;     // wraps comm->comm
public:
    CUDAGraphSum(CUDAVariable *in, CUDAVariable *out, Graph *graph, Comm *comm, Degree *degree, Buffer *buffer, int dim,
                 int workerId, int workerNum, std::string Name, int layer);
    ~CUDAGraphSum();
    void forward(bool);
    void backward();
};
