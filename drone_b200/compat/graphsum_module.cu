// CUDAGraphSum over libdrone_b200 (see graphsum_module.cuh), plus C entry points that let a test harness drive
// the C++ class.
#include "graphsum_module.cuh"

#include <cstdio>
#include <cstdlib>
#include <vector>

static void drone_check(int rc, const char *what) {   // the reference's convention: print and exit
    if (rc != 0) {
        printf("drone_b200: %s failed: %s\n", what, drone_last_error());
        exit(EXIT_FAILURE);
    }
}

template <typename T>
static std::vector<T> to_host(const T *p, size_t n) {   // works for device and managed memory alike
    std::vector<T> h(n > 0 ? n : 1);
    if (n > 0 && cudaMemcpy(h.data(), p, sizeof(T) * n, cudaMemcpyDefault) != cudaSuccess) {
        printf("drone_b200: cannot read a routing table\n");
        exit(EXIT_FAILURE);
    }
    return h;
}

CUDAGraphSum::CUDAGraphSum(CUDAVariable *in, CUDAVariable *out, Graph *graph, Comm *comm, Degree *degree, Buffer *buffer,
                           int dim, int workerId, int workerNum, std::string Name, int layer)
    : in(in), out(out), graph(graph), comm(comm), degree(degree), buffer(buffer), dim(dim), workerId(workerId),
      workerNum(workerNum), layer(layer) {
    ModuleName = Name;
    cudaSetDevice(graph->GID);
    const int n = *graph->localVertexSize;
    // was: cuda_compute_csr_values, cusparseCreateCsr x2, cusparseCsr2cscEx2, cusparseCreateDnMat x4
    // (cuda_gcn/src/cuda/cuda_module.cu:160-194)
    drone_check(drone_plan_create(&plan, n, *graph->edgeSize, graph->index, graph->dst, nullptr, degree->inDegree,
                                  degree->outDegree, DRONE_PLAN_BOTH, comm ? comm->s : nullptr),
                "drone_plan_create");
    // was: cusparseSpMM_bufferSize + cudaMalloc of the workspace on the first training step (cuda_module.cu:234-244);
    // padded staging lets class-width layers (41, 47 columns) run on the 16-byte kernels
    drone_check(drone_plan_reserve(plan, dim, dim % 4 ? DRONE_RESERVE_PADDED_ROWS : 0), "drone_plan_reserve");
    if (workerNum > 1) {
        const std::vector<int> l2g = to_host(graph->Local2Global, (size_t)n);
        const std::vector<int> mir = to_host(graph->Mirror2Worker, (size_t)n);
        const std::vector<int> mwi = to_host(graph->MasterWorkerIndex, (size_t)n + 1);
        const std::vector<int> m2w = to_host(graph->Master2Workers, (size_t)graph->MirrorWorkerSize);
        drone_check(drone_xplan_create(&xplan, workerId, workerNum, n, l2g.data(), mir.data(), mwi.data(), m2w.data(), dim),
                    "drone_xplan_create");
        drone_check(drone_comm_adopt(&dcomm, comm->comm, workerId, workerNum), "drone_comm_adopt");
    }
}

CUDAGraphSum::~CUDAGraphSum() {
    drone_comm_destroy(dcomm);
    drone_xplan_destroy(xplan);
    drone_plan_destroy(plan);
}

// out = A^T in, then mirrors -> masters (sum), masters -> mirrors (assign).
// was: out->zero(); cusparseSpMM(matAT, ...); GraphSum_sync_value_nccl   (cuda_module.cu:214-272)
void CUDAGraphSum::forward(bool) {
    cudaStream_t st = comm ? comm->s : nullptr;
    drone_check(drone_spmm(plan, DRONE_OP_AT, dim, in->data, dim, out->data, dim, st), "drone_spmm");
    if (workerNum > 1) drone_check(drone_exchange_sum(xplan, dcomm, out->data, dim, dim, st), "drone_exchange_sum");
    cudaStreamSynchronize(st);   // the reference synchronises after every module
}

// in.grad = A out.grad, then the same exchange on the gradient.
// was: in->zero_grad(); cusparseSpMM(matA, ...); GraphSum_sync_grad_nccl   (cuda_module.cu:315-368)
void CUDAGraphSum::backward() {
    cudaStream_t st = comm ? comm->s : nullptr;
    drone_check(drone_spmm(plan, DRONE_OP_A, dim, out->grad, dim, in->grad, dim, st), "drone_spmm");
    if (workerNum > 1) drone_check(drone_exchange_sum(xplan, dcomm, in->grad, dim, dim, st), "drone_exchange_sum");
    cudaStreamSynchronize(st);
}

// ---- C entry points for harnesses (ctypes): build the reference-shaped arguments, own the module ----
struct CompatGraphSum {
    Graph graph;
    Comm comm;
    Degree degree;
    CUDAVariable in, out;
    int scalars[3];
    CUDAModule *module;
};

extern "C" {

// All pointers are device pointers on the current device; routing tables may be NULL when worker_num == 1.
void *drone_compat_graphsum_create(int n_local, int n_edges, int global_v, int *d_index, int *d_dst, int *d_in_degree,
                                   int *d_out_degree, int *d_local2global, int *d_mirror2worker,
                                   int *d_master_worker_index, int *d_master2workers, int mirror_worker_size,
                                   float *d_in_data, float *d_in_grad, float *d_out_data, float *d_out_grad, int dim,
                                   int worker_id, int worker_num, void *nccl_comm, void *stream) {
    CompatGraphSum *c = new CompatGraphSum();
    Graph &g = c->graph;
    g = Graph();
    cudaGetDevice(&g.GID);
    g.index = d_index;
    g.dst = d_dst;
    g.Local2Global = d_local2global;
    g.Mirror2Worker = d_mirror2worker;
    g.MasterWorkerIndex = d_master_worker_index;
    g.Master2Workers = d_master2workers;
    g.MirrorWorkerSize = mirror_worker_size;
    c->scalars[0] = n_local;
    c->scalars[1] = global_v;
    c->scalars[2] = n_edges;
    g.localVertexSize = &c->scalars[0];
    g.globalVertexSize = &c->scalars[1];
    g.edgeSize = &c->scalars[2];
    c->comm.comm = (ncclComm_t)nccl_comm;
    c->comm.s = (cudaStream_t)stream;
    c->degree.inDegree = d_in_degree;
    c->degree.outDegree = d_out_degree;
    c->in = CUDAVariable{d_in_data, d_in_grad, true, false, n_local * dim};
    c->out = CUDAVariable{d_out_data, d_out_grad, true, false, n_local * dim};
    c->module = new CUDAGraphSum(&c->in, &c->out, &c->graph, &c->comm, &c->degree, nullptr, dim, worker_id, worker_num,
                                 "graphSum_compat", 0);
    return c;
}

void drone_compat_graphsum_forward(void *h) { static_cast<CompatGraphSum *>(h)->module->forward(true); }
void drone_compat_graphsum_backward(void *h) { static_cast<CompatGraphSum *>(h)->module->backward(); }
void drone_compat_graphsum_destroy(void *h) {
    CompatGraphSum *c = static_cast<CompatGraphSum *>(h);
    delete c->module;
    delete c;
}

}  // extern "C"
