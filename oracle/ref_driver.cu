// Drives the REFERENCE's own GraphSum layer (class CUDAGraphSum over cuSPARSE, cuda_gcn/src/cuda/cuda_module.cu:149-389)
// on one worker: builds the reference's Graph with its build_graph / addMasterRoute / addMirrorRoute, its Degree,
// Buffer and CUDAVariable objects, runs forward() and backward(), and copies the results out.
// Compiled together with the reference sources, where they lie, by `make ref` into oracle/_ref/ (never committed).
// TEST INFRASTRUCTURE: validates the oracle and the CUDA library against the reference itself on a GPU box.
#include <cstdio>
#include <cstring>
#include <vector>

#include "cuda_module.cuh"

// One worker of worker_num (one process per GPU; several workers need the file-based MPI_Bcast stand-in of
// ref_shim/mpi.h).  The Master.<p> / Mirror.<p> rows are passed as the reference's parser passes them
// (cuda_gcn/src/common/parser.cu:86-131).
extern "C" int ref_graphsum_run_worker(int global_v, int n_edges, int *u, int *v, int worker_id, int worker_num,
                                       int *master_vertex, int *mirror_number, int *mirror_workers, int master_size,
                                       int mirror_worker_size, int *mirror_vertex, int *master_worker, int mirror_size,
                                       const int *global_in_degree, const int *global_out_degree, int dim,
                                       const float *h_in_data, const float *h_out_grad, float *h_out_data,
                                       float *h_in_grad, float *h_values, int *h_local2global, int *n_local_out) {
    Comm *comm = new Comm();
    Graph *g = build_graph(global_v, n_edges, u, v, worker_id, worker_num, comm);
    addMasterRoute(g, master_vertex, mirror_number, mirror_workers, master_size, mirror_worker_size);
    addMirrorRoute(g, mirror_vertex, master_worker, mirror_size);
    const int n = getLocalVertexSize(g);
    *n_local_out = n;
    std::vector<int> l2g(n), ind(n), outd(n);
    cudaMemcpy(l2g.data(), g->Local2Global, sizeof(int) * n, cudaMemcpyDeviceToHost);
    for (int i = 0; i < n; ++i) {
        h_local2global[i] = l2g[i];
        ind[i] = global_in_degree[l2g[i]];      // what loadInOutDegree / setDegree do (common/parser.cu:25-50)
        outd[i] = global_out_degree[l2g[i]];
    }
    Degree *degree = new Degree();
    cudaMalloc(&degree->inDegree, sizeof(int) * n);
    cudaMalloc(&degree->outDegree, sizeof(int) * n);
    cudaMemcpy(degree->inDegree, ind.data(), sizeof(int) * n, cudaMemcpyHostToDevice);
    cudaMemcpy(degree->outDegree, outd.data(), sizeof(int) * n, cudaMemcpyHostToDevice);

    CUDAVariable *in = new CUDAVariable(n * dim, true, false);
    CUDAVariable *out = new CUDAVariable(n * dim, true, false);
    Buffer *buffer = new Buffer();
    buffer->maxDim = dim;
    buffer_init(buffer, g, worker_id, worker_num);
    // local rows are in the reference's first-seen order; the caller passes operands by GLOBAL id
    std::vector<float> tmp((size_t)n * dim);
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < dim; ++j) tmp[(size_t)i * dim + j] = h_in_data[(size_t)l2g[i] * dim + j];
    cudaMemcpy(in->data, tmp.data(), sizeof(float) * tmp.size(), cudaMemcpyHostToDevice);
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < dim; ++j) tmp[(size_t)i * dim + j] = h_out_grad[(size_t)l2g[i] * dim + j];
    cudaMemcpy(out->grad, tmp.data(), sizeof(float) * tmp.size(), cudaMemcpyHostToDevice);

    CUDAGraphSum *layer = new CUDAGraphSum(in, out, g, comm, degree, buffer, dim, worker_id, worker_num, "graphSum_ref", 0);
    // forward and backward each end in an exchange that, with one worker, launches over zero rows; the launch errors
    // are cleared here and the reference's exit() on them is caught (see ref_shim/utils_override.h)
    try {
        layer->forward(true);
    } catch (const DroneRefExit &) {
    }
    cudaDeviceSynchronize();
    cudaGetLastError();
    try {
        layer->backward();
    } catch (const DroneRefExit &) {
    }
    cudaGetLastError();
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    cudaMemcpy(h_out_data, out->data, sizeof(float) * (size_t)n * dim, cudaMemcpyDeviceToHost);   // by LOCAL id
    cudaMemcpy(h_in_grad, in->grad, sizeof(float) * (size_t)n * dim, cudaMemcpyDeviceToHost);
    cudaMemcpy(h_values, g->edgeLen, sizeof(float) * n_edges, cudaMemcpyDeviceToHost);           // CSR order
    // the reference's destructor deletes an uninitialised pointer when batch_type != SEMI_BATCH: the layer is leaked
    cudaGetLastError();
    return 0;
}

extern "C" int ref_graphsum_run(int global_v, int n_edges, int *u, int *v, const int *global_in_degree,
                                const int *global_out_degree, int dim, const float *h_in_data,
                                const float *h_out_grad, float *h_out_data, float *h_in_grad, float *h_values,
                                int *h_local2global, int *n_local_out) {
    int none = 0;
    return ref_graphsum_run_worker(global_v, n_edges, u, v, 0, 1, &none, &none, &none, 0, 0, &none, &none, 0,
                                   global_in_degree, global_out_degree, dim, h_in_data, h_out_grad, h_out_data, h_in_grad,
                                   h_values, h_local2global, n_local_out);
}

// ---------------------------------------------------------------------------------------------------------------
// The REFERENCE's own training epoch (class CUDAGCN, cuda_gcn/src/cuda/cuda_gcn.cu:8-99, train_epoch :287-306) on one
// worker, over a graph, features, labels and starting weights handed in by the caller: the same objects the
// reference's parser would build from its dataset files (cuda_gcn/src/common/parser.cu:59-295), built in memory.
// Times `epochs` calls of train_epoch() (which ends in cudaDeviceSynchronize) with the host clock, and separately the
// parts of train_epoch that are bookkeeping rather than training (set_truth's two cudaMalloc + copies every epoch,
// get_accuracy's copy of all logits to the host and host loop, get_l2_penalty): :211-260.
// With one worker the exchange inside every GraphSum launches kernels over zero rows and the reference's error checks
// would end the run; drone_ref_tolerate_exit makes those checks clear the (non-sticky) launch error and carry on, and
// the device is synchronised and checked at the end.
#include "cuda_gcn.cuh"

#include <chrono>

int drone_ref_tolerate_exit = 0;
extern "C" int cudaGetLastError_for_ref_shim(void) { return (int)cudaGetLastError(); }

extern "C" int ref_gcn_epochs(int global_v, int n_edges, int *u, int *v, const int *global_in_degree,
                              const int *global_out_degree, int input_dim, int hidden_dim, int output_dim,
                              const float *h_features, const int *h_labels, const float *h_w1, const float *h_w2,
                              int warmup, int epochs, double *ms_per_epoch, double *ms_bookkeeping_per_epoch,
                              float *first_loss) {
    Comm *comm = new Comm();
    Graph *g = build_graph(global_v, n_edges, u, v, 0, 1, comm);
    int none = 0;
    addMasterRoute(g, &none, &none, &none, 0, 0);
    addMirrorRoute(g, &none, &none, 0);
    const int n = getLocalVertexSize(g);
    std::vector<int> l2g(n), ind(n), outd(n);
    cudaMemcpy(l2g.data(), g->Local2Global, sizeof(int) * n, cudaMemcpyDeviceToHost);
    for (int i = 0; i < n; ++i) {
        ind[i] = global_in_degree[l2g[i]];
        outd[i] = global_out_degree[l2g[i]];
    }
    Degree *degree = new Degree();
    cudaMalloc(&degree->inDegree, sizeof(int) * n);
    cudaMalloc(&degree->outDegree, sizeof(int) * n);
    cudaMemcpy(degree->inDegree, ind.data(), sizeof(int) * n, cudaMemcpyHostToDevice);
    cudaMemcpy(degree->outDegree, outd.data(), sizeof(int) * n, cudaMemcpyHostToDevice);

    GCNData *data = new GCNData();
    data->graph = g;
    data->degree = degree;
    data->comm = comm;
    data->split.assign(n, 1);                      // every vertex in the training split
    data->label.resize(n);
    data->feature_value.resize((size_t)n * input_dim);
    for (int i = 0; i < n; ++i) {                  // operands arrive by GLOBAL id, the reference holds them by local id
        data->label[i] = h_labels[l2g[i]];
        memcpy(&data->feature_value[(size_t)i * input_dim], h_features + (size_t)l2g[i] * input_dim,
               sizeof(float) * input_dim);
    }
    GCNParams params = GCNParams::get_default();
    params.globalVertexSize = global_v;
    params.localVertexSize = n;
    params.input_dim = input_dim;
    params.hidden_dim = hidden_dim;
    params.output_dim = output_dim;

    drone_ref_tolerate_exit = 1;
    int rc = 0;
    try {
        CUDAGCN *gcn = new CUDAGCN(params, data, 0, 1);
        // variables: 0 input, 1 X·W1, 2 W1, 3 GraphSum 1, 4 (.)·W2, 5 W2, 6 GraphSum 2 (cuda_gcn.cu:33-79)
        cudaMemcpy(gcn->variables[2].data, h_w1, sizeof(float) * (size_t)input_dim * hidden_dim, cudaMemcpyHostToDevice);
        cudaMemcpy(gcn->variables[5].data, h_w2, sizeof(float) * (size_t)hidden_dim * output_dim, cudaMemcpyHostToDevice);
        for (int e = 0; e < warmup + epochs; ++e) {
            if (e == warmup) {
                cudaDeviceSynchronize();
                const auto t0 = std::chrono::steady_clock::now();
                for (int k = 0; k < epochs; ++k) gcn->train_epoch();
                cudaDeviceSynchronize();
                *ms_per_epoch = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / epochs;
                break;
            }
            gcn->train_epoch();
            if (e == 0) *first_loss = gcn->loss;     // the cross-entropy loss alone (train_epoch returns it plus the L2 penalty)
        }
        cudaDeviceSynchronize();
        const auto t0 = std::chrono::steady_clock::now();
        for (int k = 0; k < epochs; ++k) {
            cudaDeviceSynchronize();
            gcn->set_truth(1);
            cudaDeviceSynchronize();
            gcn->get_l2_penalty();
            gcn->get_accuracy();
        }
        *ms_bookkeeping_per_epoch = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / epochs;
    } catch (const DroneRefExit &) {
        rc = -2;
    }
    drone_ref_tolerate_exit = 0;
    cudaGetLastError();
    if (cudaDeviceSynchronize() != cudaSuccess) rc = -1;
    return rc;
}
