// The cgo-facing C interface of DRONE's pr_cuda job (drone_pr_compat.h) implemented over libdrone_b200's C ABI.
// Error convention of the reference: print and exit (DRONE/src/cuda/algorithm/common.h:4-21); the library's status
// codes are translated to that here and nowhere else.
#include "drone_pr_compat.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <ctime>
#include <sys/stat.h>
#include <unistd.h>

#include "../../include/drone_b200.h"

namespace {

// What the shim keeps beside the public struct (the Go side only ever holds the Graph pointer).
struct GraphImpl {
    Graph pub;                       // must stay first: &impl->pub == (Graph*)impl
    int n_local = 0, global_v = 0, n_edges = 0;
    int worker_id = 0, worker_num = 1;
    int scalars[3] = {0, 0, 0};      // localVertexSize, globalVertexSize, edgeSize live here
    std::vector<int> g2l, l2g;
    std::vector<int> master_vertex, mirror_number, mirror_workers, mirror_vertex, master_worker;
    bool routes_built = false;
    bool have_master_route = false, have_mirror_route = false;   // addMasterRoute / addMirrorRoute were called
    drone_xplan *xplan = nullptr;
    drone_comm *dcomm = nullptr;
    drone_pr *pr = nullptr;
    drone_mp *cc = nullptr, *sssp = nullptr;
};

GraphImpl *impl_of(Graph *g) { return reinterpret_cast<GraphImpl *>(g); }

void check(int rc, const char *what) {
    if (rc != 0) {
        printf("Failed: %s: %s\n", what, drone_last_error());
        exit(EXIT_FAILURE);
    }
}

void check_cuda(cudaError_t e, const char *what) {
    if (e != cudaSuccess) {
        printf("Failed: Cuda error in %s: '%s'\n", what, cudaGetErrorString(e));
        exit(EXIT_FAILURE);
    }
}

template <typename T>
T *to_device(const std::vector<T> &h, size_t min_elems = 1) {
    T *d = nullptr;
    const size_t n = h.size() > min_elems ? h.size() : min_elems;
    check_cuda(cudaMalloc(&d, sizeof(T) * n), "cudaMalloc");
    if (!h.empty()) check_cuda(cudaMemcpy(d, h.data(), sizeof(T) * h.size(), cudaMemcpyHostToDevice), "cudaMemcpy");
    return d;
}

// Mirror2Worker / MasterWorkerIndex / Master2Workers by local id, and the exchange plan built from them.
void build_routes(GraphImpl *g) {
    if (g->routes_built) return;
    std::vector<int> mwi((size_t)g->n_local + 1, 0), m2w(g->mirror_workers.size() + 1, 0), mir((size_t)g->n_local + 1, -1);
    check(drone_route_tables_host(g->n_local, g->g2l.data(), g->master_vertex.data(), g->mirror_number.data(),
                                  g->mirror_workers.data(), (int)g->master_vertex.size(), (int)g->mirror_workers.size(),
                                  g->mirror_vertex.data(), g->master_worker.data(), (int)g->mirror_vertex.size(),
                                  mwi.data(), m2w.data(), mir.data()),
          "drone_route_tables_host");
    m2w.resize(g->mirror_workers.size());
    mir.resize((size_t)g->n_local);
    check(drone_xplan_create(&g->xplan, g->worker_id, g->worker_num, g->n_local, g->l2g.data(), mir.data(), mwi.data(),
                             m2w.data(), 1),
          "drone_xplan_create");
    g->pub.MasterWorkerIndex = to_device(mwi);
    g->pub.Master2Workers = to_device(m2w);
    g->pub.Mirror2Worker = to_device(mir);
    g->routes_built = true;
}

}  // namespace

extern "C" {

Graph *build_graph(int globalVertexSize, int edgeSize, int *u, int *v, int workerId, int workerNum, Comm *comm) {
    GraphImpl *g = new GraphImpl();
    memset(&g->pub, 0, sizeof(Graph));
    g->worker_id = workerId;
    g->worker_num = workerNum;
    g->global_v = globalVertexSize;
    g->n_edges = edgeSize;

    int n_devices = 0;
    check_cuda(cudaGetDeviceCount(&n_devices), "cudaGetDeviceCount");
    g->pub.GID = workerId % (n_devices > 0 ? n_devices : 1);   // the reference hard-wires 4 GPUs per node
    check_cuda(cudaSetDevice(g->pub.GID), "cudaSetDevice");

    const size_t cap = (size_t)(globalVertexSize < 2 * (long long)edgeSize ? globalVertexSize : 2 * edgeSize) + 1;
    g->g2l.assign((size_t)globalVertexSize, -1);
    g->l2g.assign(cap, 0);
    std::vector<int> index(cap + 1, 0), dst((size_t)edgeSize + 1, 0);
    check(drone_graph_build_host(globalVertexSize, edgeSize, u, v, g->g2l.data(), g->l2g.data(), index.data(), dst.data(),
                                 &g->n_local),
          "drone_graph_build_host");
    g->l2g.resize((size_t)g->n_local);
    index.resize((size_t)g->n_local + 1);
    dst.resize((size_t)edgeSize);

    g->pub.Global2Local = to_device(g->g2l);
    g->pub.Local2Global = to_device(g->l2g);
    g->pub.index = to_device(index);
    g->pub.dst = to_device(dst);
    std::vector<float> ones((size_t)edgeSize, 1.0f);
    g->pub.edgeLen = to_device(ones);
    g->scalars[0] = g->n_local;
    g->scalars[1] = globalVertexSize;
    g->scalars[2] = edgeSize;
    g->pub.localVertexSize = &g->scalars[0];
    g->pub.globalVertexSize = &g->scalars[1];
    g->pub.edgeSize = &g->scalars[2];
    g->pub.blockSize = 256;
    g->pub.gridSize = (g->n_local - 1) / 256 + 1;
    if (g->pub.gridSize > 1024) g->pub.gridSize = 1024;

    // communicator: worker 0 publishes the id through ./nccl.id, the others wait for the file
    unsigned char id[DRONE_UNIQUE_ID_BYTES];
    // A file left by an earlier run must not be taken for this run's id: worker 0 removes it before it makes the new
    // one, and the others only accept a file written less than a minute before they got here.
    const time_t entered = time(nullptr);
    if (workerId == 0) {
        unlink("./nccl.id");
        check(drone_comm_unique_id(id, sizeof(id)), "drone_comm_unique_id");
        FILE *fp = fopen("./nccl.id.tmp", "wb");
        if (!fp || fwrite(id, sizeof(id), 1, fp) != 1) { printf("Failed: cannot write ./nccl.id\n"); exit(EXIT_FAILURE); }
        fclose(fp);
        rename("./nccl.id.tmp", "./nccl.id");
    } else {
        FILE *fp = nullptr;
        for (int tries = 0; tries < 600 && !fp; ++tries) {
            struct stat info;
            if (stat("./nccl.id", &info) == 0 && info.st_mtime >= entered - 60) fp = fopen("./nccl.id", "rb");
            if (!fp) usleep(100000);
        }
        if (!fp || fread(id, sizeof(id), 1, fp) != 1) { printf("Failed: cannot read ./nccl.id\n"); exit(EXIT_FAILURE); }
        fclose(fp);
    }
    drone_comm *owned = nullptr;
    if (workerNum > 1) {
        ncclUniqueId nid;
        memcpy(&nid, id, sizeof(nid));
        ncclResult_t r = ncclCommInitRank(&comm->comm, workerNum, nid, workerId);
        if (r != ncclSuccess) { printf("Failed, NCCL error '%s'\n", ncclGetErrorString(r)); exit(EXIT_FAILURE); }
        check(drone_comm_adopt(&owned, comm->comm, workerId, workerNum), "drone_comm_adopt");
    } else {
        comm->comm = nullptr;
    }
    g->dcomm = owned;
    check_cuda(cudaStreamCreate(&comm->s), "cudaStreamCreate");
    return &g->pub;
}

int getLocalVertexSize(Graph *g) {
    cudaSetDevice(g->GID);
    return impl_of(g)->n_local;
}

int getGlobalVertexSize(Graph *g) {
    cudaSetDevice(g->GID);
    return impl_of(g)->global_v;
}

void addMasterRoute(Graph *gp, int *masterVertex, int *mirrorNumber, int *mirrorWorkers, int masterSize,
                    int mirrorWorkerSize) {
    GraphImpl *g = impl_of(gp);
    cudaSetDevice(gp->GID);
    gp->MasterSize = masterSize;
    gp->MirrorWorkerSize = mirrorWorkerSize;
    g->have_master_route = true;
    g->master_vertex.assign(masterVertex, masterVertex + masterSize);
    g->mirror_number.assign(mirrorNumber, mirrorNumber + masterSize);
    g->mirror_workers.assign(mirrorWorkers, mirrorWorkers + mirrorWorkerSize);
}

void addMirrorRoute(Graph *gp, int *mirrorVertex, int *masterWorker, int mirrorSize) {
    GraphImpl *g = impl_of(gp);
    cudaSetDevice(gp->GID);
    gp->MirrorSize = mirrorSize;
    g->have_mirror_route = true;
    g->mirror_vertex.assign(mirrorVertex, mirrorVertex + mirrorSize);
    g->master_worker.assign(masterWorker, masterWorker + mirrorSize);
}

// The PageRank job of a graph: transposed graph, work lists and state arrays.  Made when the out-degrees arrive
// (the routes are known by then in the order the Go worker calls: build_graph, addMasterRoute, addMirrorRoute,
// loadOutDegree), so that the first PR_PEVal only runs its superstep.
static void ensure_pr_job(GraphImpl *g, Graph *gp, PRValues *values) {
    if (g->pr) return;
    build_routes(g);
    check(drone_pr_create(&g->pr, g->n_local, g->global_v, g->n_edges, gp->index, gp->dst, values->outDegree,
                          gp->Mirror2Worker, g->xplan, g->dcomm, /*use_double*/ 0, /*eps*/ 1e-6),
          "drone_pr_create");
    void *p = nullptr, *a = nullptr, *d = nullptr;
    check(drone_pr_device_arrays(g->pr, &p, &a, &d, &gp->active, &gp->updateByMessage), "drone_pr_device_arrays");
    values->prValue = (float *)p;
    values->accValue = (float *)a;
    values->diffValue = (float *)d;
    values->sendID = values->recvID = nullptr;
    values->sendDiff = values->recvDiff = nullptr;
    values->globalAcc = values->globalDiff = nullptr;
}

void loadOutDegree(Graph *gp, PRValues *values, int *globalOutDegree) {
    GraphImpl *g = impl_of(gp);
    cudaSetDevice(gp->GID);
    std::vector<int> local((size_t)g->n_local);
    for (int i = 0; i < g->n_local; ++i) local[i] = globalOutDegree[g->l2g[i]];
    values->outDegree = to_device(local);
    if (g->have_master_route && g->have_mirror_route) ensure_pr_job(g, gp, values);
}

static Response run_step(Graph *gp, PRValues *values, int workerId, int workerNum, Comm *comm, bool peval) {
    GraphImpl *g = impl_of(gp);
    check_cuda(cudaSetDevice(gp->GID), "cudaSetDevice");   // calls arrive on arbitrary OS threads
    (void)workerId;
    (void)workerNum;
    ensure_pr_job(g, gp, values);      // only when the degrees were loaded before the routes
    drone_pr_response r;
    check(peval ? drone_pr_peval(g->pr, &r, comm->s) : drone_pr_inceval(g->pr, &r, comm->s),
          peval ? "drone_pr_peval" : "drone_pr_inceval");
    Response res;
    static_assert(sizeof(Response) == sizeof(drone_pr_response), "Response layout");
    memcpy(&res, &r, sizeof(res));
    return res;
}

// CC / SSSP: one drone_mp handle per job kind and graph, made at the first PEval.
static Response run_mp(Graph *gp, int kind, drone_mp **job, void **value_out, int start_id, Comm *comm, bool peval) {
    GraphImpl *g = impl_of(gp);
    check_cuda(cudaSetDevice(gp->GID), "cudaSetDevice");   // calls arrive on arbitrary OS threads
    if (!*job) {
        build_routes(g);
        check(drone_mp_create(job, kind, g->n_local, g->n_edges, gp->index, gp->dst,
                              kind == DRONE_MP_SSSP ? gp->edgeLen : nullptr, gp->Local2Global, g->xplan, g->dcomm),
              "drone_mp_create");
    }
    check(drone_mp_device_arrays(*job, value_out, &gp->active, &gp->updateByMessage), "drone_mp_device_arrays");
    drone_pr_response r;
    check(peval ? drone_mp_peval(*job, start_id, &r, comm->s) : drone_mp_inceval(*job, &r, comm->s),
          peval ? "drone_mp_peval" : "drone_mp_inceval");
    Response res;
    memcpy(&res, &r, sizeof(res));
    return res;
}

Response CC_PEVal(Graph *g, CCValues *values, int workerId, int workerNum, Comm *comm) {
    (void)workerId; (void)workerNum;
    values->sendID = values->recvID = values->sendCCValue = values->recvCCValue = nullptr;
    return run_mp(g, DRONE_MP_CC, &impl_of(g)->cc, (void **)&values->ccValue, -1, comm, true);
}

Response CC_IncEVal(Graph *g, CCValues *values, int workerId, int workerNum, Comm *comm) {
    (void)workerId; (void)workerNum;
    return run_mp(g, DRONE_MP_CC, &impl_of(g)->cc, (void **)&values->ccValue, -1, comm, false);
}

Response SSSP_PEVal(Graph *g, SSSPValues *values, int startId, int workerId, int workerNum, Comm *comm) {
    (void)workerId; (void)workerNum;
    values->sendID = values->recvID = nullptr;
    values->sendDis = values->recvDis = nullptr;
    return run_mp(g, DRONE_MP_SSSP, &impl_of(g)->sssp, (void **)&values->distance, startId, comm, true);
}

Response SSSP_IncEVal(Graph *g, SSSPValues *values, int workerId, int workerNum, Comm *comm) {
    (void)workerId; (void)workerNum;
    return run_mp(g, DRONE_MP_SSSP, &impl_of(g)->sssp, (void **)&values->distance, -1, comm, false);
}

Response PR_PEVal(Graph *g, PRValues *values, int workerId, int workerNum, Comm *comm) {
    return run_step(g, values, workerId, workerNum, comm, true);
}

Response PR_IncEVal(Graph *g, PRValues *values, int workerId, int workerNum, Comm *comm) {
    return run_step(g, values, workerId, workerNum, comm, false);
}

}  // extern "C"
