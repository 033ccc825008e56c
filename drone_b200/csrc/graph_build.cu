// Host-side construction of one rank's local graph and routing tables from the
// partition files' contents (edge list of G.<p>, rows of Master.<p> and Mirror.<p>).
#include "common.cuh"

#include <vector>

using namespace drone;

extern "C" {

// Local numbering and CSR of one part.  Local ids are handed out in first-seen order
// over the edge list, source before destination (cuda_gcn/src/cuda/graph.cu:67-70);
// the CSR is by source vertex with destinations in edge-list order (:94-103).
// h_g2l[global_v] receives -1 for vertices that do not occur; h_l2g and h_index need
// room for min(global_v, 2*n_edges) (+1) entries, h_dst for n_edges.
int drone_graph_build_host(int global_v, int n_edges, const int *h_u, const int *h_v, int *h_g2l, int *h_l2g,
                           int *h_index, int *h_dst, int *n_local_out) {
    DRONE_REQUIRE(global_v > 0 && n_edges >= 0, "drone_graph_build_host: bad sizes (V=%d, E=%d)", global_v, n_edges);
    DRONE_REQUIRE(h_g2l && h_l2g && h_index && n_local_out, "drone_graph_build_host: NULL output");
    DRONE_REQUIRE(n_edges == 0 || (h_u && h_v && h_dst), "drone_graph_build_host: NULL edge arrays");
    for (int i = 0; i < global_v; ++i) h_g2l[i] = -1;
    int n = 0;
    for (int i = 0; i < n_edges; ++i) {
        const int u = h_u[i], v = h_v[i];
        DRONE_REQUIRE(u >= 0 && u < global_v && v >= 0 && v < global_v,
                      "drone_graph_build_host: edge %d (%d,%d) outside 0..%d", i, u, v, global_v - 1);
        if (h_g2l[u] < 0) { h_g2l[u] = n; h_l2g[n++] = u; }
        if (h_g2l[v] < 0) { h_g2l[v] = n; h_l2g[n++] = v; }
    }
    for (int i = 0; i <= n; ++i) h_index[i] = 0;
    for (int i = 0; i < n_edges; ++i) h_index[h_g2l[h_u[i]] + 1]++;
    for (int i = 0; i < n; ++i) h_index[i + 1] += h_index[i];
    std::vector<int> fill((size_t)n, 0);
    for (int i = 0; i < n_edges; ++i) {
        const int lu = h_g2l[h_u[i]];
        h_dst[h_index[lu] + fill[lu]++] = h_g2l[h_v[i]];
    }
    *n_local_out = n;
    return DRONE_OK;
}

// Routing tables by local id from the rows of Master.<p> (vertex, then the ranks holding
// its mirrors) and Mirror.<p> (vertex, rank of its master):
//   h_master_worker_index[n_local+1] / h_master2workers[mirror_worker_size]  (CSR) and
//   h_mirror2worker[n_local] (-1 where the local vertex is not a mirror).
// Same content as addMasterRoute / addMirrorRoute build on the device,
// cuda_gcn/src/cuda/graph.cu:242-367.
int drone_route_tables_host(int n_local, const int *h_g2l, const int *master_vertex, const int *mirror_number,
                            const int *mirror_workers, int master_size, int mirror_worker_size,
                            const int *mirror_vertex, const int *master_worker, int mirror_size,
                            int *h_master_worker_index, int *h_master2workers, int *h_mirror2worker) {
    DRONE_REQUIRE(n_local >= 0 && master_size >= 0 && mirror_size >= 0 && mirror_worker_size >= 0,
                  "drone_route_tables_host: negative size");
    DRONE_REQUIRE(h_g2l && h_master_worker_index && h_mirror2worker, "drone_route_tables_host: NULL table");
    DRONE_REQUIRE(mirror_worker_size == 0 || h_master2workers, "drone_route_tables_host: NULL Master2Workers");
    for (int i = 0; i <= n_local; ++i) h_master_worker_index[i] = 0;
    for (int i = 0; i < n_local; ++i) h_mirror2worker[i] = -1;
    long long total = 0;
    for (int i = 0; i < master_size; ++i) {
        const int l = h_g2l[master_vertex[i]];
        DRONE_REQUIRE(l >= 0 && l < n_local, "drone_route_tables_host: master vertex %d is not in this part", master_vertex[i]);
        DRONE_REQUIRE(h_master_worker_index[l + 1] == 0, "drone_route_tables_host: master vertex %d listed twice",
                      master_vertex[i]);
        h_master_worker_index[l + 1] = mirror_number[i];
        total += mirror_number[i];
    }
    DRONE_REQUIRE(total == mirror_worker_size, "drone_route_tables_host: mirror counts sum to %lld, list has %d", total,
                  mirror_worker_size);
    for (int i = 0; i < n_local; ++i) h_master_worker_index[i + 1] += h_master_worker_index[i];
    int src = 0;
    for (int i = 0; i < master_size; ++i) {
        const int l = h_g2l[master_vertex[i]];
        for (int j = 0; j < mirror_number[i]; ++j) h_master2workers[h_master_worker_index[l] + j] = mirror_workers[src + j];
        src += mirror_number[i];
    }
    for (int i = 0; i < mirror_size; ++i) {
        const int l = h_g2l[mirror_vertex[i]];
        DRONE_REQUIRE(l >= 0 && l < n_local, "drone_route_tables_host: mirror vertex %d is not in this part", mirror_vertex[i]);
        h_mirror2worker[l] = master_worker[i];
    }
    return DRONE_OK;
}

}  // extern "C"
