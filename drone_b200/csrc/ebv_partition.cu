// EBV vertex-cut partitioner on the host, single process.
//
// Restates the algorithm of the reference's MPI partitioner (EBV_mpi.cpp) as a
// simulation of its P ranks in one address space, so that partitions in the
// reference's format can be produced without MPI:
//   * edges are dealt round-robin to P ranks (EBV_mpi.cpp:212-253, rank = index % P);
//   * every rank sorts its share by deg(u)+deg(v) ascending, degrees counted over
//     its own share only (:259-265);
//   * in lock-step rounds of 10, 13, 16, ... up to 1000 edges per rank (:273,372)
//     each rank scores every part for each of its edges from the state at the start
//     of the round (:284-331):
//         score[p] = -[u not in p] - [v not in p] - edges_p/edges_of_this_rank
//                    - vertices_p / |V| * P   (+0.1 for the rank's own part)
//     and sends the edge to the first part with the highest score (:50-61);
//   * parts append what they receive in sender order and update their vertex sets
//     and counters (:334-370);
//   * a vertex held by several parts gets as master the replica number
//     (id mod #replicas) in ascending part order (:567-581); the others are mirrors.
// The per-rank sort is stable by default (the reference uses std::sort, whose order
// among equal keys is unspecified), which makes the result independent of the C++
// library.  With DRONE_EBV_STD_SORT_TIES the shares are sorted by std::sort itself,
// the call the reference makes (:265): built with the same standard library, the
// parts then equal the reference's edge for edge.
#include "common.cuh"

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <functional>
#include <thread>
#include <vector>

namespace drone {

struct EbvEdge {
    int u, v, key;
};

// Runs job(i) for i in [0, n) on up to `threads` host threads, repeatedly, with the workers kept alive
// between calls (the partitioner has tens of thousands of short parallel phases).
class PhasePool {
public:
    explicit PhasePool(int threads) : n_threads_(threads > 1 ? threads : 1) {
        for (int t = 1; t < n_threads_; ++t) workers_.emplace_back([this, t] { loop(t); });
    }
    ~PhasePool() {
        stop_.store(true);
        generation_.fetch_add(1);
        for (auto &w : workers_) w.join();
    }
    void run(int n, const std::function<void(int)> &job) {
        job_ = &job;
        n_items_ = n;
        next_.store(0);
        pending_.store(n_threads_ - 1);
        generation_.fetch_add(1);
        work();
        while (pending_.load(std::memory_order_acquire) != 0) std::this_thread::yield();
    }

private:
    void work() {
        for (int i = next_.fetch_add(1); i < n_items_; i = next_.fetch_add(1)) (*job_)(i);
    }
    void loop(int) {
        unsigned long long seen = 0;
        for (;;) {
            while (generation_.load(std::memory_order_acquire) == seen) std::this_thread::yield();
            seen = generation_.load();
            if (stop_.load()) return;
            work();
            pending_.fetch_sub(1, std::memory_order_release);
        }
    }
    int n_threads_;
    std::vector<std::thread> workers_;
    const std::function<void(int)> *job_ = nullptr;
    int n_items_ = 0;
    std::atomic<int> next_{0}, pending_{0};
    std::atomic<unsigned long long> generation_{0};
    std::atomic<bool> stop_{false};
};

static inline int pool_slices(int n) { return n >= (1 << 16) ? 64 : 1; }

// Stable sort of a rank's edges by key (ascending): least-significant-digit radix passes of 11 bits, as many as the
// largest key needs.  Same order as std::stable_sort on the key, several times faster on 10^8 edges.
static void sort_by_key(std::vector<EbvEdge> &edges, int max_key) {
    const size_t n = edges.size();
    if (n < 2) return;
    constexpr int kBits = 11, kBuckets = 1 << kBits;
    std::vector<EbvEdge> other(n);
    EbvEdge *src = edges.data(), *dst = other.data();
    for (int shift = 0; shift == 0 || (max_key >> shift) != 0; shift += kBits) {
        size_t count[kBuckets + 1] = {0};
        for (size_t i = 0; i < n; ++i) ++count[(((unsigned)src[i].key >> shift) & (kBuckets - 1)) + 1];
        for (int b = 0; b < kBuckets; ++b) count[b + 1] += count[b];
        for (size_t i = 0; i < n; ++i) dst[count[((unsigned)src[i].key >> shift) & (kBuckets - 1)]++] = src[i];
        std::swap(src, dst);
    }
    if (src != edges.data()) edges.swap(other);
}

// The reference's own call (EBV_mpi.cpp:46-48,265): std::sort over the array with a comparator on the key alone.
// Equal keys end up in whatever order the library's algorithm leaves them.
static bool key_less(EbvEdge a, EbvEdge b) { return a.key < b.key; }
static void sort_by_key_as_reference(std::vector<EbvEdge> &edges) {
    std::sort(edges.data(), edges.data() + edges.size(), key_less);
}

// The partitioner proper.  Mask is an unsigned type of at least n_parts bits: held[v] has bit p set when part p holds
// vertex v, so that scoring an edge costs two random reads whatever the number of parts.
template <typename Mask>
static int ebv_run(int n_vertices, long long n_edges, const int *h_u, const int *h_v, int P, int flags,
                   int *h_out_u, int *h_out_v, long long *h_part_offset, int *h_owner, int *h_replicas) {
    const int max_batch = 1000;
    const bool keep_self_loops = (flags & DRONE_EBV_KEEP_SELF_LOOPS) != 0;
    const bool std_sort_ties = (flags & DRONE_EBV_STD_SORT_TIES) != 0;
    int hw = (int)std::thread::hardware_concurrency();
    if (hw < 1) hw = 1;
    PhasePool pool(std::min(P, hw));

    // deal + per-rank degree + per-rank stable sort by degree sum
    std::vector<std::vector<EbvEdge>> share(P);
    std::vector<long long> bad_edge(P, -1);
    pool.run(P, [&](int r) {
        share[r].reserve((size_t)(n_edges / P + 1));
        for (long long i = r; i < n_edges; i += P) {
            const int u = h_u[i], v = h_v[i];
            if (u < 0 || u >= n_vertices || v < 0 || v >= n_vertices) {
                if (bad_edge[r] < 0) bad_edge[r] = i;
                continue;
            }
            if (!keep_self_loops && u == v) continue;
            share[r].push_back({u, v, 0});
        }
    });
    for (int r = 0; r < P; ++r)
        if (bad_edge[r] >= 0) {
            const long long i = bad_edge[r];
            return set_error(DRONE_E_INVALID, "drone_ebv_partition: edge %lld (%d,%d) outside 0..%d", i, h_u[i], h_v[i],
                             n_vertices - 1);
        }
    long long kept = 0;
    pool.run(P, [&](int r) {
        std::vector<int> deg((size_t)n_vertices, 0);
        for (const EbvEdge &e : share[r]) { deg[e.u]++; deg[e.v]++; }
        int max_key = 0;
        for (EbvEdge &e : share[r]) {
            e.key = deg[e.u] + deg[e.v];
            max_key = std::max(max_key, e.key);
        }
        if (std_sort_ties) sort_by_key_as_reference(share[r]);
        else sort_by_key(share[r], max_key);
    });
    for (int r = 0; r < P; ++r) kept += (long long)share[r].size();

    std::vector<Mask> held((size_t)n_vertices, 0);
    std::vector<long long> edge_count(P, 0), vertex_count(P, 0);
    std::vector<std::vector<int>> part_u(P), part_v(P);
    for (int p = 0; p < P; ++p) {
        part_u[p].reserve((size_t)(kept / P + kept / (16 * P) + 1024));
        part_v[p].reserve((size_t)(kept / P + kept / (16 * P) + 1024));
    }
    // assignments of the current scoring step: for each (sender, part) the edges in sender order
    std::vector<std::vector<int>> sent((size_t)P * P);

    long long longest = 0;
    for (int r = 0; r < P; ++r) longest = std::max<long long>(longest, (long long)share[r].size());
    int batch = 10;
    for (long long start = 0; start < longest; start += batch,
                   batch = batch < max_batch ? std::min((int)(batch * 1.3), max_batch) : batch) {
        for (auto &s : sent) s.clear();
        // scoring: every simulated rank reads the state left by the previous round only
        pool.run(P, [&](int r) {
            const long long edges_r = (long long)share[r].size();
            const long long end = std::min<long long>(start + batch, edges_r);
            double load[64], spread[64];   // the terms of the score that do not depend on the edge
            for (int p = 0; p < P; ++p) {
                load[p] = 1.0 * edge_count[p] / (double)edges_r;
                spread[p] = 1.0 * vertex_count[p] / n_vertices * P;
            }
            for (long long i = start; i < end; ++i) {
                const EbvEdge &e = share[r][(size_t)i];
                const Mask hu = held[e.u], hv = held[e.v];
                int best = -1;
                double best_w = -100;
                for (int p = 0; p < P; ++p) {
                    double w = 0;
                    if (!((hu >> p) & 1)) w -= 1;
                    if (!((hv >> p) & 1)) w -= 1;
                    w = w - load[p] - spread[p];
                    if (p == r) w += 0.1;
                    if (best_w < w) { best_w = w; best = p; }
                }
                sent[(size_t)r * P + best].push_back(e.u);
                sent[(size_t)r * P + best].push_back(e.v);
            }
        });
        // hand-over: every part appends what it was sent, in sender order, and updates its own state.  Parts run
        // side by side and may meet on one vertex's mask word, hence the atomic OR; bit p is only ever set by part p.
        pool.run(P, [&](int p) {
            const Mask bit = (Mask)((Mask)1 << p);
            for (int r = 0; r < P; ++r) {
                const std::vector<int> &s = sent[(size_t)r * P + p];
                for (size_t k = 0; k < s.size(); k += 2) {
                    const int u = s[k], v = s[k + 1];
                    part_u[p].push_back(u);
                    part_v[p].push_back(v);
                    if (!(__atomic_load_n(&held[u], __ATOMIC_RELAXED) & bit)) {
                        __atomic_fetch_or(&held[u], bit, __ATOMIC_RELAXED);
                        vertex_count[p]++;
                    }
                    if (!(__atomic_load_n(&held[v], __ATOMIC_RELAXED) & bit)) {
                        __atomic_fetch_or(&held[v], bit, __ATOMIC_RELAXED);
                        vertex_count[p]++;
                    }
                }
                edge_count[p] += (long long)(s.size() / 2);
            }
        });
    }

    long long off = 0;
    for (int p = 0; p < P; ++p) {
        h_part_offset[p] = off;
        off += (long long)part_u[p].size();
    }
    h_part_offset[P] = off;
    if (off != kept) return set_error(DRONE_E_STATE, "drone_ebv_partition: %lld edges in, %lld out", kept, off);
    pool.run(P, [&](int p) {
        std::copy(part_u[p].begin(), part_u[p].end(), h_out_u + h_part_offset[p]);
        std::copy(part_v[p].begin(), part_v[p].end(), h_out_v + h_part_offset[p]);
    });

    const int slices = pool_slices(n_vertices);
    pool.run(slices, [&](int s) {
        const int v0 = (int)((long long)n_vertices * s / slices), v1 = (int)((long long)n_vertices * (s + 1) / slices);
        for (int v = v0; v < v1; ++v) {
            const Mask m = held[v];
            int reps = 0;
            for (int p = 0; p < P; ++p) reps += (int)((m >> p) & 1);
            h_replicas[v] = reps;
            h_owner[v] = -1;
            if (reps == 0) continue;
            const int want = reps > 1 ? v % reps : 0;
            int seen = 0;
            for (int p = 0; p < P; ++p)
                if ((m >> p) & 1) {
                    if (seen == want) { h_owner[v] = p; break; }
                    ++seen;
                }
        }
    });
    return DRONE_OK;
}

}  // namespace drone

using namespace drone;

extern "C" int drone_ebv_partition(int n_vertices, long long n_edges, const int *h_u, const int *h_v, int n_parts,
                                   int flags, int *h_out_u, int *h_out_v, long long *h_part_offset,
                                   int *h_owner, int *h_replicas) {
    DRONE_REQUIRE(n_vertices > 0 && n_edges >= 0, "drone_ebv_partition: bad sizes (V=%d, E=%lld)", n_vertices, n_edges);
    DRONE_REQUIRE(n_parts >= 1 && n_parts <= 64, "drone_ebv_partition: n_parts=%d outside 1..64", n_parts);
    DRONE_REQUIRE(n_edges == 0 || (h_u && h_v), "drone_ebv_partition: NULL edge list");
    DRONE_REQUIRE(h_out_u && h_out_v && h_part_offset && h_owner && h_replicas, "drone_ebv_partition: NULL output");
    if (n_parts <= 8)
        return ebv_run<uint8_t>(n_vertices, n_edges, h_u, h_v, n_parts, flags, h_out_u, h_out_v, h_part_offset,
                                h_owner, h_replicas);
    if (n_parts <= 16)
        return ebv_run<uint16_t>(n_vertices, n_edges, h_u, h_v, n_parts, flags, h_out_u, h_out_v, h_part_offset,
                                 h_owner, h_replicas);
    if (n_parts <= 32)
        return ebv_run<uint32_t>(n_vertices, n_edges, h_u, h_v, n_parts, flags, h_out_u, h_out_v, h_part_offset,
                                 h_owner, h_replicas);
    return ebv_run<uint64_t>(n_vertices, n_edges, h_u, h_v, n_parts, flags, h_out_u, h_out_v, h_part_offset,
                             h_owner, h_replicas);
}

// bits[v] gets bit p set when vertex v is an endpoint of an edge of part p (the parts lie one after the other in
// h_u / h_v, part p at [h_part_offset[p], h_part_offset[p+1])).
extern "C" int drone_presence_bits_host(int n_vertices, int n_parts, const int *h_u, const int *h_v,
                                        const long long *h_part_offset, unsigned long long *h_bits) {
    DRONE_REQUIRE(n_vertices > 0 && n_parts >= 1 && n_parts <= 64, "drone_presence_bits_host: bad sizes");
    DRONE_REQUIRE(h_u && h_v && h_part_offset && h_bits, "drone_presence_bits_host: NULL argument");
    int hw = (int)std::thread::hardware_concurrency();
    if (hw < 1) hw = 1;
    PhasePool pool(std::min(std::max(n_parts, 8), hw));
    const int slices = pool_slices(n_vertices);
    pool.run(slices, [&](int s) {
        const long long v0 = (long long)n_vertices * s / slices, v1 = (long long)n_vertices * (s + 1) / slices;
        std::fill(h_bits + v0, h_bits + v1, 0ULL);
    });
    std::atomic<int> bad{0};
    pool.run(n_parts, [&](int p) {
        const unsigned long long bit = 1ULL << p;
        for (long long i = h_part_offset[p]; i < h_part_offset[p + 1]; ++i) {
            const int u = h_u[i], v = h_v[i];
            if (u < 0 || u >= n_vertices || v < 0 || v >= n_vertices) { bad.store(1); continue; }
            if (!(__atomic_load_n(&h_bits[u], __ATOMIC_RELAXED) & bit)) __atomic_fetch_or(&h_bits[u], bit, __ATOMIC_RELAXED);
            if (!(__atomic_load_n(&h_bits[v], __ATOMIC_RELAXED) & bit)) __atomic_fetch_or(&h_bits[v], bit, __ATOMIC_RELAXED);
        }
    });
    if (bad.load()) return set_error(DRONE_E_INVALID, "drone_presence_bits_host: an edge names a vertex outside 0..%d", n_vertices - 1);
    return DRONE_OK;
}
