// Order of a partitioner rank's edges as the reference leaves it: std::sort over {u, v, degree sum} records with a
// comparator on the degree sum alone, the call of EBV_mpi.cpp:46-48,265.  Which of two edges with equal sums comes
// first is whatever the C++ library's algorithm does, so the Python restatement of the partitioner asks this
// helper (built with the same library as the reference's partitioner) when it has to reproduce the reference's
// files edge for edge.  TEST INFRASTRUCTURE ONLY.
#include <algorithm>

namespace {
struct Edge {
    int u, v, key;
};
bool key_less(Edge a, Edge b) { return a.key < b.key; }
}  // namespace

extern "C" void ebv_std_sort(int *u, int *v, int *key, long n) {
    Edge *e = new Edge[n > 0 ? n : 1];
    for (long i = 0; i < n; ++i) e[i] = {u[i], v[i], key[i]};
    std::sort(e, e + n, key_less);
    for (long i = 0; i < n; ++i) {
        u[i] = e[i].u;
        v[i] = e[i].v;
        key[i] = e[i].key;
    }
    delete[] e;
}
