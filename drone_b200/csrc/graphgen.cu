// Seeded R-MAT edge generator, identical on host and device: the edge with
// index e is a pure function of (seed, e), so any range of edges can be produced
// anywhere and the two entry points agree bit for bit.
#include "common.cuh"

namespace drone {

__host__ __device__ inline unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}

// One edge: `scale` quadrant draws with probabilities a, b, c, 1-a-b-c given as
// cumulative 32-bit thresholds (ta = a, tb = a+b, tc = a+b+c, each times 2^32).
__host__ __device__ inline void rmat_edge(int scale, unsigned long long seed, unsigned long long e,
                                          unsigned int ta, unsigned int tb, unsigned int tc, int *u, int *v) {
    unsigned long long state = splitmix64(seed ^ (e * 0xD1342543DE82EF95ULL));
    unsigned int row = 0, col = 0;
    for (int level = 0; level < scale; ++level) {
        state = splitmix64(state);
        const unsigned int r = (unsigned int)(state >> 32);
        const unsigned int rb = (r >= tb) ? 1u : 0u;                    // quadrants c, d: lower half
        const unsigned int cb = ((r >= ta && r < tb) || r >= tc) ? 1u : 0u;  // quadrants b, d: right half
        row = (row << 1) | rb;
        col = (col << 1) | cb;
    }
    *u = (int)row;
    *v = (int)col;
}

__global__ void rmat_edges_kernel(int scale, unsigned long long seed, unsigned long long first, long long n,
                                  unsigned int ta, unsigned int tb, unsigned int tc, int *u, int *v) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        rmat_edge(scale, seed, first + (unsigned long long)i, ta, tb, tc, u + i, v + i);
}

static int thresholds(double a, double b, double c, unsigned int *ta, unsigned int *tb, unsigned int *tc) {
    if (!(a > 0 && b >= 0 && c >= 0 && a + b + c < 1.0 + 1e-12))
        return set_error(DRONE_E_INVALID, "rmat: probabilities a=%g b=%g c=%g are not a sub-distribution", a, b, c);
    const double two32 = 4294967296.0;
    auto clamp = [&](double x) { return (unsigned int)(x >= two32 - 1 ? two32 - 1 : x); };
    *ta = clamp(a * two32);
    *tb = clamp((a + b) * two32);
    *tc = clamp((a + b + c) * two32);
    return DRONE_OK;
}

}  // namespace drone

using namespace drone;

extern "C" {

int drone_rmat_edges(int scale, long long n_edges, unsigned long long seed, double a, double b, double c,
                     long long first_edge, int *d_u, int *d_v, void *stream) {
    DRONE_REQUIRE(scale >= 1 && scale <= 30, "drone_rmat_edges: scale=%d outside 1..30", scale);
    DRONE_REQUIRE(n_edges >= 0 && first_edge >= 0, "drone_rmat_edges: negative edge range");
    unsigned int ta, tb, tc;
    const int rc = thresholds(a, b, c, &ta, &tb, &tc);
    if (rc) return rc;
    if (n_edges == 0) return DRONE_OK;
    DRONE_REQUIRE(d_u && d_v, "drone_rmat_edges: NULL output");
    long long grid = (n_edges + 255) / 256;
    if (grid > 148 * 64) grid = 148 * 64;
    rmat_edges_kernel<<<(int)grid, 256, 0, (cudaStream_t)stream>>>(scale, seed, (unsigned long long)first_edge,
                                                                  n_edges, ta, tb, tc, d_u, d_v);
    DRONE_LAUNCH_CHECK("rmat_edges_kernel");
    return DRONE_OK;
}

int drone_rmat_edges_host(int scale, long long n_edges, unsigned long long seed, double a, double b, double c,
                          long long first_edge, int *h_u, int *h_v) {
    DRONE_REQUIRE(scale >= 1 && scale <= 30, "drone_rmat_edges_host: scale=%d outside 1..30", scale);
    DRONE_REQUIRE(n_edges >= 0 && first_edge >= 0, "drone_rmat_edges_host: negative edge range");
    unsigned int ta, tb, tc;
    const int rc = thresholds(a, b, c, &ta, &tb, &tc);
    if (rc) return rc;
    if (n_edges == 0) return DRONE_OK;
    DRONE_REQUIRE(h_u && h_v, "drone_rmat_edges_host: NULL output");
    for (long long i = 0; i < n_edges; ++i)
        rmat_edge(scale, seed, (unsigned long long)(first_edge + i), ta, tb, tc, h_u + i, h_v + i);
    return DRONE_OK;
}

}  // extern "C"
