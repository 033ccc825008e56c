/*
 * pagerank_oracle.c — CPU restatement of DRONE's PageRank jobs over an
 * EBV-partitioned graph.
 *
 * TEST INFRASTRUCTURE ONLY (same rules as drone_oracle.c).
 * Parity status: the reference holds no golden PageRank values.  The GPU job
 * is pinned by running the reference's own sources (compiled into oracle/_ref)
 * on a GPU box next to the library, on one and two workers
 * (tests/test_reference_jobs_gpu.py: values within 5e-4, float atomics in
 * another order).  The Go job cannot be built here (no Go toolchain, its
 * gRPC/protobuf dependencies are neither vendored nor version-pinned): its
 * restatement below stays unpinned and is cross-checked against the other
 * procedures and against a dense power iteration in tests/test_oracle.py.
 *
 * Three procedures:
 *   oracle_pr_drone_cpu      — the CPU job "pr":   DRONE/src/algorithm/PageRank.go:22-125,
 *                              DRONE/src/worker/PRWorker.go:185-224,281-320,348-363,
 *                              stop rule DRONE/src/master.go:430-463 and :283-287.
 *   oracle_pr_drone_cuda_*   — the GPU job "pr_cuda": DRONE/src/cuda/algorithm/pr.cu:14-87,
 *                              :215-373 (exchange), :375-488 (PEval / IncEval),
 *                              stop rule DRONE/src/tools/cuda_convert.go:47-52.
 *   oracle_pagerank_power_f64 — synchronous power iteration (damping d, fixed
 *                              iteration count, uniform start 1/|V|) in double.
 *
 * A partition is given as P edge lists in global vertex ids (concatenated,
 * eoff[P+1]) plus owner[v] = the part holding the master copy of v (any value
 * for vertices present in a single part).  A vertex is present in part p when
 * one of p's edges touches it.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int P, V;
    const int *eoff, *eu, *ev, *outdeg, *owner;
    uint8_t *present; /* [P][V] */
    int *nrep;        /* [V] number of parts holding v */
    int **rowptr;     /* per part CSR by source over global ids, edge-list order inside a row */
    int **col;
} Parts;

static void parts_init(Parts *g, int P, int V, const int *eoff, const int *eu, const int *ev,
                       const int *outdeg, const int *owner) {
    g->P = P; g->V = V; g->eoff = eoff; g->eu = eu; g->ev = ev; g->outdeg = outdeg; g->owner = owner;
    g->present = (uint8_t *)calloc((size_t)P * V, 1);
    g->nrep = (int *)calloc((size_t)V, sizeof(int));
    g->rowptr = (int **)calloc((size_t)P, sizeof(int *));
    g->col = (int **)calloc((size_t)P, sizeof(int *));
    for (int p = 0; p < P; ++p) {
        uint8_t *pr = g->present + (size_t)p * V;
        const int e0 = eoff[p], e1 = eoff[p + 1];
        g->rowptr[p] = (int *)calloc((size_t)V + 1, sizeof(int));
        g->col[p] = (int *)malloc(sizeof(int) * (size_t)(e1 - e0 + 1));
        int *fill = (int *)calloc((size_t)V, sizeof(int));
        for (int i = e0; i < e1; ++i) {
            pr[eu[i]] = 1; pr[ev[i]] = 1;
            g->rowptr[p][eu[i] + 1]++;
        }
        for (int v = 0; v < V; ++v) g->rowptr[p][v + 1] += g->rowptr[p][v];
        for (int i = e0; i < e1; ++i) g->col[p][g->rowptr[p][eu[i]] + fill[eu[i]]++] = ev[i];
        free(fill);
        for (int v = 0; v < V; ++v) g->nrep[v] += pr[v];
    }
}

static void parts_free(Parts *g) {
    for (int p = 0; p < g->P; ++p) { free(g->rowptr[p]); free(g->col[p]); }
    free(g->rowptr); free(g->col); free(g->present); free(g->nrep);
}

static inline int is_present(const Parts *g, int p, int v) { return g->present[(size_t)p * g->V + v]; }
static inline int is_mirror(const Parts *g, int p, int v) {
    return is_present(g, p, v) && g->nrep[v] > 1 && g->owner[v] != p;
}
static inline int is_master(const Parts *g, int p, int v) {
    return is_present(g, p, v) && g->nrep[v] > 1 && g->owner[v] == p;
}

/* ------------------------------------------------------------------------- */
/* CPU job "pr", float32.  Iteration over Go maps is in random order in the    */
/* reference; here every loop runs in ascending vertex id and messages arrive  */
/* in ascending sender order.                                                  */
/* pr_out[v] = value at the master (or only) copy; vertices in no part get 0.  */
/* Returns the number of supersteps run (PEval counts as step 0).              */
/* ------------------------------------------------------------------------- */
int oracle_pr_drone_cpu(int P, int V, const int *eoff, const int *eu, const int *ev, const int *outdeg,
                        const int *owner, float eps, int max_steps, float *pr_out, long long *messages_out) {
    const float alpha = 0.85f; /* DRONE/src/algorithm/PageRank.go:11 */
    Parts g;
    parts_init(&g, P, V, eoff, eu, ev, outdeg, owner);
    const size_t PV = (size_t)P * V;
    float *pr = (float *)calloc(PV, sizeof(float));
    float *acc = (float *)calloc(PV, sizeof(float));
    float *diff = (float *)calloc(PV, sizeof(float));
    uint8_t *updated = (uint8_t *)calloc(PV, 1), *next_updated = (uint8_t *)calloc(PV, 1);
    uint8_t *upd_master = (uint8_t *)calloc(PV, 1), *upd_mirror = (uint8_t *)calloc(PV, 1);
    /* exchangeBuffer as a dense per-part array with a flag */
    float *exch_val = (float *)calloc(PV, sizeof(float));
    uint8_t *exch_flag = (uint8_t *)calloc(PV, 1);
    long long messages = 0;

#define IDX(p, v) ((size_t)(p) * V + (v))
    /* PEval: PageRank.go:22-57 */
    for (int p = 0; p < P; ++p)
        for (int u = 0; u < V; ++u)
            if (is_present(&g, p, u)) { pr[IDX(p, u)] = 1.0f; acc[IDX(p, u)] = 0.0f; }
    for (int p = 0; p < P; ++p)
        for (int u = 0; u < V; ++u) {
            if (!is_present(&g, p, u)) continue;
            const float temp = pr[IDX(p, u)] / (float)outdeg[u];
            for (int k = g.rowptr[p][u]; k < g.rowptr[p][u + 1]; ++k) {
                const int v = g.col[p][k];
                diff[IDX(p, v)] += temp;
                updated[IDX(p, v)] = 1;
                if (is_mirror(&g, p, v)) upd_mirror[IDX(p, v)] = 1;
                if (is_master(&g, p, v)) upd_master[IDX(p, v)] = 1;
            }
        }
    int any_message = 1; /* PRWorker.go peval reports MessageToSend: true unconditionally */
    int step = 0;
    for (;;) {
        if (!any_message) break;           /* master.go:446-448: no worker had messages -> stop */
        /* Mirror -> master messages (PageRank.go:46-54 / :113-122, delivered by MessageSend,
           PRWorker.go:348-363) carry diff[v] of every vertex in the mirror set; the master adds
           them one by one in ExchangeMessage (PRWorker.go:185-200), here in ascending sender order.
           The worker clears its mirror set after IncEval only (PRWorker.go:297), not after PEval. */
        for (int q = 0; q < P; ++q)
            for (int v = 0; v < V; ++v)
                if (upd_mirror[IDX(q, v)]) {
                    const int o = owner[v];
                    diff[IDX(o, v)] += diff[IDX(q, v)];
                    upd_master[IDX(o, v)] = 1;
                    updated[IDX(o, v)] = 1;
                    ++messages;
                }
        if (step > 0) memset(upd_mirror, 0, PV);
        /* masters send the total to every mirror (PRWorker.go:202-213) */
        for (int p = 0; p < P; ++p)
            for (int v = 0; v < V; ++v)
                if (upd_master[IDX(p, v)]) {
                    for (int q = 0; q < P; ++q)
                        if (q != p && is_present(&g, q, v)) {
                            exch_flag[IDX(q, v)] = 1;
                            exch_val[IDX(q, v)] = diff[IDX(p, v)];
                            ++messages;
                        }
                    upd_master[IDX(p, v)] = 0;
                }
        ++step;
        if (step == max_steps) break;      /* master.go:432-440: "pr" stops at step 200 */

        /* IncEval: PageRank.go:59-125 */
        any_message = 0;
        for (int p = 0; p < P; ++p) {
            for (int v = 0; v < V; ++v)
                if (exch_flag[IDX(p, v)]) {
                    diff[IDX(p, v)] = exch_val[IDX(p, v)];
                    updated[IDX(p, v)] = 1;
                    exch_flag[IDX(p, v)] = 0;
                }
            for (int u = 0; u < V; ++u)
                if (updated[IDX(p, u)]) { acc[IDX(p, u)] += diff[IDX(p, u)]; diff[IDX(p, u)] = 0.0f; }
            for (int u = 0; u < V; ++u) {
                if (!updated[IDX(p, u)]) continue;
                const float prn = alpha * acc[IDX(p, u)] + 1 - alpha;
                const float err = fabsf(pr[IDX(p, u)] - prn);
                if (err > eps) {
                    const float push = (prn - pr[IDX(p, u)]) / (float)outdeg[u];
                    for (int k = g.rowptr[p][u]; k < g.rowptr[p][u + 1]; ++k) {
                        const int v = g.col[p][k];
                        next_updated[IDX(p, v)] = 1;
                        diff[IDX(p, v)] += push;
                        if (is_mirror(&g, p, v)) upd_mirror[IDX(p, v)] = 1;
                        if (is_master(&g, p, v)) upd_master[IDX(p, v)] = 1;
                    }
                }
                pr[IDX(p, u)] = prn;
            }
            memcpy(updated + IDX(p, 0), next_updated + IDX(p, 0), (size_t)V);
            memset(next_updated + IDX(p, 0), 0, (size_t)V);
            for (int v = 0; v < V; ++v)
                if (upd_mirror[IDX(p, v)]) any_message = 1;
        }
    }
    for (int v = 0; v < V; ++v) {
        pr_out[v] = 0.0f;
        for (int p = 0; p < P; ++p)
            if (is_present(&g, p, v) && !is_mirror(&g, p, v)) pr_out[v] = pr[IDX(p, v)];
    }
    if (messages_out) *messages_out = messages;
#undef IDX
    free(pr); free(acc); free(diff); free(updated); free(next_updated); free(upd_master); free(upd_mirror);
    free(exch_val); free(exch_flag);
    parts_free(&g);
    return step;
}

/* ------------------------------------------------------------------------- */
/* The same job with every worker's state in hash maps keyed by global vertex  */
/* id, as the Go program keeps it (map[int]float32 for pr / acc / diff, sets    */
/* for updated / updateMaster / updateMirror; PRWorker.go:30-60), and loops     */
/* over a worker's own vertices instead of over all ids.  Same order of         */
/* operations as oracle_pr_drone_cpu, hence the same bits; it exists to time    */
/* the job with the data structures of the original.                            */
/* ------------------------------------------------------------------------- */
typedef struct { int *keys; float *vals; int cap; } FMap;   /* open addressing, key -1 = empty */

static void fmap_init(FMap *m, int expected) {
    int cap = 16;
    while (cap < 2 * expected + 2) cap <<= 1;
    m->cap = cap;
    m->keys = (int *)malloc(sizeof(int) * (size_t)cap);
    m->vals = (float *)calloc((size_t)cap, sizeof(float));
    for (int i = 0; i < cap; ++i) m->keys[i] = -1;
}
static void fmap_free(FMap *m) { free(m->keys); free(m->vals); }
static inline float *fmap_at(FMap *m, int key) {     /* pointer to the value, inserted as 0 when absent */
    unsigned h = ((unsigned)key * 2654435761u) & (unsigned)(m->cap - 1);
    while (m->keys[h] != key) {
        if (m->keys[h] == -1) { m->keys[h] = key; m->vals[h] = 0.0f; break; }
        h = (h + 1) & (unsigned)(m->cap - 1);
    }
    return &m->vals[h];
}
static void fmap_clear_values(FMap *m) { memset(m->vals, 0, sizeof(float) * (size_t)m->cap); }

int oracle_pr_drone_cpu_maps(int P, int V, const int *eoff, const int *eu, const int *ev, const int *outdeg,
                             const int *owner, float eps, int max_steps, float *pr_out, long long *messages_out) {
    const float alpha = 0.85f;
    Parts g;
    parts_init(&g, P, V, eoff, eu, ev, outdeg, owner);
    /* every worker's own vertices, ascending */
    int **mine = (int **)calloc((size_t)P, sizeof(int *));
    int *n_mine = (int *)calloc((size_t)P, sizeof(int));
    for (int p = 0; p < P; ++p) {
        for (int v = 0; v < V; ++v) n_mine[p] += is_present(&g, p, v);
        mine[p] = (int *)malloc(sizeof(int) * (size_t)(n_mine[p] + 1));
        int k = 0;
        for (int v = 0; v < V; ++v)
            if (is_present(&g, p, v)) mine[p][k++] = v;
    }
    enum { PR, ACC, DIFF, UPD, NEXT, UMASTER, UMIRROR, XVAL, XFLAG, NMAPS };
    FMap *m = (FMap *)calloc((size_t)P * NMAPS, sizeof(FMap));
    for (int p = 0; p < P; ++p)
        for (int k = 0; k < NMAPS; ++k) fmap_init(&m[p * NMAPS + k], n_mine[p]);
#define M(p, which, v) (*fmap_at(&m[(p) * NMAPS + (which)], (v)))
    long long messages = 0;
    for (int p = 0; p < P; ++p)
        for (int i = 0; i < n_mine[p]; ++i) { const int u = mine[p][i]; M(p, PR, u) = 1.0f; M(p, ACC, u) = 0.0f; }
    for (int p = 0; p < P; ++p)
        for (int i = 0; i < n_mine[p]; ++i) {
            const int u = mine[p][i];
            const float temp = M(p, PR, u) / (float)outdeg[u];
            for (int k = g.rowptr[p][u]; k < g.rowptr[p][u + 1]; ++k) {
                const int v = g.col[p][k];
                M(p, DIFF, v) += temp;
                M(p, UPD, v) = 1.0f;
                if (is_mirror(&g, p, v)) M(p, UMIRROR, v) = 1.0f;
                if (is_master(&g, p, v)) M(p, UMASTER, v) = 1.0f;
            }
        }
    int any_message = 1, step = 0;
    for (;;) {
        if (!any_message) break;
        for (int q = 0; q < P; ++q)
            for (int i = 0; i < n_mine[q]; ++i) {
                const int v = mine[q][i];
                if (M(q, UMIRROR, v) != 0.0f) {
                    const int o = owner[v];
                    M(o, DIFF, v) += M(q, DIFF, v);
                    M(o, UMASTER, v) = 1.0f;
                    M(o, UPD, v) = 1.0f;
                    ++messages;
                }
            }
        if (step > 0)
            for (int p = 0; p < P; ++p) fmap_clear_values(&m[p * NMAPS + UMIRROR]);
        for (int p = 0; p < P; ++p)
            for (int i = 0; i < n_mine[p]; ++i) {
                const int v = mine[p][i];
                if (M(p, UMASTER, v) != 0.0f) {
                    for (int q = 0; q < P; ++q)
                        if (q != p && is_present(&g, q, v)) {
                            M(q, XFLAG, v) = 1.0f;
                            M(q, XVAL, v) = M(p, DIFF, v);
                            ++messages;
                        }
                    M(p, UMASTER, v) = 0.0f;
                }
            }
        ++step;
        if (step == max_steps) break;
        any_message = 0;
        for (int p = 0; p < P; ++p) {
            for (int i = 0; i < n_mine[p]; ++i) {
                const int v = mine[p][i];
                if (M(p, XFLAG, v) != 0.0f) { M(p, DIFF, v) = M(p, XVAL, v); M(p, UPD, v) = 1.0f; M(p, XFLAG, v) = 0.0f; }
            }
            for (int i = 0; i < n_mine[p]; ++i) {
                const int u = mine[p][i];
                if (M(p, UPD, u) != 0.0f) { M(p, ACC, u) += M(p, DIFF, u); M(p, DIFF, u) = 0.0f; }
            }
            for (int i = 0; i < n_mine[p]; ++i) {
                const int u = mine[p][i];
                if (M(p, UPD, u) == 0.0f) continue;
                const float prn = alpha * M(p, ACC, u) + 1 - alpha;
                const float err = fabsf(M(p, PR, u) - prn);
                if (err > eps) {
                    const float push = (prn - M(p, PR, u)) / (float)outdeg[u];
                    for (int k = g.rowptr[p][u]; k < g.rowptr[p][u + 1]; ++k) {
                        const int v = g.col[p][k];
                        M(p, NEXT, v) = 1.0f;
                        M(p, DIFF, v) += push;
                        if (is_mirror(&g, p, v)) M(p, UMIRROR, v) = 1.0f;
                        if (is_master(&g, p, v)) M(p, UMASTER, v) = 1.0f;
                    }
                }
                M(p, PR, u) = prn;
            }
            for (int i = 0; i < n_mine[p]; ++i) {
                const int v = mine[p][i];
                M(p, UPD, v) = M(p, NEXT, v);
                M(p, NEXT, v) = 0.0f;
                if (M(p, UMIRROR, v) != 0.0f) any_message = 1;
            }
        }
    }
    for (int v = 0; v < V; ++v) {
        pr_out[v] = 0.0f;
        for (int p = 0; p < P; ++p)
            if (is_present(&g, p, v) && !is_mirror(&g, p, v)) pr_out[v] = M(p, PR, v);
    }
    if (messages_out) *messages_out = messages;
#undef M
    for (int p = 0; p < P; ++p) {
        for (int k = 0; k < NMAPS; ++k) fmap_free(&m[p * NMAPS + k]);
        free(mine[p]);
    }
    free(m); free(mine); free(n_mine);
    parts_free(&g);
    return step;
}

/* ------------------------------------------------------------------------- */
/* GPU job "pr_cuda".  REAL is float (the reference) or double (same schedule  */
/* without float rounding).  nvcc contracts alpha*(acc+globalAcc)+(1-alpha)    */
/* into one fused multiply-add, so fma() is used there; sums that the          */
/* reference forms with atomicAdd in arbitrary order are formed in ascending   */
/* vertex / part order.                                                        */
/* sizes_out (optional) receives, per superstep, the four exchange counts      */
/* summed over parts: m2m_send, m2m_recv, M2m_send, M2m_recv.                  */
/* ------------------------------------------------------------------------- */
#define DEFINE_PR_CUDA(NAME, REAL, FMA, FABS)                                                          \
    int NAME(int P, int V, const int *eoff, const int *eu, const int *ev, const int *outdeg,            \
             const int *owner, REAL eps, int max_steps, REAL *pr_out, long long *sizes_out) {           \
        const REAL alpha = (REAL)0.85f; /* pr.cu:12: const float alpha = 0.85 */                         \
        const REAL one_minus_alpha = (REAL)1 - alpha;                                                   \
        Parts g;                                                                                        \
        parts_init(&g, P, V, eoff, eu, ev, outdeg, owner);                                              \
        const size_t PV = (size_t)P * V;                                                                \
        REAL *pr = (REAL *)calloc(PV, sizeof(REAL)), *acc = (REAL *)calloc(PV, sizeof(REAL));           \
        REAL *diff = (REAL *)calloc(PV, sizeof(REAL));                                                  \
        REAL *gdiff = (REAL *)calloc((size_t)P, sizeof(REAL)), *gacc = (REAL *)calloc((size_t)P, sizeof(REAL)); \
        uint8_t *active = (uint8_t *)calloc(PV, 1), *ubm = (uint8_t *)calloc(PV, 1);                    \
        int step = 0;                                                                                   \
        for (;;) {                                                                                      \
            if (step == 0) { /* PR_PEVal, pr.cu:375-428 with pr_init :14-37 */                          \
                for (int p = 0; p < P; ++p)                                                             \
                    for (int u = 0; u < V; ++u)                                                         \
                        if (is_present(&g, p, u)) { pr[(size_t)p * V + u] = 1; }                        \
                for (int p = 0; p < P; ++p)                                                             \
                    for (int u = 0; u < V; ++u) {                                                       \
                        if (!is_present(&g, p, u)) continue;                                            \
                        if (outdeg[u] == 0) {                                                           \
                            if (!is_mirror(&g, p, u)) gdiff[p] += pr[(size_t)p * V + u] / V;            \
                        } else {                                                                        \
                            const REAL t = pr[(size_t)p * V + u] / outdeg[u];                           \
                            for (int k = g.rowptr[p][u]; k < g.rowptr[p][u + 1]; ++k) {                 \
                                const int v = g.col[p][k];                                              \
                                diff[(size_t)p * V + v] += t;                                           \
                                active[(size_t)p * V + v] = 1;                                          \
                            }                                                                           \
                        }                                                                               \
                    }                                                                                   \
            } else { /* PR_IncEVal, pr.cu:450-488: pr_process_messages :430-448, pr_increment :51-87 */  \
                for (int p = 0; p < P; ++p) {                                                           \
                    gacc[p] += gdiff[p];                                                                \
                    gdiff[p] = 0;                                                                       \
                    for (int u = 0; u < V; ++u) {                                                       \
                        const size_t i = (size_t)p * V + u;                                             \
                        active[i] = 0; ubm[i] = 0;                                                      \
                        acc[i] += diff[i]; diff[i] = 0;                                                 \
                    }                                                                                   \
                }                                                                                       \
                for (int p = 0; p < P; ++p)                                                             \
                    for (int u = 0; u < V; ++u) {                                                       \
                        if (!is_present(&g, p, u)) continue;                                            \
                        const size_t i = (size_t)p * V + u;                                             \
                        const REAL prn = FMA(alpha, acc[i] + gacc[p], one_minus_alpha);                 \
                        REAL d = prn - pr[i];                                                           \
                        if (d < 0) d = -d;                                                              \
                        if (d < eps) continue;                                                          \
                        if (outdeg[u] == 0) {                                                           \
                            if (!is_mirror(&g, p, u)) gdiff[p] += (prn - pr[i]) / V;                    \
                        } else {                                                                        \
                            const REAL t = (prn - pr[i]) / outdeg[u];                                   \
                            for (int k = g.rowptr[p][u]; k < g.rowptr[p][u + 1]; ++k) {                 \
                                const int v = g.col[p][k];                                              \
                                diff[(size_t)p * V + v] += t;                                           \
                                active[(size_t)p * V + v] = 1;                                          \
                            }                                                                           \
                        }                                                                               \
                        pr[i] = prn;                                                                    \
                    }                                                                                   \
            }                                                                                           \
            /* Mirror2MasterSend, pr.cu:215-297: active mirrors -> owner, added there */                 \
            long long m2m = 0, M2m = 0;                                                                 \
            for (int q = 0; q < P; ++q)                                                                 \
                for (int v = 0; v < V; ++v)                                                             \
                    if (active[(size_t)q * V + v] && is_mirror(&g, q, v)) {                             \
                        const int o = owner[v];                                                         \
                        diff[(size_t)o * V + v] += diff[(size_t)q * V + v];                             \
                        ubm[(size_t)o * V + v] = 1;                                                     \
                        ++m2m;                                                                          \
                    }                                                                                   \
            /* Master2MirrorSend, pr.cu:299-373: masters that changed -> every mirror, assigned */       \
            for (int p = 0; p < P; ++p)                                                                 \
                for (int v = 0; v < V; ++v)                                                             \
                    if (is_master(&g, p, v) && (active[(size_t)p * V + v] || ubm[(size_t)p * V + v]))   \
                        for (int q = 0; q < P; ++q)                                                     \
                            if (q != p && is_present(&g, q, v)) {                                       \
                                diff[(size_t)q * V + v] = diff[(size_t)p * V + v];                      \
                                ubm[(size_t)q * V + v] = 1;                                             \
                                ++M2m;                                                                  \
                            }                                                                           \
            { /* ncclAllReduce(globalDiff), pr.cu:365 */                                                \
                REAL s = 0;                                                                             \
                for (int p = 0; p < P; ++p) s += gdiff[p];                                              \
                for (int p = 0; p < P; ++p) gdiff[p] = s;                                               \
            }                                                                                           \
            if (sizes_out) {                                                                            \
                sizes_out[4 * step + 0] = m2m; sizes_out[4 * step + 1] = m2m;                           \
                sizes_out[4 * step + 2] = M2m; sizes_out[4 * step + 3] = M2m;                           \
            }                                                                                           \
            ++step;                                                                                     \
            /* cuda_convert.go:47-52 + master.go:283-287,446-448: stop when nobody exchanged anything */ \
            if ((m2m == 0 && M2m == 0) || step >= max_steps) break;                                     \
        }                                                                                               \
        for (int v = 0; v < V; ++v) {                                                                   \
            pr_out[v] = 0;                                                                              \
            for (int p = 0; p < P; ++p)                                                                 \
                if (is_present(&g, p, v) && !is_mirror(&g, p, v)) pr_out[v] = pr[(size_t)p * V + v];    \
        }                                                                                               \
        free(pr); free(acc); free(diff); free(gdiff); free(gacc); free(active); free(ubm);              \
        parts_free(&g);                                                                                 \
        return step;                                                                                    \
    }

DEFINE_PR_CUDA(oracle_pr_drone_cuda_f32, float, fmaf, fabsf)
DEFINE_PR_CUDA(oracle_pr_drone_cuda_f64, double, fma, fabs)

/* ------------------------------------------------------------------------- */
/* Synchronous power iteration on the whole graph (CSR by source), double:     */
/*   pr0 = 1/V;  pr' = (1-d)/V + d * (sum_{u->v} pr[u]/outdeg[u] + dangling/V)  */
/* ------------------------------------------------------------------------- */
void oracle_pagerank_power_f64(int V, const int *rowptr, const int *col, int iterations, double d,
                               double *pr_out) {
    double *pr = (double *)malloc(sizeof(double) * (size_t)V);
    double *nx = (double *)malloc(sizeof(double) * (size_t)V);
    for (int v = 0; v < V; ++v) pr[v] = 1.0 / V;
    for (int it = 0; it < iterations; ++it) {
        double dangling = 0.0;
        for (int v = 0; v < V; ++v) nx[v] = 0.0;
        for (int u = 0; u < V; ++u) {
            const int deg = rowptr[u + 1] - rowptr[u];
            if (deg == 0) { dangling += pr[u]; continue; }
            const double t = pr[u] / deg;
            for (int k = rowptr[u]; k < rowptr[u + 1]; ++k) nx[col[k]] += t;
        }
        for (int v = 0; v < V; ++v) nx[v] = (1.0 - d) / V + d * (nx[v] + dangling / V);
        double *tmp = pr; pr = nx; nx = tmp;
    }
    memcpy(pr_out, pr, sizeof(double) * (size_t)V);
    free(pr); free(nx);
}
