/*
 * minprop_oracle.c — CPU restatement of DRONE's GPU jobs "cc_cuda" and "sssp_cuda"
 * (minimum propagation along out-edges over an EBV-partitioned graph).
 *
 * TEST INFRASTRUCTURE ONLY (same rules as drone_oracle.c).
 * Parity status: the reference holds no golden labels or distances for these jobs.  The
 * restatement is pinned by running the reference's own sources (compiled into oracle/_ref) on
 * a GPU box: distances, labels (one worker, ids in first-seen order) and the Response sizes of
 * every superstep are identical on one and two workers (tests/test_reference_jobs_gpu.py).  On
 * the CPU it is cross-checked against plain single-graph fixed points
 * (tests/test_minprop_oracle.py).
 *
 * What is restated:
 *   local run      — DRONE/src/cuda/algorithm/cc.cu:9-46 (cc_init, cc_exec) and :320-345 / :398-420 (the loops of
 *                    CC_PEVal / CC_IncEVal); sssp.cu:23-74 (sssp_init, sssp_exec) and :398-430 / :494-523.
 *   exchange       — cc.cu:48-157 (which vertices are sent, how received values are applied) and :160-317 (the two
 *                    phases); sssp.cu:76-185 and :187-396 are the same with float distances.
 *   message sweep  — cc_process_messages, cc.cu:385-398; sssp_process_messages, sssp.cu:478-492.
 *   counters       — struct Response, DRONE/src/cuda/algorithm/common.h:23-27; countActive, common.cu:6-31.
 *   stop rule      — all four sizes zero on every worker, DRONE/src/tools/cuda_convert.go:47-52.
 *
 * Two deliberate differences from the GPU reference, both stated in the tests as well:
 *   * labels start as the GLOBAL vertex id (as the CPU job does, DRONE/src/algorithm/CC.go:73-79); cc_init
 *     (cc.cu:14) writes the LOCAL index, which makes labels of different workers incomparable;
 *   * a shorter distance always re-activates the vertex; sssp_exec (sssp.cu:67) asks for an improvement above
 *     1e-6, which leaves results that depend on the order of the atomics.  With unit edge lengths (what
 *     build_graph stores, DRONE/src/cuda/graph.cu:100) the two rules agree.
 *
 * A partition is given as P edge lists in global vertex ids (concatenated, eoff[P+1]) plus owner[v].
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MP_CC 0
#define MP_SSSP 1
#define MP_FAR 1e8f /* sssp_init, sssp.cu:33 */

/* Single graph, labels: label[v] = smallest id among the vertices that reach v (v included). */
void oracle_cc_fixed_point(int V, const int *rowptr, const int *col, int *label) {
    int *queue = (int *)malloc(sizeof(int) * (size_t)(V > 0 ? V : 1));
    for (int v = 0; v < V; ++v) label[v] = v;
    /* ascending seeds: a vertex relabelled by a smaller seed is never a seed itself, and inside one seed's
       search every vertex is relabelled (and queued) at most once, so the queue never holds more than V ids */
    for (int s = 0; s < V; ++s) {
        if (label[s] != s) continue;
        int head = 0, tail = 0;
        queue[tail++] = s;
        while (head < tail) {
            const int u = queue[head++];
            for (int k = rowptr[u]; k < rowptr[u + 1]; ++k) {
                const int w = col[k];
                if (label[w] > s) {
                    label[w] = s;
                    queue[tail++] = w;
                }
            }
        }
    }
    free(queue);
}

/* Single graph, float distances from `source` (edge lengths len[k], NULL = 1.0f), Bellman-Ford with a FIFO. */
void oracle_sssp_f32(int V, const int *rowptr, const int *col, const float *len, int source, float *dist) {
    int *queue = (int *)malloc(sizeof(int) * (size_t)(V > 0 ? V : 1));
    uint8_t *queued = (uint8_t *)calloc((size_t)(V > 0 ? V : 1), 1);
    for (int v = 0; v < V; ++v) dist[v] = MP_FAR;
    if (source >= 0 && source < V) {
        int head = 0, count = 0;
        dist[source] = 0.0f;
        queue[(head + count++) % V] = source;
        queued[source] = 1;
        while (count > 0) {
            const int u = queue[head];
            head = (head + 1) % V;
            --count;
            queued[u] = 0;
            const float du = dist[u];
            for (int k = rowptr[u]; k < rowptr[u + 1]; ++k) {
                const int w = col[k];
                const float nd = du + (len ? len[k] : 1.0f);
                if (nd < dist[w]) {
                    dist[w] = nd;
                    if (!queued[w]) {
                        queued[w] = 1;
                        queue[(head + count++) % V] = w;
                    }
                }
            }
        }
    }
    free(queue);
    free(queued);
}

/* ------------------------------------------------------------------------- */
/* The job over a partition.                                                  */
/* ------------------------------------------------------------------------- */
typedef struct {
    int P, V;
    uint8_t *present; /* [P][V] */
    int *nrep;        /* [V] */
    const int *owner;
    int **rowptr, **col;
    float **len;
} MpParts;

static void mp_parts_init(MpParts *g, int P, int V, const int *eoff, const int *eu, const int *ev, const float *elen,
                          const int *owner) {
    g->P = P; g->V = V; g->owner = owner;
    g->present = (uint8_t *)calloc((size_t)P * V, 1);
    g->nrep = (int *)calloc((size_t)V, sizeof(int));
    g->rowptr = (int **)calloc((size_t)P, sizeof(int *));
    g->col = (int **)calloc((size_t)P, sizeof(int *));
    g->len = (float **)calloc((size_t)P, sizeof(float *));
    for (int p = 0; p < P; ++p) {
        uint8_t *pr = g->present + (size_t)p * V;
        const int e0 = eoff[p], e1 = eoff[p + 1];
        g->rowptr[p] = (int *)calloc((size_t)V + 1, sizeof(int));
        g->col[p] = (int *)malloc(sizeof(int) * (size_t)(e1 - e0 + 1));
        g->len[p] = (float *)malloc(sizeof(float) * (size_t)(e1 - e0 + 1));
        int *fill = (int *)calloc((size_t)V, sizeof(int));
        for (int i = e0; i < e1; ++i) { pr[eu[i]] = 1; pr[ev[i]] = 1; g->rowptr[p][eu[i] + 1]++; }
        for (int v = 0; v < V; ++v) g->rowptr[p][v + 1] += g->rowptr[p][v];
        for (int i = e0; i < e1; ++i) {
            const int at = g->rowptr[p][eu[i]] + fill[eu[i]]++;
            g->col[p][at] = ev[i];
            g->len[p][at] = elen ? elen[i] : 1.0f;
        }
        free(fill);
        for (int v = 0; v < V; ++v) g->nrep[v] += pr[v];
    }
}

static void mp_parts_free(MpParts *g) {
    for (int p = 0; p < g->P; ++p) { free(g->rowptr[p]); free(g->col[p]); free(g->len[p]); }
    free(g->rowptr); free(g->col); free(g->len); free(g->present); free(g->nrep);
}

/* values are kept as float for both kinds: labels below 2^24 are exact in a float, and the tests stay below that */
typedef struct { float *val; int *active, *ubm; } MpState;

/* cc_exec / sssp_exec repeated until nothing changes (the while loops of *_PEVal / *_IncEVal) */
static void mp_local_run(const MpParts *g, int p, int kind, MpState *s) {
    const int V = g->V;
    const uint8_t *pr = g->present + (size_t)p * V;
    int step = 0, changed = 1;
    while (changed) {
        changed = 0;
        for (int u = 0; u < V; ++u) {
            if (!pr[u] || s->active[u] != step) continue;
            const float now = s->val[u];
            for (int k = g->rowptr[p][u]; k < g->rowptr[p][u + 1]; ++k) {
                const int w = g->col[p][k];
                const float nv = kind == MP_CC ? now : now + g->len[p][k];
                if (nv < s->val[w]) {
                    s->val[w] = nv;
                    s->active[w] = step + 1;
                    changed = 1;
                }
            }
        }
        ++step;
    }
}

/*
 * Runs the job to its stop rule.  out[v] = value at the master (or only) copy, as float (labels are integers
 * stored in floats); vertices in no part get -1.  sizes[(step * P + p) * 5 + 0..4] = the four exchange sizes and
 * VisitedSize of worker p in superstep `step` (PEval = step 0).  Returns the number of supersteps run.
 */
int oracle_mp_drone_cuda(int kind, int P, int V, const int *eoff, const int *eu, const int *ev, const float *elen,
                         const int *owner, int source, int max_steps, float *out, long long *sizes) {
    MpParts g;
    mp_parts_init(&g, P, V, eoff, eu, ev, elen, owner);
    MpState *st = (MpState *)calloc((size_t)P, sizeof(MpState));
    for (int p = 0; p < P; ++p) {
        st[p].val = (float *)malloc(sizeof(float) * (size_t)V);
        st[p].active = (int *)malloc(sizeof(int) * (size_t)V);
        st[p].ubm = (int *)calloc((size_t)V, sizeof(int));
    }
    int steps = 0;
    for (int step = 0; step <= max_steps; ++step) {
        long long total = 0;
        for (int p = 0; p < P; ++p) {
            const uint8_t *pr = g.present + (size_t)p * V;
            if (step == 0) {
                for (int v = 0; v < V; ++v) {
                    if (kind == MP_CC) { st[p].val[v] = (float)v; st[p].active[v] = 0; }
                    else { st[p].val[v] = v == source ? 0.0f : MP_FAR; st[p].active[v] = v == source ? 0 : -1; }
                    if (!pr[v]) st[p].active[v] = -2; /* not a local vertex: never matches a step, never counted */
                }
            } else {
                for (int v = 0; v < V; ++v) {
                    if (!pr[v]) continue;
                    if (st[p].ubm[v]) { st[p].active[v] = 0; st[p].ubm[v] = 0; }
                    else st[p].active[v] = -1;
                }
            }
            mp_local_run(&g, p, kind, &st[p]);
        }
        long long *row = sizes + (size_t)step * P * 5;
        memset(row, 0, sizeof(long long) * (size_t)P * 5);
        /* mirror -> master: mirrors lowered in this run */
        for (int p = 0; p < P; ++p)
            for (int v = 0; v < V; ++v) {
                if (!(g.present[(size_t)p * V + v] && g.nrep[v] > 1 && owner[v] != p)) continue;
                if (st[p].active[v] <= 0) continue;
                const int o = owner[v];
                row[p * 5 + 0]++;
                row[o * 5 + 1]++;
                if (st[p].val[v] < st[o].val[v]) { st[o].val[v] = st[p].val[v]; st[o].ubm[v] = 1; }
            }
        /* master -> mirrors: masters lowered in this run or by a message */
        for (int p = 0; p < P; ++p)
            for (int v = 0; v < V; ++v) {
                if (!(g.present[(size_t)p * V + v] && g.nrep[v] > 1 && owner[v] == p)) continue;
                if (st[p].active[v] <= 0 && st[p].ubm[v] == 0) continue;
                for (int q = 0; q < P; ++q) {
                    if (q == p || !g.present[(size_t)q * V + v]) continue;
                    row[p * 5 + 2]++;
                    row[q * 5 + 3]++;
                    if (st[p].val[v] < st[q].val[v]) { st[q].val[v] = st[p].val[v]; st[q].ubm[v] = 1; }
                }
            }
        for (int p = 0; p < P; ++p) {
            long long visited = 0;
            for (int v = 0; v < V; ++v)
                if (g.present[(size_t)p * V + v] && st[p].active[v] != 0) ++visited;
            row[p * 5 + 4] = visited;
            for (int k = 0; k < 4; ++k) total += row[p * 5 + k];
        }
        steps = step + 1;
        if (total == 0) break;
    }
    for (int v = 0; v < V; ++v) {
        out[v] = -1.0f;
        if (g.nrep[v] == 0) continue;
        int holder = owner[v];
        if (g.nrep[v] == 1 || holder < 0 || holder >= P || !g.present[(size_t)holder * V + v])
            for (int p = 0; p < P; ++p)
                if (g.present[(size_t)p * V + v]) { holder = p; break; }
        out[v] = st[holder].val[v];
    }
    for (int p = 0; p < P; ++p) { free(st[p].val); free(st[p].active); free(st[p].ubm); }
    free(st);
    mp_parts_free(&g);
    return steps;
}
