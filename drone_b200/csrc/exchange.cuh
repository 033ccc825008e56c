// Internal layout of the communicator and exchange-plan handles of the C ABI.
#pragma once

#include "common.cuh"

#include <nccl.h>
#include <vector>

struct drone_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, nranks = 1;
    bool owned = false;
};

struct drone_xplan {
    int rank = 0, nranks = 1, n_local = 0, max_features = 0;
    // host lists, grouped by peer (offsets have nranks+1 entries)
    std::vector<int> up_rows, up_off;        // my mirror rows, by owner, ascending global id
    std::vector<int> down_rows, down_off;    // my master rows, by mirroring peer, ascending global id
    // master rows that have at least one mirror, with the positions of their
    // contributions in the received buffer (CSR: m_off / m_pos), peers ascending
    std::vector<int> m_rows, m_off, m_pos;
    // device copies
    int device = -1;
    int *d_up_rows = nullptr, *d_down_rows = nullptr, *d_m_rows = nullptr, *d_m_off = nullptr, *d_m_pos = nullptr;
    float *d_send = nullptr, *d_recv = nullptr;   // each max(up, down) * max_features floats
    size_t buf_floats = 0;
    struct drone_p2p *p2p = nullptr;              // peer-memory transport, when enabled
};

// Peer-memory transport of one rank (one process per GPU on one NVLink domain).  Every rank owns a segment
//   [ flags: 2 x nranks epochs | up-receive: n_down rows x max_features | down-receive: n_up rows x max_features ]
// that its peers map through CUDA IPC.  Senders store rows straight into the receiver's segment and then publish
// the call's epoch in the receiver's flag word; receivers poll their own flags with a bounded wait.
struct drone_p2p {
    unsigned epoch = 0;
    char *segment = nullptr;            // my segment (cudaMalloc)
    size_t segment_bytes = 0;
    std::vector<char *> peer_segment;   // peers' segments mapped into this process (NULL for self / unused)
    // device tables, all indexed as documented in exchange_p2p.cu
    float **d_peer_up_recv = nullptr, **d_peer_down_recv = nullptr;   // [nranks] bases inside peers' segments
    unsigned **d_peer_flag_up = nullptr, **d_peer_flag_down = nullptr;   // [nranks] address of "my" word in the peer's flags
    int4 *d_walk = nullptr;             // [n_up] mirror rows in the order push_up walks them: {local row, owner, row in the owner's up-receive, 0}
    int4 *d_pairs = nullptr;            // [n_down] (master, mirror) pairs in m_pos order: {row in my up-receive, peer, row in its down-receive, 0}
    int *d_need_up = nullptr, *d_need_down = nullptr;         // [nranks] 1 where a flag from that peer is expected
    int *h_error = nullptr;             // pinned, mapped: set by a kernel whose wait ran out
    int *d_host_error = nullptr;        // device alias of h_error (written only when a wait runs out)
    int *d_error = nullptr;             // the same word in device memory: what the kernels poll
    unsigned *d_done = nullptr;         // [2] blocks of push_up / add_push_down that have finished (last one publishes the flags)
    int2 *d_route = nullptr;            // [n_local] {owner, row in the owner's up-receive} for my mirror rows, {-1, 0} for the others
    bool push_pending = false;          // the upward half of an exchange was done by an aggregation call; the rest is due
};

namespace drone {
// One direction of the peer-memory exchange for 8- or 16-byte elements per boundary vertex (exchange_p2p.cu).
int p2p_move_elements(drone_xplan *x, const void *d_send, size_t bytes, bool up, cudaStream_t st, const void **recv_out);

// The exchange in two halves, for an aggregation that stores its mirror rows straight into their owners' receive
// areas (exchange_p2p.cu).  p2p_route_begin opens a new epoch and returns the tables the aggregation kernels need;
// when those kernels are in the stream, p2p_route_publish tells the owners that this rank's rows are there (or
// p2p_push_up sends them with the copy kernel, for a call whose kernels could not route); exchange_finish_p2p is the
// rest of the exchange (masters add and send the totals down, mirror rows take them).
int p2p_route_begin(drone_xplan *x, int n_rows, int F, const int2 **route, float *const **peer_rows);
int p2p_route_publish(drone_xplan *x, cudaStream_t st);
int p2p_push_up(drone_xplan *x, const float *d_rows, int F, int ld, cudaStream_t st);
int exchange_finish_p2p(drone_xplan *x, float *d_rows, int F, int ld, cudaStream_t st);
}  // namespace drone

#define DRONE_NCCL(call)                                                                 \
    do {                                                                                 \
        ncclResult_t r__ = (call);                                                       \
        if (r__ != ncclSuccess)                                                          \
            return drone::set_error(DRONE_E_NCCL, "%s failed at %s:%d: %s", #call,       \
                                    __FILE__, __LINE__, ncclGetErrorString(r__));        \
    } while (0)

