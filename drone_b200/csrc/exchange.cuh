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
};

#define DRONE_NCCL(call)                                                                 \
    do {                                                                                 \
        ncclResult_t r__ = (call);                                                       \
        if (r__ != ncclSuccess)                                                          \
            return drone::set_error(DRONE_E_NCCL, "%s failed at %s:%d: %s", #call,       \
                                    __FILE__, __LINE__, ncclGetErrorString(r__));        \
    } while (0)

