/* Stand-in for the MPI calls the reference's partitioner makes (EBV_mpi.cpp:87-117,140,233-239,436-449,713), so that
 * the unmodified source file runs as P ranks on one machine without an MPI installation.  Test infrastructure for
 * oracle/_ref only.
 *
 * MPI_Init reads the number of ranks from the environment (EBV_STANDIN_RANKS, default 1), maps one shared anonymous
 * region and forks: the calling process becomes rank 0, the children ranks 1..P-1.  Every ordered pair of ranks owns
 * one mailbox of 10,000 ints (the partitioner's largest message, EBV_mpi.cpp:34,37); a message waits in it until the
 * receiver takes it, so messages between two ranks keep their order, which is all the partitioner relies on (every
 * rank issues the same sequence of exchanges).  Non-blocking calls only record the request; MPI_Waitall moves the
 * data.  Every wait gives up after two minutes and ends the process with a message.
 */
#ifndef DRONE_ORACLE_EBV_MPI_STANDIN_H
#define DRONE_ORACLE_EBV_MPI_STANDIN_H
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <sched.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

typedef int MPI_Comm;
typedef int MPI_Datatype;
#define MPI_COMM_WORLD 0
#define MPI_INT 4
#define MPI_SUCCESS 0

struct MPI_Status {
    int count;
    int MPI_SOURCE, MPI_TAG;
};
#define MPI_STATUS_IGNORE ((MPI_Status *)0)

struct MPI_Request {
    int kind;       /* 0 = nothing pending, 1 = send, 2 = receive */
    void *buf;
    int count, peer, tag, received;
};

namespace ebv_standin {

constexpr int kMaxInts = 10000;
constexpr int kMaxRanks = 16;

struct Mailbox {
    std::atomic<int> full;
    int tag, count;
    int data[kMaxInts];
};

struct World {
    std::atomic<int> arrived;
    std::atomic<int> generation;
    Mailbox box[kMaxRanks * kMaxRanks];   /* box[from * ranks + to] */
};

struct State {
    World *world = nullptr;
    int rank = 0, ranks = 1;
    pid_t children[kMaxRanks] = {0};
};

inline State &state() {
    static State s;
    return s;
}

[[noreturn]] inline void give_up(const char *what) {
    std::fprintf(stderr, "MPI stand-in, rank %d: %s\n", state().rank, what);
    std::fflush(nullptr);
    _exit(3);
}

/* Spins on `ready` with a yield between polls; two minutes at most. */
template <typename Ready>
inline void wait_until(Ready ready, const char *what) {
    const time_t start = time(nullptr);
    for (unsigned long long spin = 0; !ready(); ++spin) {
        sched_yield();
        if ((spin & 0xffff) == 0xffff && time(nullptr) - start > 120) give_up(what);
    }
}

inline Mailbox &mailbox(int from, int to) { return state().world->box[from * state().ranks + to]; }

inline bool try_send(MPI_Request &r) {
    Mailbox &m = mailbox(state().rank, r.peer);
    if (m.full.load(std::memory_order_acquire)) return false;
    m.tag = r.tag;
    m.count = r.count;
    std::memcpy(m.data, r.buf, sizeof(int) * (size_t)r.count);
    m.full.store(1, std::memory_order_release);
    r.kind = 0;
    return true;
}

inline bool try_receive(MPI_Request &r) {
    Mailbox &m = mailbox(r.peer, state().rank);
    if (!m.full.load(std::memory_order_acquire)) return false;
    if (m.tag != r.tag) give_up("message tag differs from the posted receive");
    if (m.count > r.count) give_up("message longer than the posted receive");
    std::memcpy(r.buf, m.data, sizeof(int) * (size_t)m.count);
    r.received = m.count;
    m.full.store(0, std::memory_order_release);
    r.kind = 0;
    return true;
}

inline bool progress(MPI_Request &r) {
    if (r.kind == 1) return try_send(r);
    if (r.kind == 2) return try_receive(r);
    return true;
}

inline MPI_Request make_request(int kind, const void *buf, int count, int peer, int tag) {
    if (count < 0 || count > kMaxInts) give_up("message larger than a mailbox");
    if (peer < 0 || peer >= state().ranks) give_up("peer outside the world");
    MPI_Request r;
    r.kind = kind;
    r.buf = const_cast<void *>(buf);
    r.count = count;
    r.peer = peer;
    r.tag = tag;
    r.received = 0;
    return r;
}

}  // namespace ebv_standin

inline int MPI_Init(int *, char ***) {
    using namespace ebv_standin;
    State &s = state();
    const char *env = std::getenv("EBV_STANDIN_RANKS");
    s.ranks = env ? std::atoi(env) : 1;
    if (s.ranks < 1 || s.ranks > kMaxRanks) give_up("EBV_STANDIN_RANKS must be 1..16");
    void *mem = mmap(nullptr, sizeof(World), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
    if (mem == MAP_FAILED) give_up("mmap of the shared region failed");
    s.world = new (mem) World;   /* the mapping is zero-filled: all mailboxes empty, counters zero */
    std::fflush(nullptr);
    for (int r = 1; r < s.ranks; ++r) {
        const pid_t pid = fork();
        if (pid < 0) give_up("fork failed");
        if (pid == 0) {
            s.rank = r;
            return MPI_SUCCESS;
        }
        s.children[r] = pid;
    }
    s.rank = 0;
    return MPI_SUCCESS;
}

inline int MPI_Comm_rank(MPI_Comm, int *rank) { *rank = ebv_standin::state().rank; return MPI_SUCCESS; }
inline int MPI_Comm_size(MPI_Comm, int *size) { *size = ebv_standin::state().ranks; return MPI_SUCCESS; }

inline int MPI_Barrier(MPI_Comm) {
    using namespace ebv_standin;
    World &w = *state().world;
    const int gen = w.generation.load(std::memory_order_acquire);
    if (w.arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == state().ranks) {
        w.arrived.store(0, std::memory_order_relaxed);
        w.generation.store(gen + 1, std::memory_order_release);
    } else {
        wait_until([&] { return w.generation.load(std::memory_order_acquire) != gen; }, "barrier timed out");
    }
    return MPI_SUCCESS;
}

inline int MPI_Isend(const void *buf, int count, MPI_Datatype, int dest, int tag, MPI_Comm, MPI_Request *req) {
    *req = ebv_standin::make_request(1, buf, count, dest, tag);
    return MPI_SUCCESS;
}

inline int MPI_Irecv(void *buf, int count, MPI_Datatype, int source, int tag, MPI_Comm, MPI_Request *req) {
    *req = ebv_standin::make_request(2, buf, count, source, tag);
    return MPI_SUCCESS;
}

inline int MPI_Waitall(int n, MPI_Request *reqs, MPI_Status *statuses) {
    using namespace ebv_standin;
    wait_until([&] {
        bool all = true;
        for (int i = 0; i < n; ++i) {
            const bool was_receive = reqs[i].kind == 2;
            if (!progress(reqs[i])) { all = false; continue; }
            if (was_receive && statuses) {
                statuses[i].count = reqs[i].received;
                statuses[i].MPI_SOURCE = reqs[i].peer;
                statuses[i].MPI_TAG = reqs[i].tag;
            }
        }
        return all;
    }, "MPI_Waitall timed out");
    return MPI_SUCCESS;
}

inline int MPI_Send(const void *buf, int count, MPI_Datatype, int dest, int tag, MPI_Comm) {
    using namespace ebv_standin;
    MPI_Request r = make_request(1, buf, count, dest, tag);
    wait_until([&] { return try_send(r); }, "MPI_Send timed out");
    return MPI_SUCCESS;
}

inline int MPI_Recv(void *buf, int count, MPI_Datatype, int source, int tag, MPI_Comm, MPI_Status *status) {
    using namespace ebv_standin;
    MPI_Request r = make_request(2, buf, count, source, tag);
    wait_until([&] { return try_receive(r); }, "MPI_Recv timed out");
    if (status) {
        status->count = r.received;
        status->MPI_SOURCE = source;
        status->MPI_TAG = tag;
    }
    return MPI_SUCCESS;
}

inline int MPI_Get_count(const MPI_Status *status, MPI_Datatype, int *count) {
    *count = status->count;
    return MPI_SUCCESS;
}

/* Children leave here (their files are closed by then, EBV_mpi.cpp:677-685); rank 0 collects them and returns. */
inline int MPI_Finalize() {
    using namespace ebv_standin;
    State &s = state();
    MPI_Barrier(MPI_COMM_WORLD);
    std::fflush(nullptr);
    if (s.rank != 0) _exit(0);
    int failed = 0;
    for (int r = 1; r < s.ranks; ++r) {
        int st = 0;
        if (waitpid(s.children[r], &st, 0) < 0 || !WIFEXITED(st) || WEXITSTATUS(st) != 0) failed = 1;
    }
    if (failed) give_up("a rank ended abnormally");
    return MPI_SUCCESS;
}
#endif
