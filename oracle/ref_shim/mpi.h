/* Single-process stand-in for the one MPI call on the reference's aggregation path
 * (MPI_Bcast of the NCCL unique id, cuda_gcn/src/cuda/graph.cu:41): with one worker the id is already where it
 * is needed.  Test infrastructure for oracle/_ref only. */
#ifndef DRONE_ORACLE_MPI_SHIM_H
#define DRONE_ORACLE_MPI_SHIM_H
typedef int MPI_Comm;
typedef int MPI_Datatype;
#define MPI_COMM_WORLD 0
#define MPI_BYTE 1
static inline int MPI_Bcast(void *buffer, int count, MPI_Datatype type, int root, MPI_Comm comm) {
    (void)buffer; (void)count; (void)type; (void)root; (void)comm;
    return 0;
}
#endif
