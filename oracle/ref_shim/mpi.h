/* Stand-in for the one MPI call on the reference's aggregation path (MPI_Bcast of the NCCL unique id,
 * cuda_gcn/src/cuda/graph.cu:41).  With one worker the id is already where it is needed.  With several workers (one
 * process per GPU, started by the test) the bytes travel through a file, the way the reference's other build_graph
 * does it (DRONE/src/cuda/graph.cu:31-37,122-128): the environment names the file (DRONE_REF_ID_FILE) and this
 * process's rank (DRONE_REF_RANK); the root writes a temporary file and renames it, the others wait for the name to
 * appear (at most 60 s).  Test infrastructure for oracle/_ref only. */
#ifndef DRONE_ORACLE_MPI_SHIM_H
#define DRONE_ORACLE_MPI_SHIM_H
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
typedef int MPI_Comm;
typedef int MPI_Datatype;
#define MPI_COMM_WORLD 0
#define MPI_BYTE 1
static inline int MPI_Bcast(void *buffer, int count, MPI_Datatype type, int root, MPI_Comm comm) {
    (void)type; (void)comm;
    const char *path = getenv("DRONE_REF_ID_FILE");
    const char *rank_s = getenv("DRONE_REF_RANK");
    if (!path || !rank_s) return 0;                     /* single worker */
    const int rank = atoi(rank_s);
    if (rank == root) {
        char tmp[4096];
        snprintf(tmp, sizeof(tmp), "%s.tmp", path);
        FILE *f = fopen(tmp, "wb");
        if (!f) return 1;
        fwrite(buffer, 1, (size_t)count, f);
        fclose(f);
        return rename(tmp, path) == 0 ? 0 : 1;
    }
    for (int tries = 0; tries < 6000; ++tries) {
        FILE *f = fopen(path, "rb");
        if (f) {
            const size_t got = fread(buffer, 1, (size_t)count, f);
            fclose(f);
            if (got == (size_t)count) return 0;
        }
        usleep(10000);
    }
    fprintf(stderr, "MPI_Bcast stand-in: %s did not appear\n", path);
    exit(1);
}
#endif
