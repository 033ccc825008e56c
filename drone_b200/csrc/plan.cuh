// Internal layout of an aggregation plan (opaque drone_plan of the C ABI).
#pragma once

#include "common.cuh"

namespace drone {

// One chunk of a long row: nonzeros [k0, k0+len) of `row`.  slot >= 0 means the
// chunk's sum goes to partial-sum slot `slot` (the row has several chunks);
// slot < 0 means the chunk is the whole row and its sum goes straight to Y.
struct Chunk {
    int row;
    int k0;
    int len;
    int slot;
};

// A row whose chunks were summed separately: partial sums slot0 .. slot0+nslots-1,
// added in that order into Y[row].
struct SplitRow {
    int row;
    int slot0;
    int nslots;
    int pad;
};

// CSR of one orientation plus the work lists of its long rows.
struct Side {
    bool ready = false;
    int *rowptr = nullptr;     // [n_rows + 1]
    int *col = nullptr;        // [nnz]
    float *val = nullptr;      // [nnz]
    Chunk *chunks = nullptr;   // [n_chunks]
    SplitRow *split = nullptr; // [n_split_rows]
    int n_long_rows = 0;
    int n_chunks = 0;
    int n_split_rows = 0;
    int n_partials = 0;
    int max_nslots = 0;        // largest nslots over split rows
};

}  // namespace drone

struct drone_plan {
    int device = 0;
    int n_rows = 0;
    int nnz = 0;
    int short_row_limit = 0;   // rows with deg <= this are summed by one lane group
    int chunk_nnz = 0;         // nonzeros per chunk of longer rows
    drone::Side side[2];       // [DRONE_OP_A], [DRONE_OP_AT]
    // partial sums of split rows, [n_partials, F] floats, grown on demand
    float *scratch = nullptr;
    size_t scratch_bytes = 0;
    // device staging for drone_spmm_host
    float *stage_x = nullptr, *stage_y = nullptr;
    size_t stage_bytes = 0;
    cudaStream_t own_stream = nullptr;
};
