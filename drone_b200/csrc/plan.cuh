// Internal layout of an aggregation plan (opaque drone_plan of the C ABI).
#pragma once

#include "common.cuh"

namespace drone {

constexpr int kWideSlots = 64;              // split rows above this many partial slots are reduced by a whole block
constexpr int kShortRangeNnz = 64;          // stream entries per lane group (plus at most one more row)
constexpr unsigned kLastInRow = 0x80000000u; // flag on s_col: last entry of its row
constexpr unsigned kPlaceholder = 0x40000000u; // flag on s_col: row has no nonzeros, entry carries no data
constexpr unsigned kColMask = 0x3fffffffu;
// Plans of very large graphs tag their most often gathered columns (bit 29 on the entries of col and s_col): the
// remaining bits of a tagged entry are the column's position in the plan's table of hot rows instead of the column.
constexpr unsigned kHotTag = 0x20000000u;
constexpr unsigned kHotMask = 0x1fffffffu;
constexpr int kMaxRowClasses = 16;         // row classes a plan can be given (drone_plan_set_row_classes)

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
    int *col = nullptr;        // [nnz]; in a tagged plan the hot columns carry kHotTag | position
    float *val = nullptr;      // [nnz]
    // tagged plans only: hot_ids[pos] = column that position pos of the table of hot rows stands for, most often
    // gathered first; col_plain = untagged copy of col, made when a caller asks for the CSR arrays
    int *hot_ids = nullptr;    // [n_hot]
    int n_hot = 0;
    int *col_plain = nullptr;  // [nnz] or NULL
    Chunk *chunks = nullptr;   // [n_chunks]
    SplitRow *split = nullptr; // [n_split_rows]
    SplitRow *wide = nullptr;  // [n_wide_rows] the split rows with more than kWideSlots slots (any order)
    int n_wide_rows = 0;
    // Short rows (at most short_row_limit nonzeros) as one contiguous stream: their nonzeros copied
    // in row order, bit 31 of the column marking the last nonzero of a row.  A row without nonzeros
    // contributes one placeholder entry (bit 30) so that it is still written.  The stream is cut into
    // ranges of about kShortRangeNnz entries at row boundaries; range i starts at row s_range_row[i].
    int *s_rows = nullptr;      // [n_short_rows] row id of each short row
    int *s_rowptr = nullptr;    // [n_short_rows + 1] start of each short row in the stream
    int *s_col = nullptr;       // [n_short_entries] column | flags
    float *s_val = nullptr;     // [n_short_entries]
    int *s_range_row = nullptr; // [n_short_ranges + 1]
    int n_short_rows = 0;
    int n_short_entries = 0;
    int n_short_ranges = 0;
    int n_long_rows = 0;
    int n_chunks = 0;
    int n_split_rows = 0;
    int n_partials = 0;
    int max_nslots = 0;        // largest nslots over split rows
    // With row classes the four lists are class-major (all work of class 0 first, then class 1, ...; rows ascending
    // inside a class) and list x of class c is [x_start[c], x_start[c+1]).  Without classes everything is class 0.
    int n_classes = 1;
    int range_start[kMaxRowClasses + 1] = {0}, chunk_start[kMaxRowClasses + 1] = {0};
    int split_start[kMaxRowClasses + 1] = {0}, wide_start[kMaxRowClasses + 1] = {0};
};

}  // namespace drone

struct drone_plan;
namespace drone {
// drone_plan_create for users inside the library that read the plan's lists with kernels of their own (the
// PageRank pull): never tags columns.
int plan_create_untagged(drone_plan **out, int n_rows, int nnz, const int *d_index, const int *d_dst, const float *d_values,
                         const int *d_in_degree, const int *d_out_degree, int orientations, void *stream);
// Renumbers the columns of one orientation of an untagged plan by how often they occur, most frequent first (the
// frequencies are the row lengths of d_other_rowptr, the row pointer of the opposite orientation): afterwards column c of
// the plan's lists means position (*d_place_out)[c], a device array of n_rows ints the caller owns.  For users inside
// the library whose gathered operand is their own array and can be laid out in that order (the PageRank pull).
int plan_order_columns_by_frequency(drone_plan *p, int orientation, const int *d_other_rowptr, int **d_place_out, void *stream);
}  // namespace drone

struct drone_plan {
    int device = 0;
    int n_rows = 0;
    int nnz = 0;
    int short_row_limit = 0;   // rows with deg <= this are summed by one lane group
    int chunk_nnz = 0;         // nonzeros per chunk of longer rows
    int last_slice_width = 0;  // what the most recent call used (reported by drone_plan_get_stats)
    int slice_forced = -1;     // column-slice width of a call: -1 chosen per call, 0 never slice, w > 0 slices of w columns
    drone::Side side[2];       // [DRONE_OP_A], [DRONE_OP_AT]
    // partial sums of split rows, [n_partials, F] floats, grown on demand
    float *scratch = nullptr;
    size_t scratch_bytes = 0;
    // device staging for drone_spmm_host
    float *stage_x = nullptr, *stage_y = nullptr;
    size_t stage_bytes = 0;
    // row classes: rows in class-major order and where each class starts in that order (NULL / 1 class: none set)
    int *row_order = nullptr;  // [n_rows]
    int n_classes = 1;
    int class_start[drone::kMaxRowClasses + 1] = {0};
    // one word: the chunk kernel's work counter (set to 0 in front of every launch)
    unsigned *counter = nullptr;
    // tagged plans: the table of hot rows, refilled from X by every call
    float *hot_table = nullptr;
    size_t hot_table_bytes = 0;
    // Staging for operands whose rows cannot be read as float4 (a width that is not a multiple of 4, odd leading
    // dimensions or addresses): [pad_rows, pad_width] floats each, made by drone_plan_reserve on request.  When
    // present and large enough, such a call copies X into pad_x with rows padded to a multiple of 4 floats, runs the
    // float4 kernels on the padded copies and copies the result out of pad_y.
    float *pad_x = nullptr, *pad_y = nullptr;
    int pad_width = 0;
    int chunk_blocks_per_sm = 0;   // cap on resident blocks of the chunk kernel per SM (0: as many as fit)
    cudaStream_t own_stream = nullptr;
    // drone_spmm_host with pinned operands: second stream and one event per column half for the copy that runs ahead
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t half_loaded[2] = {nullptr, nullptr};
    // drone_spmm_host_submit / _wait: a second pair of staging buffers, a stream for the copies out, and per slot the
    // events "operand landed", "aggregation done", "result copied out"; `submitted` counts the calls queued so far
    float *queue_x[2] = {nullptr, nullptr}, *queue_y[2] = {nullptr, nullptr};
    size_t queue_bytes = 0;
    cudaStream_t out_stream = nullptr;
    cudaEvent_t queue_in[2] = {nullptr, nullptr}, queue_done[2] = {nullptr, nullptr}, queue_out[2] = {nullptr, nullptr};
    long long submitted = 0;
    // second stream and fork/join events: the short-row kernel runs beside the chunk kernels of the same call
    cudaStream_t side_stream = nullptr;
    cudaEvent_t fork_event = nullptr, join_event = nullptr;
};
