// Internal definition of the opaque cgnn_plan and the helpers shared between translation
// units (the public contract is include/cgnn_b200.h).
#pragma once
#include "cgnn_common.cuh"

struct cgnn_plan {
    int device = 0;
    int nterms = 1;
    int64_t rows = 0;
    int64_t nnz[2] = {0, 0};
    int32_t *rowptr[2] = {nullptr, nullptr};  // device int32[rows+1], owned
    int32_t *col[2] = {nullptr, nullptr};     // device int32[nnz], owned
    int split = 0;                            // longest row a single lane group owns
    int64_t n_long = 0;                       // rows longer than split
    int64_t n_items = 0;                      // chunks of long rows (one partial-sum slot each)
    int64_t n_direct = 0;                     // work units that are whole rows
    int4 *items = nullptr;                    // device {long row index, term, e0, e1}
    int4 *longs = nullptr;                    // device {row, first item, items, 0}
    int32_t *row_ids = nullptr;               // device compact list of short non-empty rows, or null
};

namespace cgnn {

// Takes ownership of p->rowptr[t] / p->col[t] (device int32 arrays, already filled on
// `stream`), reads the row pointers back, validates them and cuts the rows into work units.
int plan_analyze(cgnn_plan *p, int split, cudaStream_t stream);

// Device status word of the segment-reduce translation unit (read-and-clear).
int segreduce_status(int *out);
int gather_status(int *out);
int cluster_status(int *out);

}  // namespace cgnn
