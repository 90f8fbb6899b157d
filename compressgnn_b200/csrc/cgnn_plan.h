// Internal definition of the opaque cgnn_plan and the helpers shared between translation
// units (the public contract is include/cgnn_b200.h).
#pragma once
#include "cgnn_common.cuh"

// A plan owns a re-laid-out copy of the block's (or the two fused blocks') entries:
//   entries[0 .. direct_entries)        the entries of the short rows, row after row in the
//                                       order of the direct row list (a row's term-0 entries
//                                       first, then its term-1 entries);
//   entries[direct_entries .. total)    the entries of the long rows, cut into chunks.
// An entry is the 32-bit source row with the term in bit 31.  `vperm` records where each entry
// came from (index into the concatenation of the callers' two value arrays) so that values
// can be brought into the same order once.
struct cgnn_plan {
    int device = 0;
    int nterms = 1;
    int64_t rows = 0;
    int64_t nnz[2] = {0, 0};
    int64_t total = 0;             // nnz[0] + nnz[1]
    int32_t *entries = nullptr;    // device int32[total]
    int32_t *vperm = nullptr;      // device int32[total]
    int32_t *uptr = nullptr;       // device int32[n_direct + 1]: entry offset of each listed row
    int32_t *urow = nullptr;       // device int32[n_direct]: row id of each listed row, or null = identity
    int split = 0;                 // longest row kept in the direct list
    int64_t n_direct = 0;          // rows in the direct list
    int64_t n_long = 0;            // rows longer than split
    int64_t n_items = 0;           // chunks of long rows (one partial-sum slot each)
    int4 *items = nullptr;         // device {long row index, first entry, end entry, 0}
    int4 *longs = nullptr;         // device {row, first item, items, first entry of the row}
    int compact = 0;               // 1: empty rows are not listed (a fresh output is cleared first)
    int64_t degree_p50 = 0, degree_p99 = 0, degree_max = 0;  // row-length histogram the split was chosen from
    int64_t source_rows[2] = {0, 0};  // 1 + the largest source row each term refers to (0: no entries)
    void *block = nullptr;         // the one device allocation all arrays above live in
    cudaStream_t home = nullptr;   // stream the block was allocated on (stream-ordered allocator)
    bool pooled = false;           // block came from cudaMallocAsync
};

namespace cgnn {

// Build the plan's work lists and entry layout from device int32 CSR arrays of one or two
// blocks over the same rows (p->rows, p->nterms, p->nnz set by the caller).  The inputs are
// only read; synchronises `stream`.
// `host_rowptr0`, when given, is a host copy of rowptr[0] the caller already has (saves a
// device-to-host copy and a synchronisation); `want_vperm` = false skips the value permutation
// (plans whose entries carry no values).
int plan_build(cgnn_plan *p, const int32_t *const rowptr[2], const int32_t *const col[2], int split,
               cudaStream_t stream, const int32_t *host_rowptr0 = nullptr, bool want_vperm = true);

// The same plan built WITHOUT host loops, for blocks whose row pointers only exist on the device (the
// bucket plan of an assignment refresh), in two steps around the caller's one synchronisation:
//   plan_stats_on_device   (queued before the wait) reads the row count from device memory, takes the
//                          row-length histogram, chooses the chunk length and counts the work lists;
//                          the figures land in header[0 .. PLAN_HEADER_WORDS), which the caller copies
//                          to the host together with whatever else it waits for;
//   plan_fill_on_device    (after the wait, header on the host) allocates the plan and lets kernels
//                          write its lists and entries; no further wait, no host-side pass over the rows.
// Rows are limited to PLAN_DEVICE_MAX_ROWS (one CTA scans them); the block has no values.
constexpr int PLAN_HEADER_WORDS = 16;
constexpr int64_t PLAN_DEVICE_MAX_ROWS = 1 << 20;
enum PlanHeader { PH_ROWS = 0, PH_SPLIT, PH_COMPACT, PH_IDENTITY, PH_DIRECT, PH_LONG, PH_ITEMS, PH_P50, PH_P99,
                  PH_MAX, PH_SHORT_ENTRIES, PH_VALID };
int plan_stats_on_device(const int32_t *rowptr, const int32_t *last_row_dev, int64_t nnz, int split,
                         int32_t *header_dev, cudaStream_t stream);
int plan_fill_on_device(cgnn_plan *p, const int32_t *rowptr, const int32_t *col, const int32_t *header_host,
                        cudaStream_t stream);

// Device status word of each translation unit (read-and-clear).
int segreduce_status(int *out);
int gather_status(int *out);
int cluster_status(int *out);

}  // namespace cgnn
