/*
 * cgnn_b200 -- C ABI of the B200 (sm_100a) kernels behind CompressGNN's runtime operators.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, returns an int
 * status (0 = ok) and never throws, traps or blocks the device.  The message for the last
 * non-zero status of the calling thread is returned by cgnn_last_error().  Paths cited as
 * "ref:" are files of ZhengChenCS/CompressGNN whose operator the entry point replaces.
 *
 * dtype: CGNN_F32 or CGNN_F64 (the reference dispatches both, ref:
 * src/runtime/csrc/sparse/cuda/spmm_gpu.cu:37).  All matrices are dense row-major with
 * row stride == width.  Index arrays handed to plan constructors may be 4 or 8 bytes wide;
 * plans keep private 32-bit copies.
 */
#ifndef CGNN_B200_H
#define CGNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *cgnn_stream_t; /* a cudaStream_t */

enum { CGNN_OK = 0, CGNN_ERR_INVALID = 1, CGNN_ERR_CUDA = 2, CGNN_ERR_CAPACITY = 3 };
enum { CGNN_F32 = 0, CGNN_F64 = 1 };

int cgnn_version(void);
const char *cgnn_last_error(void);

/* OR of the status bits recorded by kernels since the last call (1 = an index outside its
 * range was met and skipped, 2 = a bounded wait ran out, 4 = malformed CSR); clears the
 * word.  Synchronises the device.  When bit 2 is set, the output of the launch that set it is
 * undefined (rows of the unit that gave up were not written); every launch still leaves the
 * plan's ticket words zero.  The reference traps the GPU on a bad index instead
 * (ref: src/runtime/csrc/cluster/cuda/cluster_kernel.cu:66,82,92,104). */
int cgnn_device_status(int *status_out);

/* ---------------------------------------------------------------------------------------
 * Segment plans.  A plan describes "rows that sum gathered source rows": a CSR block (or
 * two blocks over the same rows whose sums are fused), cut into work units by the row
 * degree histogram: rows up to `split` entries are owned by one lane group; longer rows
 * are cut into chunks of `split` entries whose partial sums are combined in chunk order
 * by the last chunk to finish (deterministic; no floating-point atomics).
 * ------------------------------------------------------------------------------------- */
typedef struct cgnn_plan cgnn_plan;

/* Build a plan from device CSR arrays (rowptr[rows+1], col[nnz]); term 1 may be absent
 * (rowptr1 == NULL).  split == 0 picks the chunk length from the degree histogram.
 * Allocates plan-owned device memory and synchronises `stream` (one-off, at graph load).
 * Replaces the per-call kernel choice of ref: layer/CompressgnnSPMM.py:14-19. */
int cgnn_plan_create(cgnn_plan **plan_out, int64_t rows, int index_bytes,
                     const void *rowptr0, const void *col0, int64_t nnz0,
                     const void *rowptr1, const void *col1, int64_t nnz1,
                     int split, cgnn_stream_t stream);

/* Build a plan that groups the positions of index[n] (values in [0, groups)) by value,
 * positions ascending inside a group: the segments the mean / reconstruct-backward
 * reductions run over.  Sorts on the device; synchronises `stream`. */
int cgnn_plan_create_from_index(cgnn_plan **plan_out, const int64_t *index, int64_t n,
                                int64_t groups, int split, cgnn_stream_t stream);

/* Plan memory is released in the order of the stream the plan was created on; do not destroy
 * a plan while a launch that uses it may still run on a different stream. */
void cgnn_plan_destroy(cgnn_plan *plan);

/* info[0..7] = rows, entries (both terms), split, long rows, chunks, rows in the direct
 * list, terms, 1 if empty rows are left out of the list. */
int cgnn_plan_info(const cgnn_plan *plan, int64_t info[8]);

/* out[0..3] = median, 99th percentile and maximum of the row lengths (entries per output row, both
 * blocks together; the percentiles saturate at 4096) and the chunk length chosen from them: rows
 * longer than the chunk length are cut into chunks that run as work units of their own.
 * (The reference picks its kernel from nnz and the width alone, layer/CompressgnnSPMM.py:14-19.) */
int cgnn_plan_degrees(const cgnn_plan *plan, int64_t out[4]);

/* rows[t] = 1 + the largest source row that block t of the plan refers to (0 when the block has
 * no entries).  The SpMM entry points take raw pointers and cannot see how many rows `src`
 * has: a caller passes only matrices with at least this many rows.  (The reference's kernels
 * index `mat` with elist unchecked, src/runtime/csrc/sparse/cuda/row_balance.cuh:82-128.) */
int cgnn_plan_source_rows(const cgnn_plan *plan, int64_t rows[2]);

/* A plan keeps its entries in its own order (short rows back to back, then the chunks of
 * long rows; for two blocks a row's entries of block 0 precede those of block 1).  This
 * brings the caller's value arrays (val0[nnz0], val1[nnz1] or NULL) into that order:
 * out[nnz0+nnz1].  Done once per graph; cgnn_spmm / cgnn_spmm_pair take the result. */
int cgnn_plan_permute_values(const cgnn_plan *plan, int dtype, const void *val0,
                             const void *val1, void *out, cgnn_stream_t stream);

/* Bytes of caller-provided scratch a launch over `width` columns needs.  The first
 * cgnn_plan_ticket_bytes() bytes hold chunk tickets: they must be zero before the first
 * launch and are left zero by every launch, so one zero-initialised buffer can serve any
 * number of plans as long as their launches do not overlap on the device. */
size_t cgnn_plan_scratch_bytes(const cgnn_plan *plan, int64_t width, int dtype);
size_t cgnn_plan_ticket_bytes(const cgnn_plan *plan, int64_t width, int dtype);

/* ---------------------------------------------------------------------------------------
 * SpMM:  out[r,:] (+)= sum_e val[e] * src[col[e],:]
 * ref: spmm_func, src/runtime/csrc/sparse/spmm.cpp:11-23 and
 *      src/runtime/csrc/sparse/cuda/spmm_gpu.cu:8-107 (all six kernel variants).
 * val holds the entry values IN PLAN ORDER (cgnn_plan_permute_values) or is NULL (all
 * ones).  accumulate != 0 adds to the existing out (the reference's
 * optional_out contract); out may alias src when the rows written are never read (the
 * in-place rule-level updates of ref: layer/CompressgnnSPMM.py:57-58).
 * ------------------------------------------------------------------------------------- */
int cgnn_spmm(const cgnn_plan *plan, int dtype, int64_t width, const void *val,
              const void *src, void *out, int accumulate, void *scratch,
              size_t scratch_bytes, cgnn_stream_t stream);

/* cgnn_spmm for callers that cannot allocate.  (No counterpart in the reference, whose
 * operators allocate through torch on every call.)
 *
 * Some hosts cannot hand cgnn_spmm a scratch buffer because they cannot create one when the
 * call is made: a serving process that gave the whole GPU to its own memory pool at start-up,
 * so that any further cudaMalloc fails; or a latency-critical loop that must never run into
 * the device-wide synchronisation cudaMalloc and cudaFree can cause.  For them the library
 * carries its own scratch: CGNN_STATIC_SCRATCH_BYTES of device memory inside the library
 * image, held by every GPU that loads the library until the process exits.
 *
 * Same result as cgnn_spmm (bit for bit).  The call allocates nothing -- no cudaMalloc,
 * cudaFree or allocating library routine.  Limits and rules:
 *   - a plan is accepted when cgnn_plan_ticket_bytes(plan, width, dtype) + chunks * width *
 *     sizeof(element) <= CGNN_STATIC_SCRATCH_BYTES, with chunks = info[4] of cgnn_plan_info;
 *     anything larger is rejected with CGNN_ERR_INVALID and a message.  (cgnn_plan_scratch_bytes
 *     is an upper bound of that sum: it also counts alignment padding and the bias-gradient
 *     stage this entry point does not use);
 *   - the buffer is shared by every call on a device and keeps the previous call's contents;
 *     each call clears the ticket words it needs itself, but two calls that overlap on the
 *     GPU (different streams, no dependency) race on it -- order them;
 *   - the first call on each device looks up the buffer's address with that device current;
 *     make that first call outside of any stream capture;
 *   - the plan must have been created on the current device. */
#define CGNN_STATIC_SCRATCH_BYTES (8u << 20)
int cgnn_spmm_static_scratch(const cgnn_plan *plan, int dtype, int64_t width, const void *val,
                             const void *src, void *out, int accumulate, cgnn_stream_t stream);

/* Two blocks over the same output rows in one pass:
 *   out[r,:] (+)= sum_e val0[e]*src0[col0[e],:] + sum_e val1[e]*src1[col1[e],:]
 * (the plan must have been built with two terms; val = both value arrays in plan order).
 * Fastest when src1 starts a whole number of rows (width elements) away from src0, which a
 * caller that allocates one of the two can arrange; any other placement works, slower.  Fuses the last two calls of the
 * reference's forward (v2r then v2v, ref: layer/CompressgnnSPMM.py:59-60) and of its
 * backward (:84-85) so that out is written once. */
int cgnn_spmm_pair(const cgnn_plan *plan, int dtype, int64_t width, const void *val,
                   const void *src0, const void *src1, void *out, int accumulate,
                   void *scratch, size_t scratch_bytes, cgnn_stream_t stream);

/* One direction of the compressed propagation in ONE call: the launch sequence of the reference's
 * Compressgnn_SPMM_Function (ref: layer/CompressgnnSPMM.py:47-60 forward, :65-85 backward), issued
 * back to back on `stream` without returning to the host language in between.
 *   launch 0            rule_out  = A[0] x                      (rules gather vertices: r2v, or v2r^T)
 *   launch 1 .. n-2     rule_out += A[i] rule_out               (the rule levels, in place)
 *   launch n-1          out       = pair(A[n-1]) (s0, s1)       (the fused two-block vertex pass)
 * where (s0, s1) = (rule_out, x) when rule_term_of_last is 0 (forward: v2r | v2v) and (x, rule_out)
 * when it is 1 (backward: v2v^T | r2v^T).  plans[i] / vals[i] (values in plan order, or NULL for
 * ones) / scratch[i] / scratch_bytes[i] describe launch i as for cgnn_spmm and cgnn_spmm_pair.
 * Only the launches first <= i <= last are issued, so that a caller can time one of them between
 * two calls.  The host language pays its call overhead once per pass instead of once per block: with
 * the feature columns sharded over several GPUs a block's kernel takes 15-80 us, less than an
 * interpreter needs to issue it. */
int cgnn_propagate(int n_launches, const cgnn_plan *const *plans, const void *const *vals,
                   void *const *scratch, const size_t *scratch_bytes, int dtype, int64_t width,
                   const void *x, void *rule_out, void *out, int rule_term_of_last, int first,
                   int last, cgnn_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * LSH cluster assignment.
 * ref: cluster_assign_cuda, src/runtime/csrc/cluster/cuda/cluster_kernel.cu:118-153;
 *      CPU LSH, src/runtime/csrc/cluster/cpu/cluster_cpu.cpp:27-70.
 * ------------------------------------------------------------------------------------- */

/* proj[n,bits] = x[n,width] . planes[width,bits], each entry accumulated as
 * p = fma(x[r,k], planes[k,h], p) for k ascending from p = +0 (the documented order the
 * CPU oracle restates).  Used alone by the column-sharded path, whose partial
 * projections are summed across GPUs before sign packing. */
int cgnn_cluster_project(int dtype, const void *x, const void *planes, int64_t n,
                         int64_t width, int bits, void *proj, cgnn_stream_t stream);

/* codes[r] = sign bits of proj[r,:], MSB first, bit = (p > 0)  (ref: hash_ids,
 * cluster_kernel.cu:41-50). */
int cgnn_cluster_codes_from_projection(int dtype, const void *proj, int64_t n, int bits,
                                       int32_t *codes, cgnn_stream_t stream);

/* Fused projection + sign packing; the n x bits projection never reaches memory. */
int cgnn_cluster_codes(int dtype, const void *x, const void *planes, int64_t n,
                       int64_t width, int bits, int32_t *codes, cgnn_stream_t stream);

/* Bytes of workspace cgnn_cluster_assign needs for n rows. */
size_t cgnn_cluster_workspace_bytes(int64_t n, int bits);

/* Compact the raw codes: ids[r] in 1..active ascend with the raw code; returns `active`
 * through *active_out after one stream synchronisation (the reference's single .item(),
 * cluster_kernel.cu:147).  The workspace afterwards holds the per-bucket counts and the
 * bucket permutation; read them with cgnn_cluster_assign_export. */
int cgnn_cluster_assign(const int32_t *codes, int64_t n, int bits, void *workspace,
                        size_t workspace_bytes, int64_t *ids, int64_t *active_out,
                        cgnn_stream_t stream);

/* counts[active+1] (counts[0] == 0, ref: tests/test_transformation.py:39) and a plan
 * over the buckets (rows = active+1) built from the permutation already in the workspace. */
int cgnn_cluster_assign_export(const void *workspace, int64_t n, int64_t active,
                               int32_t *counts, cgnn_plan **plan_out, int split,
                               cgnn_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Mean representatives and reconstruction.
 * ------------------------------------------------------------------------------------- */

/* out[g,:] = sum_{index[r]==g} x[r,:] / max(count[g],1); plan from
 * cgnn_cluster_assign_export or cgnn_plan_create_from_index.
 * ref: cluster_mean_cuda, cluster_kernel.cu:158-170 (float atomics there). */
int cgnn_cluster_mean(const cgnn_plan *plan, int dtype, int64_t width, const void *x,
                      const int32_t *count, void *out, void *scratch, size_t scratch_bytes,
                      cgnn_stream_t stream);

/* out[r,:] = grad[index[r],:] / max(count[index[r]],1)
 * ref: cluster_mean_backward_cuda, cluster_kernel.cu:171-181.
 * `scaled` is optional scratch of groups*width elements: when given, the division is done
 * once per group row into it and the node rows are a pure gather (same bits, far fewer
 * divisions); when NULL every output element is divided on the fly. */
int cgnn_cluster_mean_backward(int dtype, int64_t n, int64_t width, int64_t groups,
                               const void *grad, const int64_t *index, const int32_t *count,
                               void *out, void *scaled, cgnn_stream_t stream);

/* out[r,:] = act(reps[index[r],:] + bias[:]); bias may be NULL; relu: v < 0 ? 0 : v.
 * ref: cluster_reconstruct_cuda, cluster_kernel.cu:182-195. */
int cgnn_cluster_reconstruct(int dtype, int64_t n, int64_t width, int64_t groups,
                             const void *reps, const int64_t *index, const void *bias,
                             int relu, void *out, cgnn_stream_t stream);

/* The hidden-layer epilogue of the reference's model in one pass:
 *   out[r,:] = dropout_p(relu(reps[index[r],:] + bias))
 * (ref: model/compressgnn/gcn.py:54-61 applies F.relu and F.dropout to the reconstructed [N,F]
 * matrix as two further elementwise passes.)  An element is dropped with probability drop_p, the
 * others are scaled by 1/(1-drop_p); element e of `out` takes word e % 4 of the Philox4x32 block
 * counted e / 4 under the key `seed`, so the mask depends on (seed, element index) only.  The
 * backward pass needs no mask tensor: with ReLU in front, a dropped element and a clamped one both
 * read 0 in `out`, which cgnn_cluster_reconstruct_backward's exact-mask mode (relu = 1) turns into
 * a zero gradient; the caller multiplies the result by 1/(1-drop_p). */
int cgnn_cluster_reconstruct_dropout(int dtype, int64_t n, int64_t width, int64_t groups,
                                     const void *reps, const int64_t *index, const void *bias,
                                     double drop_p, uint64_t seed, void *out, cgnn_stream_t stream);

/* d_reps[g,:] = sum_{index[r]==g} (relu && output[r,:] <= 0 ? 0 : grad[r,:]);
 * relu: 0 = no mask; 1 = mask read per node row from `output` (the reference's semantics for
 * any `output`); 2 = `output` is known to be the forward result of cgnn_cluster_reconstruct,
 * whose rows are identical inside a group, so one output row per group is read and the
 * group sum is masked once -- half the memory traffic, same result.
 * bias_grad (optional, [width]) = column sums of d_reps, the value the reference derives
 * in Python (ref: layer/CompressgnnReconstruct.py:26).
 * ref: cluster_reconstruct_backward_cuda, cluster_kernel.cu:196-208 (float atomics there). */
int cgnn_cluster_reconstruct_backward(const cgnn_plan *plan, int dtype, int64_t width,
                                      const void *grad, const void *output, int relu,
                                      void *d_reps, void *bias_grad, void *scratch,
                                      size_t scratch_bytes, cgnn_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Grammar compression of a CSR graph on the device (graph preparation, once per graph).
 * ref: compress_csr_batch of the module compressgnn_batch_cuda, src/offline/bindings/batch_cuda.cpp:3-9,
 * selected by loader/compression_backend.py:6-40.  The compressor behind that binding is an external
 * project; the contract the reference's tests hold it to (tests/test_batch_compression.py:15-59) is:
 * int32 arrays, rows n.. are rule bodies made of smaller symbols, every vertex row expands to its
 * input row in order, and the CUDA result equals the CPU result.  Here the CPU result is this
 * package's host compressor (rounds of digram substitution), and the device code reproduces its
 * arrays exactly.
 *
 * vlist [n+1] and elist [vlist[n]] are DEVICE arrays of int64; values of elist must lie in [0, n)
 * and n + vlist[n] must stay below 2^31 (CGNN_ERR_INVALID otherwise).  The call synchronises
 * `stream` a few times per round and allocates its work arrays with cudaMalloc (about 60 bytes per
 * input edge, released before it returns).  The result holds
 *   vlist int32 [n + rules + 1], elist int32 [entries]   (device memory)
 * cgnn_compressed_info: info = {n, rules, entries}.  cgnn_compressed_copy copies both arrays to
 * host or device buffers of those sizes on `stream` (asynchronously: synchronise before reading). */
typedef struct cgnn_compressed cgnn_compressed;
int cgnn_compress_csr_batch(const int64_t *vlist, const int64_t *elist, int64_t n, int rounds,
                            int min_frequency, cgnn_compressed **out, cgnn_stream_t stream);
int cgnn_compressed_info(const cgnn_compressed *c, int64_t info[3]);
int cgnn_compressed_copy(const cgnn_compressed *c, int32_t *vlist_out, int32_t *elist_out,
                         cgnn_stream_t stream);
void cgnn_compressed_destroy(cgnn_compressed *c);

/* ---------------------------------------------------------------------------------------
 * Neighbour sampling on the compressed graph, one hop at a time.
 * ref: neighbor_sample_sim_impl, src/sample/csrc/neighbor_sample.h:27-131 (a host function there, bound
 * as compressgnn_sample.neighbor_sample_cg_sim); get_neighbor / get_neighbor_list,
 * src/sample/csrc/storage_api.h:7-118.  Same result contract: `samples` (seeds first, then new nodes in
 * the order they are first seen), and per sampled edge the local id of the frontier node and of the
 * neighbour.  The random neighbour indices come from a counter-based generator under `seed`.
 *
 * All arrays are device arrays.  The graph is given by the CSR blocks CompressGraph holds (int64), with
 * the rule -> rule levels merged into one CSR, and the two degree arrays of gen_degree.
 * A hop over the frontier samples[begin, begin + frontier):
 *   cgnn_sample_count   count[i] = min(fanout, degree)  (degree when fanout >= degree)
 *   (caller: offset = exclusive scan of count, total = its sum)
 *   cgnn_sample_pick    picked[offset[i]..] = the neighbours, source[..] = begin + i; scratch: total int64
 *   cgnn_sample_claim   first[] / is_new[]: which pick introduces a vertex that has no local id yet
 *   (caller: rank = exclusive scan of is_new, new = its sum; samples must have room for end + new)
 *   cgnn_sample_relabel target[p] = local id of picked[p]; appends the new vertices to samples from `end`;
 *                       records their ids in local_of and restores first[] to INT32_MAX
 * local_of and first are int32[vertices], filled with INT32_MAX before the first hop;
 * cgnn_sample_seed enters the seeds (samples[0, count)) into local_of.  A vertex outside [0, vertices)
 * or a degree table that does not match the graph sets bits 1 / 4 of cgnn_device_status; nothing traps. */
typedef struct {
    const int64_t *v2v_ptr, *v2v_col;   /* [vertices + 1], direct neighbours */
    const int64_t *v2r_ptr, *v2r_col;   /* [vertices + 1], rules a vertex lists */
    const int64_t *r2v_ptr, *r2v_col;   /* [rules + 1], vertices a rule lists itself */
    const int64_t *r2r_ptr, *r2r_col;   /* [rules + 1], rules a rule lists (all levels merged) */
    const int64_t *vertex_degree, *rule_degree;
    int64_t vertices, rules;
} cgnn_sample_graph;
int cgnn_sample_seed(const int64_t *samples, int64_t count, int64_t vertices, int32_t *local_of,
                     cgnn_stream_t stream);
int cgnn_sample_count(const cgnn_sample_graph *graph, const int64_t *samples, int64_t begin,
                      int64_t frontier, int64_t fanout, int64_t *count, cgnn_stream_t stream);
int cgnn_sample_pick(const cgnn_sample_graph *graph, const int64_t *samples, int64_t begin,
                     int64_t frontier, int64_t fanout, const int64_t *count, const int64_t *offset,
                     uint32_t hop, uint64_t seed, int64_t *picked, int64_t *source, int64_t *scratch,
                     cgnn_stream_t stream);
int cgnn_sample_claim(const int64_t *picked, int64_t total, int64_t vertices, const int32_t *local_of,
                      int32_t *first, int64_t *is_new, cgnn_stream_t stream);
int cgnn_sample_relabel(const int64_t *picked, int64_t total, int64_t vertices, const int64_t *is_new,
                        const int64_t *rank, int64_t end, int32_t *local_of, int32_t *first,
                        int64_t *target, int64_t *samples, cgnn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CGNN_B200_H */
