// Segment reduce: out[r,:] (+)= sum over the entries of row r of  val[e] * src[col[e],:].
//
// One kernel serves the compressed-propagation SpMM blocks, the fused two-block pass, the
// per-bucket mean and the reconstruct backward.  Design points (B200, HBM-bound):
//   * a row is owned by a group of LPR lanes; every lane keeps VPL 16-byte vectors of the
//     row in registers, so one gathered feature row is LPR*VPL coalesced 128-bit loads;
//   * the group reads LPR (col,val) pairs with one coalesced load and broadcasts them by
//     shuffle; U gathered rows are in flight per lane before the FMAs are issued;
//   * rows longer than `split` are cut into chunks (work units of their own); a chunk
//     writes its partial sum to scratch, takes a ticket, and the chunk that draws the last
//     ticket adds the partials in chunk order -- deterministic, no float atomics, and no
//     unit ever waits for another.
#include <algorithm>
#include <vector>

#include "cgnn_plan.h"

namespace cgnn {

static __device__ int g_seg_status = 0;

int segreduce_status(int *out) {
    int zero = 0;
    CGNN_CUDA(cudaMemcpyFromSymbol(out, g_seg_status, sizeof(int)));
    CGNN_CUDA(cudaMemcpyToSymbol(g_seg_status, &zero, sizeof(int)));
    return CGNN_OK;
}

template <typename T>
struct SegArgs {
    const int32_t *rowptr[2];
    const int32_t *col[2];
    const T *val[2];
    const T *src[2];
    int nterms;
    const T *mask_src;          // MASKED: entries whose mask_src value is <= 0 contribute 0
    const int32_t *div_counts;  // optional: divide the row by max(div_counts[row], 1)
    T *out;
    int accumulate;
    int64_t width;
    const int32_t *row_ids;
    int64_t n_direct;
    int split;
    const int4 *items;
    int64_t n_items;
    const int4 *longs;
    T *partial;
    int *tickets;
};

template <typename T, int VW, int LPR, int VPL, int U, bool MASKED>
__device__ __forceinline__ void gather_edges(Vec<T, VW> (&acc)[VPL], const int32_t *col,
                                             const T *val, const T *src, const T *mask,
                                             int64_t width, int64_t colbase,
                                             const bool (&colok)[VPL], int e0, int e1, int gl,
                                             unsigned gmask) {
    using V = Vec<T, VW>;
    for (int base = e0; base < e1; base += LPR) {
        const int mine = base + gl;
        int c = 0;
        T v = T(0);
        if (mine < e1) {
            c = col[mine];
            v = val ? val[mine] : T(1);
        }
        const int cnt = min(LPR, e1 - base);
        for (int j = 0; j < cnt; j += U) {
            V x[U][VPL];
            T w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int cj = __shfl_sync(gmask, c, j + u, LPR);
                w[u] = __shfl_sync(gmask, v, j + u, LPR);
                if (j + u < cnt) {
                    const int64_t off = (int64_t)cj * width + colbase;
#pragma unroll
                    for (int p = 0; p < VPL; ++p) {
                        if (colok[p]) {
                            x[u][p] = vec_load<T, VW>(src + off + p * (LPR * VW));
                            if constexpr (MASKED) {
                                const V m = vec_load<T, VW>(mask + off + p * (LPR * VW));
#pragma unroll
                                for (int i = 0; i < VW; ++i)
                                    if (m.v[i] <= T(0)) x[u][p].v[i] = T(0);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (j + u < cnt) {
#pragma unroll
                    for (int p = 0; p < VPL; ++p) {
                        if (colok[p]) {
#pragma unroll
                            for (int i = 0; i < VW; ++i)
                                acc[p].v[i] = fma(x[u][p].v[i], w[u], acc[p].v[i]);
                        }
                    }
                }
            }
        }
    }
}

template <typename T, int VW, int LPR, int VPL, bool MASKED>
__global__ void __launch_bounds__(256) seg_kernel(const SegArgs<T> a) {
    using V = Vec<T, VW>;
    constexpr int GPW = 32 / LPR;
    constexpr int U0 = VPL >= 8 ? 1 : 8 / VPL;
    constexpr int U = U0 < LPR ? U0 : LPR;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (LPR - 1);
    const unsigned gmask =
        LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (lane & ~(LPR - 1)));
    const int64_t g =
        ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * GPW + lane / LPR;
    const int64_t width = a.width;
    const int64_t colbase = (int64_t)blockIdx.y * (LPR * VPL * VW) + gl * VW;
    bool colok[VPL];
    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) {
        colok[p] = colbase + p * (LPR * VW) < width;
        acc[p] = vec_zero<T, VW>();
    }

    int32_t row;
    if (g < a.n_direct) {
        row = a.row_ids ? a.row_ids[g] : (int32_t)g;
        const int a0 = a.rowptr[0][row], a1 = a.rowptr[0][row + 1];
        int b0 = 0, b1 = 0;
        if (a.nterms > 1) {
            b0 = a.rowptr[1][row];
            b1 = a.rowptr[1][row + 1];
        }
        if ((a1 - a0) + (b1 - b0) > a.split) return;  // cut into chunks; see below
        gather_edges<T, VW, LPR, VPL, U, MASKED>(acc, a.col[0], a.val[0], a.src[0], a.mask_src,
                                                 width, colbase, colok, a0, a1, gl, gmask);
        if (a.nterms > 1)
            gather_edges<T, VW, LPR, VPL, U, MASKED>(acc, a.col[1], a.val[1], a.src[1],
                                                     a.mask_src, width, colbase, colok, b0, b1,
                                                     gl, gmask);
    } else {
        const int64_t it = g - a.n_direct;
        if (it >= a.n_items) return;
        const int4 item = a.items[it];
        const int t = item.y;
        gather_edges<T, VW, LPR, VPL, U, MASKED>(acc, a.col[t], a.val[t], a.src[t], a.mask_src,
                                                 width, colbase, colok, item.z, item.w, gl,
                                                 gmask);
        const int4 lr = a.longs[item.x];
        T *part = a.partial + it * width + colbase;
#pragma unroll
        for (int p = 0; p < VPL; ++p)
            if (colok[p]) vec_store<T, VW>(part + p * (LPR * VW), acc[p]);
        __threadfence();
        __syncwarp(gmask);
        int *tk = a.tickets + (int64_t)item.x * gridDim.y + blockIdx.y;
        int ticket = 0;
        if (gl == 0) ticket = atomicAdd(tk, 1);
        ticket = __shfl_sync(gmask, ticket, 0, LPR);
        if (ticket != lr.z - 1) return;
        // Last chunk of this row (for this column tile): add the partials in chunk order.
        __threadfence();
#pragma unroll
        for (int p = 0; p < VPL; ++p) acc[p] = vec_zero<T, VW>();
        for (int s = 0; s < lr.z; ++s) {
            const T *ps = a.partial + (int64_t)(lr.y + s) * width + colbase;
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                if (colok[p]) {
                    const V q = vec_load_cg<T, VW>(ps + p * (LPR * VW));
#pragma unroll
                    for (int i = 0; i < VW; ++i) acc[p].v[i] += q.v[i];
                }
            }
        }
        if (gl == 0) *tk = 0;  // leave the ticket ready for the next launch
        row = lr.x;
    }

    T *orow = a.out + (int64_t)row * width + colbase;
    T divisor = T(1);
    const bool divide = a.div_counts != nullptr;
    if (divide) divisor = (T)max(a.div_counts[row], 1);
#pragma unroll
    for (int p = 0; p < VPL; ++p) {
        if (colok[p]) {
            V r = acc[p];
            if (a.accumulate) {
                const V o = vec_load<T, VW>(orow + p * (LPR * VW));
#pragma unroll
                for (int i = 0; i < VW; ++i) r.v[i] = o.v[i] + r.v[i];
            }
            if (divide) {
#pragma unroll
                for (int i = 0; i < VW; ++i) r.v[i] = r.v[i] / divisor;
            }
            vec_store<T, VW>(orow + p * (LPR * VW), r);
        }
    }
}

template <typename T, int VW, int LPR, int VPL, bool MASKED>
static int launch_cfg(const SegArgs<T> &a, cudaStream_t stream) {
    const int64_t groups = a.n_direct + a.n_items;
    const int64_t per_block = 8 * (32 / LPR);
    const int64_t gx = ceil_div(groups, per_block);
    const int64_t gy = ceil_div(a.width, (int64_t)LPR * VPL * VW);
    CGNN_REQUIRE(gx < (1ll << 31) && gy < 65536, "segment reduce: grid too large");
    seg_kernel<T, VW, LPR, VPL, MASKED><<<dim3((unsigned)gx, (unsigned)gy), 256, 0, stream>>>(a);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

template <typename T, int VW, bool MASKED>
static int launch_vw(const SegArgs<T> &a, cudaStream_t stream) {
    const int64_t vecs = a.width / VW;
    if (vecs <= 4) return launch_cfg<T, VW, 4, 1, MASKED>(a, stream);
    if (vecs <= 8) return launch_cfg<T, VW, 8, 1, MASKED>(a, stream);
    if (vecs <= 16) return launch_cfg<T, VW, 16, 1, MASKED>(a, stream);
    if (vecs <= 32) return launch_cfg<T, VW, 32, 1, MASKED>(a, stream);
    if (vecs <= 64) return launch_cfg<T, VW, 32, 2, MASKED>(a, stream);
    if (vecs <= 128) return launch_cfg<T, VW, 32, 4, MASKED>(a, stream);
    return launch_cfg<T, VW, 32, 8, MASKED>(a, stream);
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Tickets are kept per (long row, column tile).  The scalar path has the narrowest tiles
// (256 columns), so this bounds gridDim.y of every configuration launch_vw can pick.
static int64_t ticket_tiles(int64_t width) { return std::max<int64_t>(1, ceil_div(width, 256)); }

template <typename T>
static int run_typed(const cgnn_plan *p, int64_t width, const T *val0, const T *src0,
                     const T *val1, const T *src1, const T *mask, const int32_t *div_counts,
                     T *out, int accumulate, void *scratch, size_t scratch_bytes,
                     cudaStream_t stream) {
    constexpr int VWMAX = 16 / (int)sizeof(T);
    if (p->rows == 0 || width == 0) return CGNN_OK;
    SegArgs<T> a;
    for (int t = 0; t < 2; ++t) {
        a.rowptr[t] = p->rowptr[t];
        a.col[t] = p->col[t];
    }
    a.val[0] = val0; a.val[1] = val1;
    a.src[0] = src0; a.src[1] = src1;
    a.nterms = p->nterms;
    a.mask_src = mask;
    a.div_counts = div_counts;
    a.out = out;
    a.accumulate = accumulate;
    a.width = width;
    a.row_ids = p->row_ids;
    a.n_direct = p->n_direct;
    a.split = p->split;
    a.items = p->items;
    a.n_items = p->n_items;
    a.longs = p->longs;

    const bool vec = width % VWMAX == 0 && aligned16(src0) && aligned16(src1) &&
                     aligned16(mask) && aligned16(out);
    const size_t ticket_bytes =
        align_up((size_t)p->n_long * (size_t)ticket_tiles(width) * sizeof(int), 256);
    const size_t need = ticket_bytes + (size_t)p->n_items * (size_t)width * sizeof(T);
    if (p->n_items > 0) {
        CGNN_REQUIRE(scratch != nullptr && scratch_bytes >= need,
                     "segment reduce: scratch of %zu bytes needed, %zu given", need,
                     scratch_bytes);
        CGNN_REQUIRE(aligned16(scratch), "segment reduce: scratch must be 16-byte aligned");
    }
    a.tickets = reinterpret_cast<int *>(scratch);
    a.partial = reinterpret_cast<T *>(reinterpret_cast<char *>(scratch) + ticket_bytes);

    // A compact row list skips empty rows, so a fresh result has to be cleared first.
    if (!accumulate && p->row_ids)
        CGNN_CUDA(cudaMemsetAsync(out, 0, (size_t)p->rows * (size_t)width * sizeof(T), stream));
    if (p->n_direct + p->n_items == 0) return CGNN_OK;
    if (vec) {
        if (mask) return launch_vw<T, VWMAX, true>(a, stream);
        return launch_vw<T, VWMAX, false>(a, stream);
    }
    if (mask) return launch_vw<T, 1, true>(a, stream);
    return launch_vw<T, 1, false>(a, stream);
}

static int run(const cgnn_plan *p, int dtype, int64_t width, const void *val0, const void *src0,
               const void *val1, const void *src1, const void *mask,
               const int32_t *div_counts, void *out, int accumulate, void *scratch,
               size_t scratch_bytes, cudaStream_t stream) {
    CGNN_REQUIRE(p != nullptr, "segment reduce: null plan");
    CGNN_REQUIRE(width >= 0, "segment reduce: negative width");
    CGNN_REQUIRE(dtype == CGNN_F32 || dtype == CGNN_F64, "segment reduce: unknown dtype %d", dtype);
    if (p->rows > 0 && width > 0) {
        CGNN_REQUIRE(out != nullptr, "segment reduce: null output");
        CGNN_REQUIRE(src0 != nullptr || p->nnz[0] == 0, "segment reduce: null source");
        CGNN_REQUIRE(p->nterms == 1 || src1 != nullptr || p->nnz[1] == 0,
                     "segment reduce: null second source");
    }
    if (dtype == CGNN_F32)
        return run_typed<float>(p, width, (const float *)val0, (const float *)src0,
                                (const float *)val1, (const float *)src1, (const float *)mask,
                                div_counts, (float *)out, accumulate, scratch, scratch_bytes,
                                stream);
    return run_typed<double>(p, width, (const double *)val0, (const double *)src0,
                             (const double *)val1, (const double *)src1, (const double *)mask,
                             div_counts, (double *)out, accumulate, scratch, scratch_bytes,
                             stream);
}

// ---------------------------------------------------------------------------------------
// Column sums of a small [rows, width] matrix in two fixed-order stages (bias gradient).
// ---------------------------------------------------------------------------------------
constexpr int COLSUM_ROWS = 64;

template <typename T>
__global__ void colsum_stage1(const T *x, int64_t rows, int64_t width, T *part) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int64_t r0 = (int64_t)blockIdx.y * COLSUM_ROWS;
    const int64_t r1 = min(rows, r0 + COLSUM_ROWS);
    T s = T(0);
    for (int64_t r = r0; r < r1; ++r) s += x[r * width + c];
    part[(int64_t)blockIdx.y * width + c] = s;
}

template <typename T>
__global__ void colsum_stage2(const T *part, int64_t blocks, int64_t width, T *out) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    T s = T(0);
    for (int64_t b = 0; b < blocks; ++b) s += part[b * width + c];
    out[c] = s;
}

template <typename T>
static int colsum(const T *x, int64_t rows, int64_t width, T *part, T *out, cudaStream_t stream) {
    if (width == 0) return CGNN_OK;
    const int64_t blocks = ceil_div(rows, COLSUM_ROWS);
    if (blocks == 0) {
        CGNN_CUDA(cudaMemsetAsync(out, 0, (size_t)width * sizeof(T), stream));
        return CGNN_OK;
    }
    CGNN_REQUIRE(blocks < 65536, "column sum: too many rows");
    colsum_stage1<T><<<dim3((unsigned)ceil_div(width, 128), (unsigned)blocks), 128, 0, stream>>>(
        x, rows, width, part);
    CGNN_LAUNCH_CHECK();
    colsum_stage2<T><<<(unsigned)ceil_div(width, 128), 128, 0, stream>>>(part, blocks, width, out);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

// ---------------------------------------------------------------------------------------
// Plan analysis (host side, once per graph block or per assignment refresh).
// ---------------------------------------------------------------------------------------
int plan_analyze(cgnn_plan *p, int split, cudaStream_t stream) {
    const int64_t rows = p->rows;
    std::vector<int32_t> h[2];
    for (int t = 0; t < p->nterms; ++t) {
        h[t].resize((size_t)rows + 1);
        CGNN_CUDA(cudaMemcpyAsync(h[t].data(), p->rowptr[t], sizeof(int32_t) * ((size_t)rows + 1),
                                  cudaMemcpyDeviceToHost, stream));
    }
    CGNN_CUDA(cudaStreamSynchronize(stream));
    for (int t = 0; t < p->nterms; ++t) {
        CGNN_REQUIRE(h[t][0] == 0, "plan: rowptr[0] must be 0 (term %d)", t);
        for (int64_t r = 0; r < rows; ++r)
            CGNN_REQUIRE(h[t][r + 1] >= h[t][r], "plan: rowptr not monotone at row %lld (term %d)",
                         (long long)r, t);
        CGNN_REQUIRE(h[t][rows] == p->nnz[t], "plan: rowptr[rows]=%d but nnz=%lld (term %d)",
                     h[t][rows], (long long)p->nnz[t], t);
    }
    const int64_t total = p->nnz[0] + p->nnz[1];
    if (split <= 0) {
        // Degree histogram in one number: rows are short on average -> short chunks keep the
        // tail of a power-law row small; rows are long on average (bucket segments) ->
        // longer chunks halve the partial-sum traffic.
        const double avg = rows > 0 ? (double)total / (double)rows : 0.0;
        split = avg > 64.0 ? 128 : 64;
    }
    p->split = split;
    std::vector<int4> longs, items;
    std::vector<int32_t> row_ids;
    int64_t short_nonempty = 0;
    for (int64_t r = 0; r < rows; ++r) {
        int64_t deg = 0;
        for (int t = 0; t < p->nterms; ++t) deg += h[t][r + 1] - h[t][r];
        if (deg > split) {
            const int first = (int)items.size();
            for (int t = 0; t < p->nterms; ++t)
                for (int e = h[t][r]; e < h[t][r + 1]; e += split)
                    items.push_back(make_int4((int)longs.size(), t, e,
                                              (int)std::min<int64_t>((int64_t)e + split, h[t][r + 1])));
            longs.push_back(make_int4((int)r, first, (int)items.size() - first, 0));
        } else if (deg > 0) {
            ++short_nonempty;
        }
    }
    p->n_long = (int64_t)longs.size();
    p->n_items = (int64_t)items.size();
    const bool compact = rows >= 1024 && short_nonempty * 2 < rows;
    if (compact) {
        row_ids.reserve((size_t)short_nonempty);
        for (int64_t r = 0; r < rows; ++r) {
            int64_t deg = 0;
            for (int t = 0; t < p->nterms; ++t) deg += h[t][r + 1] - h[t][r];
            if (deg > 0 && deg <= split) row_ids.push_back((int32_t)r);
        }
        p->n_direct = short_nonempty;
        if (short_nonempty > 0) {
            CGNN_CUDA(cudaMalloc(&p->row_ids, sizeof(int32_t) * row_ids.size()));
            CGNN_CUDA(cudaMemcpy(p->row_ids, row_ids.data(), sizeof(int32_t) * row_ids.size(),
                                 cudaMemcpyHostToDevice));
        } else {
            // Nothing short to do, but the list must still be "present" so that a fresh
            // output is cleared: keep a one-element dummy.
            CGNN_CUDA(cudaMalloc(&p->row_ids, sizeof(int32_t)));
        }
    } else {
        p->n_direct = rows;
    }
    if (!items.empty()) {
        CGNN_CUDA(cudaMalloc(&p->items, sizeof(int4) * items.size()));
        CGNN_CUDA(cudaMemcpy(p->items, items.data(), sizeof(int4) * items.size(),
                             cudaMemcpyHostToDevice));
        CGNN_CUDA(cudaMalloc(&p->longs, sizeof(int4) * longs.size()));
        CGNN_CUDA(cudaMemcpy(p->longs, longs.data(), sizeof(int4) * longs.size(),
                             cudaMemcpyHostToDevice));
    }
    return CGNN_OK;
}

template <typename InT>
__global__ void convert_index_kernel(const InT *in, int32_t *out, int64_t n, int64_t limit) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)blockDim.x * gridDim.x) {
        const int64_t v = (int64_t)in[i];
        if (v < 0 || v > limit) atomicOr(&g_seg_status, STATUS_BAD_CSR);
        out[i] = (int32_t)v;
    }
}

static int convert_index(const void *in, int index_bytes, int32_t *out, int64_t n,
                         cudaStream_t stream) {
    if (n == 0) return CGNN_OK;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n, 256), 148 * 16);
    if (index_bytes == 8)
        convert_index_kernel<int64_t><<<blocks, 256, 0, stream>>>((const int64_t *)in, out, n,
                                                                   0x7fffffffll);
    else
        convert_index_kernel<int32_t><<<blocks, 256, 0, stream>>>((const int32_t *)in, out, n,
                                                                   0x7fffffffll);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

}  // namespace cgnn

using namespace cgnn;

extern "C" {

int cgnn_plan_create(cgnn_plan **plan_out, int64_t rows, int index_bytes, const void *rowptr0,
                     const void *col0, int64_t nnz0, const void *rowptr1, const void *col1,
                     int64_t nnz1, int split, cgnn_stream_t stream) {
    CGNN_REQUIRE(plan_out != nullptr, "plan: null output");
    *plan_out = nullptr;
    CGNN_REQUIRE(index_bytes == 4 || index_bytes == 8, "plan: index_bytes must be 4 or 8");
    CGNN_REQUIRE(rows >= 0 && rows < 0x7fffffffll, "plan: row count out of range");
    CGNN_REQUIRE(nnz0 >= 0 && nnz1 >= 0 && nnz0 + nnz1 < 0x7fffffffll,
                 "plan: entry count out of 32-bit range");
    CGNN_REQUIRE(rowptr0 != nullptr, "plan: null rowptr");
    CGNN_REQUIRE(col0 != nullptr || nnz0 == 0, "plan: null col");
    CGNN_REQUIRE(split >= 0, "plan: negative split");
    cgnn_plan *p = new cgnn_plan();
    CGNN_CUDA(cudaGetDevice(&p->device));
    p->rows = rows;
    p->nterms = rowptr1 ? 2 : 1;
    p->nnz[0] = nnz0;
    p->nnz[1] = rowptr1 ? nnz1 : 0;
    const void *rp[2] = {rowptr0, rowptr1};
    const void *cl[2] = {col0, col1};
    int rc = CGNN_OK;
    for (int t = 0; t < p->nterms && rc == CGNN_OK; ++t) {
        if (cudaMalloc(&p->rowptr[t], sizeof(int32_t) * ((size_t)rows + 1)) != cudaSuccess ||
            cudaMalloc(&p->col[t], sizeof(int32_t) * (size_t)std::max<int64_t>(p->nnz[t], 1)) !=
                cudaSuccess) {
            set_error("plan: device allocation failed");
            rc = CGNN_ERR_CUDA;
            break;
        }
        rc = convert_index(rp[t], index_bytes, p->rowptr[t], rows + 1, (cudaStream_t)stream);
        if (rc == CGNN_OK)
            rc = convert_index(cl[t], index_bytes, p->col[t], p->nnz[t], (cudaStream_t)stream);
    }
    if (rc == CGNN_OK) rc = plan_analyze(p, split, (cudaStream_t)stream);
    if (rc != CGNN_OK) {
        cgnn_plan_destroy(p);
        return rc;
    }
    *plan_out = p;
    return CGNN_OK;
}

void cgnn_plan_destroy(cgnn_plan *p) {
    if (!p) return;
    for (int t = 0; t < 2; ++t) {
        if (p->rowptr[t]) cudaFree(p->rowptr[t]);
        if (p->col[t]) cudaFree(p->col[t]);
    }
    if (p->items) cudaFree(p->items);
    if (p->longs) cudaFree(p->longs);
    if (p->row_ids) cudaFree(p->row_ids);
    delete p;
}

int cgnn_plan_info(const cgnn_plan *p, int64_t info[8]) {
    CGNN_REQUIRE(p != nullptr && info != nullptr, "plan info: null argument");
    info[0] = p->rows;
    info[1] = p->nnz[0] + p->nnz[1];
    info[2] = p->split;
    info[3] = p->n_long;
    info[4] = p->n_items;
    info[5] = p->n_direct;
    info[6] = p->nterms;
    info[7] = p->row_ids ? 1 : 0;
    return CGNN_OK;
}

size_t cgnn_plan_ticket_bytes(const cgnn_plan *p, int64_t width, int dtype) {
    if (!p || width <= 0) return 0;
    (void)dtype;
    return align_up((size_t)p->n_long * (size_t)ticket_tiles(width) * sizeof(int), 256);
}

size_t cgnn_plan_scratch_bytes(const cgnn_plan *p, int64_t width, int dtype) {
    if (!p || width <= 0) return 0;
    const size_t elt = dtype == CGNN_F64 ? 8 : 4;
    // tickets + one partial row per chunk + the column-sum stage of the bias gradient
    return cgnn_plan_ticket_bytes(p, width, dtype) +
           align_up((size_t)p->n_items * (size_t)width * elt, 256) +
           (size_t)ceil_div(std::max<int64_t>(p->rows, 1), COLSUM_ROWS) * (size_t)width * elt;
}

int cgnn_spmm(const cgnn_plan *plan, int dtype, int64_t width, const void *val, const void *src,
              void *out, int accumulate, void *scratch, size_t scratch_bytes,
              cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 1, "spmm: plan must hold one block");
    return run(plan, dtype, width, val, src, nullptr, nullptr, nullptr, nullptr, out, accumulate,
               scratch, scratch_bytes, (cudaStream_t)stream);
}

int cgnn_spmm_pair(const cgnn_plan *plan, int dtype, int64_t width, const void *val0,
                   const void *src0, const void *val1, const void *src1, void *out,
                   int accumulate, void *scratch, size_t scratch_bytes, cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 2, "spmm_pair: plan must hold two blocks");
    return run(plan, dtype, width, val0, src0, val1, src1, nullptr, nullptr, out, accumulate,
               scratch, scratch_bytes, (cudaStream_t)stream);
}

int cgnn_cluster_mean(const cgnn_plan *plan, int dtype, int64_t width, const void *x,
                      const int32_t *count, void *out, void *scratch, size_t scratch_bytes,
                      cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 1, "cluster_mean: bad plan");
    CGNN_REQUIRE(count != nullptr, "cluster_mean: null counts");
    return run(plan, dtype, width, nullptr, x, nullptr, nullptr, nullptr, count, out, 0, scratch,
               scratch_bytes, (cudaStream_t)stream);
}

int cgnn_cluster_reconstruct_backward(const cgnn_plan *plan, int dtype, int64_t width,
                                      const void *grad, const void *output, int relu,
                                      void *d_reps, void *bias_grad, void *scratch,
                                      size_t scratch_bytes, cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 1, "reconstruct_backward: bad plan");
    CGNN_REQUIRE(!relu || output != nullptr || plan->nnz[0] == 0,
                 "reconstruct_backward: relu needs the forward output");
    int rc = run(plan, dtype, width, nullptr, grad, nullptr, nullptr, relu ? output : nullptr,
                 nullptr, d_reps, 0, scratch, scratch_bytes, (cudaStream_t)stream);
    if (rc != CGNN_OK || bias_grad == nullptr || width == 0) return rc;
    const size_t elt = dtype == CGNN_F64 ? 8 : 4;
    const size_t off = cgnn_plan_ticket_bytes(plan, width, dtype) +
                       align_up((size_t)plan->n_items * (size_t)width * elt, 256);
    CGNN_REQUIRE(scratch != nullptr && scratch_bytes >= cgnn_plan_scratch_bytes(plan, width, dtype),
                 "reconstruct_backward: scratch too small for the bias gradient");
    void *part = reinterpret_cast<char *>(scratch) + off;
    if (dtype == CGNN_F32)
        return colsum<float>((const float *)d_reps, plan->rows, width, (float *)part,
                             (float *)bias_grad, (cudaStream_t)stream);
    return colsum<double>((const double *)d_reps, plan->rows, width, (double *)part,
                          (double *)bias_grad, (cudaStream_t)stream);
}

}  // extern "C"
