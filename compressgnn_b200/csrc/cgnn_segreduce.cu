// Segment reduce: out[r,:] (+)= sum over the entries of row r of  val[e] * src[col[e],:].
//
// One kernel serves the compressed-propagation SpMM blocks, the fused two-block pass, the
// per-bucket mean and the reconstruct backward.  Design points (B200, HBM-bound):
//   * a group of LPR lanes owns up to LPR consecutive rows; every lane keeps VPL 16-byte
//     vectors of the current row in registers, so one gathered feature row is LPR*VPL
//     coalesced 128-bit loads;
//   * the entries of the group's rows are read as one stream: LPR (col,val) pairs per
//     coalesced load (the next batch is requested before the current one is consumed),
//     broadcast by shuffle; U gathered rows are in flight per lane before the FMAs issue,
//     across row boundaries;
//   * rows longer than `split` are cut into chunks (work units of their own); a chunk
//     writes its partial sum to scratch, takes a ticket, and the chunk that draws the last
//     ticket adds the partials in chunk order -- deterministic, no float atomics, and no
//     unit ever waits for another.
#include <algorithm>
#include <vector>

#include "cgnn_plan.h"

// Build-time tuning knobs (defaults are the measured best; see profiles/).
#ifndef CGNN_SEG_USCALE
#define CGNN_SEG_USCALE 8   // 16-byte gather loads a lane keeps in flight
#endif
#ifndef CGNN_SEG_LDMODE
#define CGNN_SEG_LDMODE 0   // 0 plain ld.global, 1 ld.global.cg (bypass L1), 2 ld.global.nc
#endif
#ifndef CGNN_SEG_RPU
#define CGNN_SEG_RPU 8      // rows per direct work unit (capped by the lane-group width)
#endif
#ifndef CGNN_SEG_STREAMHINT
#define CGNN_SEG_STREAMHINT 0  // 1: evict-first loads of indices and streaming stores of rows
#endif
#ifndef CGNN_SEG_THREADS
#define CGNN_SEG_THREADS 128
#endif
#ifndef CGNN_SEG_MINBLOCKS
#define CGNN_SEG_MINBLOCKS 5
#endif

namespace cgnn {

static __device__ int g_seg_status = 0;

template <typename T, int VW>
__device__ __forceinline__ Vec<T, VW> gather_load(const T *p) {
#if CGNN_SEG_LDMODE == 1
    return vec_load_cg<T, VW>(p);
#elif CGNN_SEG_LDMODE == 2
    Vec<T, VW> r;
    if constexpr (sizeof(T) * VW == 16) {
        float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        r = *reinterpret_cast<Vec<T, VW> *>(&t);
    } else if constexpr (sizeof(T) * VW == 8) {
        float2 t = __ldg(reinterpret_cast<const float2 *>(p));
        r = *reinterpret_cast<Vec<T, VW> *>(&t);
    } else {
        float t = __ldg(reinterpret_cast<const float *>(p));
        r = *reinterpret_cast<Vec<T, VW> *>(&t);
    }
    return r;
#else
    return vec_load<T, VW>(p);
#endif
}

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
    const T *seg_mask;          // optional: the finished row is zeroed where the mask row of its
                                // FIRST entry is <= 0 (all entries of a row share one mask row)
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

// Sum of one contiguous entry range [e0, e1) of one block into acc: LPR (col,val) pairs per
// coalesced load, U gathered rows in flight per lane.  Used for the chunks of long rows.
template <typename T, int VW, int LPR, int VPL, int U, bool MASKED>
__device__ __forceinline__ void gather_range(Vec<T, VW> (&acc)[VPL], const int32_t *col,
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
                            x[u][p] = gather_load<T, VW>(src + off + p * (LPR * VW));
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

// Store (or accumulate, or divide) one finished row.
template <typename T, int VW, int LPR, int VPL>
__device__ __forceinline__ void finish_row(const SegArgs<T> &a, int32_t row, Vec<T, VW> (&acc)[VPL],
                                           int64_t colbase, const bool (&colok)[VPL]) {
    using V = Vec<T, VW>;
    T *orow = a.out + (int64_t)row * a.width + colbase;
    if (a.seg_mask) {
        const int first = a.rowptr[0][row];
        if (first < a.rowptr[0][row + 1]) {
            const T *mrow = a.seg_mask + (int64_t)a.col[0][first] * a.width + colbase;
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                if (colok[p]) {
                    const V m = vec_load<T, VW>(mrow + p * (LPR * VW));
#pragma unroll
                    for (int i = 0; i < VW; ++i)
                        if (m.v[i] <= T(0)) acc[p].v[i] = T(0);
                }
            }
        }
    }
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
#if CGNN_SEG_STREAMHINT
            vec_store_cs<T, VW>(orow + p * (LPR * VW), r);
#else
            vec_store<T, VW>(orow + p * (LPR * VW), r);
#endif
        }
    }
}

// One work unit per group of LPR lanes: either up to LPR rows of the direct row list (their
// entries are streamed as ONE sequence, so the loads of a row's gathered feature rows are in
// flight together with its neighbours' and a short row costs no pipeline restart), or one
// chunk of a long row.  Lane q of the group keeps the extent of row slot q; an entry's slot is
// found by a shuffle binary search over the slots' prefix sums.
template <typename T, int VW, int LPR, int VPL, bool MASKED>
__global__ void __launch_bounds__(CGNN_SEG_THREADS, CGNN_SEG_MINBLOCKS) seg_kernel(const SegArgs<T> a) {
    using V = Vec<T, VW>;
    constexpr int GPW = 32 / LPR;
    constexpr int U0 = VPL >= CGNN_SEG_USCALE ? 1 : CGNN_SEG_USCALE / VPL;
    constexpr int U = U0 < LPR ? U0 : LPR;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (LPR - 1);
    const unsigned gmask =
        LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (lane & ~(LPR - 1)));
    const int64_t unit =
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

    constexpr int RPU = CGNN_SEG_RPU < LPR ? CGNN_SEG_RPU : LPR;
    const int64_t direct_units = (a.n_direct + RPU - 1) / RPU;

    if (unit >= direct_units) {
        // ---- chunk of a long row: sum it, publish the partial sum, last ticket adds them up
        const int64_t item_index = unit - direct_units;
        if (item_index >= a.n_items) return;
        const int4 item = a.items[item_index];
        const int4 lr = a.longs[item.x];
        const int t = item.y;
        gather_range<T, VW, LPR, VPL, U, MASKED>(acc, a.col[t], a.val[t], a.src[t], a.mask_src,
                                                 width, colbase, colok, item.z, item.w, gl, gmask);
        T *part = a.partial + item_index * width + colbase;
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
        finish_row<T, VW, LPR, VPL>(a, lr.x, acc, colbase, colok);
        return;
    }

    // ---- row slots of this unit: up to RPU rows of the direct row list --------------------
    int my_row = 0, s0 = 0, d0 = 0, s1 = 0, d1 = 0;
    bool my_write = false;
    const int64_t first = unit * RPU;
    const int nr = (int)min((int64_t)RPU, a.n_direct - first);
    if (gl < nr) {
        my_row = a.row_ids ? a.row_ids[first + gl] : (int32_t)(first + gl);
        s0 = a.rowptr[0][my_row];
        d0 = a.rowptr[0][my_row + 1] - s0;
        if (a.nterms > 1) {
            s1 = a.rowptr[1][my_row];
            d1 = a.rowptr[1][my_row + 1] - s1;
        }
        my_write = d0 + d1 <= a.split;  // longer rows are served by chunk units
        if (!my_write) d0 = d1 = 0;
    }
    // exclusive prefix of the slot lengths inside the group
    const int deg = d0 + d1;
    int incl = deg;
#pragma unroll
    for (int o = 1; o < LPR; o <<= 1) {
        const int t = __shfl_up_sync(gmask, incl, o, LPR);
        if (gl >= o) incl += t;
    }
    const int P = incl - deg;
    const int total = __shfl_sync(gmask, incl, LPR - 1, LPR);

    // entry k of the unit's stream -> (column, value, slot | term << 8)
    auto fetch = [&](int k, int &c, T &v, int &qt) {
        int q = 0;
#pragma unroll
        for (int step = LPR / 2; step >= 1; step >>= 1) {
            const int cand = q + step;
            const int pc = __shfl_sync(gmask, P, cand & (LPR - 1), LPR);
            if (cand < nr && pc <= k) q = cand;
        }
        const int pq = __shfl_sync(gmask, P, q, LPR);
        const int s0q = __shfl_sync(gmask, s0, q, LPR);
        const int d0q = __shfl_sync(gmask, d0, q, LPR);
        const int s1q = __shfl_sync(gmask, s1, q, LPR);
        c = 0;
        v = T(0);
        qt = q;
        if (k < total) {
            const int o = k - pq;
            const int term = o >= d0q ? 1 : 0;
            const int e = term ? s1q + (o - d0q) : s0q + o;
            const T *vp = a.val[term];
#if CGNN_SEG_STREAMHINT
            c = __ldcs(a.col[term] + e);
            v = vp ? __ldcs(vp + e) : T(1);
#else
            c = a.col[term][e];
            v = vp ? vp[e] : T(1);
#endif
            qt = q | (term << 8);
        }
    };

    int cur = 0;  // slot whose sum is in acc
    auto flush_until = [&](int upto) {  // finish slots cur .. upto-1 (all but the first are empty)
        for (; cur < upto; ++cur) {
            const int row = __shfl_sync(gmask, my_row, cur, LPR);
            const int wr = __shfl_sync(gmask, (int)my_write, cur, LPR);
            if (wr) finish_row<T, VW, LPR, VPL>(a, row, acc, colbase, colok);
#pragma unroll
            for (int p = 0; p < VPL; ++p) acc[p] = vec_zero<T, VW>();
        }
    };

    int c, qt, c_next = 0, qt_next = 0;
    T v, v_next = T(0);
    fetch(gl, c, v, qt);
    for (int base = 0; base < total; base += LPR) {
        if (base + LPR < total) fetch(base + LPR + gl, c_next, v_next, qt_next);
        const int cnt = min(LPR, total - base);
        // bit j: entry j of this batch starts a new row slot (bit 0 always set: compare with cur)
        const int prev_slot = __shfl_up_sync(gmask, qt, 1, LPR) & 0xff;
        const unsigned ballot = __ballot_sync(gmask, gl == 0 || (qt & 0xff) != prev_slot);
        const unsigned bmask = LPR == 32 ? ballot : ((ballot >> (lane & ~(LPR - 1))) & ((1u << LPR) - 1u));
        for (int j = 0; j < cnt; j += U) {
            V x[U][VPL];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int cj = __shfl_sync(gmask, c, j + u, LPR);
                const int term = __shfl_sync(gmask, qt, j + u, LPR) >> 8;
                if (j + u < cnt) {
                    const T *src = term ? a.src[1] : a.src[0];
                    const int64_t off = (int64_t)cj * width + colbase;
#pragma unroll
                    for (int p = 0; p < VPL; ++p) {
                        if (colok[p]) {
                            x[u][p] = gather_load<T, VW>(src + off + p * (LPR * VW));
                            if constexpr (MASKED) {
                                const V m = vec_load<T, VW>(a.mask_src + off + p * (LPR * VW));
#pragma unroll
                                for (int i = 0; i < VW; ++i)
                                    if (m.v[i] <= T(0)) x[u][p].v[i] = T(0);
                            }
                        }
                    }
                }
            }
            // Row boundaries inside this batch are rare for long rows and absent for chunks:
            // test once per batch and keep the per-entry check out of the common path.
            if (((bmask >> j) & ((1u << U) - 1u)) == 0u) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const T w = __shfl_sync(gmask, v, j + u, LPR);
                    if (j + u < cnt) {
#pragma unroll
                        for (int p = 0; p < VPL; ++p) {
                            if (colok[p]) {
#pragma unroll
                                for (int i = 0; i < VW; ++i)
                                    acc[p].v[i] = fma(x[u][p].v[i], w, acc[p].v[i]);
                            }
                        }
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const T w = __shfl_sync(gmask, v, j + u, LPR);
                    const int q = __shfl_sync(gmask, qt, j + u, LPR) & 0xff;
                    if (j + u < cnt) {
                        if (q != cur) flush_until(q);
#pragma unroll
                        for (int p = 0; p < VPL; ++p) {
                            if (colok[p]) {
#pragma unroll
                                for (int i = 0; i < VW; ++i)
                                    acc[p].v[i] = fma(x[u][p].v[i], w, acc[p].v[i]);
                            }
                        }
                    }
                }
            }
        }
        c = c_next;
        v = v_next;
        qt = qt_next;
    }

    flush_until(nr);
}

template <typename T, int VW, int LPR, int VPL, bool MASKED>
static int launch_cfg(const SegArgs<T> &a, cudaStream_t stream) {
    constexpr int RPU = CGNN_SEG_RPU < LPR ? CGNN_SEG_RPU : LPR;
    const int64_t units = ceil_div(a.n_direct, RPU) + a.n_items;
    const int64_t per_block = (CGNN_SEG_THREADS / 32) * (32 / LPR);
    const int64_t gx = ceil_div(units, per_block);
    const int64_t gy = ceil_div(a.width, (int64_t)LPR * VPL * VW);
    CGNN_REQUIRE(gx < (1ll << 31) && gy < 65536, "segment reduce: grid too large");
    seg_kernel<T, VW, LPR, VPL, MASKED><<<dim3((unsigned)gx, (unsigned)gy), CGNN_SEG_THREADS, 0, stream>>>(a);
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
                     const T *val1, const T *src1, const T *mask, const T *seg_mask,
                     const int32_t *div_counts,
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
    a.seg_mask = seg_mask;
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
                     aligned16(mask) && aligned16(seg_mask) && aligned16(out);
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
               const void *val1, const void *src1, const void *mask, const void *seg_mask,
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
                                (const float *)seg_mask, div_counts, (float *)out, accumulate, scratch, scratch_bytes,
                                stream);
    return run_typed<double>(p, width, (const double *)val0, (const double *)src0,
                             (const double *)val1, (const double *)src1, (const double *)mask,
                             (const double *)seg_mask, div_counts, (double *)out, accumulate, scratch, scratch_bytes,
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
    return run(plan, dtype, width, val, src, nullptr, nullptr, nullptr, nullptr, nullptr, out, accumulate,
               scratch, scratch_bytes, (cudaStream_t)stream);
}

int cgnn_spmm_pair(const cgnn_plan *plan, int dtype, int64_t width, const void *val0,
                   const void *src0, const void *val1, const void *src1, void *out,
                   int accumulate, void *scratch, size_t scratch_bytes, cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 2, "spmm_pair: plan must hold two blocks");
    return run(plan, dtype, width, val0, src0, val1, src1, nullptr, nullptr, nullptr, out, accumulate,
               scratch, scratch_bytes, (cudaStream_t)stream);
}

int cgnn_cluster_mean(const cgnn_plan *plan, int dtype, int64_t width, const void *x,
                      const int32_t *count, void *out, void *scratch, size_t scratch_bytes,
                      cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 1, "cluster_mean: bad plan");
    CGNN_REQUIRE(count != nullptr, "cluster_mean: null counts");
    return run(plan, dtype, width, nullptr, x, nullptr, nullptr, nullptr, nullptr, count, out, 0, scratch,
               scratch_bytes, (cudaStream_t)stream);
}

int cgnn_cluster_reconstruct_backward(const cgnn_plan *plan, int dtype, int64_t width,
                                      const void *grad, const void *output, int relu,
                                      void *d_reps, void *bias_grad, void *scratch,
                                      size_t scratch_bytes, cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 1, "reconstruct_backward: bad plan");
    CGNN_REQUIRE(relu >= 0 && relu <= 2, "reconstruct_backward: relu mode must be 0, 1 or 2");
    CGNN_REQUIRE(!relu || output != nullptr || plan->nnz[0] == 0,
                 "reconstruct_backward: relu needs the forward output");
    int rc = run(plan, dtype, width, nullptr, grad, nullptr, nullptr, relu == 1 ? output : nullptr,
                 relu == 2 ? output : nullptr, nullptr, d_reps, 0, scratch, scratch_bytes,
                 (cudaStream_t)stream);
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
