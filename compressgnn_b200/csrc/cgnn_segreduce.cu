// Segment reduce: out[r,:] (+)= sum over the entries of row r of  val[e] * src[col[e],:].
//
// One decomposition serves the compressed-propagation SpMM blocks, the fused two-block pass, the
// per-bucket mean and the reconstruct backward.  Design points (B200, HBM-bound):
//   * the plan stores the entries of the short rows back to back, so a work unit that owns a few
//     consecutive rows reads ONE contiguous entry range, 32 (source,value) pairs per coalesced
//     load, the next window requested before the current one is consumed;
//   * rows longer than `split` are cut into chunks (work units of their own); a chunk writes its
//     partial sum to scratch, takes a ticket, and the chunk that draws the last ticket adds the
//     partials in chunk order -- deterministic, no float atomics, and no unit ever waits for another;
//   * three gather engines share that decomposition and produce the same bits:
//       seg_async_kernel  gathered rows staged through shared memory by 16-byte cp.async copies, one
//                         warp-wide instruction per 512 bytes; rows narrower than 512 bytes bring
//                         several entries per instruction.  The engine of every plain launch on
//                         16-byte aligned rows (column tiles of 128 fp32 columns).
//       seg_bulk_kernel   rows staged by one bulk copy (cp.async.bulk + mbarrier) per row; kept for
//                         the launches that also stage a mask row per entry or per output row.
//       seg_kernel        register gathers; scalar rows, unaligned operands, two source matrices
//                         that are not a whole number of rows apart.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <vector>

#include "cgnn_plan.h"

// Build-time tuning knobs (the defaults are the measured best on B200).
#ifndef CGNN_SEG_USCALE
#define CGNN_SEG_USCALE 8   // 16-byte gather loads a lane keeps in flight
#endif
#ifndef CGNN_SEG_LDMODE
#define CGNN_SEG_LDMODE 0   // 0 plain ld.global, 1 ld.global.cg (bypass L1), 2 ld.global.nc
#endif
#ifndef CGNN_SEG_RPU
#define CGNN_SEG_RPU 8      // rows per direct work unit (capped by the lane-group width)
#endif
#ifndef CGNN_SEG_PREFETCH
#define CGNN_SEG_PREFETCH 1    // request the next (source,value) batch before consuming the current
#endif
#ifndef CGNN_SEG_FFMA2
#define CGNN_SEG_FFMA2 0    // packed fma.rn.f32x2 in the row update: measured slower (148 -> 213 us at F=128)
#endif
#ifndef CGNN_SEG_VEC_META
#define CGNN_SEG_VEC_META 1 // a stage's value words read as 16-byte vectors instead of one by one
#endif
#ifndef CGNN_SEG_THREADS
#define CGNN_SEG_THREADS 128
#endif
#ifndef CGNN_SEG_MINBLOCKS
#define CGNN_SEG_MINBLOCKS 6
#endif

namespace cgnn {

// Scratch of cgnn_spmm_static_scratch: lives in the library image, so every GPU that loads the
// library holds CGNN_STATIC_SCRATCH_BYTES of it until the process exits.  In host code this
// name is only a stand-in for the symbol, never a device address; the address is looked up
// per device with cudaGetSymbolAddress (static_scratch_pointer below).
static __device__ __align__(256) unsigned char g_static_scratch[CGNN_STATIC_SCRATCH_BYTES];

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

// Store of a finished output row.  (Streaming and L2 evict-first variants of this store, alone and
// together with evict-last / evict-first hints on the gathers, changed neither the time nor the DRAM
// traffic of the vertex pass on B200; a plain store it stays.)
template <typename T, int VW>
__device__ __forceinline__ void row_store(T *p, const Vec<T, VW> &x) {
    vec_store<T, VW>(p, x);
}

int segreduce_status(int *out) {
    int zero = 0;
    CGNN_CUDA(cudaMemcpyFromSymbol(out, g_seg_status, sizeof(int)));
    CGNN_CUDA(cudaMemcpyToSymbol(g_seg_status, &zero, sizeof(int)));
    return CGNN_OK;
}

template <typename T>
struct SegArgs {
    const int32_t *entries;     // source row | term << 31, in plan order
    const T *val;               // values in plan order, or null (all ones)
    const T *src0;              // source matrix of block 0
    int32_t delta_rows;         // (source matrix of block 1) - src0 in whole rows, when aligned
    int64_t delta_elems;        // the same distance in elements (GENERIC kernels)
    const T *mask_src;          // MASKED: entries whose mask_src value is <= 0 contribute 0
    const T *seg_mask;          // optional: the finished row is zeroed where the mask row of its
                                // FIRST entry is <= 0 (all entries of a row share one mask row)
    const int32_t *div_counts;  // optional: divide the row by max(div_counts[row], 1)
    T *out;
    int accumulate;
    int64_t width;
    const int32_t *uptr;
    const int32_t *urow;
    int64_t n_direct;
    const int4 *items;
    int64_t n_items;
    const int4 *longs;
    T *partial;
    int *tickets;
};

// Source-row index of an entry relative to src0.  Entries of the second block (bit 31 set)
// live in another matrix; when that matrix starts a whole number of rows away from src0
// (delta_rows), adding it here -- once, in the lane that loaded the entry -- lets every
// gather use the plain address row * width + column.  (Any per-gather select or extra 64-bit
// term in that address costs about a third of the kernel's throughput on B200.)
template <typename T>
__device__ __forceinline__ int32_t entry_row(const SegArgs<T> &a, int32_t c) {
    return (c & 0x7fffffff) + ((c >> 31) & a.delta_rows);
}

// Load U gathered feature rows (entries j .. j+U of the current batch) into registers.
// GENERIC: the second matrix is not row-aligned with the first; its entries (flag kept in
// bit 31 of r) add an element remainder.
template <typename T, int VW, int LPR, int VPL, int U, bool MASKED, bool GENERIC>
__device__ __forceinline__ void load_batch(const SegArgs<T> &a, Vec<T, VW> (&x)[U][VPL], int32_t r, int j,
                                           int cnt, int64_t colbase, const bool (&colok)[VPL],
                                           unsigned gmask) {
    using V = Vec<T, VW>;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int32_t rj = __shfl_sync(gmask, r, j + u, LPR);
        if (j + u < cnt) {
            int64_t off;
            if constexpr (GENERIC)
                off = (int64_t)(rj & 0x7fffffff) * a.width + colbase + (rj < 0 ? a.delta_elems : (int64_t)0);
            else
                off = (int64_t)rj * a.width + colbase;
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                if (colok[p]) {
                    x[u][p] = gather_load<T, VW>(a.src0 + off + p * (LPR * VW));
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
}

template <typename T, int VW, int VPL>
__device__ __forceinline__ void fma_row(Vec<T, VW> (&acc)[VPL], const Vec<T, VW> (&x)[VPL], T w,
                                        const bool (&colok)[VPL]) {
#pragma unroll
    for (int p = 0; p < VPL; ++p) {
        if (colok[p]) {
            if constexpr (CGNN_SEG_FFMA2 && sizeof(T) == 4 && VW == 4) {
                // two packed fma.rn.f32x2 (sm_100): each half is the IEEE fma of the scalar form
                const float2 ww = make_float2(w, w);
                const float2 lo = __ffma2_rn(make_float2(x[p].v[0], x[p].v[1]), ww, make_float2(acc[p].v[0], acc[p].v[1]));
                const float2 hi = __ffma2_rn(make_float2(x[p].v[2], x[p].v[3]), ww, make_float2(acc[p].v[2], acc[p].v[3]));
                acc[p].v[0] = lo.x;
                acc[p].v[1] = lo.y;
                acc[p].v[2] = hi.x;
                acc[p].v[3] = hi.y;
            } else {
#pragma unroll
                for (int i = 0; i < VW; ++i) acc[p].v[i] = fma(x[p].v[i], w, acc[p].v[i]);
            }
        }
    }
}

// Store (or accumulate, or divide) one finished row; first_entry < 0 means the row is empty.
template <typename T, int VW, int LPR, int VPL>
__device__ __forceinline__ void finish_row(const SegArgs<T> &a, int32_t row, int first_entry,
                                           Vec<T, VW> (&acc)[VPL], int64_t colbase,
                                           const bool (&colok)[VPL]) {
    using V = Vec<T, VW>;
    if (first_entry < 0 && a.accumulate) return;  // nothing to add
    T *orow = a.out + (int64_t)row * a.width + colbase;
    if (a.seg_mask && first_entry >= 0) {
        const T *mrow = a.seg_mask + (int64_t)(a.entries[first_entry] & 0x7fffffff) * a.width + colbase;
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
            row_store<T, VW>(orow + p * (LPR * VW), r);
        }
    }
}

// One work unit per group of LPR lanes: a few consecutive rows of the direct list (one
// contiguous entry range), or one chunk of a long row.
template <typename T, int VW, int LPR, int VPL, bool MASKED, bool GENERIC>
__global__ void __launch_bounds__(CGNN_SEG_THREADS, CGNN_SEG_MINBLOCKS) seg_kernel(const SegArgs<T> a) {
    using V = Vec<T, VW>;
    constexpr int GPW = 32 / LPR;
    constexpr int U0 = VPL >= CGNN_SEG_USCALE ? 1 : CGNN_SEG_USCALE / VPL;
    constexpr int U = U0 < LPR ? U0 : LPR;
    constexpr int RPU = CGNN_SEG_RPU < LPR ? CGNN_SEG_RPU : LPR - 1;
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
    const int64_t direct_units = (a.n_direct + RPU - 1) / RPU;

    int e_begin, e_end, nr = 0, myptr = 0;
    int32_t myrow = 0;  // row id of listed row `gl` of this unit (fetched up front: a load at
                        // flush time would stall the store that needs it as its address)
    int64_t first = 0;
    int64_t item_index = -1;
    if (unit < direct_units) {
        first = unit * RPU;
        nr = (int)min((int64_t)RPU, a.n_direct - first);
        if (gl <= nr) myptr = a.uptr[first + gl];
        if (gl < nr) myrow = a.urow ? a.urow[first + gl] : (int32_t)(first + gl);
        e_begin = __shfl_sync(gmask, myptr, 0, LPR);
        e_end = __shfl_sync(gmask, myptr, nr, LPR);
    } else {
        item_index = unit - direct_units;
        if (item_index >= a.n_items) return;
        const int4 item = a.items[item_index];
        e_begin = item.y;
        e_end = item.z;
    }

    // ---- stream the entry range -------------------------------------------------------
    int cur = 0;              // listed row whose sum is in acc (direct units)
    int row_begin = e_begin;  // its entry range
    int row_end = item_index >= 0 ? e_end : __shfl_sync(gmask, myptr, 1, LPR);
    auto flush = [&]() {  // finish listed row `cur` and move to the next one
        const int32_t row = __shfl_sync(gmask, myrow, cur, LPR);
        finish_row<T, VW, LPR, VPL>(a, row, row_begin < row_end ? row_begin : -1, acc, colbase, colok);
#pragma unroll
        for (int p = 0; p < VPL; ++p) acc[p] = vec_zero<T, VW>();
        ++cur;
        row_begin = row_end;
        row_end = __shfl_sync(gmask, myptr, (cur + 1) & (LPR - 1), LPR);
    };
    auto row_of = [&](int32_t c) { return GENERIC ? c : entry_row(a, c); };
    int32_t o = 0, o_next = 0;  // source row of this lane's entry of the batch
    T v = T(0), v_next = T(0);
    if (e_begin + gl < e_end) {
        o = row_of(a.entries[e_begin + gl]);
        v = a.val ? a.val[e_begin + gl] : T(1);
    }
    for (int base = e_begin; base < e_end; base += LPR) {
#if CGNN_SEG_PREFETCH
        const int nxt = base + LPR + gl;
        if (nxt < e_end) {
            o_next = row_of(a.entries[nxt]);
            v_next = a.val ? a.val[nxt] : T(1);
        }
#else
        if (base != e_begin && base + gl < e_end) {
            o = row_of(a.entries[base + gl]);
            v = a.val ? a.val[base + gl] : T(1);
        }
#endif
        const int cnt = min(LPR, e_end - base);
        for (int j = 0; j < cnt; j += U) {
            V x[U][VPL];
            load_batch<T, VW, LPR, VPL, U, MASKED, GENERIC>(a, x, o, j, cnt, colbase, colok, gmask);
            if (base + j + U <= row_end) {  // no row boundary inside this batch
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const T w = __shfl_sync(gmask, v, j + u, LPR);
                    if (j + u < cnt) fma_row<T, VW, VPL>(acc, x[u], w, colok);
                }
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const T w = __shfl_sync(gmask, v, j + u, LPR);
                    if (j + u < cnt) {
                        while (base + j + u >= row_end) flush();
                        fma_row<T, VW, VPL>(acc, x[u], w, colok);
                    }
                }
            }
        }
#if CGNN_SEG_PREFETCH
        o = o_next;
        v = v_next;
#endif
    }
    if (item_index < 0) {
        while (cur < nr) flush();
        return;
    }

    // ---- chunk of a long row: publish the partial sum, the last ticket adds them up --------
    const int4 item = a.items[item_index];
    const int4 lr = a.longs[item.x];
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
    finish_row<T, VW, LPR, VPL>(a, lr.x, lr.w, acc, colbase, colok);
}

// Rows of at most 16 vectors (F <= 64 in fp32) go through the cp.async engine below with several
// entries per warp-wide copy; a direct work unit of such rows holds this many of them.
#ifndef CGNN_SEG_NARROW_RPU
#define CGNN_SEG_NARROW_RPU 8    // 8 against 16: the rule launches of a column shard (few tens of thousands of short rows) run 15-25 % faster, the vertex pass the same
#endif

// ---------------------------------------------------------------------------------------
// Rows staged by bulk copies (at least 272 bytes of a row per column tile): the gathered rows are
// brought into shared memory by bulk asynchronous copies (cp.async.bulk, completion counted on an
// mbarrier).  A warp owns a ring of S stages x B rows; the lane that holds an entry of the unit's
// stream issues the copy of its source row (so the address of an entry, including the choice between
// the two source matrices, is computed once by one lane); when a stage's barrier completes the warp
// moves the stage to registers, refills it at once and then adds the rows to its row sums.  CTAs are
// ONE warp with an 8 KB ring (about 24 per SM): units differ in length, and a CTA's shared memory is
// idle from the moment its first warp finishes until its last one does.  MASKED: every entry also
// brings the tile of its mask row (same row index in mask_src) into the second half of the stage, and
// values whose mask is <= 0 are dropped as the stage moves to registers.
//
// What bounds this engine on B200: an SM's bulk-copy unit accepts about one copy per ten cycles (27 G
// copies/s on the whole GPU), each lane's copy is issued as an instruction of its own, and the
// barrier is polled.  For 1 KB rows that is enough to saturate DRAM (the masked reconstruct backward
// runs at the copy bandwidth); for 512-byte rows and less the cp.async engine below is faster
// (154 -> 113 us on the 128-column vertex pass of the 325 k-node graph), and it took over every plain
// launch.
// ---------------------------------------------------------------------------------------
#ifndef CGNN_SEG_BULK
#define CGNN_SEG_BULK 1
#endif
#ifndef CGNN_SEG_BULK_WARPS
#define CGNN_SEG_BULK_WARPS 1        // warps per CTA: one, so that a finished unit frees its ring at once
#endif
#ifndef CGNN_SEG_BULK_STAGE_BYTES
#define CGNN_SEG_BULK_STAGE_BYTES 4096  // one stage: 4 rows of a 1 KB tile, 8 rows of a 512-byte tile
#endif
#ifndef CGNN_SEG_BULK_S
#define CGNN_SEG_BULK_S 2
#endif
#ifndef CGNN_SEG_BULK_MIN_VECS
#define CGNN_SEG_BULK_MIN_VECS 17    // narrowest row (in 16-byte vectors) that is staged
#endif
#ifndef CGNN_SEG_BULK_RPU
#define CGNN_SEG_BULK_RPU CGNN_SEG_RPU  // rows per direct work unit of the staged kernel
#endif
constexpr int BULK_WAIT_LIMIT = 1 << 20;  // mbarrier polls before a stage is given up

__device__ __forceinline__ uint32_t shared_addr(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, int arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_addr(bar)), "r"(arrivals));
}
__device__ __forceinline__ void mbar_arrive_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(shared_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Poll with a limit; true when the phase completed.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (int i = 0; i < BULK_WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned) that
// reports to `bar`.  The destination is this CTA's own shared memory.
__device__ __forceinline__ void bulk_copy_to_shared(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     shared_addr(dst)),
                 "l"(src), "r"(bytes), "r"(shared_addr(bar))
                 : "memory");
}

template <typename T, int VPL, bool MASKED>
struct BulkLayout {
    static constexpr int SLOT = 32 * VPL * 16;  // bytes of one staged row tile
    static constexpr int W = CGNN_SEG_BULK_WARPS, B = CGNN_SEG_BULK_STAGE_BYTES / SLOT, S = CGNN_SEG_BULK_S;
    static constexpr int PARTS = MASKED ? 2 : 1;  // a stage holds B source tiles, then their B mask tiles
    static constexpr size_t RING = (size_t)S * PARTS * B * SLOT;
    static constexpr size_t BARS = (size_t)W * RING;
    static constexpr size_t META = (BARS + (size_t)W * S * 8 + 15) / 16 * 16;
    static constexpr size_t BYTES = META + (size_t)W * S * B * sizeof(T);
};

template <typename T, int VW, int VPL, bool MASKED>
__global__ void __launch_bounds__(CGNN_SEG_BULK_WARPS * 32) seg_bulk_kernel(const SegArgs<T> a) {
    using V = Vec<T, VW>;
    using L = BulkLayout<T, VPL, MASKED>;
    constexpr int PARTS = L::PARTS;
    static_assert(sizeof(T) * VW == 16, "bulk staging moves 16-byte vectors");
    static_assert(32 % L::B == 0, "a stage must not straddle two entry windows");
    constexpr int LPR = 32, B = L::B, S = L::S, SLOT = L::SLOT;
    constexpr int TILE = 32 * VPL * VW;  // columns of one tile
    constexpr int RPU = CGNN_SEG_BULK_RPU;
    constexpr unsigned FULL = 0xffffffffu;
    extern __shared__ __align__(128) unsigned char bulk_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *ring = bulk_smem + (size_t)warp * L::RING;
    uint64_t *bars = reinterpret_cast<uint64_t *>(bulk_smem + L::BARS) + warp * S;
    T *meta = reinterpret_cast<T *>(bulk_smem + L::META) + warp * (S * B);

    const int64_t unit = (int64_t)blockIdx.x * L::W + warp;
    const int64_t width = a.width;
    const int64_t col0 = (int64_t)blockIdx.y * TILE;
    const int64_t colbase = col0 + lane * VW;
    const uint32_t slot_bytes = (uint32_t)(min((int64_t)TILE, width - col0) * (int64_t)sizeof(T));
    bool colok[VPL];
    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) {
        colok[p] = colbase + p * (LPR * VW) < width;
        acc[p] = vec_zero<T, VW>();
    }
    const int64_t direct_units = (a.n_direct + RPU - 1) / RPU;

    int e_begin, e_end, nr = 0, myptr = 0;
    int32_t myrow = 0;
    int64_t item_index = -1;
    if (unit < direct_units) {
        const int64_t first = unit * RPU;
        nr = (int)min((int64_t)RPU, a.n_direct - first);
        if (lane <= nr) myptr = a.uptr[first + lane];
        if (lane < nr) myrow = a.urow ? a.urow[first + lane] : (int32_t)(first + lane);
        e_begin = __shfl_sync(FULL, myptr, 0);
        e_end = __shfl_sync(FULL, myptr, nr);
    } else {
        item_index = unit - direct_units;
        if (item_index >= a.n_items) return;  // whole warp
        const int4 item = a.items[item_index];
        e_begin = item.y;
        e_end = item.z;
    }
    if (lane < S) mbar_init(&bars[lane], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();

    int cur = 0;
    int row_begin = e_begin;
    int row_end = item_index >= 0 ? e_end : __shfl_sync(FULL, myptr, 1);
    auto flush = [&]() {  // finish listed row `cur` and move to the next one
        const int32_t row = __shfl_sync(FULL, myrow, cur);
        finish_row<T, VW, LPR, VPL>(a, row, row_begin < row_end ? row_begin : -1, acc, colbase, colok);
#pragma unroll
        for (int p = 0; p < VPL; ++p) acc[p] = vec_zero<T, VW>();
        ++cur;
        row_begin = row_end;
        row_end = __shfl_sync(FULL, myptr, (cur + 1) & 31);
    };

    // ---- issue side: a window of 32 entries in registers (lane l holds entry window*32 + l) ----
    const int n_ent = e_end - e_begin;
    const int nb = (n_ent + B - 1) / B;
    const T *src1 = a.src0 + a.delta_elems;
    int32_t o = 0, o_next = 0;
    T v = T(1), v_next = T(1);
    if (lane < n_ent) {
        o = a.entries[e_begin + lane];
        if (a.val) v = a.val[e_begin + lane];
    }
    if (32 + lane < n_ent) {
        o_next = a.entries[e_begin + 32 + lane];
        if (a.val) v_next = a.val[e_begin + 32 + lane];
    }
    int window = 0;
    auto issue = [&](int b) {
        const int first = b * B;  // position of the stage's first entry in the unit's stream
        if ((first >> 5) != window) {
            window = first >> 5;
            o = o_next;
            v = v_next;
            const int nxt = (window + 1) * 32 + lane;
            if (nxt < n_ent) {
                o_next = a.entries[e_begin + nxt];
                if (a.val) v_next = a.val[e_begin + nxt];
            }
        }
        const int st = b % S;
        const int j = lane - (first & 31);
        const int cnt = min(B, n_ent - first);
        if (j == 0) mbar_arrive_expect(&bars[st], (uint32_t)(cnt * PARTS) * slot_bytes);
        __syncwarp();
        if (j >= 0 && j < cnt) {
            const int64_t off = (int64_t)(o & 0x7fffffff) * width + col0;
            meta[st * B + j] = v;
            bulk_copy_to_shared(ring + (size_t)(st * PARTS * B + j) * SLOT, (o < 0 ? src1 : a.src0) + off, slot_bytes,
                                &bars[st]);
            if constexpr (MASKED)
                bulk_copy_to_shared(ring + (size_t)(st * PARTS * B + B + j) * SLOT, a.mask_src + off, slot_bytes,
                                    &bars[st]);
        }
    };
    for (int b = 0; b < S && b < nb; ++b) issue(b);

    // ---- consume side ---------------------------------------------------------------------------
    int b = 0;
    bool expired = false;
    for (; b < nb; ++b) {
        const int st = b % S;
        if (!__all_sync(FULL, mbar_wait_bounded(&bars[st], (uint32_t)(b / S) & 1u))) {
            expired = true;
            break;
        }
        __syncwarp();  // the issuing lanes' value words are visible to the whole warp
        const int ebase = e_begin + b * B;
        const int cnt = min(B, e_end - ebase);
        const unsigned char *stage = ring + (size_t)st * PARTS * B * SLOT + lane * 16;
        // the stage moves to registers and is handed back for refilling before the arithmetic
        V x[B][VPL];
        T w[B];
#if CGNN_SEG_VEC_META
        static_assert(B % VW == 0, "a stage's value words are read as whole vectors");
#pragma unroll
        for (int j = 0; j < B; j += VW) {
            const V wv = *reinterpret_cast<const V *>(meta + st * B + j);
#pragma unroll
            for (int i = 0; i < VW; ++i) w[j + i] = wv.v[i];
        }
#else
#pragma unroll
        for (int j = 0; j < B; ++j) w[j] = meta[st * B + j];
#endif
#pragma unroll
        for (int j = 0; j < B; ++j) {
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                x[j][p] = *reinterpret_cast<const V *>(stage + j * SLOT + p * 512);
                if constexpr (MASKED) {  // entries whose mask value is <= 0 contribute 0
                    const V m = *reinterpret_cast<const V *>(stage + (B + j) * SLOT + p * 512);
#pragma unroll
                    for (int i = 0; i < VW; ++i)
                        if (m.v[i] <= T(0)) x[j][p].v[i] = T(0);
                }
            }
        }
        __syncwarp();  // every lane has read the stage
        if (b + S < nb) issue(b + S);
        if (ebase + cnt <= row_end) {  // no row ends inside this stage
#pragma unroll
            for (int j = 0; j < B; ++j)
                if (j < cnt) fma_row<T, VW, VPL>(acc, x[j], w[j], colok);
        } else {
#pragma unroll
            for (int j = 0; j < B; ++j) {
                if (j < cnt) {
                    while (ebase + j >= row_end) flush();
                    fma_row<T, VW, VPL>(acc, x[j], w[j], colok);
                }
            }
        }
    }
    if (expired) {
        // give up on this unit: record it and let the copies still in flight land (bounded).  Rows of a
        // direct unit stay unwritten; a chunk still publishes a (zero) partial sum and draws its ticket, so
        // that the row's ticket word returns to zero for the next launch.  Either way the status word
        // tells the host that this launch's output is not to be used.
        if (lane == 0) atomicOr(&g_seg_status, STATUS_WAIT_EXPIRED);
        for (int bb = b + 1; bb < nb && bb < b + S; ++bb) mbar_wait_bounded(&bars[bb % S], (uint32_t)(bb / S) & 1u);
        if (item_index < 0) return;
#pragma unroll
        for (int p = 0; p < VPL; ++p) acc[p] = vec_zero<T, VW>();
    }
    if (item_index < 0) {
        while (cur < nr) flush();
        return;
    }

    // ---- chunk of a long row: publish the partial sum, the last ticket adds them up --------
    const int4 item = a.items[item_index];
    const int4 lr = a.longs[item.x];
    T *part = a.partial + item_index * width + colbase;
#pragma unroll
    for (int p = 0; p < VPL; ++p)
        if (colok[p]) vec_store<T, VW>(part + p * (LPR * VW), acc[p]);
    __threadfence();
    __syncwarp();
    int *tk = a.tickets + (int64_t)item.x * gridDim.y + blockIdx.y;
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(tk, 1);
    ticket = __shfl_sync(FULL, ticket, 0);
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
    if (lane == 0) *tk = 0;  // leave the ticket ready for the next launch
    finish_row<T, VW, LPR, VPL>(a, lr.x, lr.w, acc, colbase, colok);
}

// ---------------------------------------------------------------------------------------
// Rows of at most a few hundred bytes per column tile: staged through shared memory by 16-byte
// asynchronous copies (cp.async, one warp-wide instruction per 512 bytes of a gathered row) instead
// of one bulk copy per row.  The bulk-copy engine of an SM accepts about one copy every ten cycles,
// which caps 512-byte rows well below what L2 delivers; cp.async goes through the load/store path,
// needs no registers for the data in flight and no barrier polling: a lane later reads exactly the
// 16 bytes it copied itself, so `cp.async.wait_group` (the hardware parks the warp) is all the
// synchronisation there is.  A warp owns a ring of S stages of K gathered rows; the source rows of
// a 32-entry window sit in registers on the issue side, the values of the window being consumed on
// the consume side.  Unit decomposition, row order, chunk tickets and summation order are those of
// seg_kernel, so all engines produce the same bits.  A feature row wider than the tile is covered
// by blockIdx.y; the tiles of one unit run as separate CTAs, tile 0 of every unit first, which makes
// the slice of the source matrix that one sweep touches smaller than the whole matrix.
// ---------------------------------------------------------------------------------------
#ifndef CGNN_SEG_ASYNC
#define CGNN_SEG_ASYNC 1
#endif
#ifndef CGNN_SEG_ASYNC_K
#define CGNN_SEG_ASYNC_K 4    // gathered rows per stage
#endif
#ifndef CGNN_SEG_ASYNC_S
#define CGNN_SEG_ASYNC_S 4    // stages per warp
#endif
#ifndef CGNN_SEG_ASYNC_RPU
#define CGNN_SEG_ASYNC_RPU CGNN_SEG_RPU
#endif
#ifndef CGNN_SEG_ASYNC_MAX_VECS
#define CGNN_SEG_ASYNC_MAX_VECS 32   // widest row (in 16-byte vectors) handled as ONE tile by this engine
#endif

__device__ __forceinline__ void async_copy16(uint32_t dst_shared, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_shared), "l"(src) : "memory");
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Steps (warp-wide copies per vector) of one stage: a stage never holds more than the 32 entries of a window.
__host__ __device__ constexpr int async_steps(int lpr) {
    return CGNN_SEG_ASYNC_K * (32 / lpr) > 32 ? 32 / (32 / lpr) : CGNN_SEG_ASYNC_K;
}
template <int N>
__device__ __forceinline__ void async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// PLAIN: fresh output, no divide, no mask, the width a whole number of tiles -- the propagation
// passes.  The instantiation drops every per-lane column test and the row epilogue is one store.
// LPR < 32 (rows of at most 256 bytes): a row needs only LPR lanes, so one warp-wide copy brings
// G = 32 / LPR consecutive entries of the unit's stream, lane group k taking entry k of the step.
// Every group keeps a partial sum of the current row (its entries in ascending order) and a row is
// finished by adding the groups' sums with a fixed shuffle tree -- the arrangement of
// seg_narrow_kernel, fed from shared memory instead of registers.
template <typename T, int VW, int LPR, int VPL, bool PLAIN>
__global__ void __launch_bounds__(32) seg_async_kernel(const SegArgs<T> a) {
    using V = Vec<T, VW>;
    static_assert(sizeof(T) * VW == 16, "cp.async staging moves 16-byte vectors");
    static_assert(LPR == 32 || VPL == 1, "several vectors per lane only for full-warp rows");
    constexpr int G = 32 / LPR;               // entries per step (one warp-wide copy per vector)
    constexpr int K = async_steps(LPR), S = CGNN_SEG_ASYNC_S, RPU = LPR == 32 ? CGNN_SEG_ASYNC_RPU : CGNN_SEG_NARROW_RPU;
    constexpr int KE = K * G;                 // entries per stage
    static_assert(32 % KE == 0, "a stage must not straddle two entry windows");
    constexpr int TILE = LPR * VPL * VW;      // columns of one tile
    constexpr int SLOT = 32 * VPL * 16;       // bytes of one staged step
    constexpr unsigned FULL = 0xffffffffu;
    extern __shared__ __align__(128) unsigned char async_smem[];
    const int lane = threadIdx.x;
    const int gl = lane & (LPR - 1), gk = lane / LPR;
    const uint32_t ring = shared_addr(async_smem) + lane * 16;  // this lane's 16 bytes of slot 0, vector 0

    const int64_t unit = blockIdx.x;
    const int64_t width = a.width;
    const int row_bytes = (int)(width * (int64_t)sizeof(T));  // < 2^31: checked by the launcher
    const int64_t col0 = (int64_t)blockIdx.y * TILE;
    const int64_t colbase = col0 + gl * VW;
    bool colok[VPL];
    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) {
        colok[p] = PLAIN || colbase + p * (LPR * VW) < width;
        acc[p] = vec_zero<T, VW>();
    }
    const int64_t direct_units = (a.n_direct + RPU - 1) / RPU;

    int e_begin, e_end, nr = 0, myptr = 0;
    int32_t myrow = 0;
    int64_t item_index = -1;
    if (unit < direct_units) {
        const int64_t first = unit * RPU;
        nr = (int)min((int64_t)RPU, a.n_direct - first);
        if (lane <= nr) myptr = a.uptr[first + lane];
        if (lane < nr) myrow = a.urow ? a.urow[first + lane] : (int32_t)(first + lane);
        e_begin = __shfl_sync(FULL, myptr, 0);
        e_end = __shfl_sync(FULL, myptr, nr);
    } else {
        item_index = unit - direct_units;
        if (item_index >= a.n_items) return;  // whole warp
        const int4 item = a.items[item_index];
        e_begin = item.y;
        e_end = item.z;
    }

    // sum of the groups' partial sums, the same value in every group (fixed tree)
    auto reduce_groups = [&]() {
        if constexpr (G > 1) {
#pragma unroll
            for (int m = LPR; m < 32; m <<= 1) {
#pragma unroll
                for (int i = 0; i < VW; ++i) acc[0].v[i] += __shfl_xor_sync(FULL, acc[0].v[i], m);
            }
        }
    };
    int cur = 0;
    int row_begin = e_begin;
    int row_end = item_index >= 0 ? e_end : __shfl_sync(FULL, myptr, 1);
    char *const obase = reinterpret_cast<char *>(a.out + colbase);  // this lane's first vector of output row 0
    auto flush = [&]() {  // finish listed row `cur` and move to the next one
        const int32_t row = __shfl_sync(FULL, myrow, cur);
        reduce_groups();
        if (G == 1 || gk == 0) {
            if constexpr (PLAIN) {
                T *orow = reinterpret_cast<T *>(obase + (int64_t)row * row_bytes);
#pragma unroll
                for (int p = 0; p < VPL; ++p) row_store<T, VW>(orow + p * (LPR * VW), acc[p]);
            } else {
                finish_row<T, VW, LPR, VPL>(a, row, row_begin < row_end ? row_begin : -1, acc, colbase, colok);
            }
        }
#pragma unroll
        for (int p = 0; p < VPL; ++p) acc[p] = vec_zero<T, VW>();
        ++cur;
        row_begin = row_end;
        row_end = __shfl_sync(FULL, myptr, (cur + 1) & 31);
    };

    const int n_ent = e_end - e_begin;
    const int nb = (n_ent + KE - 1) / KE;
    const char *const gbase = reinterpret_cast<const char *>(a.src0 + colbase);  // this lane's first vector of source row 0

    // ---- issue side: source rows of a 32-entry window (lane l holds entry window*32 + l) --------------
    int32_t o = 0, o_next = 0;
    if (lane < n_ent) o = entry_row(a, a.entries[e_begin + lane]);
    if (32 + lane < n_ent) o_next = entry_row(a, a.entries[e_begin + 32 + lane]);
    int iwindow = 0;
    auto copy_row = [&](uint32_t slot, int32_t rj) {
        const char *src = gbase + (int64_t)rj * row_bytes;  // one widening multiply-add
#pragma unroll
        for (int p = 0; p < VPL; ++p)
            if (colok[p]) async_copy16(slot + (uint32_t)(p * 512), src + p * 512);
    };
    auto issue = [&](int b) {
        if (b < nb) {
            const int first = b * KE;
            if ((first >> 5) != iwindow) {
                iwindow = first >> 5;
                o = o_next;
                const int nxt = (iwindow + 1) * 32 + lane;
                if (nxt < n_ent) o_next = entry_row(a, a.entries[e_begin + nxt]);
            }
            const int cnt = n_ent - first;  // >= 1
            const uint32_t stage = ring + (uint32_t)((b % S) * K) * SLOT;
            const int pos = (first & 31) + gk;
            if (cnt >= KE) {
#pragma unroll
                for (int j = 0; j < K; ++j) copy_row(stage + (uint32_t)(j * SLOT), __shfl_sync(FULL, o, pos + j * G));
            } else {
#pragma unroll
                for (int j = 0; j < K; ++j) {
                    const int32_t rj = __shfl_sync(FULL, o, (pos + j * G) & 31);
                    if (j * G + gk < cnt) copy_row(stage + (uint32_t)(j * SLOT), rj);
                }
            }
        }
        async_commit();  // one group per stage, empty past the end, so that the wait below can count groups
    };
#pragma unroll
    for (int b = 0; b < S; ++b) issue(b);

    // ---- consume side: values of the window being consumed ------------------------------------------
    T v = T(1), v_next = T(1);
    if (a.val) {
        if (lane < n_ent) v = a.val[e_begin + lane];
        if (32 + lane < n_ent) v_next = a.val[e_begin + 32 + lane];
    }
    int cwindow = 0;
    for (int b = 0; b < nb; ++b) {
        const int first = b * KE;
        if ((first >> 5) != cwindow) {
            cwindow = first >> 5;
            v = v_next;
            const int nxt = (cwindow + 1) * 32 + lane;
            if (a.val && nxt < n_ent) v_next = a.val[e_begin + nxt];
        }
        async_wait<S - 1>();  // all but the S-1 youngest groups have landed: stage b is in shared memory
        const int ebase = e_begin + first;
        const int cnt = n_ent - first;
        const uint32_t stage = ring + (uint32_t)((b % S) * K) * SLOT;
        const int pos = (first & 31) + gk;
        V x[K][VPL];
#pragma unroll
        for (int j = 0; j < K; ++j) {
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                if (colok[p]) {
                    float4 t;
                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w)
                                 : "r"(stage + (uint32_t)(j * SLOT + p * 512)));
                    x[j][p] = *reinterpret_cast<V *>(&t);
                }
            }
        }
        if (cnt >= KE && ebase + KE <= row_end && ebase < row_end) {  // a full stage inside the current row
#pragma unroll
            for (int j = 0; j < K; ++j) fma_row<T, VW, VPL>(acc, x[j], __shfl_sync(FULL, v, pos + j * G), colok);
        } else if constexpr (G == 1) {  // one entry per step: finish the rows that end before it, then add it
#pragma unroll
            for (int j = 0; j < K; ++j) {
                const T w = __shfl_sync(FULL, v, (pos + j) & 31);
                if (j < cnt) {
                    while (ebase + j >= row_end) flush();
                    fma_row<T, VW, VPL>(acc, x[j], w, colok);
                }
            }
        } else {
            const int stage_end = ebase + min(cnt, KE);
#pragma unroll
            for (int j = 0; j < K; ++j) {
                const T w = __shfl_sync(FULL, v, (pos + j * G) & 31);
                const int s0 = ebase + j * G;           // the step's entries are [s0, s1)
                const int s1 = min(s0 + G, stage_end);
                const int mine = s0 + gk;               // this lane group's entry
                if (s0 < s1) {                          // uniform: the step holds entries of this unit
                    if (row_end >= s1 && row_end > s0) {  // the current row covers the whole step
                        if (G == 1 || mine < s1) fma_row<T, VW, VPL>(acc, x[j], w, colok);
                    } else {                            // one or more rows end inside this step
                        int lo = s0;
                        while (true) {
                            const int hi = min(row_end, s1);
                            if (mine >= lo && mine < hi) fma_row<T, VW, VPL>(acc, x[j], w, colok);
                            if (row_end > s1) break;    // the current row goes on in the next step
                            flush();
                            lo = hi;
                            if (cur >= nr) break;
                        }
                    }
                }
            }
        }
        issue(b + S);  // the stage's rows are summed: its slots can be refilled
    }
    async_wait<0>();
    if (item_index < 0) {
        while (cur < nr) flush();
        return;
    }

    // ---- chunk of a long row: publish the partial sum, the last ticket adds them up --------
    reduce_groups();
    if (G > 1 && gk != 0) return;
    const unsigned gmask = LPR == 32 ? FULL : (1u << LPR) - 1u;
    const int4 item = a.items[item_index];
    const int4 lr = a.longs[item.x];
    T *part = a.partial + item_index * width + colbase;
#pragma unroll
    for (int p = 0; p < VPL; ++p)
        if (colok[p]) vec_store<T, VW>(part + p * (LPR * VW), acc[p]);
    __threadfence();
    __syncwarp(gmask);
    int *tk = a.tickets + (int64_t)item.x * gridDim.y + blockIdx.y;
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(tk, 1);
    ticket = __shfl_sync(gmask, ticket, 0);
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
    if (lane == 0) *tk = 0;  // leave the ticket ready for the next launch
    finish_row<T, VW, LPR, VPL>(a, lr.x, lr.w, acc, colbase, colok);
}

template <typename T, int VW, int LPR, int VPL, bool PLAIN>
static int launch_async_as(const SegArgs<T> &a, cudaStream_t stream) {
    constexpr size_t BYTES = (size_t)CGNN_SEG_ASYNC_S * async_steps(LPR) * 32 * VPL * 16;
    constexpr int RPU = LPR == 32 ? CGNN_SEG_ASYNC_RPU : CGNN_SEG_NARROW_RPU;
    static std::mutex mu;
    static uint64_t configured = 0;  // one bit per device: the kernel may use BYTES of shared memory
    int device = 0;
    CGNN_CUDA(cudaGetDevice(&device));
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 64 || !(configured >> device & 1)) {
            CGNN_CUDA(cudaFuncSetAttribute(seg_async_kernel<T, VW, LPR, VPL, PLAIN>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BYTES));
            if (device < 64) configured |= 1ull << device;
        }
    }
    const int64_t gx = ceil_div(a.n_direct, RPU) + a.n_items;
    const int64_t gy = ceil_div(a.width, (int64_t)LPR * VPL * VW);
    CGNN_REQUIRE(gx < (1ll << 31) && gy < 65536, "segment reduce: grid too large");
    seg_async_kernel<T, VW, LPR, VPL, PLAIN><<<dim3((unsigned)gx, (unsigned)gy), 32, BYTES, stream>>>(a);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

template <typename T, int VW, int LPR, int VPL>
static int launch_async(const SegArgs<T> &a, cudaStream_t stream) {
    const bool plain = !a.accumulate && a.div_counts == nullptr && a.seg_mask == nullptr &&
                       a.width % (LPR * VPL * VW) == 0;
    return plain ? launch_async_as<T, VW, LPR, VPL, true>(a, stream)
                 : launch_async_as<T, VW, LPR, VPL, false>(a, stream);
}

template <typename T, int VW, int VPL, bool MASKED>
static int launch_bulk(const SegArgs<T> &a, cudaStream_t stream) {
    using L = BulkLayout<T, VPL, MASKED>;
    static std::mutex mu;
    static uint64_t configured = 0;  // one bit per device: the kernel may use L::BYTES of shared memory
    int device = 0;
    CGNN_CUDA(cudaGetDevice(&device));
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 64 || !(configured >> device & 1)) {
            CGNN_CUDA(cudaFuncSetAttribute(seg_bulk_kernel<T, VW, VPL, MASKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)L::BYTES));
            if (device < 64) configured |= 1ull << device;
        }
    }
    const int64_t units = ceil_div(a.n_direct, CGNN_SEG_BULK_RPU) + a.n_items;
    const int64_t gx = ceil_div(units, L::W);
    const int64_t gy = ceil_div(a.width, (int64_t)32 * VPL * VW);
    CGNN_REQUIRE(gx < (1ll << 31) && gy < 65536, "segment reduce: grid too large");
    seg_bulk_kernel<T, VW, VPL, MASKED><<<dim3((unsigned)gx, (unsigned)gy), L::W * 32, L::BYTES, stream>>>(a);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

template <typename T, int VW, int LPR, int VPL, bool MASKED, bool GENERIC>
static int launch_cfg(const SegArgs<T> &a, cudaStream_t stream) {
    constexpr int RPU = CGNN_SEG_RPU < LPR ? CGNN_SEG_RPU : LPR - 1;
    const int64_t units = ceil_div(a.n_direct, RPU) + a.n_items;
    const int64_t per_block = (CGNN_SEG_THREADS / 32) * (32 / LPR);
    const int64_t gx = ceil_div(units, per_block);
    const int64_t gy = ceil_div(a.width, (int64_t)LPR * VPL * VW);
    CGNN_REQUIRE(gx < (1ll << 31) && gy < 65536, "segment reduce: grid too large");
    seg_kernel<T, VW, LPR, VPL, MASKED, GENERIC><<<dim3((unsigned)gx, (unsigned)gy), CGNN_SEG_THREADS, 0, stream>>>(a);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

template <typename T, int VW, bool MASKED, bool GENERIC>
static int launch_vw(const SegArgs<T> &a, cudaStream_t stream) {
    const int64_t vecs = a.width / VW;
#if CGNN_SEG_ASYNC
    if constexpr (sizeof(T) * VW == 16 && !MASKED && !GENERIC) {
        if (a.seg_mask == nullptr && a.width * (int64_t)sizeof(T) < 0x7fffffffll) {
            if (vecs <= 4) return launch_async<T, VW, 4, 1>(a, stream);
            if (vecs <= 8) return launch_async<T, VW, 8, 1>(a, stream);
            if (vecs <= 16) return launch_async<T, VW, 16, 1>(a, stream);
            if (vecs >= CGNN_SEG_BULK_MIN_VECS) {
                if (vecs <= 32 || vecs > CGNN_SEG_ASYNC_MAX_VECS) return launch_async<T, VW, 32, 1>(a, stream);
                if (vecs <= 64) return launch_async<T, VW, 32, 2>(a, stream);
            }
        }
    }
#endif
#if CGNN_SEG_BULK
    if constexpr (sizeof(T) * VW == 16) {
        // staged rows: measured faster than register gathers from 17 vectors (272 bytes) up
        if (vecs > 32) return launch_bulk<T, VW, 2, MASKED>(a, stream);
        if (vecs >= CGNN_SEG_BULK_MIN_VECS) return launch_bulk<T, VW, 1, MASKED>(a, stream);
    }
#endif
    if (vecs <= 4) return launch_cfg<T, VW, 4, 1, MASKED, GENERIC>(a, stream);
    if (vecs <= 8) return launch_cfg<T, VW, 8, 1, MASKED, GENERIC>(a, stream);
    if (vecs <= 16) return launch_cfg<T, VW, 16, 1, MASKED, GENERIC>(a, stream);
    if (vecs <= 32) return launch_cfg<T, VW, 32, 1, MASKED, GENERIC>(a, stream);
    if (vecs <= 64) return launch_cfg<T, VW, 32, 2, MASKED, GENERIC>(a, stream);
    if (vecs <= 128) return launch_cfg<T, VW, 32, 4, MASKED, GENERIC>(a, stream);
    return launch_cfg<T, VW, 32, 8, MASKED, GENERIC>(a, stream);
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Tickets are kept per (long row, column tile).  The cp.async path in fp64 has the narrowest tiles
// of a multi-tile launch (64 columns), so this bounds gridDim.y of every configuration
// launch_vw can pick.
static int64_t ticket_tiles(int64_t width) { return std::max<int64_t>(1, ceil_div(width, 64)); }

// Bytes at the start of a scratch buffer that must be zero before the first launch (and are
// left zero by every launch): the tickets.
static size_t zero_prefix_bytes(const cgnn_plan *p, int64_t width) {
    return align_up((size_t)p->n_long * (size_t)ticket_tiles(width) * sizeof(int), 256);
}

template <typename T>
static int run_typed(const cgnn_plan *p, int64_t width, const T *val, const T *src0, const T *src1,
                     const T *mask, const T *seg_mask, const int32_t *div_counts, T *out,
                     int accumulate, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
    constexpr int VWMAX = 16 / (int)sizeof(T);
    if (p->rows == 0 || width == 0) return CGNN_OK;
    SegArgs<T> a;
    a.entries = p->entries;
    a.val = val;
    a.src0 = src0 ? src0 : src1;
    a.delta_elems = (src0 && src1) ? (int64_t)(src1 - src0) : 0;
    const bool row_aligned = a.delta_elems % width == 0 && a.delta_elems / width > -0x7fffffffll &&
                             a.delta_elems / width < 0x3fffffffll;
    a.delta_rows = row_aligned ? (int32_t)(a.delta_elems / width) : 0;
    a.mask_src = mask;
    a.seg_mask = seg_mask;
    a.div_counts = div_counts;
    a.out = out;
    a.accumulate = accumulate;
    a.width = width;
    a.uptr = p->uptr;
    a.urow = p->urow;
    a.n_direct = p->n_direct;
    a.items = p->items;
    a.n_items = p->n_items;
    a.longs = p->longs;

    const bool vec = width % VWMAX == 0 && aligned16(src0) && aligned16(src1) &&
                     aligned16(mask) && aligned16(seg_mask) && aligned16(out);
    // scratch: [tickets][one partial row per chunk]
    const size_t ticket_bytes = zero_prefix_bytes(p, width);
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
    if (!accumulate && p->compact)
        CGNN_CUDA(cudaMemsetAsync(out, 0, (size_t)p->rows * (size_t)width * sizeof(T), stream));
    if (p->n_direct + p->n_items == 0) return CGNN_OK;
    if (!row_aligned) {  // two sources that are not a whole number of rows apart
        if (vec) return launch_vw<T, VWMAX, false, true>(a, stream);
        return launch_vw<T, 1, false, true>(a, stream);
    }
    if (vec) {
        if (mask) return launch_vw<T, VWMAX, true, false>(a, stream);
        return launch_vw<T, VWMAX, false, false>(a, stream);
    }
    if (mask) return launch_vw<T, 1, true, false>(a, stream);
    return launch_vw<T, 1, false, false>(a, stream);
}

static int run(const cgnn_plan *p, int dtype, int64_t width, const void *val, const void *src0,
               const void *src1, const void *mask, const void *seg_mask,
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
        return run_typed<float>(p, width, (const float *)val, (const float *)src0, (const float *)src1,
                                (const float *)mask, (const float *)seg_mask, div_counts, (float *)out,
                                accumulate, scratch, scratch_bytes, stream);
    return run_typed<double>(p, width, (const double *)val, (const double *)src0, (const double *)src1,
                             (const double *)mask, (const double *)seg_mask, div_counts, (double *)out,
                             accumulate, scratch, scratch_bytes, stream);
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
// Plan construction (once per graph block or per assignment refresh): the host cuts the rows
// into work units from the row pointers alone; a kernel then copies the entries into the
// plan's order.
// ---------------------------------------------------------------------------------------
__global__ void scatter_entries_kernel(const int32_t *rowptr, const int32_t *col, const int32_t *dst,
                                       const int32_t *lead, int64_t rows, int term, int32_t value_base,
                                       int32_t *entries, int32_t *vperm, int32_t *max_source) {
    // one warp per row; `lead` holds the row's term-0 length when this is term 1
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    int32_t largest = -1;  // largest source row this thread has seen
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const int b = rowptr[r], e = rowptr[r + 1];
        if (b == e) continue;
        const int d = dst[r] + (lead ? lead[r + 1] - lead[r] : 0);
        for (int k = b + lane; k < e; k += 32) {
            const int32_t cv = col[k];
            if (cv < 0) atomicOr(&g_seg_status, STATUS_BAD_CSR);
            largest = max(largest, cv);
            entries[d + (k - b)] = cv | (term ? (int32_t)0x80000000 : 0);
            if (vperm) vperm[d + (k - b)] = value_base + k;
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, m));
    if (lane == 0 && largest >= 0) atomicMax(&max_source[term], largest);
}

template <typename T>
__global__ void permute_values_kernel(const int32_t *vperm, int64_t total, int64_t nnz0, const T *val0,
                                      const T *val1, T *out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)blockDim.x * gridDim.x) {
        const int32_t k = vperm[i];
        out[i] = k < nnz0 ? val0[k] : val1[k - nnz0];
    }
}

int plan_build(cgnn_plan *p, const int32_t *const rowptr[2], const int32_t *const col[2], int split,
               cudaStream_t stream, const int32_t *host_rowptr0, bool want_vperm) {
    const int64_t rows = p->rows;
    std::vector<int32_t> h[2];
    const int32_t *hp[2] = {nullptr, nullptr};
    bool copied = false;
    for (int t = 0; t < p->nterms; ++t) {
        if (t == 0 && host_rowptr0) {
            hp[0] = host_rowptr0;
            continue;
        }
        h[t].resize((size_t)rows + 1);
        CGNN_CUDA(cudaMemcpyAsync(h[t].data(), rowptr[t], sizeof(int32_t) * ((size_t)rows + 1),
                                  cudaMemcpyDeviceToHost, stream));
        hp[t] = h[t].data();
        copied = true;
    }
    if (copied) CGNN_CUDA(cudaStreamSynchronize(stream));
    // Pass 1: row lengths (both blocks together), validation, and the row-length histogram (lengths
    // of HIST_CAP and more share the last bin); median, 99th percentile and maximum are kept with the
    // plan (cgnn_plan_degrees).
    constexpr int64_t HIST_CAP = 4096;
    std::vector<int32_t> deg((size_t)rows);
    std::vector<int64_t> hist((size_t)HIST_CAP + 1, 0);
    int64_t longest = 0;
    for (int t = 0; t < p->nterms; ++t) {
        const int32_t *rp = hp[t];
        CGNN_REQUIRE(rp[0] == 0, "plan: rowptr[0] must be 0 (term %d)", t);
        int64_t bad = -1;
        for (int64_t r = 0; r < rows; ++r) {
            const int32_t d = rp[r + 1] - rp[r];
            if (d < 0 && bad < 0) bad = r;
            deg[(size_t)r] = t == 0 ? d : deg[(size_t)r] + d;
        }
        CGNN_REQUIRE(bad < 0, "plan: rowptr not monotone at row %lld (term %d)", (long long)bad, t);
        CGNN_REQUIRE(rp[rows] == p->nnz[t], "plan: rowptr[rows]=%d but nnz=%lld (term %d)", rp[rows],
                     (long long)p->nnz[t], t);
    }
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t d = deg[(size_t)r];
        ++hist[(size_t)std::min(d, HIST_CAP)];
        longest = std::max(longest, d);
    }
    const int64_t total = p->nnz[0] + p->nnz[1];
    p->total = total;
    auto percentile = [&](double q) {
        const int64_t want = (int64_t)std::ceil(q * (double)rows);
        int64_t seen = 0;
        for (int64_t d = 0; d <= HIST_CAP; ++d) {
            seen += hist[(size_t)d];
            if (seen >= want) return d;
        }
        return HIST_CAP;
    };
    p->degree_p50 = rows > 0 ? percentile(0.50) : 0;
    p->degree_p99 = rows > 0 ? percentile(0.99) : 0;
    p->degree_max = longest;
    if (split <= 0) {
        // Chunk length of the long rows, from the histogram.  Mostly short rows with a thin tail (a
        // power-law graph block: p99 a few dozen): chunks of 64 keep the tail's work units close to the
        // direct units in size.  Rows that are long as a rule (bucket segments of an assignment, mean
        // length above 64) or a heavy tail (one row in a hundred beyond 512 entries): chunks of 128
        // halve the partial sums that have to be written and added up.
        const double avg = rows > 0 ? (double)total / (double)rows : 0.0;
        split = (avg > 64.0 || p->degree_p99 > 512) ? 128 : 64;
    }
    p->split = split;

    // Pass 2: sizes of the work lists.
    int64_t short_nonempty = 0, long_rows = 0, n_items = 0;
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t d = deg[(size_t)r];
        if (d > split) {
            ++long_rows;
            n_items += (d + split - 1) / split;
        } else if (d > 0) {
            ++short_nonempty;
        }
    }
    p->compact = rows >= 1024 && short_nonempty * 2 < rows ? 1 : 0;
    const bool identity = !p->compact && long_rows == 0;
    p->n_direct = p->compact ? short_nonempty : rows - long_rows;
    p->n_long = long_rows;
    p->n_items = n_items;

    // One device block holds every array; the small ones are written straight into a page-locked
    // stage (slot 0 of the thread's arena; slot 1 takes the two words that come back) and go up in
    // one copy.
    auto span = [](size_t bytes) { return align_up(std::max<size_t>(bytes, 16), 256); };
    const size_t o_uptr = 0;
    const size_t o_urow = o_uptr + span(((size_t)p->n_direct + 1) * 4);
    const size_t o_items = o_urow + span(identity ? 0 : (size_t)p->n_direct * 4);
    const size_t o_longs = o_items + span((size_t)n_items * 16);
    const size_t o_dst = o_longs + span((size_t)long_rows * 16);
    const size_t o_maxsrc = o_dst + span((size_t)rows * 4);  // largest source row of each term, filled by the scatter
    const size_t staged = o_maxsrc + span(2 * 4);
    std::vector<char> pageable;
    char *stage = static_cast<char *>(pinned_scratch(staged, 0));
    if (stage == nullptr) {
        pageable.resize(staged);
        stage = pageable.data();
    }
    int32_t *const uptr = reinterpret_cast<int32_t *>(stage + o_uptr);
    int32_t *const urow = reinterpret_cast<int32_t *>(stage + o_urow);
    int4 *const items = reinterpret_cast<int4 *>(stage + o_items);
    int4 *const longs = reinterpret_cast<int4 *>(stage + o_longs);
    int32_t *const dst = reinterpret_cast<int32_t *>(stage + o_dst);

    // Pass 3: the direct list (short rows back to back), then the long rows cut into chunks.
    int64_t pos = 0, listed = 0;
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t d = deg[(size_t)r];
        dst[r] = 0;
        if (d > split || (p->compact && d == 0)) continue;
        uptr[listed] = (int32_t)pos;
        if (!identity) urow[listed] = (int32_t)r;
        ++listed;
        dst[r] = (int32_t)pos;
        pos += d;
    }
    uptr[listed] = (int32_t)pos;
    CGNN_REQUIRE(listed == p->n_direct, "plan: internal row count mismatch");
    if (long_rows > 0) {
        int64_t item = 0, lrow = 0;
        for (int64_t r = 0; r < rows; ++r) {
            const int64_t d = deg[(size_t)r];
            if (d <= split) continue;
            const int64_t first = item;
            for (int64_t o = 0; o < d; o += split)
                items[item++] = make_int4((int)lrow, (int)(pos + o), (int)(pos + std::min<int64_t>(o + split, d)), 0);
            longs[lrow++] = make_int4((int)r, (int)first, (int)(item - first), (int)pos);
            dst[r] = (int32_t)pos;
            pos += d;
        }
    }
    CGNN_REQUIRE(pos == total, "plan: internal entry count mismatch");
    int32_t fallback_words[2];
    int32_t *max_source = static_cast<int32_t *>(pinned_scratch(sizeof(fallback_words), 1));
    if (max_source == nullptr) max_source = fallback_words;
    max_source[0] = max_source[1] = -1;
    std::memcpy(stage + o_maxsrc, max_source, 2 * sizeof(int32_t));
    const size_t o_entries = staged;
    const size_t o_vperm = o_entries + span((size_t)total * 4);
    const size_t bytes = o_vperm + (want_vperm ? span((size_t)total * 4) : 0);
    // Stream-ordered allocation: an assignment refresh builds and drops a plan every few epochs,
    // and cudaMalloc / cudaFree would each stall the whole device.
    p->home = stream;
    p->pooled = pool_alloc(&p->block, bytes, stream) == cudaSuccess;
    if (!p->pooled) {
        cudaGetLastError();
        if (cudaMalloc(&p->block, bytes) != cudaSuccess) {
            cudaGetLastError();
            p->block = nullptr;
            set_error("plan: device allocation of %zu bytes failed", bytes);
            return CGNN_ERR_CUDA;
        }
    }
    char *base = reinterpret_cast<char *>(p->block);
    CGNN_CUDA(cudaMemcpyAsync(base, stage, staged, cudaMemcpyHostToDevice, stream));
    p->uptr = reinterpret_cast<int32_t *>(base + o_uptr);
    p->urow = identity ? nullptr : reinterpret_cast<int32_t *>(base + o_urow);
    p->items = reinterpret_cast<int4 *>(base + o_items);
    p->longs = reinterpret_cast<int4 *>(base + o_longs);
    p->entries = reinterpret_cast<int32_t *>(base + o_entries);
    p->vperm = want_vperm ? reinterpret_cast<int32_t *>(base + o_vperm) : nullptr;
    const int32_t *dst_dev = reinterpret_cast<const int32_t *>(base + o_dst);
    if (total > 0) {
        const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(rows, 8), 148 * 16));
        for (int t = 0; t < p->nterms; ++t) {
            if (p->nnz[t] == 0) continue;
            scatter_entries_kernel<<<blocks, 256, 0, stream>>>(rowptr[t], col[t], dst_dev, t ? rowptr[0] : nullptr,
                                                               rows, t, t ? (int32_t)p->nnz[0] : 0, p->entries,
                                                               p->vperm, reinterpret_cast<int32_t *>(base + o_maxsrc));
        }
        CGNN_LAUNCH_CHECK();
        if (want_vperm)
            CGNN_CUDA(cudaMemcpyAsync(max_source, base + o_maxsrc, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    }
    if (!want_vperm && pageable.empty()) {
        // A plan over an index array (no values): its "columns" are the positions 0 .. nnz-1, so the
        // source row count is known, and the page-locked stage is handed back with an event behind the
        // copy instead of a wait -- an assignment refresh then synchronises once, for the bucket count.
        pinned_scratch_in_use(0, stream);
        p->source_rows[0] = p->nnz[0];
        p->source_rows[1] = 0;
        return CGNN_OK;
    }
    // the staged host buffer must outlive the copy
    CGNN_CUDA(cudaStreamSynchronize(stream));
    if (want_vperm) {
        p->source_rows[0] = (int64_t)max_source[0] + 1;
        p->source_rows[1] = (int64_t)max_source[1] + 1;
    } else {
        p->source_rows[0] = p->nnz[0];
    }
    return CGNN_OK;
}

// ---------------------------------------------------------------------------------------
// Plan construction on the device (see cgnn_plan.h): the decisions of plan_build, taken by one CTA.
// ---------------------------------------------------------------------------------------
constexpr int PLAN_CTA = 1024;
constexpr int PLAN_HIST_CAP = 4096;

__global__ void __launch_bounds__(PLAN_CTA) plan_stats_kernel(const int32_t *rowptr, const int32_t *last_row_dev,
                                                              int64_t nnz, int split_request, int32_t *header) {
    __shared__ int hist[PLAN_HIST_CAP + 1];
    __shared__ int s_max, s_split, s_short, s_long, s_items, s_short_entries;
    const int rows = *last_row_dev + 1;
    for (int i = threadIdx.x; i <= PLAN_HIST_CAP; i += PLAN_CTA) hist[i] = 0;
    if (threadIdx.x == 0) s_max = s_short = s_long = s_items = s_short_entries = 0;
    __syncthreads();
    int longest = 0;
    for (int r = threadIdx.x; r < rows; r += PLAN_CTA) {
        const int d = rowptr[r + 1] - rowptr[r];
        atomicAdd(&hist[min(d, PLAN_HIST_CAP)], 1);
        longest = max(longest, d);
    }
    atomicMax(&s_max, longest);
    __syncthreads();
    if (threadIdx.x == 0) {
        // smallest length whose cumulative count reaches ceil(q * rows): the host path's percentile
        const int want50 = (rows + 1) / 2, want99 = (int)((99ll * rows + 99) / 100);
        int seen = 0, p50 = -1, p99 = -1;
        for (int d = 0; d <= PLAN_HIST_CAP && p99 < 0; ++d) {
            seen += hist[d];
            if (p50 < 0 && seen >= want50) p50 = d;
            if (seen >= want99) p99 = d;
        }
        header[PH_P50] = max(p50, 0);
        header[PH_P99] = max(p99, 0);
        s_split = split_request > 0 ? split_request : ((nnz > 64ll * rows || p99 > 512) ? 128 : 64);
    }
    __syncthreads();
    const int split = s_split;
    int n_short = 0, n_long = 0, n_items = 0, short_entries = 0;
    for (int r = threadIdx.x; r < rows; r += PLAN_CTA) {
        const int d = rowptr[r + 1] - rowptr[r];
        if (d > split) {
            ++n_long;
            n_items += (d + split - 1) / split;
        } else {
            n_short += d > 0;
            short_entries += d;
        }
    }
    atomicAdd(&s_short, n_short);
    atomicAdd(&s_long, n_long);
    atomicAdd(&s_items, n_items);
    atomicAdd(&s_short_entries, short_entries);
    __syncthreads();
    if (threadIdx.x == 0) {
        const int compact = rows >= 1024 && 2ll * s_short < rows;
        header[PH_ROWS] = rows;
        header[PH_SPLIT] = split;
        header[PH_COMPACT] = compact;
        header[PH_IDENTITY] = !compact && s_long == 0;
        header[PH_DIRECT] = compact ? s_short : rows - s_long;
        header[PH_LONG] = s_long;
        header[PH_ITEMS] = s_items;
        header[PH_MAX] = s_max;
        header[PH_SHORT_ENTRIES] = s_short_entries;
        header[PH_VALID] = 1;
    }
}

// One CTA: thread t owns a contiguous slice of the rows; five block-wide prefix sums place its listed
// rows, long rows, chunks and entries; a second walk over the slice writes the lists.
constexpr int PLAN_STAGED_ROWS = 50000;  // (rows + 1) * 4 bytes of dynamic shared memory beside the 20 KB of `scan`
__global__ void __launch_bounds__(PLAN_CTA) plan_fill_kernel(const int32_t *rowptr, int rows, int split, int compact,
                                                             int identity, int staged, int32_t *uptr, int32_t *urow,
                                                             int4 *longs, int32_t *dst) {
    __shared__ int scan[5][PLAN_CTA + 1];
    extern __shared__ int32_t staged_rowptr[];
    // A thread's slice of the row pointers is contiguous, so its reads from global memory are a chain of
    // uncoalesced loads (about 90 us for 30 k rows); when the array fits it is first copied to shared memory
    // with coalesced loads and both walks read it from there.
    if (staged) {
        for (int i = threadIdx.x; i <= rows; i += PLAN_CTA) staged_rowptr[i] = rowptr[i];
        __syncthreads();
        rowptr = staged_rowptr;
    }
    const int per = (rows + PLAN_CTA - 1) / PLAN_CTA;
    const int r0 = min(rows, (int)threadIdx.x * per), r1 = min(rows, r0 + per);
    int mine[5] = {0, 0, 0, 0, 0};  // listed rows, their entries, long rows, their entries, chunks
    for (int r = r0; r < r1; ++r) {
        const int d = rowptr[r + 1] - rowptr[r];
        if (d > split) {
            ++mine[2];
            mine[3] += d;
            mine[4] += (d + split - 1) / split;
        } else if (!(compact && d == 0)) {
            ++mine[0];
            mine[1] += d;
        }
    }
#pragma unroll
    for (int q = 0; q < 5; ++q) scan[q][threadIdx.x + 1] = mine[q];
    if (threadIdx.x == 0)
        for (int q = 0; q < 5; ++q) scan[q][0] = 0;
    __syncthreads();
    // inclusive prefix sums in place (Hillis-Steele over PLAN_CTA + 1 slots, slot 0 stays 0)
    for (int step = 1; step <= PLAN_CTA; step <<= 1) {
        int add[5];
        const int i = threadIdx.x + 1;
#pragma unroll
        for (int q = 0; q < 5; ++q) add[q] = i >= step ? scan[q][i - step] : 0;
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 5; ++q) scan[q][i] += add[q];
        __syncthreads();
    }
    int listed = scan[0][threadIdx.x], pos = scan[1][threadIdx.x], lrow = scan[2][threadIdx.x];
    const int short_total = scan[1][PLAN_CTA];
    int lpos = short_total + scan[3][threadIdx.x], item = scan[4][threadIdx.x];
    for (int r = r0; r < r1; ++r) {
        const int d = rowptr[r + 1] - rowptr[r];
        if (d > split) {
            const int chunks = (d + split - 1) / split;
            longs[lrow++] = make_int4(r, item, chunks, lpos);
            dst[r] = lpos;
            item += chunks;
            lpos += d;
        } else if (!(compact && d == 0)) {
            uptr[listed] = pos;
            if (!identity) urow[listed] = r;
            ++listed;
            dst[r] = pos;
            pos += d;
        } else {
            dst[r] = 0;
        }
    }
    if (threadIdx.x == PLAN_CTA - 1) uptr[scan[0][PLAN_CTA]] = short_total;
}

// One thread per chunk: find its long row (the last one whose first chunk is not beyond it).
__global__ void plan_items_kernel(const int32_t *rowptr, const int4 *longs, int n_long, int4 *items, int n_items,
                                  int split) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_items; i += blockDim.x * gridDim.x) {
        int lo = 0, hi = n_long - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (longs[mid].y <= i) lo = mid;
            else hi = mid - 1;
        }
        const int4 lr = longs[lo];
        const int d = rowptr[lr.x + 1] - rowptr[lr.x];
        const int o = (i - lr.y) * split;
        items[i] = make_int4(lo, lr.w + o, lr.w + min(o + split, d), 0);
    }
}

int plan_stats_on_device(const int32_t *rowptr, const int32_t *last_row_dev, int64_t nnz, int split,
                         int32_t *header_dev, cudaStream_t stream) {
    CGNN_CUDA(cudaMemsetAsync(header_dev, 0, sizeof(int32_t) * PLAN_HEADER_WORDS, stream));
    plan_stats_kernel<<<1, PLAN_CTA, 0, stream>>>(rowptr, last_row_dev, nnz, split, header_dev);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

int plan_fill_on_device(cgnn_plan *p, const int32_t *rowptr, const int32_t *col, const int32_t *h,
                        cudaStream_t stream) {
    CGNN_REQUIRE(h[PH_VALID] == 1 && h[PH_ROWS] == p->rows, "plan: the device-side row statistics do not match");
    const int64_t rows = p->rows, total = p->nnz[0];
    p->total = total;
    p->split = h[PH_SPLIT];
    p->compact = h[PH_COMPACT];
    p->n_direct = h[PH_DIRECT];
    p->n_long = h[PH_LONG];
    p->n_items = h[PH_ITEMS];
    p->degree_p50 = h[PH_P50];
    p->degree_p99 = h[PH_P99];
    p->degree_max = h[PH_MAX];
    p->source_rows[0] = total;  // the columns of an index plan are the positions 0 .. nnz-1
    p->source_rows[1] = 0;
    const bool identity = h[PH_IDENTITY] != 0;
    auto span = [](size_t bytes) { return align_up(std::max<size_t>(bytes, 16), 256); };
    const size_t o_uptr = 0;
    const size_t o_urow = o_uptr + span(((size_t)p->n_direct + 1) * 4);
    const size_t o_items = o_urow + span(identity ? 0 : (size_t)p->n_direct * 4);
    const size_t o_longs = o_items + span((size_t)p->n_items * 16);
    const size_t o_dst = o_longs + span((size_t)p->n_long * 16);
    const size_t o_maxsrc = o_dst + span((size_t)rows * 4);
    const size_t o_entries = o_maxsrc + span(2 * 4);
    const size_t bytes = o_entries + span((size_t)total * 4);
    p->home = stream;
    p->pooled = pool_alloc(&p->block, bytes, stream) == cudaSuccess;
    if (!p->pooled) {
        cudaGetLastError();
        if (cudaMalloc(&p->block, bytes) != cudaSuccess) {
            cudaGetLastError();
            p->block = nullptr;
            set_error("plan: device allocation of %zu bytes failed", bytes);
            return CGNN_ERR_CUDA;
        }
    }
    char *base = reinterpret_cast<char *>(p->block);
    p->uptr = reinterpret_cast<int32_t *>(base + o_uptr);
    p->urow = identity ? nullptr : reinterpret_cast<int32_t *>(base + o_urow);
    p->items = reinterpret_cast<int4 *>(base + o_items);
    p->longs = reinterpret_cast<int4 *>(base + o_longs);
    p->entries = reinterpret_cast<int32_t *>(base + o_entries);
    p->vperm = nullptr;
    int32_t *dst = reinterpret_cast<int32_t *>(base + o_dst);
    int32_t *max_source = reinterpret_cast<int32_t *>(base + o_maxsrc);
    CGNN_CUDA(cudaMemsetAsync(max_source, 0xff, 2 * sizeof(int32_t), stream));
    const bool staged = rows < PLAN_STAGED_ROWS;
    const size_t staged_bytes = staged ? ((size_t)rows + 1) * sizeof(int32_t) : 0;
    if (staged)  // per device and cheap: repeated at every call rather than tracked
        CGNN_CUDA(cudaFuncSetAttribute(plan_fill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       PLAN_STAGED_ROWS * (int)sizeof(int32_t)));
    plan_fill_kernel<<<1, PLAN_CTA, staged_bytes, stream>>>(rowptr, (int)rows, p->split, p->compact, identity ? 1 : 0,
                                                            staged ? 1 : 0, p->uptr,
                                                            reinterpret_cast<int32_t *>(base + o_urow), p->longs, dst);
    CGNN_LAUNCH_CHECK();
    if (p->n_items > 0) {
        const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(p->n_items, 256), 148 * 8);
        plan_items_kernel<<<blocks, 256, 0, stream>>>(rowptr, p->longs, (int)p->n_long, p->items, (int)p->n_items,
                                                      p->split);
        CGNN_LAUNCH_CHECK();
    }
    if (total > 0) {
        const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(rows, 8), 148 * 16));
        scatter_entries_kernel<<<blocks, 256, 0, stream>>>(rowptr, col, dst, nullptr, rows, 0, 0, p->entries, nullptr,
                                                           max_source);
        CGNN_LAUNCH_CHECK();
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

// Device address of g_static_scratch on the current device, looked up once per device.
static int static_scratch_pointer(int device, void **out) {
    constexpr int MAX_DEVICES = 64;
    static std::mutex lock;
    static void *address[MAX_DEVICES] = {};
    CGNN_REQUIRE(device >= 0 && device < MAX_DEVICES, "static scratch: device ordinal %d not supported", device);
    std::lock_guard<std::mutex> guard(lock);
    if (address[device] == nullptr) {
        void *p = nullptr;
        CGNN_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        address[device] = p;
    }
    *out = address[device];
    return CGNN_OK;
}

}  // namespace cgnn

using namespace cgnn;

extern "C" {

int cgnn_spmm_static_scratch(const cgnn_plan *plan, int dtype, int64_t width, const void *val,
                             const void *src, void *out, int accumulate, cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 1, "spmm_static_scratch: plan must hold one block");
    CGNN_REQUIRE(dtype == CGNN_F32 || dtype == CGNN_F64, "spmm_static_scratch: unknown dtype %d", dtype);
    CGNN_REQUIRE(width >= 0, "spmm_static_scratch: negative width");
    int device = -1;
    CGNN_CUDA(cudaGetDevice(&device));
    CGNN_REQUIRE(device == plan->device, "spmm_static_scratch: the plan was built on device %d, current is %d",
                 plan->device, device);
    const size_t ticket_bytes = cgnn_plan_ticket_bytes(plan, width, dtype);
    const size_t need = ticket_bytes + (size_t)plan->n_items * (size_t)width * (dtype == CGNN_F64 ? 8 : 4);
    CGNN_REQUIRE(need <= (size_t)CGNN_STATIC_SCRATCH_BYTES,
                 "spmm_static_scratch: this plan and width need %zu bytes of scratch, the built-in "
                 "buffer holds %zu; use cgnn_spmm with caller-provided scratch",
                 need, (size_t)CGNN_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    int rc = static_scratch_pointer(device, &scratch);
    if (rc != CGNN_OK) return rc;
    // The buffer keeps whatever the previous call left; the ticket words must start at zero.
    if (plan->n_items > 0 && ticket_bytes > 0)
        CGNN_CUDA(cudaMemsetAsync(scratch, 0, ticket_bytes, (cudaStream_t)stream));
    return run(plan, dtype, width, val, src, nullptr, nullptr, nullptr, nullptr, out, accumulate,
               scratch, (size_t)CGNN_STATIC_SCRATCH_BYTES, (cudaStream_t)stream);
}

int cgnn_plan_create(cgnn_plan **plan_out, int64_t rows, int index_bytes, const void *rowptr0,
                     const void *col0, int64_t nnz0, const void *rowptr1, const void *col1,
                     int64_t nnz1, int split, cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
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
    p->rows = rows;
    p->nterms = rowptr1 ? 2 : 1;
    p->nnz[0] = nnz0;
    p->nnz[1] = rowptr1 ? nnz1 : 0;
    const void *rp[2] = {rowptr0, rowptr1};
    const void *cl[2] = {col0, col1};
    int32_t *rp32[2] = {nullptr, nullptr}, *cl32[2] = {nullptr, nullptr};
    int rc = cudaGetDevice(&p->device) == cudaSuccess ? CGNN_OK : CGNN_ERR_CUDA;
    for (int t = 0; t < p->nterms && rc == CGNN_OK; ++t) {
        if (cudaMalloc(&rp32[t], sizeof(int32_t) * ((size_t)rows + 1)) != cudaSuccess ||
            cudaMalloc(&cl32[t], sizeof(int32_t) * (size_t)std::max<int64_t>(p->nnz[t], 1)) != cudaSuccess) {
            set_error("plan: device allocation failed");
            rc = CGNN_ERR_CUDA;
            break;
        }
        rc = convert_index(rp[t], index_bytes, rp32[t], rows + 1, stream);
        if (rc == CGNN_OK) rc = convert_index(cl[t], index_bytes, cl32[t], p->nnz[t], stream);
    }
    if (rc == CGNN_OK) rc = plan_build(p, rp32, cl32, split, stream);
    for (int t = 0; t < 2; ++t) {
        if (rp32[t]) cudaFree(rp32[t]);
        if (cl32[t]) cudaFree(cl32[t]);
    }
    if (rc == CGNN_OK) {
        int status = 0;
        rc = segreduce_status(&status);
        if (rc == CGNN_OK && (status & STATUS_BAD_CSR)) {
            set_error("plan: an index is negative or exceeds 32 bits");
            rc = CGNN_ERR_INVALID;
        }
    }
    if (rc != CGNN_OK) {
        cgnn_plan_destroy(p);
        return rc;
    }
    *plan_out = p;
    return CGNN_OK;
}

void cgnn_plan_destroy(cgnn_plan *p) {
    if (!p) return;
    if (p->block) {
        // released in the order of the stream the plan was built on; a launch that still uses
        // the plan on ANOTHER stream must have been waited for by the caller
        if (!p->pooled || cudaFreeAsync(p->block, p->home) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(p->block);
        }
    }
    delete p;
}

int cgnn_plan_info(const cgnn_plan *p, int64_t info[8]) {
    CGNN_REQUIRE(p != nullptr && info != nullptr, "plan info: null argument");
    info[0] = p->rows;
    info[1] = p->total;
    info[2] = p->split;
    info[3] = p->n_long;
    info[4] = p->n_items;
    info[5] = p->n_direct;
    info[6] = p->nterms;
    info[7] = p->compact;
    return CGNN_OK;
}

int cgnn_plan_degrees(const cgnn_plan *p, int64_t out[4]) {
    CGNN_REQUIRE(p != nullptr && out != nullptr, "plan degrees: null argument");
    out[0] = p->degree_p50;
    out[1] = p->degree_p99;
    out[2] = p->degree_max;
    out[3] = p->split;
    return CGNN_OK;
}

int cgnn_plan_source_rows(const cgnn_plan *p, int64_t rows[2]) {
    CGNN_REQUIRE(p != nullptr && rows != nullptr, "plan source rows: null argument");
    rows[0] = p->source_rows[0];
    rows[1] = p->source_rows[1];
    return CGNN_OK;
}

int cgnn_plan_permute_values(const cgnn_plan *p, int dtype, const void *val0, const void *val1,
                             void *out, cgnn_stream_t stream) {
    CGNN_REQUIRE(p != nullptr, "permute_values: null plan");
    CGNN_REQUIRE(p->vperm != nullptr || p->total == 0, "permute_values: this plan carries no value order");
    CGNN_REQUIRE(dtype == CGNN_F32 || dtype == CGNN_F64, "permute_values: unknown dtype %d", dtype);
    if (p->total == 0) return CGNN_OK;
    CGNN_REQUIRE(out != nullptr && (val0 != nullptr || p->nnz[0] == 0) &&
                     (val1 != nullptr || p->nnz[1] == 0), "permute_values: null pointer");
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(p->total, 256), 148 * 16);
    if (dtype == CGNN_F32)
        permute_values_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>(
            p->vperm, p->total, p->nnz[0], (const float *)val0, (const float *)val1, (float *)out);
    else
        permute_values_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>(
            p->vperm, p->total, p->nnz[0], (const double *)val0, (const double *)val1, (double *)out);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

size_t cgnn_plan_ticket_bytes(const cgnn_plan *p, int64_t width, int dtype) {
    if (!p || width <= 0) return 0;
    (void)dtype;
    return zero_prefix_bytes(p, width);
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

int cgnn_spmm_pair(const cgnn_plan *plan, int dtype, int64_t width, const void *val,
                   const void *src0, const void *src1, void *out, int accumulate, void *scratch,
                   size_t scratch_bytes, cgnn_stream_t stream) {
    CGNN_REQUIRE(plan != nullptr && plan->nterms == 2, "spmm_pair: plan must hold two blocks");
    return run(plan, dtype, width, val, src0, src1, nullptr, nullptr, nullptr, out, accumulate,
               scratch, scratch_bytes, (cudaStream_t)stream);
}

int cgnn_propagate(int n_launches, const cgnn_plan *const *plans, const void *const *vals,
                   void *const *scratch, const size_t *scratch_bytes, int dtype, int64_t width,
                   const void *x, void *rule_out, void *out, int rule_term_of_last, int first,
                   int last, cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    CGNN_REQUIRE(n_launches >= 2, "propagate: a pass has at least the rule launch and the vertex launch");
    CGNN_REQUIRE(plans != nullptr && vals != nullptr && scratch != nullptr && scratch_bytes != nullptr,
                 "propagate: null launch table");
    CGNN_REQUIRE(rule_term_of_last == 0 || rule_term_of_last == 1, "propagate: rule_term_of_last must be 0 or 1");
    for (int i = 0; i < n_launches; ++i) {
        CGNN_REQUIRE(plans[i] != nullptr, "propagate: null plan of launch %d", i);
        CGNN_REQUIRE(plans[i]->nterms == (i == n_launches - 1 ? 2 : 1), "propagate: launch %d has the wrong kind of plan", i);
    }
    first = std::max(first, 0);
    last = std::min(last, n_launches - 1);
    for (int i = first; i <= last; ++i) {
        int rc;
        if (i == 0)
            rc = run(plans[0], dtype, width, vals[0], x, nullptr, nullptr, nullptr, nullptr, rule_out, 0,
                     scratch[0], scratch_bytes[0], stream);
        else if (i < n_launches - 1)
            rc = run(plans[i], dtype, width, vals[i], rule_out, nullptr, nullptr, nullptr, nullptr, rule_out, 1,
                     scratch[i], scratch_bytes[i], stream);
        else
            rc = run(plans[i], dtype, width, vals[i], rule_term_of_last == 0 ? rule_out : x,
                     rule_term_of_last == 0 ? x : rule_out, nullptr, nullptr, nullptr, out, 0, scratch[i],
                     scratch_bytes[i], stream);
        if (rc != CGNN_OK) return rc;
    }
    return CGNN_OK;
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
    CGNN_REQUIRE(relu >= 0 && relu <= 2, "reconstruct_backward: relu mode must be 0, 1 or 2");
    CGNN_REQUIRE(!relu || output != nullptr || plan->nnz[0] == 0,
                 "reconstruct_backward: relu needs the forward output");
    int rc = run(plan, dtype, width, nullptr, grad, nullptr, relu == 1 ? output : nullptr,
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
