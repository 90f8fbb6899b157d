// LSH cluster assignment: projection onto the random hyperplanes, sign packing, and the
// compaction of raw bucket codes into dense 1-based ids with per-bucket counts and the
// bucket permutation the deterministic mean runs over.
//
// Projection kernel (the only heavy part: it reads all of X once).  fp32 with 16-byte aligned rows,
// a width that is a multiple of 16 and a multiple of four planes takes project_tma_kernel: a producer
// lane moves each (row tile, 16 columns) box of X and the matching 16 plane rows into shared memory with
// one TMA tile copy (64-byte swizzle, so the per-row 128-bit reads are conflict-free without padding)
// and one bulk copy, a full/empty mbarrier pair per stage hands the stages to four consumer warps, and
// no CTA-wide barrier sits between a copy and the FMAs that overlap it.  Measured at 2.45 M x 128,
// 16 planes: 243 us against 340 us for the cp.async kernel below (memory alone 190 us; the FMAs alone,
// with their shared-memory operand loads, 214 us).  Every other case takes project_kernel:
//   * a CTA walks row tiles of TR rows; X arrives in k-chunks of KC columns through a
//     multi-stage cp.async pipeline into padded shared memory (conflict-free 128-bit reads);
//   * each thread owns RPT rows and all `bits` accumulators of them, so the n x bits
//     projection never leaves registers in the fused path; plane values are broadcast
//     128-bit shared loads shared by the RPT rows;
//   * every accumulator is the chain p = fma(x[r,k], w[k,h], p), k ascending from +0 --
//     the order the CPU oracle restates, which makes the sign bits reproducible bit for bit.
// Compaction sorts (code,row) pairs with a stable radix sort (CUB), so neither a 2^bits
// histogram nor any atomic is involved and the permutation is deterministic.
#include <algorithm>
#include <mutex>
#include <type_traits>
#include <vector>
#include <cub/cub.cuh>
#include <cuda.h>

#include "cgnn_plan.h"

namespace cgnn {

static __device__ int g_cluster_status = 0;

int cluster_status(int *out) {
    int zero = 0;
    CGNN_CUDA(cudaMemcpyFromSymbol(out, g_cluster_status, sizeof(int)));
    CGNN_CUDA(cudaMemcpyToSymbol(g_cluster_status, &zero, sizeof(int)));
    return CGNN_OK;
}

#ifndef CGNN_PROJ_TMA
#define CGNN_PROJ_TMA 1   // 0: every projection takes the cp.async kernel
#endif
constexpr int PROJ_THREADS = 128;
constexpr int KC = 16;         // columns per pipeline stage
constexpr int XS_STRIDE = 20;  // padded row stride of the X stage (elements): odd in 16-byte units
#ifndef CGNN_PROJ_STAGES
#define CGNN_PROJ_STAGES 2
#endif
constexpr int PROJ_STAGES = CGNN_PROJ_STAGES;   // cp.async pipeline depth
constexpr int PROJ_CTAS_PER_SM = PROJ_STAGES == 2 ? 5 : 3;  // shared-memory limited at 16 planes

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, int src_bytes) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    // .L2::256B: the 64-byte slice of a feature row this stage needs pulls the surrounding
    // 256 bytes into L2, so the following k-stages of the same rows hit L2 and DRAM sees
    // whole-page bursts instead of scattered 64-byte reads.
    asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

template <typename T, int HB, int RPT>
struct ProjSmem {
    static constexpr int TR = PROJ_THREADS * RPT;
    T xs[PROJ_STAGES][TR][XS_STRIDE];
    T ws[PROJ_STAGES][KC][HB];
};

// Stage loader: X[row0 .. row0+TR, k0 .. k0+KC) and planes[k0 .. k0+KC, 0..bits) -> shared,
// zero-filled outside the matrix.  On the vector path (16-byte aligned rows) a thread always
// moves the same 16-byte column slot of rows (t / VPR) + j * (THREADS / VPR), so its global
// and shared offsets are a fixed base plus a constant stride per j: a handful of integer
// instructions per 16-byte cp.async instead of a div/mod per element.
template <typename T, int HB, int RPT>
__device__ __forceinline__ void load_stage(ProjSmem<T, HB, RPT> &sm, int stage, const T *x,
                                           const T *planes, int64_t n, int64_t width, int bits,
                                           int64_t row0, int64_t k0, bool vec_ok) {
    constexpr int TR = PROJ_THREADS * RPT;
    constexpr int VW = 16 / (int)sizeof(T);
    constexpr int VPR = KC / VW;                   // 16-byte slots per row of the stage
    constexpr int ROWS_PER_PASS = PROJ_THREADS / VPR;
    constexpr int PASSES = TR / ROWS_PER_PASS;
    if (vec_ok) {
        const int r0 = threadIdx.x / VPR, c = (threadIdx.x % VPR) * VW;
        const bool col_ok = k0 + c < width;  // width % VW == 0 on this path
        const T *g = x + (row0 + r0) * width + k0 + c;
        T *sdst = &sm.xs[stage][r0][c];
        const int64_t rows_left = n - row0 - r0;
#pragma unroll
        for (int j = 0; j < PASSES; ++j) {
            const bool ok = col_ok && (int64_t)j * ROWS_PER_PASS < rows_left;
            cp_async16(sdst + j * (ROWS_PER_PASS * XS_STRIDE),
                       ok ? (const void *)(g + (int64_t)j * ROWS_PER_PASS * width) : (const void *)x,
                       ok ? 16 : 0);
        }
        if (bits == HB && k0 + KC <= width) {
            // the KC plane rows of this stage are one contiguous block of KC*HB elements
            constexpr int SLOTS = KC * HB / VW;
            const T *pg = planes + k0 * HB;
            T *ps = &sm.ws[stage][0][0];
            for (int i = threadIdx.x; i < SLOTS; i += PROJ_THREADS) cp_async16(ps + i * VW, pg + i * VW, 16);
            return;
        }
    } else {
        for (int i = threadIdx.x; i < TR * KC; i += PROJ_THREADS) {
            const int r = i / KC, c = i % KC;
            const int64_t gr = row0 + r, gk = k0 + c;
            sm.xs[stage][r][c] = (gr < n && gk < width) ? x[gr * width + gk] : T(0);
        }
    }
    for (int i = threadIdx.x; i < KC * HB; i += PROJ_THREADS) {
        const int k = i / HB, h = i % HB;
        const int64_t gk = k0 + k;
        sm.ws[stage][k][h] = (gk < width && h < bits) ? planes[gk * bits + h] : T(0);
    }
}

template <typename T, int HB, int RPT>
__global__ void __launch_bounds__(PROJ_THREADS)
project_kernel(const T *__restrict__ x, const T *__restrict__ planes, int64_t n, int64_t width,
               int bits, T *__restrict__ proj, int32_t *__restrict__ codes, int vec_ok_i) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    using Smem = ProjSmem<T, HB, RPT>;
    Smem &sm = *reinterpret_cast<Smem *>(smem_raw);
    constexpr int TR = PROJ_THREADS * RPT;
    constexpr int VW = 16 / (int)sizeof(T);
    using V = Vec<T, VW>;
    const bool vec_ok = vec_ok_i != 0;
    const int64_t tiles = (n + TR - 1) / TR;
    const int64_t nk = (width + KC - 1) / KC;
    // Stages of this CTA: (tile, k-chunk) pairs, tiles strided by the grid.
    const int64_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t stages = my_tiles * nk;
    if (stages == 0) return;

    // fp32 accumulators are kept as pairs of adjacent planes and updated with the packed
    // two-wide FMA of sm_100 (fma.rn.f32x2): each half is an IEEE fused multiply-add, so the
    // per-plane chain p = fma(x, w, p) -- and with it every sign bit -- is unchanged, at half
    // the issue slots.  fp64 uses scalar FMAs.
    constexpr bool PACKED = sizeof(T) == 4;
    using Acc = typename std::conditional<PACKED, float2, T>::type;
    constexpr int NACC = PACKED ? HB / 2 : HB;
    Acc acc[RPT][NACC] = {};
    auto plane = [&](int i, int h) -> T {
        if constexpr (PACKED) return (h & 1) ? acc[i][h >> 1].y : acc[i][h >> 1].x;
        else return acc[i][h];
    };
    // prologue: the first PROJ_STAGES-1 stages are requested up front
#pragma unroll
    for (int pre = 0; pre < PROJ_STAGES - 1; ++pre) {
        if (pre < stages) {
            const int64_t ptile = blockIdx.x + (pre / nk) * gridDim.x;
            load_stage<T, HB, RPT>(sm, pre, x, planes, n, width, bits, ptile * TR, (pre % nk) * KC, vec_ok);
        }
        cp_async_commit();
    }
    for (int64_t s = 0; s < stages; ++s) {
        const int cur = (int)(s % PROJ_STAGES);
        const int64_t tile = blockIdx.x + (s / nk) * gridDim.x;
        const int64_t kc = s % nk;
        const int64_t ahead = s + PROJ_STAGES - 1;
        if (ahead < stages) {
            const int64_t ntile = blockIdx.x + (ahead / nk) * gridDim.x;
            load_stage<T, HB, RPT>(sm, (int)(ahead % PROJ_STAGES), x, planes, n, width, bits, ntile * TR,
                                   (ahead % nk) * KC, vec_ok);
        }
        cp_async_commit();
        cp_async_wait<PROJ_STAGES - 1>();
        __syncthreads();
        if (kc == 0) {
#pragma unroll
            for (int i = 0; i < RPT; ++i)
#pragma unroll
                for (int h = 0; h < NACC; ++h) {
                    if constexpr (PACKED) acc[i][h] = make_float2(0.f, 0.f);
                    else acc[i][h] = T(0);
                }
        }
#pragma unroll
        for (int kk = 0; kk < KC; kk += VW) {
            V xv[RPT];
#pragma unroll
            for (int i = 0; i < RPT; ++i)
                xv[i] = *reinterpret_cast<const V *>(&sm.xs[cur][threadIdx.x + i * PROJ_THREADS][kk]);
#pragma unroll
            for (int q = 0; q < VW; ++q) {
#pragma unroll
                for (int h4 = 0; h4 < HB; h4 += VW) {
                    const V w = *reinterpret_cast<const V *>(&sm.ws[cur][kk + q][h4]);
                    if constexpr (PACKED) {
#pragma unroll
                        for (int j = 0; j < VW; j += 2)
#pragma unroll
                            for (int i = 0; i < RPT; ++i)
                                acc[i][(h4 + j) >> 1] =
                                    __ffma2_rn(make_float2(xv[i].v[q], xv[i].v[q]),
                                               make_float2(w.v[j], w.v[j + 1]), acc[i][(h4 + j) >> 1]);
                    } else {
#pragma unroll
                        for (int j = 0; j < VW; ++j)
#pragma unroll
                            for (int i = 0; i < RPT; ++i)
                                acc[i][h4 + j] = fma(xv[i].v[q], w.v[j], acc[i][h4 + j]);
                    }
                }
            }
        }
        if (kc == nk - 1) {
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                const int64_t row = tile * TR + threadIdx.x + i * PROJ_THREADS;
                if (row < n) {
                    if (proj) {
#pragma unroll
                        for (int h = 0; h < HB; ++h)
                            if (h < bits) proj[row * bits + h] = plane(i, h);
                    }
                    if (codes) {
                        int32_t id = 0;
#pragma unroll
                        for (int h = 0; h < HB; ++h)
                            if (h < bits) id = (id << 1) | (plane(i, h) > T(0) ? 1 : 0);
                        codes[row] = id;
                    }
                }
            }
        }
        __syncthreads();
    }
}

template <typename T, int HB>
static int launch_project(const T *x, const T *planes, int64_t n, int64_t width, int bits,
                          T *proj, int32_t *codes, cudaStream_t stream) {
    constexpr int RPT = sizeof(T) == 4 ? 2 : 1;
    using Smem = ProjSmem<T, HB, RPT>;
    constexpr int TR = PROJ_THREADS * RPT;
    constexpr int VW = 16 / (int)sizeof(T);
    const size_t smem = sizeof(Smem);
    auto kernel = project_kernel<T, HB, RPT>;
    CGNN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CGNN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   cudaSharedmemCarveoutMaxShared));
    const int64_t tiles = ceil_div(n, TR);
    const int64_t grid = std::min<int64_t>(tiles, 148 * PROJ_CTAS_PER_SM);
    const bool vec_ok = width % VW == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                        (reinterpret_cast<uintptr_t>(planes) & 15) == 0;
    kernel<<<(unsigned)grid, PROJ_THREADS, smem, stream>>>(x, planes, n, width, bits, proj, codes,
                                                          vec_ok ? 1 : 0);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

// ---------------------------------------------------------------------------------------
// TMA-staged projection (fp32)
// ---------------------------------------------------------------------------------------
constexpr int TMA_CONSUMERS = 128;   // four consumer warps; a fifth warp holds the producer lane
constexpr int TMA_BOX_ROWS = 256;    // rows per TMA box (the hardware limit of a box dimension)
constexpr int TMA_STAGES = 3;
constexpr int TMA_WAIT_LIMIT = 1 << 20;  // mbarrier polls before a wait is given up

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbarrier_init(uint64_t *bar, int arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals));
}
__device__ __forceinline__ void mbarrier_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Bounded wait: false when the phase did not complete within TMA_WAIT_LIMIT polls.
__device__ __forceinline__ bool mbarrier_wait(uint64_t *bar, uint32_t parity) {
    for (int i = 0; i < TMA_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// One box of the tensor map, starting at (column c0, row c1); c0 * 4 bytes is a multiple of 16.
__device__ __forceinline__ void tma_load_box(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar))
        : "memory");
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

template <int HB, int RPT>
struct TmaLayout {
    static constexpr int TR = TMA_CONSUMERS * RPT;      // rows per tile
    static constexpr int XS_BYTES = TR * KC * 4;        // dense: 64 bytes per row, swizzled by the copy
    static constexpr int WS_BYTES = KC * HB * 4;
    static constexpr int BAR_OFFSET = TMA_STAGES * (XS_BYTES + WS_BYTES);
    static constexpr int BYTES = BAR_OFFSET + (2 * TMA_STAGES + 1) * 8;
};

// Thread t of the consumers owns rows t + i * 128 of the tile and all HB accumulators of them, as pairs
// of adjacent planes updated by fma.rn.f32x2: per plane the chain p = fma(x[r,k], w[k,h], p), k ascending
// from +0, exactly as in project_kernel.  A stage is released to the producer by one arrival per warp.
template <int HB, int RPT>
__global__ void __launch_bounds__(TMA_CONSUMERS + 32)
project_tma_kernel(const __grid_constant__ CUtensorMap xmap, const float *__restrict__ planes, int64_t n,
                   int64_t width, float *__restrict__ proj, int32_t *__restrict__ codes) {
    using L = TmaLayout<HB, RPT>;
    extern __shared__ __align__(1024) unsigned char tma_smem[];
    unsigned char *xs = tma_smem;                                                   // [STAGES][XS_BYTES]
    float *ws = reinterpret_cast<float *>(tma_smem + TMA_STAGES * L::XS_BYTES);      // [STAGES][KC][HB]
    uint64_t *full = reinterpret_cast<uint64_t *>(tma_smem + L::BAR_OFFSET);
    uint64_t *empty = full + TMA_STAGES;
    volatile int *gave_up = reinterpret_cast<volatile int *>(empty + TMA_STAGES);
    const int64_t tiles = (n + L::TR - 1) / L::TR;
    const int64_t nk = width / KC;
    const int64_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t stages = my_tiles * nk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < TMA_STAGES; ++s) {
            mbarrier_init(&full[s], 1);
            mbarrier_init(&empty[s], TMA_CONSUMERS / 32);
        }
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == TMA_CONSUMERS / 32) {
        if (lane == 0) {
            for (int64_t s = 0; s < stages && !*gave_up; ++s) {
                const int st = (int)(s % TMA_STAGES);
                if (s >= TMA_STAGES && !mbarrier_wait(&empty[st], (uint32_t)(s / TMA_STAGES - 1) & 1u)) {
                    atomicOr(&g_cluster_status, STATUS_WAIT_EXPIRED);
                    *gave_up = 1;
                    break;
                }
                const int64_t tile = blockIdx.x + (s / nk) * gridDim.x;
                const int64_t kc = s % nk;
                mbarrier_expect(&full[st], L::XS_BYTES + L::WS_BYTES);
#pragma unroll
                for (int b = 0; b < L::TR / TMA_BOX_ROWS; ++b)
                    tma_load_box(xs + st * L::XS_BYTES + b * TMA_BOX_ROWS * KC * 4, &xmap, (int)(kc * KC),
                                 (int)(tile * L::TR + b * TMA_BOX_ROWS), &full[st]);
                bulk_load(ws + st * KC * HB, planes + kc * KC * HB, L::WS_BYTES, &full[st]);
            }
        }
    } else {
        float2 acc[RPT][HB / 2];
        const int t = threadIdx.x;
        for (int64_t s = 0; s < stages; ++s) {
            const int st = (int)(s % TMA_STAGES);
            const int64_t tile = blockIdx.x + (s / nk) * gridDim.x;
            const int64_t kc = s % nk;
            if (!mbarrier_wait(&full[st], (uint32_t)(s / TMA_STAGES) & 1u)) {
                // the copies of this stage never landed: report, stop the producer, and give the copies that
                // were already requested one more bounded wait each before the CTA leaves its shared memory
                atomicOr(&g_cluster_status, STATUS_WAIT_EXPIRED);
                *gave_up = 1;
                for (int64_t r = s; r < stages && r < s + TMA_STAGES; ++r)
                    if (!mbarrier_wait(&full[r % TMA_STAGES], (uint32_t)(r / TMA_STAGES) & 1u)) break;
                break;
            }
            if (kc == 0) {
#pragma unroll
                for (int i = 0; i < RPT; ++i)
#pragma unroll
                    for (int h = 0; h < HB / 2; ++h) acc[i][h] = make_float2(0.f, 0.f);
            }
            const unsigned char *xst = xs + st * L::XS_BYTES;
            const float *wst = ws + st * KC * HB;
#pragma unroll
            for (int c = 0; c < KC / 4; ++c) {
                float4 xv[RPT];
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    // 64-byte swizzle: the 16-byte slot index is xor-ed with bits 7..8 of the byte address
                    const int r = t + i * TMA_CONSUMERS;
                    xv[i] = *reinterpret_cast<const float4 *>(xst + r * (KC * 4) + ((c ^ ((r >> 1) & 3)) << 4));
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
#pragma unroll
                    for (int h4 = 0; h4 < HB; h4 += 4) {
                        const float4 w = *reinterpret_cast<const float4 *>(wst + (c * 4 + q) * HB + h4);
#pragma unroll
                        for (int i = 0; i < RPT; ++i) {
                            const float xq = q == 0 ? xv[i].x : q == 1 ? xv[i].y : q == 2 ? xv[i].z : xv[i].w;
                            acc[i][h4 / 2] = __ffma2_rn(make_float2(xq, xq), make_float2(w.x, w.y), acc[i][h4 / 2]);
                            acc[i][h4 / 2 + 1] =
                                __ffma2_rn(make_float2(xq, xq), make_float2(w.z, w.w), acc[i][h4 / 2 + 1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbarrier_arrive(&empty[st]);
            if (kc == nk - 1) {
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    const int64_t row = tile * L::TR + t + i * TMA_CONSUMERS;
                    if (row < n) {
                        if (proj) {
#pragma unroll
                            for (int h = 0; h < HB; h += 4)
                                *reinterpret_cast<float4 *>(proj + row * HB + h) = make_float4(
                                    acc[i][h / 2].x, acc[i][h / 2].y, acc[i][h / 2 + 1].x, acc[i][h / 2 + 1].y);
                        }
                        if (codes) {
                            int32_t id = 0;
#pragma unroll
                            for (int h = 0; h < HB; ++h) {
                                const float p = (h & 1) ? acc[i][h >> 1].y : acc[i][h >> 1].x;
                                id = (id << 1) | (p > 0.f ? 1 : 0);
                            }
                            codes[row] = id;
                        }
                    }
                }
            }
        }
    }
    __syncthreads();  // nobody leaves while the producer may still be requesting copies
}

using TensorMapEncode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                     const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                     CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point query (no link against the driver
// library); nullptr when the driver does not export it.
static TensorMapEncode tensor_map_encoder() {
    static const TensorMapEncode fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<TensorMapEncode>(p);
    }();
    return fn;
}

// Launches the TMA kernel; CGNN_OK with *taken = false when the tensor map cannot be built here.
template <int HB, int RPT>
static int launch_project_tma(const float *x, const float *planes, int64_t n, int64_t width, float *proj,
                              int32_t *codes, cudaStream_t stream, bool *taken) {
    using L = TmaLayout<HB, RPT>;
    *taken = false;
    const TensorMapEncode encode = tensor_map_encoder();
    if (!encode) return CGNN_OK;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)n};
    const cuuint64_t strides[1] = {(cuuint64_t)width * 4};
    const cuuint32_t box[2] = {(cuuint32_t)KC, (cuuint32_t)TMA_BOX_ROWS};
    const cuuint32_t steps[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(x), dims, strides, box, steps,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return CGNN_OK;
    auto kernel = project_tma_kernel<HB, RPT>;
    static const int ctas_per_sm = [&] {
        int per_sm = 0;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, TMA_CONSUMERS + 32, L::BYTES) !=
                cudaSuccess)
            per_sm = 0;
        return per_sm;
    }();
    if (ctas_per_sm <= 0) {
        (void)cudaGetLastError();
        return CGNN_OK;
    }
    CGNN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES));
    const int64_t tiles = ceil_div(n, L::TR);
    const int64_t grid = std::min<int64_t>(tiles, (int64_t)148 * ctas_per_sm);
    kernel<<<(unsigned)grid, TMA_CONSUMERS + 32, L::BYTES, stream>>>(map, planes, n, width, proj, codes);
    CGNN_LAUNCH_CHECK();
    *taken = true;
    return CGNN_OK;
}

static int project_tma(const float *x, const float *planes, int64_t n, int64_t width, int bits, float *proj,
                       int32_t *codes, cudaStream_t stream, bool *taken) {
    *taken = false;
    const bool fits = bits % 4 == 0 && bits >= 4 && bits <= 32 && width % KC == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(planes) & 15) == 0 &&
                      (proj == nullptr || (reinterpret_cast<uintptr_t>(proj) & 15) == 0);
    if (!fits) return CGNN_OK;
    switch (bits / 4) {
        case 1: return launch_project_tma<4, 4>(x, planes, n, width, proj, codes, stream, taken);
        case 2: return launch_project_tma<8, 4>(x, planes, n, width, proj, codes, stream, taken);
        case 3: return launch_project_tma<12, 4>(x, planes, n, width, proj, codes, stream, taken);
        case 4: return launch_project_tma<16, 4>(x, planes, n, width, proj, codes, stream, taken);
        case 5: return launch_project_tma<20, 2>(x, planes, n, width, proj, codes, stream, taken);
        case 6: return launch_project_tma<24, 2>(x, planes, n, width, proj, codes, stream, taken);
        case 7: return launch_project_tma<28, 2>(x, planes, n, width, proj, codes, stream, taken);
        default: return launch_project_tma<32, 2>(x, planes, n, width, proj, codes, stream, taken);
    }
}

template <typename T>
static int project_typed(const T *x, const T *planes, int64_t n, int64_t width, int bits, T *proj,
                         int32_t *codes, cudaStream_t stream) {
    if (n == 0) return CGNN_OK;
    if (bits == 0) {
        if (codes) CGNN_CUDA(cudaMemsetAsync(codes, 0, sizeof(int32_t) * (size_t)n, stream));
        return CGNN_OK;
    }
    if (width == 0) {
        if (codes) CGNN_CUDA(cudaMemsetAsync(codes, 0, sizeof(int32_t) * (size_t)n, stream));
        if (proj) CGNN_CUDA(cudaMemsetAsync(proj, 0, sizeof(T) * (size_t)n * (size_t)bits, stream));
        return CGNN_OK;
    }
    if constexpr (std::is_same<T, float>::value) {
#if CGNN_PROJ_TMA
        bool taken = false;
        const int rc = project_tma(x, planes, n, width, bits, proj, codes, stream, &taken);
        if (rc != CGNN_OK || taken) return rc;
#endif
    }
    switch ((bits + 3) / 4) {
        case 1: return launch_project<T, 4>(x, planes, n, width, bits, proj, codes, stream);
        case 2: return launch_project<T, 8>(x, planes, n, width, bits, proj, codes, stream);
        case 3: return launch_project<T, 12>(x, planes, n, width, bits, proj, codes, stream);
        case 4: return launch_project<T, 16>(x, planes, n, width, bits, proj, codes, stream);
        case 5: return launch_project<T, 20>(x, planes, n, width, bits, proj, codes, stream);
        case 6: return launch_project<T, 24>(x, planes, n, width, bits, proj, codes, stream);
        case 7: return launch_project<T, 28>(x, planes, n, width, bits, proj, codes, stream);
        default: return launch_project<T, 32>(x, planes, n, width, bits, proj, codes, stream);
    }
}

static int project(int dtype, const void *x, const void *planes, int64_t n, int64_t width, int bits,
                   void *proj, int32_t *codes, cudaStream_t stream) {
    CGNN_REQUIRE(dtype == CGNN_F32 || dtype == CGNN_F64, "cluster: unknown dtype %d", dtype);
    CGNN_REQUIRE(bits >= 0 && bits <= 30, "cluster: hash bits must be in [0,30]");
    CGNN_REQUIRE(n >= 0 && n <= 0x7fffffffll, "cluster: node count exceeds int32 capacity");
    CGNN_REQUIRE(width >= 0, "cluster: negative width");
    if (n > 0 && width > 0 && bits > 0)
        CGNN_REQUIRE(x != nullptr && planes != nullptr, "cluster: null input");
    if (dtype == CGNN_F32)
        return project_typed<float>((const float *)x, (const float *)planes, n, width, bits,
                                    (float *)proj, codes, stream);
    return project_typed<double>((const double *)x, (const double *)planes, n, width, bits,
                                 (double *)proj, codes, stream);
}

template <typename T>
__global__ void codes_from_proj_kernel(const T *proj, int64_t n, int bits, int32_t *codes) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n;
         r += (int64_t)blockDim.x * gridDim.x) {
        int32_t id = 0;
        for (int h = 0; h < bits; ++h) id = (id << 1) | (proj[r * bits + h] > T(0) ? 1 : 0);
        codes[r] = id;
    }
}

// ---------------------------------------------------------------------------------------
// Compaction of raw codes.  Workspace layout (all int32 unless noted), n rows:
//   keys[2][n]  vals[2][n]  cid[n]  segstart[n+2]  active[1]  pad  | cub temp (bytes)
// After cgnn_cluster_assign: vals[0] = permutation (rows sorted by code, ascending row
// inside a bucket), segstart[b] = first sorted position of bucket b (b = 1..active),
// segstart[0] = 0 (bucket 0 is always empty), segstart[active+1] = n.
// ---------------------------------------------------------------------------------------
struct AssignLayout {
    int32_t *keys[2];
    int32_t *vals[2];
    int32_t *cid;
    int32_t *segstart;
    int32_t *active;
    void *temp;
    size_t temp_bytes;
    size_t total;
};

static size_t cub_temp_bytes(int64_t n) {
    size_t sort_bytes = 0, scan_bytes = 0;
    cub::DoubleBuffer<int32_t> k(nullptr, nullptr), v(nullptr, nullptr);
    const int num = (int)std::max<int64_t>(n, 1);
    cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, k, v, num, 0, 32);
    cub::DeviceScan::InclusiveSum(nullptr, scan_bytes, (const int32_t *)nullptr, (int32_t *)nullptr, num);
    cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, (const int32_t *)nullptr, (int32_t *)nullptr, num + 2);
    return align_up(std::max(sort_bytes, scan_bytes) + 256, 256);
}

static AssignLayout assign_layout(void *base, int64_t n) {
    AssignLayout L;
    const size_t nn = align_up(sizeof(int32_t) * (size_t)std::max<int64_t>(n, 1), 256);
    char *p = reinterpret_cast<char *>(base);
    size_t off = 0;
    for (int i = 0; i < 2; ++i) { L.keys[i] = reinterpret_cast<int32_t *>(p + off); off += nn; }
    for (int i = 0; i < 2; ++i) { L.vals[i] = reinterpret_cast<int32_t *>(p + off); off += nn; }
    L.cid = reinterpret_cast<int32_t *>(p + off); off += nn;
    L.segstart = reinterpret_cast<int32_t *>(p + off); off += nn + 256;
    L.active = reinterpret_cast<int32_t *>(p + off); off += 256;
    L.temp = p + off;
    L.temp_bytes = cub_temp_bytes(n);
    L.total = off + L.temp_bytes;
    return L;
}

__global__ void iota_kernel(int32_t *v, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)blockDim.x * gridDim.x)
        v[i] = (int32_t)i;
}

__global__ void head_flags_kernel(const int32_t *sorted, int32_t *flags, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)blockDim.x * gridDim.x)
        flags[i] = (i == 0 || sorted[i] != sorted[i - 1]) ? 1 : 0;
}

__global__ void scatter_ids_kernel(const int32_t *perm, const int32_t *cid, const int32_t *flags,
                                   int64_t n, int64_t *ids, int32_t *segstart, int32_t *active) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)blockDim.x * gridDim.x) {
        const int32_t c = cid[i];
        ids[perm[i]] = c;
        if (flags[i]) segstart[c] = (int32_t)i;
        if (i == 0) segstart[0] = 0;
        if (i == n - 1) {
            segstart[c + 1] = (int32_t)n;
            *active = c;
        }
    }
}

__global__ void counts_kernel(const int32_t *segstart, int64_t active, int32_t *counts) {
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b <= active;
         b += (int64_t)blockDim.x * gridDim.x)
        counts[b] = b == 0 ? 0 : segstart[b + 1] - segstart[b];
}

__global__ void index_to_key_kernel(const int64_t *index, int64_t n, int64_t groups, int32_t *keys,
                                    int32_t *hist) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)blockDim.x * gridDim.x) {
        const int64_t g = index[i];
        if (g < 0 || g >= groups) {
            atomicOr(&g_cluster_status, STATUS_BAD_INDEX);
            keys[i] = 0;
            atomicAdd(hist, 1);
        } else {
            keys[i] = (int32_t)g;
            atomicAdd(hist + g, 1);  // integer atomics: order-independent result
        }
    }
}

// Host copy of the segment starts of the latest cgnn_cluster_assign, handed to the export step.
struct HostSegments {
    std::mutex lock;
    const void *workspace = nullptr;
    int64_t n = 0, valid = 0;
    bool on_device = false;            // start[16 ..] holds the plan's row statistics instead of segment starts
    int32_t *start = nullptr;          // page-locked, grow-only (the copy into it must not be staged)
    size_t capacity = 0;               // in words
    std::vector<int32_t> pageable;     // used when page-locked memory cannot be had
    int32_t *reserve(size_t words) {
        if (capacity < words) {
            if (start && start != pageable.data()) cudaFreeHost(start);
            void *p = nullptr;
            if (cudaHostAlloc(&p, sizeof(int32_t) * words, cudaHostAllocDefault) == cudaSuccess) {
                start = static_cast<int32_t *>(p);
            } else {
                cudaGetLastError();
                pageable.resize(words);
                start = pageable.data();
            }
            capacity = words;
        }
        return start;
    }
};
static HostSegments &host_segments() {
    static HostSegments hs;
    return hs;
}

static unsigned grid_for(int64_t n) { return (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n, 256), 148 * 16)); }

// Sort (key,row) pairs by the low `bits` bits of the key; leaves sorted keys in keys_out and
// the permutation in vals[0].
static int sort_pairs(AssignLayout &L, int64_t n, int bits, int32_t **sorted_keys,
                      cudaStream_t stream) {
    iota_kernel<<<grid_for(n), 256, 0, stream>>>(L.vals[0], n);
    CGNN_LAUNCH_CHECK();
    if (bits == 0) {
        *sorted_keys = L.keys[0];
        return CGNN_OK;
    }
    cub::DoubleBuffer<int32_t> k(L.keys[0], L.keys[1]), v(L.vals[0], L.vals[1]);
    size_t bytes = L.temp_bytes;
    CGNN_CUDA(cub::DeviceRadixSort::SortPairs(L.temp, bytes, k, v, (int)n, 0, bits, stream));
    if (v.Current() != L.vals[0])
        CGNN_CUDA(cudaMemcpyAsync(L.vals[0], v.Current(), sizeof(int32_t) * (size_t)n,
                                  cudaMemcpyDeviceToDevice, stream));
    *sorted_keys = k.Current();
    return CGNN_OK;
}

}  // namespace cgnn

using namespace cgnn;

extern "C" {

int cgnn_cluster_project(int dtype, const void *x, const void *planes, int64_t n, int64_t width,
                         int bits, void *proj, cgnn_stream_t stream) {
    CGNN_REQUIRE(proj != nullptr || n == 0 || bits == 0, "cluster_project: null output");
    return project(dtype, x, planes, n, width, bits, proj, nullptr, (cudaStream_t)stream);
}

int cgnn_cluster_codes(int dtype, const void *x, const void *planes, int64_t n, int64_t width,
                       int bits, int32_t *codes, cgnn_stream_t stream) {
    CGNN_REQUIRE(codes != nullptr || n == 0, "cluster_codes: null output");
    return project(dtype, x, planes, n, width, bits, nullptr, codes, (cudaStream_t)stream);
}

int cgnn_cluster_codes_from_projection(int dtype, const void *proj, int64_t n, int bits,
                                       int32_t *codes, cgnn_stream_t stream) {
    CGNN_REQUIRE(dtype == CGNN_F32 || dtype == CGNN_F64, "cluster: unknown dtype %d", dtype);
    CGNN_REQUIRE(bits >= 0 && bits <= 30, "cluster: hash bits must be in [0,30]");
    CGNN_REQUIRE(n >= 0 && n <= 0x7fffffffll, "cluster: node count exceeds int32 capacity");
    if (n == 0) return CGNN_OK;
    CGNN_REQUIRE(codes != nullptr && (proj != nullptr || bits == 0), "cluster: null pointer");
    if (dtype == CGNN_F32)
        codes_from_proj_kernel<float><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(
            (const float *)proj, n, bits, codes);
    else
        codes_from_proj_kernel<double><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(
            (const double *)proj, n, bits, codes);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

size_t cgnn_cluster_workspace_bytes(int64_t n, int bits) {
    (void)bits;
    if (n < 0 || n > 0x7fffffffll) return 0;
    return assign_layout(nullptr, n).total;
}

int cgnn_cluster_assign(const int32_t *codes, int64_t n, int bits, void *workspace,
                        size_t workspace_bytes, int64_t *ids, int64_t *active_out,
                        cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    CGNN_REQUIRE(bits >= 0 && bits <= 30, "cluster_assign: hash bits must be in [0,30]");
    CGNN_REQUIRE(n >= 0 && n <= 0x7fffffffll, "cluster_assign: node count exceeds int32 capacity");
    CGNN_REQUIRE(active_out != nullptr, "cluster_assign: null active_out");
    *active_out = 0;
    if (n == 0) return CGNN_OK;
    CGNN_REQUIRE(codes != nullptr && ids != nullptr && workspace != nullptr,
                 "cluster_assign: null pointer");
    CGNN_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0,
                 "cluster_assign: workspace must be 256-byte aligned");
    AssignLayout L = assign_layout(workspace, n);
    CGNN_REQUIRE(workspace_bytes >= L.total, "cluster_assign: workspace of %zu bytes needed, %zu given",
                 L.total, workspace_bytes);
    CGNN_CUDA(cudaMemcpyAsync(L.keys[0], codes, sizeof(int32_t) * (size_t)n,
                              cudaMemcpyDeviceToDevice, stream));
    int32_t *sorted = nullptr;
    int rc = sort_pairs(L, n, bits, &sorted, stream);
    if (rc != CGNN_OK) return rc;
    int32_t *flags = sorted == L.keys[0] ? L.keys[1] : L.keys[0];
    head_flags_kernel<<<grid_for(n), 256, 0, stream>>>(sorted, flags, n);
    CGNN_LAUNCH_CHECK();
    size_t bytes = L.temp_bytes;
    CGNN_CUDA(cub::DeviceScan::InclusiveSum(L.temp, bytes, flags, L.cid, (int)n, stream));
    scatter_ids_kernel<<<grid_for(n), 256, 0, stream>>>(L.vals[0], L.cid, flags, n, ids, L.segstart,
                                                        L.active);
    CGNN_LAUNCH_CHECK();
    // One synchronisation fetches `active`.  With it comes what the export step needs to build the
    // bucket plan without another round trip: when the buckets are few enough for one CTA to scan
    // (at most 2^20: the usual bit counts), the row statistics of the plan, taken on the device and
    // written behind `active`; otherwise, speculatively, the head of the segment-start array.
    HostSegments &hs = host_segments();
    std::lock_guard<std::mutex> guard(hs.lock);
    hs.workspace = workspace;
    hs.n = n;
    hs.valid = 0;
    hs.on_device = std::min<int64_t>(n, (int64_t)1 << bits) + 1 <= PLAN_DEVICE_MAX_ROWS;
    if (hs.on_device) {
        int32_t *header_dev = L.active + 16;  // inside the 256-byte slot of `active`
        rc = plan_stats_on_device(L.segstart, L.active, n, 0, header_dev, stream);
        if (rc != CGNN_OK) return rc;
        int32_t *host = hs.reserve(16 + PLAN_HEADER_WORDS);
        CGNN_CUDA(cudaMemcpyAsync(host, L.active, sizeof(int32_t) * (16 + PLAN_HEADER_WORDS), cudaMemcpyDeviceToHost,
                                  stream));
        CGNN_CUDA(cudaStreamSynchronize(stream));
        *active_out = host[0];
        return CGNN_OK;
    }
    const int64_t want = std::min<int64_t>(n + 2, std::min<int64_t>(((int64_t)1 << bits) + 2, (int64_t)1 << 20));
    int32_t *host = hs.reserve((size_t)want + 1);  // [0] receives `active`, the segment starts follow
    CGNN_CUDA(cudaMemcpyAsync(host, L.active, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    CGNN_CUDA(cudaMemcpyAsync(host + 1, L.segstart, sizeof(int32_t) * (size_t)want,
                              cudaMemcpyDeviceToHost, stream));
    CGNN_CUDA(cudaStreamSynchronize(stream));
    const int32_t active = host[0];
    hs.valid = (int64_t)active + 2 <= want ? (int64_t)active + 2 : 0;
    *active_out = active;
    return CGNN_OK;
}

int cgnn_cluster_assign_export(const void *workspace, int64_t n, int64_t active, int32_t *counts,
                               cgnn_plan **plan_out, int split, cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (plan_out) *plan_out = nullptr;
    CGNN_REQUIRE(n >= 0 && active >= 0 && active <= n, "assign_export: bad sizes");
    CGNN_REQUIRE(counts != nullptr, "assign_export: null counts");
    if (n == 0) {
        CGNN_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t), stream));
        return CGNN_OK;
    }
    CGNN_REQUIRE(workspace != nullptr, "assign_export: null workspace");
    AssignLayout L = assign_layout(const_cast<void *>(workspace), n);
    counts_kernel<<<grid_for(active + 1), 256, 0, stream>>>(L.segstart, active, counts);
    CGNN_LAUNCH_CHECK();
    if (!plan_out) return CGNN_OK;
    cgnn_plan *p = new cgnn_plan();
    cudaGetDevice(&p->device);
    p->rows = active + 1;
    p->nterms = 1;
    p->nnz[0] = n;
    const int32_t *rp[2] = {L.segstart, nullptr};
    const int32_t *cl[2] = {L.vals[0], nullptr};
    int rc;
    {
        HostSegments &hs = host_segments();
        std::lock_guard<std::mutex> guard(hs.lock);
        if (hs.workspace == workspace && hs.n == n && hs.on_device && split == 0 && hs.start[0] == active) {
            rc = plan_fill_on_device(p, L.segstart, L.vals[0], hs.start + 16, stream);
        } else {
            const bool have = hs.workspace == workspace && hs.n == n && !hs.on_device && hs.valid == active + 2;
            rc = plan_build(p, rp, cl, split, stream, have ? hs.start + 1 : nullptr, false);
        }
    }
    if (rc != CGNN_OK) {
        cgnn_plan_destroy(p);
        return rc;
    }
    *plan_out = p;
    return CGNN_OK;
}

int cgnn_plan_create_from_index(cgnn_plan **plan_out, const int64_t *index, int64_t n,
                                int64_t groups, int split, cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    CGNN_REQUIRE(plan_out != nullptr, "plan_from_index: null output");
    *plan_out = nullptr;
    CGNN_REQUIRE(n >= 0 && n < 0x7fffffffll && groups >= 0 && groups < 0x7fffffffll,
                 "plan_from_index: size out of 32-bit range");
    CGNN_REQUIRE(index != nullptr || n == 0, "plan_from_index: null index");
    CGNN_REQUIRE(groups > 0 || n == 0, "plan_from_index: entries but no groups");
    cgnn_plan *p = new cgnn_plan();
    cudaGetDevice(&p->device);
    p->rows = groups;
    p->nterms = 1;
    p->nnz[0] = n;
    void *ws = nullptr;
    int32_t *hist = nullptr, *rowptr = nullptr;
    int rc = CGNN_OK;
    do {
        AssignLayout L0 = assign_layout(nullptr, n);
        if (cudaMalloc(&ws, L0.total) != cudaSuccess ||
            cudaMalloc(&hist, sizeof(int32_t) * (size_t)(groups + 1)) != cudaSuccess ||
            cudaMalloc(&rowptr, sizeof(int32_t) * (size_t)(groups + 1)) != cudaSuccess) {
            set_error("plan_from_index: device allocation failed");
            rc = CGNN_ERR_CUDA;
            break;
        }
        AssignLayout L = assign_layout(ws, n);
        cudaMemsetAsync(hist, 0, sizeof(int32_t) * (size_t)(groups + 1), stream);
        if (n > 0) {
            index_to_key_kernel<<<grid_for(n), 256, 0, stream>>>(index, n, groups, L.keys[0], hist);
            int bits = 1;
            while (bits < 31 && ((int64_t)1 << bits) < groups) ++bits;
            int32_t *sorted = nullptr;
            rc = sort_pairs(L, n, bits, &sorted, stream);
            if (rc != CGNN_OK) break;
        }
        size_t bytes = L.temp_bytes;
        // The scan temp was sized for max(n,1)+2 items; a longer histogram gets its own.
        void *temp = L.temp;
        void *own_temp = nullptr;
        size_t need = 0;
        cub::DeviceScan::ExclusiveSum(nullptr, need, hist, rowptr, (int)(groups + 1));
        if (need > bytes) {
            if (cudaMalloc(&own_temp, need) != cudaSuccess) {
                set_error("plan_from_index: device allocation failed");
                rc = CGNN_ERR_CUDA;
                break;
            }
            temp = own_temp;
            bytes = need;
        }
        cudaError_t e = cub::DeviceScan::ExclusiveSum(temp, bytes, hist, rowptr, (int)(groups + 1), stream);
        cudaStreamSynchronize(stream);
        if (own_temp) cudaFree(own_temp);
        if (e != cudaSuccess) {
            set_error("plan_from_index: scan failed: %s", cudaGetErrorString(e));
            rc = CGNN_ERR_CUDA;
            break;
        }
        int status = 0;
        rc = cluster_status(&status);
        if (rc != CGNN_OK) break;
        if (status & STATUS_BAD_INDEX) {
            set_error("plan_from_index: index value outside [0, %lld)", (long long)groups);
            rc = CGNN_ERR_INVALID;
            break;
        }
        const int32_t *rp[2] = {rowptr, nullptr};
        const int32_t *cl[2] = {L.vals[0], nullptr};
        rc = plan_build(p, rp, cl, split, stream, nullptr, false);
    } while (0);
    if (ws) cudaFree(ws);
    if (hist) cudaFree(hist);
    if (rowptr) cudaFree(rowptr);
    if (rc != CGNN_OK) {
        cgnn_plan_destroy(p);
        return rc;
    }
    *plan_out = p;
    return CGNN_OK;
}

}  // extern "C"
