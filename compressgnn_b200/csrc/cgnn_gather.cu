// Row expansion: out[r,:] = f(table[index[r],:]) for every node r.
//
// Serves the fused reconstruction (gather + bias + ReLU) and the mean backward (gather /
// bucket size).  The table of representatives is small and stays in L2; the kernel is a
// streaming writer of n*width elements, so it uses 128-bit streaming stores and keeps
// several rows per lane group in flight.  A bad index sets a status bit and yields zeros
// (the reference traps the GPU instead).
#include <algorithm>

#include "cgnn_plan.h"

#ifndef CGNN_EXPAND_WIDE
#define CGNN_EXPAND_WIDE 1
#endif
#ifndef CGNN_EXPAND_WIDE_MINBLOCKS
#define CGNN_EXPAND_WIDE_MINBLOCKS 3
#endif
#ifndef CGNN_EXPAND_RPG
#define CGNN_EXPAND_RPG 4
#endif

namespace cgnn {

static __device__ int g_gather_status = 0;

int gather_status(int *out) {
    int zero = 0;
    CGNN_CUDA(cudaMemcpyFromSymbol(out, g_gather_status, sizeof(int)));
    CGNN_CUDA(cudaMemcpyToSymbol(g_gather_status, &zero, sizeof(int)));
    return CGNN_OK;
}

template <typename T>
struct ExpandArgs {
    const T *table;
    const int64_t *index;
    const T *bias;              // optional [width]
    const int32_t *div_counts;  // optional [groups]: divide by max(count[g], 1)
    int relu;
    T *out;
    int64_t n, width, groups;
    // optional dropout after the activation: an element is dropped when its 32-bit random word is below
    // drop_threshold, the survivors are multiplied by keep_scale = 1 / (1 - p); 0 = no dropout
    uint32_t drop_threshold = 0;
    T keep_scale = T(1);
    uint64_t seed = 0;
};

// Philox4x32 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC 2011) with 7
// rounds: four 32-bit words for the counter (element-vector index, 0) under the key `seed`.  Counter
// based, so the words of an element do not depend on which thread produces them.
__device__ __forceinline__ uint4 philox4x32_7(uint64_t counter, uint64_t seed) {
    uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0x243F6A88u, c3 = 0x85A308D3u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int round = 0; round < 7; ++round) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
}

// Dropout of the VW values of the vector that starts at element `first` of the output (VW is 1, 2 or 4 and
// divides `first`).  Element e takes word e % 4 of the Philox block counted e / 4, so the mask is a
// function of (seed, element index) alone: the same whatever the element type or the kernel that writes it.
template <typename T, int VW>
__device__ __forceinline__ void drop_vector(Vec<T, VW> &y, int64_t first, uint32_t threshold, T keep_scale,
                                            uint64_t seed) {
    static_assert(VW == 1 || VW == 2 || VW == 4, "a vector lies inside one block of four random words");
    const uint4 r = philox4x32_7((uint64_t)first >> 2, seed);
    if constexpr (VW == 4) {
        const uint32_t word[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) y.v[k] = word[k] < threshold ? T(0) : y.v[k] * keep_scale;
    } else if constexpr (VW == 2) {
        const bool upper = (first & 2) != 0;
        const uint32_t w0 = upper ? r.z : r.x, w1 = upper ? r.w : r.y;
        y.v[0] = w0 < threshold ? T(0) : y.v[0] * keep_scale;
        y.v[1] = w1 < threshold ? T(0) : y.v[1] * keep_scale;
    } else {
        const int at = (int)(first & 3);
        const uint32_t w = at == 0 ? r.x : at == 1 ? r.y : at == 2 ? r.z : r.w;
        y.v[0] = w < threshold ? T(0) : y.v[0] * keep_scale;
    }
}

// A group of LPR lanes expands LPR consecutive node rows per step: lane l reads index[r0 + l]
// (one coalesced load), the indices are broadcast by shuffle, and U table rows are in flight
// per lane before any output row is stored.
template <typename T, int VW, int LPR, int U>
__global__ void __launch_bounds__(256) expand_kernel(const ExpandArgs<T> a) {
    using V = Vec<T, VW>;
    constexpr int GPW = 32 / LPR;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (LPR - 1);
    const unsigned gmask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (lane & ~(LPR - 1)));
    const int64_t group = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * GPW + lane / LPR;
    const int64_t ngroups = (int64_t)gridDim.x * (blockDim.x >> 5) * GPW;
    const int64_t vecs = a.width / VW;
    for (int64_t r0 = group * LPR; r0 < a.n; r0 += ngroups * LPR) {
        int32_t gi = -1;
        if (r0 + gl < a.n) {
            const int64_t g = a.index[r0 + gl];
            if (g < 0 || g >= a.groups) atomicOr(&g_gather_status, STATUS_BAD_INDEX);
            else gi = (int32_t)g;
        }
        const int cnt = (int)min((int64_t)LPR, a.n - r0);
        for (int64_t cbase = 0; cbase < vecs; cbase += LPR) {  // uniform trip count in the group
            const int64_t c = cbase + gl;
            const bool active = c < vecs;
            V b = vec_zero<T, VW>();
            if (a.bias && active) b = vec_load<T, VW>(a.bias + c * VW);
            for (int j = 0; j < cnt; j += U) {
                V x[U];
                T divisor[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int32_t g = __shfl_sync(gmask, gi, j + u, LPR);
                    x[u] = vec_zero<T, VW>();
                    divisor[u] = T(1);
                    if (active && j + u < cnt && g >= 0) {
                        x[u] = vec_load<T, VW>(a.table + (int64_t)g * a.width + c * VW);
                        if (a.div_counts) divisor[u] = (T)max(a.div_counts[g], 1);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (active && j + u < cnt) {
                        V y;
#pragma unroll
                        for (int k = 0; k < VW; ++k) {
                            T v = x[u].v[k];
                            if (a.bias) v += b.v[k];
                            if (a.div_counts) v = v / divisor[u];
                            y.v[k] = (a.relu && v < T(0)) ? T(0) : v;
                        }
                        if (a.drop_threshold)
                            drop_vector<T, VW>(y, (r0 + j + u) * a.width + c * VW, a.drop_threshold, a.keep_scale, a.seed);
                        vec_store_cs<T, VW>(a.out + (r0 + j + u) * a.width + c * VW, y);
                    }
                }
            }
        }
    }
}

// Rows of more than 16 vectors without a divisor (the fused reconstruction and the mean backward
// at benchmark widths): a warp expands 32 node rows per step, each lane owns VPL vectors of a row,
// and bias / ReLU are compile-time switches, so that the per-row work is one index shuffle, one
// row-base multiply, VPL loads, the epilogue and VPL streaming stores.
template <typename T, int VW, int VPL, int U, bool BIAS, bool RELU, bool DROP>
__global__ void __launch_bounds__(256, CGNN_EXPAND_WIDE_MINBLOCKS) expand_wide_kernel(const ExpandArgs<T> a) {
    using V = Vec<T, VW>;
    constexpr unsigned FULL = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int64_t vecs = a.width / VW;
    for (int64_t r0 = warp * 32; r0 < a.n; r0 += nwarps * 32) {
        int32_t gi = -1;
        if (r0 + lane < a.n) {
            const int64_t g = a.index[r0 + lane];
            if (g < 0 || g >= a.groups) atomicOr(&g_gather_status, STATUS_BAD_INDEX);
            else gi = (int32_t)g;
        }
        const int cnt = (int)min((int64_t)32, a.n - r0);
        for (int64_t cbase = 0; cbase < vecs; cbase += 32 * VPL) {  // uniform trip count
            bool act[VPL];
            int64_t col[VPL];
            V b[VPL];
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                const int64_t c = cbase + p * 32 + lane;
                act[p] = c < vecs;
                col[p] = c * VW;
                b[p] = vec_zero<T, VW>();
                if (BIAS && act[p]) b[p] = vec_load<T, VW>(a.bias + col[p]);
            }
            T *orow = a.out + r0 * a.width;
            for (int j = 0; j < cnt; j += U) {
                V x[U][VPL];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int32_t g = __shfl_sync(FULL, gi, (j + u) & 31);
                    const bool live = j + u < cnt && g >= 0;  // a bad index yields zeros
                    const T *trow = a.table + (int64_t)(live ? g : 0) * a.width;
#pragma unroll
                    for (int p = 0; p < VPL; ++p) {
                        x[u][p] = vec_zero<T, VW>();
                        if (live && act[p]) x[u][p] = vec_load<T, VW>(trow + col[p]);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (j + u < cnt) {
#pragma unroll
                        for (int p = 0; p < VPL; ++p) {
                            if (act[p]) {
                                V y;
#pragma unroll
                                for (int k = 0; k < VW; ++k) {
                                    T v = x[u][p].v[k];
                                    if (BIAS) v += b[p].v[k];
                                    y.v[k] = (RELU && v < T(0)) ? T(0) : v;
                                }
                                if constexpr (DROP)
                                    drop_vector<T, VW>(y, (orow - a.out) + col[p], a.drop_threshold, a.keep_scale, a.seed);
                                vec_store_cs<T, VW>(orow + col[p], y);
                            }
                        }
                    }
                    orow += a.width;
                }
            }
        }
    }
}

template <typename T, int VW, int VPL>
static int launch_expand_wide(const ExpandArgs<T> &a, cudaStream_t stream) {
    constexpr int U = 8 / VPL;  // 8 vectors in flight per lane
    const int64_t blocks = std::min<int64_t>(ceil_div(a.n, 32 * 8), 148 * 32);
    const bool bias = a.bias != nullptr, relu = a.relu != 0;
    if (a.drop_threshold) {  // the hidden layers of the model: always with ReLU, with or without bias
        if (bias)
            expand_wide_kernel<T, VW, VPL, U, true, true, true><<<(unsigned)blocks, 256, 0, stream>>>(a);
        else
            expand_wide_kernel<T, VW, VPL, U, false, true, true><<<(unsigned)blocks, 256, 0, stream>>>(a);
    } else if (bias && relu)
        expand_wide_kernel<T, VW, VPL, U, true, true, false><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else if (bias)
        expand_wide_kernel<T, VW, VPL, U, true, false, false><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else if (relu)
        expand_wide_kernel<T, VW, VPL, U, false, true, false><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else
        expand_wide_kernel<T, VW, VPL, U, false, false, false><<<(unsigned)blocks, 256, 0, stream>>>(a);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

// table[g,:] / max(count[g],1) for the (small) group table, one thread per element.
template <typename T>
__global__ void scale_rows_kernel(const T *table, const int32_t *count, T *out, int64_t groups,
                                  int64_t width) {
    const int64_t total = groups * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)blockDim.x * gridDim.x)
        out[i] = table[i] / (T)max(count[i / width], 1);
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, int VW, int LPR>
static int launch_expand(const ExpandArgs<T> &a, cudaStream_t stream) {
    constexpr int U = CGNN_EXPAND_RPG;  // table rows in flight per lane
    const int64_t groups_needed = ceil_div(a.n, LPR);
    const int64_t per_block = 8 * (32 / LPR);
    const int64_t blocks = std::min<int64_t>(ceil_div(groups_needed, per_block), 148 * 32);
    expand_kernel<T, VW, LPR, U><<<(unsigned)blocks, 256, 0, stream>>>(a);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

// Rows whose byte length is no multiple of 16 (47 class scores: 188 bytes): the output is written as ONE
// flat array in aligned 16-byte vectors, a vector taking its elements from up to two node rows.  The
// table rows it reads are few and stay in cache; what matters is that every store is a whole aligned vector
// instead of one element per lane with rows starting at odd offsets.
template <typename T>
__global__ void __launch_bounds__(256) expand_flat_kernel(const ExpandArgs<T> a) {
    constexpr int VW = 16 / (int)sizeof(T);
    using V = Vec<T, VW>;
    const int64_t total = a.n * a.width, vectors = total / VW;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vectors; i += (int64_t)blockDim.x * gridDim.x) {
        const int64_t first = i * VW;
        int64_t r = first / a.width;
        int64_t c = first - r * a.width;
        V y;
#pragma unroll
        for (int k = 0; k < VW; ++k) {
            const int64_t g = a.index[r];
            T v = T(0);
            if (g < 0 || g >= a.groups) atomicOr(&g_gather_status, STATUS_BAD_INDEX);
            else v = a.table[g * a.width + c];
            if (a.bias) v += a.bias[c];
            y.v[k] = (a.relu && v < T(0)) ? T(0) : v;
            if (++c == a.width) {
                c = 0;
                ++r;
            }
        }
        if (a.drop_threshold) drop_vector<T, VW>(y, first, a.drop_threshold, a.keep_scale, a.seed);
        vec_store_cs<T, VW>(a.out + first, y);
    }
    // the last total % VW elements
    if (blockIdx.x == 0 && threadIdx.x < total - vectors * VW) {
        const int64_t e = vectors * VW + threadIdx.x, r = e / a.width, c = e - r * a.width;
        const int64_t g = a.index[r];
        T v = T(0);
        if (g < 0 || g >= a.groups) atomicOr(&g_gather_status, STATUS_BAD_INDEX);
        else v = a.table[g * a.width + c];
        if (a.bias) v += a.bias[c];
        Vec<T, 1> y;
        y.v[0] = (a.relu && v < T(0)) ? T(0) : v;
        if (a.drop_threshold) drop_vector<T, 1>(y, e, a.drop_threshold, a.keep_scale, a.seed);
        a.out[e] = y.v[0];
    }
}

template <typename T>
static int expand_typed(const ExpandArgs<T> &a, cudaStream_t stream) {
    constexpr int VWMAX = 16 / (int)sizeof(T);
    if (a.n == 0 || a.width == 0) return CGNN_OK;
    const bool vec = a.width % VWMAX == 0 && aligned16(a.table) && aligned16(a.out) &&
                     aligned16(a.bias);
    if (vec) {
        const int64_t vecs = a.width / VWMAX;
#if CGNN_EXPAND_WIDE
        if (vecs > 16 && a.div_counts == nullptr) {
            if (vecs > 32) return launch_expand_wide<T, VWMAX, 2>(a, stream);
            return launch_expand_wide<T, VWMAX, 1>(a, stream);
        }
#endif
        if (vecs <= 4) return launch_expand<T, VWMAX, 4>(a, stream);
        if (vecs <= 8) return launch_expand<T, VWMAX, 8>(a, stream);
        if (vecs <= 16) return launch_expand<T, VWMAX, 16>(a, stream);
        return launch_expand<T, VWMAX, 32>(a, stream);
    }
    if (a.div_counts == nullptr && aligned16(a.out) && a.width > 4) {
        const int64_t vectors = a.n * a.width / VWMAX;
        const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(ceil_div(vectors, 256), 148 * 16));
        expand_flat_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(a);
        CGNN_LAUNCH_CHECK();
        return CGNN_OK;
    }
    if (a.width <= 4) return launch_expand<T, 1, 4>(a, stream);
    if (a.width <= 8) return launch_expand<T, 1, 8>(a, stream);
    if (a.width <= 16) return launch_expand<T, 1, 16>(a, stream);
    return launch_expand<T, 1, 32>(a, stream);
}

static int expand(int dtype, int64_t n, int64_t width, int64_t groups, const void *table,
                  const int64_t *index, const void *bias, const int32_t *div_counts, int relu,
                  void *out, cudaStream_t stream, double drop_p = 0.0, uint64_t seed = 0) {
    CGNN_REQUIRE(dtype == CGNN_F32 || dtype == CGNN_F64, "gather: unknown dtype %d", dtype);
    CGNN_REQUIRE(n >= 0 && width >= 0 && groups >= 0, "gather: negative size");
    if (n > 0 && width > 0)
        CGNN_REQUIRE(table != nullptr && index != nullptr && out != nullptr,
                     "gather: null pointer");
    uint32_t threshold = 0;
    double keep_scale = 1.0;
    if (drop_p > 0.0) {
        threshold = (uint32_t)std::min<double>(drop_p * 4294967296.0, 4294967295.0);
        keep_scale = 1.0 / (1.0 - drop_p);
    }
    if (dtype == CGNN_F32) {
        ExpandArgs<float> a{(const float *)table, index, (const float *)bias, div_counts, relu,
                            (float *)out, n, width, groups, threshold, (float)keep_scale, seed};
        return expand_typed<float>(a, stream);
    }
    ExpandArgs<double> a{(const double *)table, index, (const double *)bias, div_counts, relu,
                         (double *)out, n, width, groups, threshold, keep_scale, seed};
    return expand_typed<double>(a, stream);
}

}  // namespace cgnn

using namespace cgnn;

extern "C" {

int cgnn_cluster_mean_backward(int dtype, int64_t n, int64_t width, int64_t groups,
                               const void *grad, const int64_t *index, const int32_t *count,
                               void *out, void *scaled, cgnn_stream_t stream) {
    CGNN_REQUIRE(count != nullptr || n == 0, "mean_backward: null counts");
    CGNN_REQUIRE(dtype == CGNN_F32 || dtype == CGNN_F64, "gather: unknown dtype %d", dtype);
    if (scaled == nullptr || n == 0 || width == 0 || groups == 0)
        return expand(dtype, n, width, groups, grad, index, nullptr, count, 0, out,
                      (cudaStream_t)stream);
    CGNN_REQUIRE(grad != nullptr, "mean_backward: null gradient");
    const int64_t total = groups * width;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(total, 256), 148 * 8);
    if (dtype == CGNN_F32)
        scale_rows_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>(
            (const float *)grad, count, (float *)scaled, groups, width);
    else
        scale_rows_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>(
            (const double *)grad, count, (double *)scaled, groups, width);
    CGNN_LAUNCH_CHECK();
    return expand(dtype, n, width, groups, scaled, index, nullptr, nullptr, 0, out,
                  (cudaStream_t)stream);
}

int cgnn_cluster_reconstruct(int dtype, int64_t n, int64_t width, int64_t groups,
                             const void *reps, const int64_t *index, const void *bias, int relu,
                             void *out, cgnn_stream_t stream) {
    return expand(dtype, n, width, groups, reps, index, bias, nullptr, relu, out,
                  (cudaStream_t)stream);
}

int cgnn_cluster_reconstruct_dropout(int dtype, int64_t n, int64_t width, int64_t groups,
                                     const void *reps, const int64_t *index, const void *bias,
                                     double drop_p, uint64_t seed, void *out, cgnn_stream_t stream) {
    CGNN_REQUIRE(drop_p >= 0.0 && drop_p < 1.0, "reconstruct_dropout: the drop probability must lie in [0, 1)");
    return expand(dtype, n, width, groups, reps, index, bias, nullptr, 1, out, (cudaStream_t)stream, drop_p, seed);
}

}  // extern "C"
