/*
 * TEST INFRASTRUCTURE -- not product code.
 *
 * Plain-C, single-threaded restatement of the CPU algorithms of ZhengChenCS/CompressGNN's
 * hot path.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
 * load this file; the product (compressgnn_b200) never does.
 *
 * Each function cites the reference file:line it follows.  Index arrays are int64 and
 * values fp32/fp64, exactly as the reference stores them.
 *
 * Build: gcc -O2 -ffp-contract=off -shared -fPIC cgnn_oracle.c -lm -o libcgnn_oracle.so
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------ */
/* SpMM, method "rowbalance": src/runtime/csrc/sparse/cpu/spmm_cpu.cpp:42-70.            */
/* Per row: a zeroed row accumulator, edges in CSR order, vals[k] += mat[dst,k]*val,     */
/* then out[row,k] += vals[k] (out is pre-zeroed by the caller when no `out` is passed,  */
/* spmm_cpu.cpp:19-28).                                                                  */
/* ------------------------------------------------------------------------------------ */
#define DEF_SPMM(T, SUF)                                                                   \
    int oracle_spmm_rowbalance_##SUF(const int64_t *rowptr, const int64_t *col,           \
                                     const T *val, const T *mat, int64_t rows,            \
                                     int64_t width, T *out) {                              \
        T *acc = (T *)malloc(sizeof(T) * (size_t)(width > 0 ? width : 1));                 \
        if (!acc) return 1;                                                                \
        for (int64_t r = 0; r < rows; ++r) {                                               \
            for (int64_t k = 0; k < width; ++k) acc[k] = 0;                                \
            for (int64_t e = rowptr[r]; e < rowptr[r + 1]; ++e) {                          \
                const T v = val[e];                                                        \
                const T *src = mat + col[e] * width;                                       \
                for (int64_t k = 0; k < width; ++k) acc[k] += src[k] * v;                  \
            }                                                                              \
            for (int64_t k = 0; k < width; ++k) out[r * width + k] += acc[k];              \
        }                                                                                  \
        free(acc);                                                                         \
        return 0;                                                                          \
    }
DEF_SPMM(float, f32)
DEF_SPMM(double, f64)

/* ------------------------------------------------------------------------------------ */
/* LSH projection: the reference calls input.mm(planes)                                  */
/* (src/runtime/csrc/cluster/cpu/cluster_cpu.cpp:41, cuda/cluster_kernel.cu:136) and      */
/* leaves the summation order to the BLAS.  The restatement fixes the order that the     */
/* CUDA kernel documents: p = fma(x[r,k], w[k,h], p), k ascending, p starting at +0.     */
/* ------------------------------------------------------------------------------------ */
int oracle_project_f32(const float *x, const float *planes, int64_t n, int64_t width,
                       int bits, float *proj) {
    for (int64_t r = 0; r < n; ++r)
        for (int h = 0; h < bits; ++h) {
            float p = 0.0f;
            for (int64_t k = 0; k < width; ++k) p = fmaf(x[r * width + k], planes[k * bits + h], p);
            proj[r * bits + h] = p;
        }
    return 0;
}
int oracle_project_f64(const double *x, const double *planes, int64_t n, int64_t width,
                       int bits, double *proj) {
    for (int64_t r = 0; r < n; ++r)
        for (int h = 0; h < bits; ++h) {
            double p = 0.0;
            for (int64_t k = 0; k < width; ++k) p = fma(x[r * width + k], planes[k * bits + h], p);
            proj[r * bits + h] = p;
        }
    return 0;
}

/* Column-sharded projection: the feature axis is cut into `shards` contiguous blocks    */
/* (the last block takes the remainder); each block is reduced in the order above and    */
/* the block partials are added in ascending block order, starting from block 0's value. */
int oracle_project_sharded_f32(const float *x, const float *planes, int64_t n, int64_t width,
                               int bits, int shards, float *proj) {
    int64_t per = (width + shards - 1) / shards;
    for (int64_t r = 0; r < n; ++r)
        for (int h = 0; h < bits; ++h) {
            float total = 0.0f;
            for (int s = 0; s < shards; ++s) {
                int64_t k0 = s * per, k1 = k0 + per < width ? k0 + per : width;
                float p = 0.0f;
                for (int64_t k = k0; k < k1; ++k) p = fmaf(x[r * width + k], planes[k * bits + h], p);
                total = s == 0 ? p : total + p;
            }
            proj[r * bits + h] = total;
        }
    return 0;
}

/* Sign packing, MSB first, strict `> 0`: cluster_cpu.cpp:45-57, cluster_kernel.cu:41-50. */
#define DEF_CODES(T, SUF)                                                                  \
    int oracle_codes_##SUF(const T *proj, int64_t n, int bits, int32_t *codes) {           \
        for (int64_t r = 0; r < n; ++r) {                                                  \
            int32_t id = 0;                                                                \
            for (int h = 0; h < bits; ++h) id = (id << 1) | (proj[r * bits + h] > 0 ? 1 : 0); \
            codes[r] = id;                                                                 \
        }                                                                                  \
        return 0;                                                                          \
    }
DEF_CODES(float, f32)
DEF_CODES(double, f64)

/* Bucket compaction: flag array over 2^bits raw codes, inclusive prefix, remap, so that */
/* ids are 1-based and ascend with the raw code (cluster_cpu.cpp:58-68); counts as       */
/* torch.bincount(index, minlength=active+1) (layer/CompressgnnCluster.py:47-50), hence  */
/* counts[0] == 0.  `counts` must hold n+1 entries (active <= n).                        */
int oracle_assign(const int32_t *codes, int64_t n, int bits, int64_t *ids, int32_t *counts,
                  int64_t *active_out) {
    int64_t buckets = (int64_t)1 << bits;
    int32_t *flag = (int32_t *)calloc((size_t)buckets, sizeof(int32_t));
    if (!flag) return 1;
    for (int64_t r = 0; r < n; ++r) flag[codes[r]] = 1;
    int32_t run = 0;
    for (int64_t b = 0; b < buckets; ++b) { run += flag[b]; flag[b] = run; }
    int64_t active = n ? flag[buckets - 1] : 0;
    for (int64_t b = 0; b <= active; ++b) counts[b] = 0;
    for (int64_t r = 0; r < n; ++r) { ids[r] = flag[codes[r]]; counts[ids[r]] += 1; }
    *active_out = active;
    free(flag);
    return 0;
}

/* ------------------------------------------------------------------------------------ */
/* Mean representatives: sum rows per bucket in row order, then divide by max(count,1):  */
/* cluster_kernel.cu:60-75 (sum_features + divide_counts), CPU scatter_mean              */
/* (layer/CompressgnnCluster.py:16-19).  Backward: layer/CompressgnnCluster.py:22-25,    */
/* cluster_kernel.cu:76-85.                                                              */
/* Reconstruct: gather + bias + ReLU (`value < 0 ? 0 : value`), cluster_kernel.cu:86-97, */
/* layer/CompressgnnReconstruct.py:39-42; backward cluster_kernel.cu:98-108 (the mask is */
/* `output <= 0`), bias gradient = column sum of the representative gradient             */
/* (layer/CompressgnnReconstruct.py:26).                                                 */
/* ------------------------------------------------------------------------------------ */
#define DEF_CLUSTER(T, SUF)                                                                \
    int oracle_mean_##SUF(const T *x, const int64_t *index, const int32_t *count,          \
                          int64_t n, int64_t width, int64_t groups, T *out) {              \
        memset(out, 0, sizeof(T) * (size_t)(groups * width));                              \
        for (int64_t r = 0; r < n; ++r) {                                                  \
            if (index[r] < 0 || index[r] >= groups) return 2;                              \
            for (int64_t k = 0; k < width; ++k) out[index[r] * width + k] += x[r * width + k]; \
        }                                                                                  \
        for (int64_t g = 0; g < groups; ++g) {                                             \
            T d = (T)(count[g] > 1 ? count[g] : 1);                                        \
            for (int64_t k = 0; k < width; ++k) out[g * width + k] /= d;                   \
        }                                                                                  \
        return 0;                                                                          \
    }                                                                                      \
    int oracle_mean_backward_##SUF(const T *grad, const int64_t *index, const int32_t *count, \
                                   int64_t n, int64_t width, int64_t groups, T *out) {     \
        for (int64_t r = 0; r < n; ++r) {                                                  \
            int64_t g = index[r];                                                          \
            if (g < 0 || g >= groups) return 2;                                            \
            T d = (T)(count[g] > 1 ? count[g] : 1);                                        \
            for (int64_t k = 0; k < width; ++k) out[r * width + k] = grad[g * width + k] / d; \
        }                                                                                  \
        return 0;                                                                          \
    }                                                                                      \
    int oracle_reconstruct_##SUF(const T *reps, const int64_t *index, const T *bias,       \
                                 int relu, int64_t n, int64_t width, int64_t groups, T *out) { \
        for (int64_t r = 0; r < n; ++r) {                                                  \
            int64_t g = index[r];                                                          \
            if (g < 0 || g >= groups) return 2;                                            \
            for (int64_t k = 0; k < width; ++k) {                                          \
                T v = reps[g * width + k];                                                 \
                if (bias) v += bias[k];                                                    \
                out[r * width + k] = (relu && v < 0) ? (T)0 : v;                           \
            }                                                                              \
        }                                                                                  \
        return 0;                                                                          \
    }                                                                                      \
    int oracle_reconstruct_backward_##SUF(const T *grad, const T *output,                  \
                                          const int64_t *index, int relu, int64_t n,       \
                                          int64_t width, int64_t groups, T *out,           \
                                          T *bias_grad) {                                  \
        memset(out, 0, sizeof(T) * (size_t)(groups * width));                              \
        for (int64_t r = 0; r < n; ++r) {                                                  \
            int64_t g = index[r];                                                          \
            if (g < 0 || g >= groups) return 2;                                            \
            for (int64_t k = 0; k < width; ++k) {                                          \
                T v = (relu && output[r * width + k] <= 0) ? (T)0 : grad[r * width + k];   \
                out[g * width + k] += v;                                                   \
            }                                                                              \
        }                                                                                  \
        if (bias_grad)                                                                     \
            for (int64_t k = 0; k < width; ++k) {                                          \
                T s = 0;                                                                   \
                for (int64_t g = 0; g < groups; ++g) s += out[g * width + k];              \
                bias_grad[k] = s;                                                          \
            }                                                                              \
        return 0;                                                                          \
    }
DEF_CLUSTER(float, f32)
DEF_CLUSTER(double, f64)
