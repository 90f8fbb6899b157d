// Shared host/device helpers for the cgnn_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/cgnn_b200.h"

namespace cgnn {

// Thread-local message behind cgnn_last_error(); defined in cgnn_api.cu.
void set_error(const char *fmt, ...);

#define CGNN_CUDA(call)                                                                    \
    do {                                                                                   \
        cudaError_t cgnn_e_ = (call);                                                      \
        if (cgnn_e_ != cudaSuccess) {                                                      \
            ::cgnn::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(cgnn_e_), \
                              __FILE__, __LINE__);                                         \
            return CGNN_ERR_CUDA;                                                          \
        }                                                                                  \
    } while (0)

#define CGNN_REQUIRE(cond, ...)                                                            \
    do {                                                                                   \
        if (!(cond)) {                                                                     \
            ::cgnn::set_error(__VA_ARGS__);                                                \
            return CGNN_ERR_INVALID;                                                       \
        }                                                                                  \
    } while (0)

#define CGNN_LAUNCH_CHECK()                                                                \
    do {                                                                                   \
        cudaError_t cgnn_e_ = cudaGetLastError();                                          \
        if (cgnn_e_ != cudaSuccess) {                                                      \
            ::cgnn::set_error("kernel launch failed: %s (%s:%d)",                          \
                              cudaGetErrorString(cgnn_e_), __FILE__, __LINE__);            \
            return CGNN_ERR_CUDA;                                                          \
        }                                                                                  \
    } while (0)

// Bits of the device status word (cgnn_device_status).  A kernel that meets a bad index
// records the bit, skips the access and carries on; nothing traps.
enum : int { STATUS_BAD_INDEX = 1, STATUS_WAIT_EXPIRED = 2, STATUS_BAD_CSR = 4 };

// A VW-wide vector of T that moves with one instruction (16 bytes at most).
template <typename T, int VW>
struct alignas(sizeof(T) * VW) Vec {
    T v[VW];
};

template <typename T, int VW>
__device__ __forceinline__ Vec<T, VW> vec_zero() {
    Vec<T, VW> r;
#pragma unroll
    for (int i = 0; i < VW; ++i) r.v[i] = T(0);
    return r;
}

template <typename T, int VW>
__device__ __forceinline__ Vec<T, VW> vec_load(const T *p) {
    return *reinterpret_cast<const Vec<T, VW> *>(p);
}

// Load that bypasses L1 (data written by another SM during the same launch).
template <typename T, int VW>
__device__ __forceinline__ Vec<T, VW> vec_load_cg(const T *p) {
    Vec<T, VW> r;
    if constexpr (sizeof(T) * VW == 16) {
        float4 t = __ldcg(reinterpret_cast<const float4 *>(p));
        r = *reinterpret_cast<Vec<T, VW> *>(&t);
    } else if constexpr (sizeof(T) * VW == 8) {
        float2 t = __ldcg(reinterpret_cast<const float2 *>(p));
        r = *reinterpret_cast<Vec<T, VW> *>(&t);
    } else {
        float t = __ldcg(reinterpret_cast<const float *>(p));
        r = *reinterpret_cast<Vec<T, VW> *>(&t);
    }
    return r;
}

template <typename T, int VW>
__device__ __forceinline__ void vec_store(T *p, const Vec<T, VW> &x) {
    *reinterpret_cast<Vec<T, VW> *>(p) = x;
}

// Streaming store: written once, not read again by this kernel.
template <typename T, int VW>
__device__ __forceinline__ void vec_store_cs(T *p, const Vec<T, VW> &x) {
    if constexpr (sizeof(T) * VW == 16) {
        __stcs(reinterpret_cast<float4 *>(p), *reinterpret_cast<const float4 *>(&x));
    } else if constexpr (sizeof(T) * VW == 8) {
        __stcs(reinterpret_cast<float2 *>(p), *reinterpret_cast<const float2 *>(&x));
    } else {
        __stcs(reinterpret_cast<float *>(p), *reinterpret_cast<const float *>(&x));
    }
}

// Page-locked host scratch of the calling thread, grow-only, reused from call to call (the callers
// synchronise their stream before they return).  Copies to and from pageable memory are staged by
// the driver and cost the host ~100 us each; an assignment refresh makes four of them.  Returns
// nullptr when page-locked memory cannot be had or `bytes` exceeds the cap: use pageable memory then.
void *pinned_scratch(size_t bytes, int slot);
// Marks the slot as read by work queued on `stream` up to now: the next pinned_scratch() of the slot
// waits for that work (normally long finished) instead of the caller synchronising the stream.
void pinned_scratch_in_use(int slot, cudaStream_t stream);

// Stream-ordered device allocation from a pool the library owns (one per device, nothing is given
// back to the driver until the process ends): a plan is built and dropped at every assignment
// refresh, and with the default pool's release threshold of zero every cudaMallocAsync after a
// synchronisation went back to the driver (~250 us of host time).
cudaError_t pool_alloc(void **ptr, size_t bytes, cudaStream_t stream);

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

}  // namespace cgnn
