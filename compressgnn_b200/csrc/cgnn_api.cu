// Library-wide entry points: version, the per-thread error message, the device status word.
#include <stdarg.h>

#include <algorithm>
#include <mutex>

#include "cgnn_plan.h"

namespace cgnn {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

namespace {
constexpr int PINNED_SLOTS = 4;
constexpr size_t PINNED_CAP = (size_t)64 << 20;
struct PinnedArena {
    void *ptr[PINNED_SLOTS] = {};
    size_t cap[PINNED_SLOTS] = {};
    cudaEvent_t busy[PINNED_SLOTS] = {};  // recorded behind the last copy that reads the slot
    bool pending[PINNED_SLOTS] = {};
    ~PinnedArena() {
        for (void *p : ptr)
            if (p) cudaFreeHost(p);  // may fail at process exit, when the context is gone: ignored
    }
};
PinnedArena &arena_of_thread() {
    static thread_local PinnedArena arena;
    return arena;
}
}  // namespace

void pinned_scratch_in_use(int slot, cudaStream_t stream) {
    PinnedArena &arena = arena_of_thread();
    if (slot < 0 || slot >= PINNED_SLOTS) return;
    if (arena.busy[slot] == nullptr &&
        cudaEventCreateWithFlags(&arena.busy[slot], cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        arena.busy[slot] = nullptr;
        cudaStreamSynchronize(stream);  // no event to wait on later: wait now
        return;
    }
    arena.pending[slot] = cudaEventRecord(arena.busy[slot], stream) == cudaSuccess;
    if (!arena.pending[slot]) cudaStreamSynchronize(stream);
}

void *pinned_scratch(size_t bytes, int slot) {
    PinnedArena &arena = arena_of_thread();
    if (slot < 0 || slot >= PINNED_SLOTS || bytes > PINNED_CAP) return nullptr;
    if (arena.pending[slot]) {
        cudaEventSynchronize(arena.busy[slot]);
        arena.pending[slot] = false;
    }
    if (arena.cap[slot] < bytes) {
        if (arena.ptr[slot]) cudaFreeHost(arena.ptr[slot]);
        arena.ptr[slot] = nullptr;
        arena.cap[slot] = 0;
        const size_t want = std::max<size_t>(bytes + bytes / 2, (size_t)1 << 16);
        void *p = nullptr;
        if (cudaHostAlloc(&p, want, cudaHostAllocDefault) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        arena.ptr[slot] = p;
        arena.cap[slot] = want;
    }
    return arena.ptr[slot];
}

cudaError_t pool_alloc(void **ptr, size_t bytes, cudaStream_t stream) {
    constexpr int MAX_DEVICES = 64;
    static std::mutex lock;
    static cudaMemPool_t pools[MAX_DEVICES] = {};
    int device = 0;
    cudaError_t rc = cudaGetDevice(&device);
    if (rc != cudaSuccess) return rc;
    if (device < 0 || device >= MAX_DEVICES) return cudaMallocAsync(ptr, bytes, stream);
    cudaMemPool_t pool;
    {
        std::lock_guard<std::mutex> guard(lock);
        if (pools[device] == nullptr) {
            cudaMemPoolProps props = {};
            props.allocType = cudaMemAllocationTypePinned;
            props.location.type = cudaMemLocationTypeDevice;
            props.location.id = device;
            rc = cudaMemPoolCreate(&pools[device], &props);
            if (rc != cudaSuccess) {
                pools[device] = nullptr;
                return rc;
            }
            uint64_t keep = UINT64_MAX;  // freed blocks stay in the pool for the next plan
            cudaMemPoolSetAttribute(pools[device], cudaMemPoolAttrReleaseThreshold, &keep);
        }
        pool = pools[device];
    }
    return cudaMallocFromPoolAsync(ptr, bytes, pool, stream);
}

}  // namespace cgnn

namespace cgnn {
int sample_status(int *out);  // cgnn_sample.cu
}

extern "C" {

int cgnn_version(void) { return 100; }

const char *cgnn_last_error(void) { return cgnn::g_error; }

int cgnn_device_status(int *status_out) {
    CGNN_REQUIRE(status_out != nullptr, "device_status: null output");
    int a = 0, b = 0, c = 0;
    CGNN_CUDA(cudaDeviceSynchronize());
    int rc = cgnn::segreduce_status(&a);
    if (rc == CGNN_OK) rc = cgnn::gather_status(&b);
    if (rc == CGNN_OK) rc = cgnn::cluster_status(&c);
    int d = 0;
    if (rc == CGNN_OK) rc = cgnn::sample_status(&d);  // defined in cgnn_sample.cu
    *status_out = a | b | c | d;
    return rc;
}

}  // extern "C"
