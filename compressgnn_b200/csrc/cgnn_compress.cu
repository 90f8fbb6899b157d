// Batch pair-substitution grammar compressor on the device.
//
// The reference reaches its CUDA compressor through `compress_csr_batch` of the module
// compressgnn_batch_cuda (src/offline/bindings/batch_cuda.cpp:3-9, chosen by
// loader/compression_backend.py:6-40); the source behind that binding is an external project that is
// not part of the reference tree.  What the reference's tests pin is the contract
// (tests/test_batch_compression.py:15-59): int32 (vlist, elist, n, rules), rule bodies made of smaller
// symbols, exact in-order expansion, and the CUDA result equal to the CPU result array for array.
// This file runs the same rounds as the host compressor of this package (host/cgnn_host.cpp,
// cgnn_host_compress_csr_batch) and produces the same arrays:
//   1. key of every adjacent symbol pair of every vertex row, radix-sorted, run-length counted;
//   2. pairs seen at least `min_frequency` times become candidate rules, ids ascending with the key;
//   3. parse: a candidate is substituted where it outweighs both overlapping neighbours
//      (weight = (count, id)), what is left is taken greedily from the left of each row;
//   4. rows are compacted with a scan, candidates the parse never used are dropped and the ids closed up.
// Everything is integer work on flat arrays: sort, scan and run-length steps are CUB calls, the rest
// are one-thread-per-symbol kernels, except the left-to-right step of the parse, which is one thread
// per row.  Two small device-to-host reads per round (candidate count; new length and rules kept).
#include <cub/cub.cuh>

#include <algorithm>
#include <vector>

#include "cgnn_common.cuh"

struct cgnn_compressed {
    int32_t *vlist = nullptr;  // device, rows + 1
    int32_t *elist = nullptr;  // device, entries
    int64_t n = 0, rules = 0, entries = 0;
};

namespace cgnn {
namespace {

constexpr uint64_t NO_PAIR = ~0ull;
constexpr int THREADS = 256;
static inline unsigned blocks_for(int64_t count) {
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(count, THREADS), 148 * 64));
}
#define GRID_STRIDE(i, count) \
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (count); i += (int64_t)blockDim.x * gridDim.x)

// Device buffers of one compression: the work arrays are carved out of one allocation (sized by a dry
// pass of the same requests), the rule pairs of each round are allocated as the rounds find them.
struct Arena {
    std::vector<void *> held;
    char *block = nullptr;
    size_t used = 0, capacity = 0;
    bool sizing = true;
    ~Arena() {
        for (void *p : held) cudaFree(p);
    }
    template <typename T>
    void carve(T **p, size_t count) {
        const size_t bytes = align_up(std::max<size_t>(count, 1) * sizeof(T), 256);
        *p = sizing ? nullptr : reinterpret_cast<T *>(block + used);
        used += bytes;
    }
    cudaError_t commit() {  // end of the dry pass
        capacity = used;
        used = 0;
        sizing = false;
        void *raw = nullptr;
        cudaError_t e = cudaMalloc(&raw, std::max<size_t>(capacity, 256));
        if (e == cudaSuccess) held.push_back(raw);
        block = reinterpret_cast<char *>(raw);
        return e;
    }
    template <typename T>
    cudaError_t get(T **p, size_t count) {
        void *raw = nullptr;
        cudaError_t e = cudaMalloc(&raw, std::max<size_t>(count, 1) * sizeof(T));
        if (e == cudaSuccess) held.push_back(raw);
        *p = reinterpret_cast<T *>(raw);
        return e;
    }
};

__global__ void load_rows_kernel(const int64_t *vlist, const int64_t *elist, int64_t n, int64_t total, int32_t *rowptr,
                                 int32_t *sym, int *bad) {
    GRID_STRIDE(i, n + 1) {
        const int64_t v = vlist[i];
        if (v < 0 || v > total || (i > 0 && v < vlist[i - 1]) || (i == 0 && v != 0)) atomicOr(bad, 1);
        rowptr[i] = (int32_t)v;
    }
    GRID_STRIDE(i, total) {
        const int64_t e = elist[i];
        if (e < 0 || e >= n) atomicOr(bad, 2);
        sym[i] = (int32_t)e;
    }
}

__global__ void row_of_kernel(const int32_t *rowptr, int64_t n, int32_t *row_of) {
    GRID_STRIDE(r, n)
        for (int32_t i = rowptr[r]; i < rowptr[r + 1]; ++i) row_of[i] = (int32_t)r;
}

// key[i] = (sym[i], sym[i+1]) packed into 2 * shift bits when both belong to one row
__global__ void pair_keys_kernel(const int32_t *sym, const int32_t *row_of, int64_t total, int shift, uint64_t *key) {
    GRID_STRIDE(i, total) {
        uint64_t k = NO_PAIR;
        if (i + 1 < total && row_of[i] == row_of[i + 1]) k = ((uint64_t)(uint32_t)sym[i] << shift) | (uint32_t)sym[i + 1];
        key[i] = k;
    }
}

__global__ void flag_candidates_kernel(const uint64_t *run_key, const int32_t *run_count, const int *num_runs,
                                       int min_frequency, int32_t *flag) {
    const int64_t runs = *num_runs;
    GRID_STRIDE(r, runs) flag[r] = (run_key[r] != NO_PAIR && run_count[r] >= min_frequency) ? 1 : 0;
}

__global__ void gather_candidates_kernel(const uint64_t *run_key, const int32_t *run_count, const int32_t *flag,
                                         const int32_t *slot, const int *num_runs, uint64_t *cand_key,
                                         int32_t *cand_count, int32_t *cand_total) {
    const int64_t runs = *num_runs;
    GRID_STRIDE(r, runs) {
        if (flag[r]) {
            cand_key[slot[r]] = run_key[r];
            cand_count[slot[r]] = run_count[r];
        }
        if (r == runs - 1) *cand_total = slot[r] + flag[r];
    }
    if (runs == 0 && blockIdx.x == 0 && threadIdx.x == 0) *cand_total = 0;
}

// weight[i] = (count of the pair at i) << 32 | (its candidate id), or 0 when the pair is no candidate
__global__ void weights_kernel(const uint64_t *key, int64_t total, const uint64_t *cand_key, const int32_t *cand_count,
                               int32_t candidates, int32_t base, uint64_t *weight) {
    GRID_STRIDE(i, total) {
        const uint64_t k = key[i];
        uint64_t w = 0;
        if (k != NO_PAIR) {
            int32_t lo = 0, hi = candidates;
            while (lo < hi) {
                const int32_t mid = (lo + hi) >> 1;
                if (cand_key[mid] < k) lo = mid + 1;
                else hi = mid;
            }
            if (lo < candidates && cand_key[lo] == k) w = ((uint64_t)(uint32_t)cand_count[lo] << 32) | (uint32_t)(base + lo);
        }
        weight[i] = w;
    }
}

// First step of the parse: a candidate that outweighs the pair before it and is not outweighed by the
// pair after it (pairs of its own row only).
__global__ void take_heavier_kernel(const uint64_t *key, const uint64_t *weight, int64_t total, uint8_t *take) {
    GRID_STRIDE(i, total) {
        const uint64_t w = weight[i];
        bool t = false;
        if (w != 0) {
            const bool has_prev = i > 0 && key[i - 1] != NO_PAIR;       // a pair of the same row sits before / after
            const bool has_next = i + 1 < total && key[i] != NO_PAIR && key[i + 1] != NO_PAIR;
            t = (!has_prev || w > weight[i - 1]) && (!has_next || w >= weight[i + 1]);
        }
        take[i] = t ? 1 : 0;
    }
}

// Second step: left to right along each row, a remaining candidate whose neighbours are free.
__global__ void take_greedy_kernel(const int32_t *rowptr, int64_t n, const uint64_t *weight, uint8_t *take) {
    GRID_STRIDE(r, n) {
        const int32_t begin = rowptr[r], pairs = rowptr[r + 1] - begin - 1;
        bool prev = false;
        for (int32_t i = 0; i < pairs; ++i) {
            bool t = take[begin + i] != 0;
            if (!t && weight[begin + i] != 0 && !prev && (i + 1 == pairs || !take[begin + i + 1])) {
                t = true;
                take[begin + i] = 1;
            }
            prev = t;
        }
    }
}

// A symbol is kept unless the pair before it was substituted; a substituted pair leaves its rule id.
__global__ void emit_kernel(const int32_t *sym, const uint64_t *key, const uint64_t *weight, const uint8_t *take,
                            int64_t total, int32_t base, int32_t *keep, int32_t *value, int32_t *uses) {
    GRID_STRIDE(i, total) {
        const bool swallowed = i > 0 && key[i - 1] != NO_PAIR && take[i - 1];
        const bool head = key[i] != NO_PAIR && take[i];
        keep[i] = swallowed ? 0 : 1;
        int32_t v = sym[i];
        if (head) {
            v = (int32_t)(uint32_t)weight[i];
            atomicAdd(&uses[v - base], 1);
        }
        value[i] = v;
    }
}

__global__ void compact_kernel(const int32_t *keep, const int32_t *slot, const int32_t *value, const int32_t *row_of,
                               int64_t total, int32_t *sym_out, int32_t *row_of_out, int32_t *new_total) {
    GRID_STRIDE(i, total) {
        if (keep[i]) {
            sym_out[slot[i]] = value[i];
            row_of_out[slot[i]] = row_of[i];
        }
        if (i == total - 1) *new_total = slot[i] + keep[i];
    }
}

// The first symbol of a row is always kept, so a row starts where its old first symbol went.
__global__ void move_rowptr_kernel(const int32_t *rowptr, const int32_t *slot, const int32_t *new_total, int64_t n,
                                   int64_t total, int32_t *rowptr_out) {
    GRID_STRIDE(r, n + 1) {
        const int32_t old = rowptr[r];
        rowptr_out[r] = old < total ? slot[old] : *new_total;
    }
}

__global__ void used_flags_kernel(const int32_t *uses, int32_t candidates, int32_t *used) {
    GRID_STRIDE(k, candidates) used[k] = uses[k] > 0 ? 1 : 0;
}

__global__ void keep_rules_kernel(const uint64_t *cand_key, const int32_t *used, const int32_t *rank, int32_t candidates,
                                  int shift, int32_t base, int32_t *remap, int32_t *rule_pairs, int32_t *kept) {
    const uint64_t low = (1ull << shift) - 1;
    GRID_STRIDE(k, candidates) {
        if (used[k]) {
            remap[k] = base + rank[k];
            rule_pairs[2 * (int64_t)rank[k]] = (int32_t)(cand_key[k] >> shift);
            rule_pairs[2 * (int64_t)rank[k] + 1] = (int32_t)(cand_key[k] & low);
        } else {
            remap[k] = -1;
        }
        if (k == candidates - 1) *kept = rank[k] + used[k];
    }
}

__global__ void remap_kernel(int32_t *sym, int64_t total, int32_t base, const int32_t *remap) {
    GRID_STRIDE(i, total) {
        const int32_t s = sym[i];
        if (s >= base) sym[i] = remap[s - base];
    }
}

__global__ void final_vlist_kernel(const int32_t *rowptr, int64_t n, int64_t rules, int32_t total, int32_t *vlist) {
    GRID_STRIDE(i, n + rules + 1) vlist[i] = i <= n ? rowptr[i] : total + 2 * (int32_t)(i - n);
}

static int bits_for(int64_t largest) {
    int bits = 1;
    while ((largest >> bits) != 0) ++bits;
    return bits;
}

}  // namespace
}  // namespace cgnn

using namespace cgnn;

extern "C" {

int cgnn_compress_csr_batch(const int64_t *vlist, const int64_t *elist, int64_t n, int rounds, int min_frequency,
                            cgnn_compressed **out, cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    CGNN_REQUIRE(out != nullptr, "compress_csr_batch: null result pointer");
    *out = nullptr;
    CGNN_REQUIRE(n >= 0 && (n == 0 || vlist != nullptr), "compress_csr_batch: null row pointers");
    CGNN_REQUIRE(min_frequency >= 3, "Batch compression needs min_pair_frequency >= 3");
    CGNN_REQUIRE(rounds >= 1, "compression_rounds must be positive");
    int64_t total64 = 0;
    if (n > 0) CGNN_CUDA(cudaMemcpyAsync(&total64, vlist + n, sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
    CGNN_CUDA(cudaStreamSynchronize(stream));
    CGNN_REQUIRE(total64 >= 0 && n + total64 < INT32_MAX, "CSR array exceeds int32 capacity");
    CGNN_REQUIRE(total64 == 0 || elist != nullptr, "compress_csr_batch: null edge list");
    const int64_t cap = total64;  // rows only shrink

    Arena arena;
    int32_t *rowptr[2], *sym[2], *row_of[2], *keep, *value, *slot, *run_count, *flag, *cand_count, *uses, *remap;
    uint64_t *key, *key_sorted, *run_key, *cand_key, *weight;
    uint8_t *take, *temp;
    int32_t *scalars;  // 0: bad input, 1: runs, 2: candidates, 3: new total, 4: rules kept
    // candidate arrays: at most one candidate per min_frequency pairs
    const size_t cand_cap = (size_t)(cap / min_frequency + 1);
    size_t temp_bytes = 0, need = 0;
    const int cap32 = (int)std::max<int64_t>(cap, 1);
    for (int pass = 0; pass < 2; ++pass) {  // 0: sizes only, 1: pointers into the one allocation
        for (int b = 0; b < 2; ++b) {
            arena.carve(&rowptr[b], (size_t)n + 1);
            arena.carve(&sym[b], (size_t)cap);
            arena.carve(&row_of[b], (size_t)cap);
        }
        arena.carve(&keep, (size_t)cap);
        arena.carve(&value, (size_t)cap);
        arena.carve(&slot, (size_t)cap);
        arena.carve(&run_count, (size_t)cap);
        arena.carve(&flag, (size_t)cap);
        arena.carve(&key, (size_t)cap);
        arena.carve(&key_sorted, (size_t)cap);
        arena.carve(&run_key, (size_t)cap);
        arena.carve(&weight, (size_t)cap);
        arena.carve(&take, (size_t)cap);
        arena.carve(&scalars, 8);
        arena.carve(&cand_key, cand_cap);
        arena.carve(&cand_count, cand_cap);
        arena.carve(&uses, cand_cap);
        arena.carve(&remap, cand_cap);
        if (pass == 0) {
            cub::DeviceRadixSort::SortKeys(nullptr, need, key, key_sorted, cap32, 0, 64, stream);
            temp_bytes = std::max(temp_bytes, need);
            cub::DeviceRunLengthEncode::Encode(nullptr, need, key_sorted, run_key, run_count, scalars + 1, cap32, stream);
            temp_bytes = std::max(temp_bytes, need);
            cub::DeviceScan::ExclusiveSum(nullptr, need, flag, slot, cap32, stream);
            temp_bytes = std::max(temp_bytes, need);
        }
        arena.carve(&temp, temp_bytes);
        if (pass == 0) CGNN_CUDA(arena.commit());
    }
    CGNN_CUDA(cudaMemsetAsync(scalars, 0, 8 * sizeof(int32_t), stream));
    int32_t *used = flag, *rank = slot;  // free again once the rows are compacted

    load_rows_kernel<<<blocks_for(std::max(n + 1, cap)), THREADS, 0, stream>>>(vlist, elist, n, cap, rowptr[0], sym[0],
                                                                              scalars);
    CGNN_LAUNCH_CHECK();
    int32_t host_scalars[8];
    CGNN_CUDA(cudaMemcpyAsync(host_scalars, scalars, sizeof(host_scalars), cudaMemcpyDeviceToHost, stream));
    CGNN_CUDA(cudaStreamSynchronize(stream));
    // nothing indexes with the row pointers before they are known to be sound
    CGNN_REQUIRE(!(host_scalars[0] & 1), "compress_csr_batch: row pointers must ascend from 0 to the edge count");
    CGNN_REQUIRE(!(host_scalars[0] & 2), "CSR value exceeds vertex range");
    row_of_kernel<<<blocks_for(n), THREADS, 0, stream>>>(rowptr[0], n, row_of[0]);
    CGNN_LAUNCH_CHECK();

    std::vector<std::pair<int32_t *, int32_t>> rule_blocks;  // (device pairs, count) of every round
    int64_t total = cap, rules = 0;
    int cur = 0;
    for (int round = 0; round < rounds && total > 1; ++round) {
        const int32_t base = (int32_t)(n + rules);
        const int shift = bits_for(std::max<int64_t>(base - 1, 1));
        const int total32 = (int)total;
        pair_keys_kernel<<<blocks_for(total), THREADS, 0, stream>>>(sym[cur], row_of[cur], total, shift, key);
        CGNN_LAUNCH_CHECK();
        need = temp_bytes;
        // pair keys use 2 * shift bits and the key of "no pair" is all ones: bit 2 * shift puts it last
        CGNN_CUDA(cub::DeviceRadixSort::SortKeys(temp, need, key, key_sorted, total32, 0, std::min(64, 2 * shift + 1),
                                                 stream));
        need = temp_bytes;
        CGNN_CUDA(cub::DeviceRunLengthEncode::Encode(temp, need, key_sorted, run_key, run_count, scalars + 1, total32,
                                                     stream));
        flag_candidates_kernel<<<blocks_for(total), THREADS, 0, stream>>>(run_key, run_count, scalars + 1, min_frequency,
                                                                          flag);
        CGNN_LAUNCH_CHECK();
        // (slots past the number of runs hold stale flags; the gather below stops at the number of runs)
        need = temp_bytes;
        CGNN_CUDA(cub::DeviceScan::ExclusiveSum(temp, need, flag, slot, total32, stream));
        gather_candidates_kernel<<<blocks_for(total), THREADS, 0, stream>>>(run_key, run_count, flag, slot, scalars + 1,
                                                                            cand_key, cand_count, scalars + 2);
        CGNN_LAUNCH_CHECK();
        CGNN_CUDA(cudaMemcpyAsync(host_scalars, scalars, sizeof(host_scalars), cudaMemcpyDeviceToHost, stream));
        CGNN_CUDA(cudaStreamSynchronize(stream));
        const int32_t candidates = host_scalars[2];
        if (candidates == 0) break;
        CGNN_REQUIRE((int64_t)base + candidates < INT32_MAX, "rule ids exceed int32 capacity");
        CGNN_REQUIRE((size_t)candidates <= cand_cap, "compress_csr_batch: candidate table overflow");

        weights_kernel<<<blocks_for(total), THREADS, 0, stream>>>(key, total, cand_key, cand_count, candidates, base,
                                                                  weight);
        CGNN_LAUNCH_CHECK();
        take_heavier_kernel<<<blocks_for(total), THREADS, 0, stream>>>(key, weight, total, take);
        CGNN_LAUNCH_CHECK();
        take_greedy_kernel<<<blocks_for(n), THREADS, 0, stream>>>(rowptr[cur], n, weight, take);
        CGNN_LAUNCH_CHECK();
        CGNN_CUDA(cudaMemsetAsync(uses, 0, (size_t)candidates * sizeof(int32_t), stream));
        emit_kernel<<<blocks_for(total), THREADS, 0, stream>>>(sym[cur], key, weight, take, total, base, keep, value,
                                                               uses);
        CGNN_LAUNCH_CHECK();
        need = temp_bytes;
        CGNN_CUDA(cub::DeviceScan::ExclusiveSum(temp, need, keep, slot, total32, stream));
        compact_kernel<<<blocks_for(total), THREADS, 0, stream>>>(keep, slot, value, row_of[cur], total, sym[cur ^ 1],
                                                                  row_of[cur ^ 1], scalars + 3);
        CGNN_LAUNCH_CHECK();
        move_rowptr_kernel<<<blocks_for(n + 1), THREADS, 0, stream>>>(rowptr[cur], slot, scalars + 3, n, total,
                                                                      rowptr[cur ^ 1]);
        CGNN_LAUNCH_CHECK();
        cur ^= 1;
        // candidates the parse never used are dropped, the others keep their order
        used_flags_kernel<<<blocks_for(candidates), THREADS, 0, stream>>>(uses, candidates, used);
        CGNN_LAUNCH_CHECK();
        need = temp_bytes;
        CGNN_CUDA(cub::DeviceScan::ExclusiveSum(temp, need, used, rank, candidates, stream));
        int32_t *pairs = nullptr;
        CGNN_CUDA(arena.get(&pairs, 2 * (size_t)candidates));
        keep_rules_kernel<<<blocks_for(candidates), THREADS, 0, stream>>>(cand_key, used, rank, candidates, shift, base,
                                                                          remap, pairs, scalars + 4);
        CGNN_LAUNCH_CHECK();
        CGNN_CUDA(cudaMemcpyAsync(host_scalars, scalars, sizeof(host_scalars), cudaMemcpyDeviceToHost, stream));
        CGNN_CUDA(cudaStreamSynchronize(stream));
        total = host_scalars[3];
        const int32_t kept = host_scalars[4];
        if (kept != candidates) {
            remap_kernel<<<blocks_for(total), THREADS, 0, stream>>>(sym[cur], total, base, remap);
            CGNN_LAUNCH_CHECK();
        }
        rule_blocks.emplace_back(pairs, kept);
        rules += kept;
    }

    CGNN_REQUIRE(total + 2 * rules < INT32_MAX, "compressed arrays exceed int32 capacity");
    auto *res = new cgnn_compressed();
    res->n = n;
    res->rules = rules;
    res->entries = total + 2 * rules;
    cudaError_t e = cudaMalloc(&res->vlist, (size_t)(n + rules + 1) * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&res->elist, std::max<size_t>((size_t)res->entries, 1) * sizeof(int32_t));
    if (e != cudaSuccess) {
        cgnn_compressed_destroy(res);
        set_error("compress_csr_batch: cudaMalloc of the result failed: %s", cudaGetErrorString(e));
        return CGNN_ERR_CUDA;
    }
    final_vlist_kernel<<<blocks_for(n + rules + 1), THREADS, 0, stream>>>(rowptr[cur], n, rules, (int32_t)total,
                                                                          res->vlist);
    cudaError_t launch = cudaGetLastError();
    if (launch == cudaSuccess && total > 0)
        launch = cudaMemcpyAsync(res->elist, sym[cur], (size_t)total * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream);
    int64_t at = total;
    for (const auto &block : rule_blocks) {
        if (launch == cudaSuccess && block.second > 0)
            launch = cudaMemcpyAsync(res->elist + at, block.first, 2 * (size_t)block.second * sizeof(int32_t),
                                     cudaMemcpyDeviceToDevice, stream);
        at += 2 * (int64_t)block.second;
    }
    if (launch == cudaSuccess) launch = cudaStreamSynchronize(stream);  // the arena is freed on return
    if (launch != cudaSuccess) {
        cgnn_compressed_destroy(res);
        set_error("compress_csr_batch: assembling the result failed: %s", cudaGetErrorString(launch));
        return CGNN_ERR_CUDA;
    }
    *out = res;
    return CGNN_OK;
}

int cgnn_compressed_info(const cgnn_compressed *c, int64_t info[3]) {
    CGNN_REQUIRE(c != nullptr && info != nullptr, "compressed_info: null argument");
    info[0] = c->n;
    info[1] = c->rules;
    info[2] = c->entries;
    return CGNN_OK;
}

int cgnn_compressed_copy(const cgnn_compressed *c, int32_t *vlist_out, int32_t *elist_out, cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    CGNN_REQUIRE(c != nullptr && vlist_out != nullptr, "compressed_copy: null argument");
    CGNN_REQUIRE(c->entries == 0 || elist_out != nullptr, "compressed_copy: null edge list");
    CGNN_CUDA(cudaMemcpyAsync(vlist_out, c->vlist, (size_t)(c->n + c->rules + 1) * sizeof(int32_t), cudaMemcpyDefault,
                              stream));
    if (c->entries > 0)
        CGNN_CUDA(cudaMemcpyAsync(elist_out, c->elist, (size_t)c->entries * sizeof(int32_t), cudaMemcpyDefault, stream));
    return CGNN_OK;
}

void cgnn_compressed_destroy(cgnn_compressed *c) {
    if (!c) return;
    cudaFree(c->vlist);
    cudaFree(c->elist);
    delete c;
}

}  // extern "C"
