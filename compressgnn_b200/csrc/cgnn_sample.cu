// Neighbour sampling on the compressed graph (device side of one hop).
//
// ref: neighbor_sample_sim_impl, src/sample/csrc/neighbor_sample.h:27-131, with get_neighbor and
// get_neighbor_list of src/sample/csrc/storage_api.h:7-118 (host code there; bound as
// compressgnn_sample.neighbor_sample_cg_sim).  A node's neighbours are its v2v entries followed by the
// expansion of its v2r rules; `vertex_degree` / `rule_degree` (gen_degree) give the sizes, so the i-th
// neighbour is found by skipping whole rules.  Per hop the reference does, node by node in frontier
// order: degree <= fan-out -> all neighbours in list order (v2v, then the rules breadth first, then every
// listed rule's own vertices); otherwise Floyd's scheme draws `fan-out` distinct neighbour indices
// (for j = degree - k .. degree - 1: a uniform index below j, replaced by j if already drawn).  New nodes
// get local ids in the order they are first seen.
//
// Here a hop is four steps on the device: every frontier node picks its neighbours (one thread per node:
// the picks of a node are sequential by definition and few), then first-seen relabelling without a hash
// map: atomicMin of the pick position into a per-vertex table, a flag for the winning positions, a scan,
// and a scatter.  Random indices come from Philox4x32 counted by (hop, frontier position, draw) under the
// caller's seed instead of the host generator the reference asks, so a hop does not depend on thread
// order and the CPU restatement can draw the same numbers.
//
// The children of a rule are read from ONE rule -> rule CSR (the union of the reference's level blocks,
// each rule's children live in exactly one of them).  storage_api.h looks a rule's children up in the
// level numbered by the descent depth, which finds them only for rules without nested rules; on such
// graphs both orders below are the reference's, on deeper ones they are what its comments describe.
#include <algorithm>

#include "cgnn_common.cuh"

namespace cgnn {
namespace {

constexpr int THREADS = 128;
constexpr int32_t NO_LOCAL_ID = INT32_MAX;  // value of local_of[] and first[] for a vertex not seen yet
static inline unsigned blocks_for(int64_t count) {
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(count, THREADS), 148 * 32));
}
#define GRID_STRIDE(i, count) \
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (count); i += (int64_t)blockDim.x * gridDim.x)

static __device__ int g_sample_status = 0;

// Philox4x32 with 7 rounds (Salmon et al., SC 2011): counter (c0, c1, c2, c3), key (k0, k1).
__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint64_t seed) {
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
    return c0;
}

struct GraphView {
    const int64_t *v2v_ptr, *v2v_col, *v2r_ptr, *v2r_col, *r2v_ptr, *r2v_col, *r2r_ptr, *r2r_col;
    const int64_t *v_degree, *r_degree;
    int64_t n, r;
};

// The `index`-th neighbour of `node` (index < vertex_degree[node]); -1 if the degree tables do not match.
__device__ int64_t neighbor_at(const GraphView &g, int64_t node, int64_t index) {
    const int64_t vb = g.v2v_ptr[node], vcount = g.v2v_ptr[node + 1] - vb;
    if (index < vcount) return g.v2v_col[vb + index];
    index -= vcount;
    for (int64_t e = g.v2r_ptr[node]; e < g.v2r_ptr[node + 1]; ++e) {
        int64_t rule = g.v2r_col[e];
        const int64_t size = g.r_degree[rule];
        if (index >= size) {
            index -= size;
            continue;
        }
        for (int depth = 0; depth < 64; ++depth) {  // a rule graph is far shallower; the bound keeps the walk finite
            const int64_t rb = g.r2v_ptr[rule], own = g.r2v_ptr[rule + 1] - rb;
            if (index < own) return g.r2v_col[rb + index];
            index -= own;
            int64_t next = -1;
            for (int64_t c = g.r2r_ptr[rule]; c < g.r2r_ptr[rule + 1]; ++c) {
                const int64_t child = g.r2r_col[c], below = g.r_degree[child];
                if (index < below) {
                    next = child;
                    break;
                }
                index -= below;
            }
            if (next < 0) return -1;
            rule = next;
        }
        return -1;
    }
    return -1;
}

__global__ void count_kernel(const GraphView g, const int64_t *samples, int64_t begin, int64_t frontier, int64_t fanout,
                             int64_t *count) {
    GRID_STRIDE(i, frontier) {
        const int64_t node = samples[begin + i];
        int64_t k = 0;
        if (node >= 0 && node < g.n) {
            const int64_t degree = g.v_degree[node];
            k = degree <= 0 ? 0 : (fanout >= degree ? degree : (fanout > 0 ? fanout : 0));
        } else {
            atomicOr(&g_sample_status, STATUS_BAD_INDEX);
        }
        count[i] = k;
    }
}

// offset = exclusive scan of count.  picked[offset[i] .. +count[i]) receives the neighbours of frontier node i,
// source[...] its local id; `queue` (same layout) is scratch for the breadth-first rule list of a take-all node.
__global__ void pick_kernel(const GraphView g, const int64_t *samples, int64_t begin, int64_t frontier, int64_t fanout,
                            const int64_t *count, const int64_t *offset, uint32_t hop, uint64_t seed, int64_t *picked,
                            int64_t *source, int64_t *queue) {
    GRID_STRIDE(i, frontier) {
        const int64_t k = count[i];
        if (k == 0) continue;
        const int64_t node = samples[begin + i], at = offset[i], degree = g.v_degree[node];
        for (int64_t j = 0; j < k; ++j) source[at + j] = begin + i;
        if (k == degree) {  // everything, in list order
            int64_t out = 0;
            for (int64_t e = g.v2v_ptr[node]; e < g.v2v_ptr[node + 1] && out < k; ++e) picked[at + out++] = g.v2v_col[e];
            int64_t rules = 0;  // breadth-first list of the rules below the node (each holds >= 1 vertex: rules <= k)
            for (int64_t e = g.v2r_ptr[node]; e < g.v2r_ptr[node + 1] && rules < k; ++e) queue[at + rules++] = g.v2r_col[e];
            for (int64_t head = 0; head < rules; ++head) {
                const int64_t rule = queue[at + head];
                for (int64_t c = g.r2r_ptr[rule]; c < g.r2r_ptr[rule + 1] && rules < k; ++c) queue[at + rules++] = g.r2r_col[c];
            }
            for (int64_t head = 0; head < rules; ++head) {
                const int64_t rule = queue[at + head];
                for (int64_t e = g.r2v_ptr[rule]; e < g.r2v_ptr[rule + 1] && out < k; ++e) picked[at + out++] = g.r2v_col[e];
            }
            if (out != k) {
                atomicOr(&g_sample_status, STATUS_BAD_CSR);  // the degree table does not match the graph
                for (; out < k; ++out) picked[at + out] = node;
            }
        } else {  // Floyd: k distinct indices below degree; queue[] keeps the indices drawn so far
            for (int64_t t = 0; t < k; ++t) {
                const int64_t j = degree - k + t;  // >= 1
                const uint32_t word = philox_first_word((uint32_t)(begin + i), (uint32_t)((begin + i) >> 32), (uint32_t)t, hop, seed);
                int64_t index = (int64_t)(((uint64_t)word * (uint64_t)j) >> 32);  // uniform below j
                for (int64_t s = 0; s < t; ++s)
                    if (queue[at + s] == index) {
                        index = j;
                        break;
                    }
                queue[at + t] = index;
                int64_t v = neighbor_at(g, node, index);
                if (v < 0) {
                    atomicOr(&g_sample_status, STATUS_BAD_CSR);
                    v = node;
                }
                picked[at + t] = v;
            }
        }
    }
}

// first[v] = smallest pick position of a vertex that has no local id yet
__global__ void claim_kernel(const int64_t *picked, int64_t total, int64_t n, const int32_t *local_of, int32_t *first) {
    GRID_STRIDE(p, total) {
        const int64_t v = picked[p];
        if (v < 0 || v >= n) {
            atomicOr(&g_sample_status, STATUS_BAD_INDEX);
            continue;
        }
        if (local_of[v] == NO_LOCAL_ID) atomicMin(&first[v], (int32_t)p);
    }
}

__global__ void flag_kernel(const int64_t *picked, int64_t total, int64_t n, const int32_t *local_of, const int32_t *first,
                            int64_t *is_new) {
    GRID_STRIDE(p, total) {
        const int64_t v = picked[p];
        is_new[p] = (v >= 0 && v < n && local_of[v] == NO_LOCAL_ID && first[v] == (int32_t)p) ? 1 : 0;
    }
}

// rank = exclusive scan of is_new.  Local id of a new vertex = end + rank of its first pick.
__global__ void relabel_kernel(const int64_t *picked, int64_t total, int64_t n, const int32_t *local_of, const int32_t *first,
                               const int64_t *is_new, const int64_t *rank, int64_t end, int64_t *target,
                               int64_t *samples) {
    GRID_STRIDE(p, total) {
        const int64_t v = picked[p];
        int64_t local = 0;
        if (v >= 0 && v < n) local = local_of[v] != NO_LOCAL_ID ? local_of[v] : end + rank[first[v]];
        target[p] = local;
        if (is_new[p]) samples[end + rank[p]] = v;
    }
}

__global__ void commit_kernel(const int64_t *picked, int64_t total, const int64_t *is_new, const int64_t *rank, int64_t end,
                              int32_t *local_of, int32_t *first) {
    GRID_STRIDE(p, total) {
        if (is_new[p]) {
            const int64_t v = picked[p];
            local_of[v] = (int32_t)(end + rank[p]);
            first[v] = NO_LOCAL_ID;
        }
    }
}

__global__ void seed_kernel(const int64_t *samples, int64_t count, int64_t n, int32_t *local_of) {
    GRID_STRIDE(i, count) {
        const int64_t v = samples[i];
        if (v >= 0 && v < n) atomicMin(&local_of[v], (int32_t)i);  // a repeated seed keeps its first position
        else atomicOr(&g_sample_status, STATUS_BAD_INDEX);
    }
}

static GraphView view_of(const cgnn_sample_graph *g) {
    GraphView v;
    v.v2v_ptr = g->v2v_ptr, v.v2v_col = g->v2v_col, v.v2r_ptr = g->v2r_ptr, v.v2r_col = g->v2r_col;
    v.r2v_ptr = g->r2v_ptr, v.r2v_col = g->r2v_col, v.r2r_ptr = g->r2r_ptr, v.r2r_col = g->r2r_col;
    v.v_degree = g->vertex_degree, v.r_degree = g->rule_degree, v.n = g->vertices, v.r = g->rules;
    return v;
}

}  // namespace

int sample_status(int *out) {
    int zero = 0;
    CGNN_CUDA(cudaMemcpyFromSymbol(out, g_sample_status, sizeof(int)));
    CGNN_CUDA(cudaMemcpyToSymbol(g_sample_status, &zero, sizeof(int)));
    return CGNN_OK;
}

}  // namespace cgnn

using namespace cgnn;

extern "C" {

int cgnn_sample_seed(const int64_t *samples, int64_t count, int64_t vertices, int32_t *local_of, cgnn_stream_t stream) {
    CGNN_REQUIRE(count >= 0 && (count == 0 || (samples != nullptr && local_of != nullptr)), "sample_seed: null argument");
    if (count == 0) return CGNN_OK;
    seed_kernel<<<blocks_for(count), THREADS, 0, (cudaStream_t)stream>>>(samples, count, vertices, local_of);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

int cgnn_sample_count(const cgnn_sample_graph *graph, const int64_t *samples, int64_t begin, int64_t frontier,
                      int64_t fanout, int64_t *count, cgnn_stream_t stream) {
    CGNN_REQUIRE(graph != nullptr && frontier >= 0 && (frontier == 0 || (samples != nullptr && count != nullptr)),
                 "sample_count: null argument");
    if (frontier == 0) return CGNN_OK;
    count_kernel<<<blocks_for(frontier), THREADS, 0, (cudaStream_t)stream>>>(view_of(graph), samples, begin, frontier, fanout,
                                                                            count);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

int cgnn_sample_pick(const cgnn_sample_graph *graph, const int64_t *samples, int64_t begin, int64_t frontier, int64_t fanout,
                     const int64_t *count, const int64_t *offset, uint32_t hop, uint64_t seed, int64_t *picked,
                     int64_t *source, int64_t *scratch, cgnn_stream_t stream) {
    CGNN_REQUIRE(graph != nullptr && frontier >= 0, "sample_pick: null graph");
    if (frontier == 0) return CGNN_OK;
    CGNN_REQUIRE(samples && count && offset && picked && source && scratch, "sample_pick: null argument");
    pick_kernel<<<blocks_for(frontier), THREADS, 0, (cudaStream_t)stream>>>(view_of(graph), samples, begin, frontier, fanout,
                                                                           count, offset, hop, seed, picked, source, scratch);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

int cgnn_sample_claim(const int64_t *picked, int64_t total, int64_t vertices, const int32_t *local_of, int32_t *first,
                      int64_t *is_new, cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    CGNN_REQUIRE(total >= 0 && total < INT32_MAX, "sample_claim: too many picks for one hop");
    if (total == 0) return CGNN_OK;
    CGNN_REQUIRE(picked && local_of && first && is_new, "sample_claim: null argument");
    claim_kernel<<<blocks_for(total), THREADS, 0, stream>>>(picked, total, vertices, local_of, first);
    CGNN_LAUNCH_CHECK();
    flag_kernel<<<blocks_for(total), THREADS, 0, stream>>>(picked, total, vertices, local_of, first, is_new);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

int cgnn_sample_relabel(const int64_t *picked, int64_t total, int64_t vertices, const int64_t *is_new, const int64_t *rank,
                        int64_t end, int32_t *local_of, int32_t *first, int64_t *target, int64_t *samples,
                        cgnn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (total == 0) return CGNN_OK;
    CGNN_REQUIRE(picked && is_new && rank && local_of && first && target && samples, "sample_relabel: null argument");
    relabel_kernel<<<blocks_for(total), THREADS, 0, stream>>>(picked, total, vertices, local_of, first, is_new, rank, end,
                                                             target, samples);
    CGNN_LAUNCH_CHECK();
    commit_kernel<<<blocks_for(total), THREADS, 0, stream>>>(picked, total, is_new, rank, end, local_of, first);
    CGNN_LAUNCH_CHECK();
    return CGNN_OK;
}

}  // extern "C"
