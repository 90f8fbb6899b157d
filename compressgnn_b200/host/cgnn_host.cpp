// Host-side graph preparation for the compressed-propagation path (runs once, on the CPU,
// before training): self loops, GCN normalisation of a compressed graph, a batch
// pair-substitution grammar compressor, the two rule filters, the four-way block partition,
// the topological split of the rule-to-rule block into levels, degrees, and seeded synthetic
// graph generators.
//
// The numeric contracts follow ZhengChenCS/CompressGNN's src/offline/csrc (cited per
// function) so that the CompressGraph / CompressgnnData objects built from them have the
// reference's layout; the code is written from those contracts, with flat arrays and a C ABI
// (numpy arrays in, result handle out) instead of pybind11.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <omp.h>
#include <parallel/algorithm>
#include <random>
#include <string>
#include <vector>

#define CGNN_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;

struct Result {
    std::vector<std::vector<int64_t>> i64;
    std::vector<std::vector<float>> f32;
    int64_t scalars[8] = {0, 0, 0, 0, 0, 0, 0, 0};
};

int fail(const std::string &msg) {
    g_error = msg;
    return 1;
}

using Rows = std::vector<std::vector<int64_t>>;

Rows rows_from_csr(const int64_t *vlist, const int64_t *elist, int64_t total) {
    Rows g((size_t)total);
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < total; ++v) g[v].assign(elist + vlist[v], elist + vlist[v + 1]);
    return g;
}

// graphT[x] lists, in ascending v and with multiplicity, the rows v that contain rule x (x >= n).  The
// reference keeps these lists for vertices as well and splices them on every inlining
// (filter.h:31-67); nothing ever reads a vertex's list -- neither a decision nor the output -- and with
// hubs in thousands of rows those splices were most of the run time, so they are not kept here.
Rows referencing_rows(const int64_t *vlist, const int64_t *elist, int64_t total, int64_t n) {
    Rows t((size_t)total);
    std::vector<int32_t> uses((size_t)(total - n), 0);  // exact capacities first: no list is reallocated while it fills
    const int64_t edges = vlist[total];
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < edges; ++e)
        if (elist[e] >= n) {
#pragma omp atomic
            ++uses[(size_t)(elist[e] - n)];
        }
#pragma omp parallel for schedule(static)
    for (int64_t x = n; x < total; ++x) t[x].reserve((size_t)uses[(size_t)(x - n)]);
    for (int64_t v = 0; v < total; ++v)
        for (int64_t e = vlist[v]; e < vlist[v + 1]; ++e)
            if (elist[e] >= n) t[elist[e]].push_back(v);
    return t;
}

// Replace the first occurrence of `id` in `list` by `body` (order preserved).
void splice_first(std::vector<int64_t> &list, int64_t id, const std::vector<int64_t> &body) {
    auto it = std::find(list.begin(), list.end(), id);
    if (it == list.end()) return;
    auto pos = list.erase(it);
    list.insert(pos, body.begin(), body.end());
}

// Inline rule `id` into every row that references it and hand its references to its
// children (ref: mergeRule, src/offline/csrc/filter.h:31-67, depth_filter.h:17-40).
template <typename ParentHook, typename ChildHook>
void inline_rule(int64_t id, int64_t n, Rows &graph, Rows &graphT, ParentHook on_parent, ChildHook on_child) {
    // neither list is spliced below (a rule is no parent or child of itself), so they are read in place
    const std::vector<int64_t> &body = graph[id];
    const std::vector<int64_t> &parents = graphT[id];
    for (int64_t node : parents) {
        splice_first(graph[node], id, body);
        on_parent(node, (int64_t)body.size());
    }
    for (int64_t child : body) {
        if (child >= n) splice_first(graphT[child], id, parents);
        on_child(child);
    }
}

// Renumber the surviving rules densely and emit the CSR (ref: genNewIdForRule /
// genNewGraphCSR, src/offline/csrc/util.h:107-164).
void emit_filtered(const Rows &graph, const std::vector<char> &removed, int64_t n, int64_t r,
                   Result *res) {
    std::vector<int64_t> new_id((size_t)r);
    int64_t cur = n;
    for (int64_t i = 0; i < r; ++i) {
        new_id[i] = cur;
        if (!removed[i]) ++cur;
    }
    // row pointers of the surviving rows first, then every row copied to its place in parallel
    std::vector<int64_t> keep;
    keep.reserve((size_t)(n + r));
    for (int64_t v = 0; v < n + r; ++v)
        if (v < n || !removed[v - n]) keep.push_back(v);
    std::vector<int64_t> vl(keep.size() + 1, 0);
    for (size_t i = 0; i < keep.size(); ++i) vl[i + 1] = vl[i] + (int64_t)graph[keep[i]].size();
    std::vector<int64_t> el((size_t)vl.back());
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)keep.size(); ++i) {
        int64_t at = vl[(size_t)i];
        for (int64_t d : graph[keep[(size_t)i]]) el[(size_t)at++] = d >= n ? new_id[d - n] : d;
    }
    res->i64 = {std::move(vl), std::move(el)};
    res->scalars[0] = n;
    res->scalars[1] = cur - n;
}

// Depth of every node counted from the vertices: a rule's depth is one more than the
// deepest row that references it (ref: gen_vertex_order_csr, src/offline/csrc/gen_mask.h:187-233).
// Returns max depth + 1, the value the reference calls m_depth.
int rule_depths(const int64_t *vlist, const int64_t *elist, int64_t n, int64_t r,
                std::vector<int> &order) {
    const int INIT = 100000;
    order.assign((size_t)(n + r), INIT);
    std::vector<int64_t> indeg((size_t)r, 0);
    const int64_t edges = vlist[n + r];
    for (int64_t e = 0; e < edges; ++e)
        if (elist[e] >= n) ++indeg[elist[e] - n];
    std::vector<int64_t> work, next;
    for (int64_t v = 0; v < n; ++v) {
        order[v] = 0;
        work.push_back(v);
    }
    int step = 1;
    while (!work.empty()) {
        for (int64_t src : work)
            for (int64_t e = vlist[src]; e < vlist[src + 1]; ++e) {
                const int64_t dst = elist[e];
                if (dst >= n && order[dst] == INIT && --indeg[dst - n] == 0) {
                    order[dst] = step;
                    next.push_back(dst);
                }
            }
        ++step;
        std::swap(work, next);
        next.clear();
    }
    return step - 1;
}

}  // namespace

CGNN_HOST_API const char *cgnn_host_last_error() { return g_error.c_str(); }

CGNN_HOST_API int64_t cgnn_host_result_count(const Result *r, int kind) {
    return kind == 0 ? (int64_t)r->i64.size() : (int64_t)r->f32.size();
}
CGNN_HOST_API int64_t cgnn_host_result_size(const Result *r, int kind, int i) {
    return kind == 0 ? (int64_t)r->i64[i].size() : (int64_t)r->f32[i].size();
}
CGNN_HOST_API void cgnn_host_result_copy(const Result *r, int kind, int i, void *dst) {
    if (kind == 0)
        std::memcpy(dst, r->i64[i].data(), r->i64[i].size() * sizeof(int64_t));
    else
        std::memcpy(dst, r->f32[i].data(), r->f32[i].size() * sizeof(float));
}
CGNN_HOST_API int64_t cgnn_host_result_scalar(const Result *r, int i) { return r->scalars[i]; }
CGNN_HOST_API void cgnn_host_result_free(Result *r) { delete r; }

// ---------------------------------------------------------------------------------------
// Self loops and normalisation
// ---------------------------------------------------------------------------------------

// Insert (v,v) into every sorted row that lacks it (ref: add_self_loop_csr,
// src/offline/csrc/add_self_loop.h:17-44).
CGNN_HOST_API int cgnn_host_add_self_loop_csr(const int64_t *vlist, const int64_t *elist, int64_t n,
                                              Result **out) {
    auto *res = new Result();
    // which rows lack the loop (rows are independent), the new row pointers, then every row copied in parallel
    std::vector<int64_t> vl((size_t)n + 1, 0);
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < n; ++v) {
        const int64_t *begin = elist + vlist[v], *end = elist + vlist[v + 1];
        const int64_t *at = std::lower_bound(begin, end, v);  // rows are sorted
        vl[(size_t)v + 1] = (end - begin) + ((at == end || *at != v) ? 1 : 0);
    }
    for (int64_t v = 0; v < n; ++v) vl[(size_t)v + 1] += vl[(size_t)v];
    std::vector<int64_t> el((size_t)vl[(size_t)n]);
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < n; ++v) {
        int64_t e = vlist[v], o = vl[(size_t)v];
        const int64_t end = vlist[v + 1];
        for (; e < end && elist[e] < v; ++e) el[(size_t)o++] = elist[e];
        if (e == end || elist[e] != v) el[(size_t)o++] = v;
        for (; e < end; ++e) el[(size_t)o++] = elist[e];
    }
    res->i64 = {std::move(vl), std::move(el)};
    *out = res;
    return 0;
}

// 1/sqrt(1e-6 + in-degree), accumulated in fp32 (ref: get_norm_degree,
// src/offline/csrc/norm.h:20-45; INF is 1e-6 in util.h:16).
CGNN_HOST_API int cgnn_host_get_norm_degree(const int64_t *dst, int64_t edges, int64_t n, float *out) {
    // The reference adds 1.0f to 1e-6f once per incoming edge, in fp32: the result depends on the number of
    // additions only, so the edges are counted in parallel and every vertex repeats its own additions.
    std::vector<int32_t> count((size_t)n, 0);
    bool bad = false;
#pragma omp parallel for schedule(static) reduction(|| : bad)
    for (int64_t e = 0; e < edges; ++e) {
        if (dst[e] < 0 || dst[e] >= n) {
            bad = true;
        } else {
#pragma omp atomic
            ++count[(size_t)dst[e]];
        }
    }
    if (bad) return fail("get_norm_degree: destination out of range");
#pragma omp parallel for schedule(dynamic, 4096)
    for (int64_t v = 0; v < n; ++v) {
        float sum = 1e-6;
        for (int32_t k = 0; k < count[(size_t)v]; ++k) sum += 1;
        out[v] = 1 / std::sqrt(sum);
    }
    return 0;
}

// Edge weights of a compressed graph: vertex->vertex d_v*d_u, vertex->rule d_v,
// rule->vertex d_u, rule->rule 1 (ref: gcn_norm_csr_compress, src/offline/csrc/norm.h:179-216).
CGNN_HOST_API int cgnn_host_gcn_norm_csr_compress(const int64_t *vlist, const int64_t *elist,
                                                  const float *deg, int64_t n, int64_t r, float *w) {
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < n + r; ++v)
        for (int64_t e = vlist[v]; e < vlist[v + 1]; ++e) {
            const int64_t d = elist[e];
            if (v < n && d < n) w[e] = deg[v] * deg[d];
            else if (v < n) w[e] = deg[v];
            else if (d < n) w[e] = deg[d];
            else w[e] = 1;
        }
    return 0;
}

// Plain graph: d_v*d_u (ref: gcn_norm_csr, src/offline/csrc/norm.h:89-113).
CGNN_HOST_API int cgnn_host_gcn_norm_csr(const int64_t *vlist, const int64_t *elist, const float *deg,
                                         int64_t n, float *w) {
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < n; ++v)
        for (int64_t e = vlist[v]; e < vlist[v + 1]; ++e) w[e] = deg[v] * deg[elist[e]];
    return 0;
}

// Stable transpose of a CSR matrix with `ncols` columns: entries of an output row keep
// ascending source-row order (what torch_sparse's .csc() yields for the reference,
// loader/CompressgnnData.py:180).
CGNN_HOST_API int cgnn_host_transpose_csr(const int64_t *vlist, const int64_t *elist, const float *val,
                                          int64_t rows, int64_t ncols, int64_t *t_vlist,
                                          int64_t *t_elist, float *t_val) {
    const int64_t nnz = vlist[rows];
    std::fill(t_vlist, t_vlist + ncols + 1, 0);
    for (int64_t e = 0; e < nnz; ++e) {
        if (elist[e] < 0 || elist[e] >= ncols) return fail("transpose: column out of range");
        ++t_vlist[elist[e] + 1];
    }
    for (int64_t c = 0; c < ncols; ++c) t_vlist[c + 1] += t_vlist[c];
    std::vector<int64_t> cursor(t_vlist, t_vlist + ncols);
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t e = vlist[r]; e < vlist[r + 1]; ++e) {
            const int64_t p = cursor[elist[e]]++;
            t_elist[p] = r;
            if (val) t_val[p] = val[e];
        }
    return 0;
}

// ---------------------------------------------------------------------------------------
// Batch pair-substitution compressor.
//
// The reference delegates this step to an external project (compress_csr_batch of
// ZhengChenCS/CompressGraph, bound in src/offline/bindings/batch_cpu.cpp:2-7) whose source
// is not part of the reference tree; what the reference's tests pin is the contract
// (tests/test_batch_compression.py:15-36, tests/test_offline_compression.py:7-27): the
// result is (vlist int32, elist int32, n, rules), rows n.. are rule bodies whose symbols
// are all smaller than the rule's own id, and expanding every vertex row through the rules
// reproduces the input row in order.  This implementation meets that contract with
// rounds of digram substitution: count adjacent symbol pairs over all vertex rows, turn
// every pair seen at least `min_frequency` times into a rule (ids ascend with the pair
// key, so the output is deterministic), substitute non-overlapping occurrences preferring
// the more frequent pair, drop rules the parse never used.
// ---------------------------------------------------------------------------------------
CGNN_HOST_API int cgnn_host_compress_csr_batch(const int64_t *vlist, const int64_t *elist, int64_t n,
                                               int threads, int rounds, int min_frequency,
                                               Result **out) {
    if (min_frequency < 3) return fail("Batch compression needs min_pair_frequency >= 3");
    if (rounds < 1) return fail("compression_rounds must be positive");
    const int64_t edges = n > 0 ? vlist[n] : 0;
    if (n + edges >= INT32_MAX) return fail("CSR array exceeds int32 capacity");
    std::vector<std::vector<int32_t>> rows((size_t)n);
    for (int64_t v = 0; v < n; ++v) {
        rows[v].reserve((size_t)(vlist[v + 1] - vlist[v]));
        for (int64_t e = vlist[v]; e < vlist[v + 1]; ++e) {
            if (elist[e] < 0 || elist[e] >= n) return fail("CSR value exceeds vertex range");
            rows[v].push_back((int32_t)elist[e]);
        }
    }
    std::vector<std::pair<int32_t, int32_t>> rules;
    if (threads > 0) omp_set_num_threads(threads);
    std::vector<uint64_t> keys;      // every adjacent pair of every row, then sorted
    std::vector<uint64_t> cand_key;  // pairs seen often enough, ascending
    std::vector<int32_t> cand_count;
    std::vector<int64_t> offset((size_t)n + 1);
    for (int round = 0; round < rounds; ++round) {
        // 1. all adjacent pairs, gathered in parallel and sorted: counting is a run-length pass
        offset[0] = 0;
        for (int64_t v = 0; v < n; ++v)
            offset[v + 1] = offset[v] + (rows[v].size() > 1 ? (int64_t)rows[v].size() - 1 : 0);
        keys.resize((size_t)offset[n]);
        if (keys.empty()) break;
#pragma omp parallel for schedule(static)
        for (int64_t v = 0; v < n; ++v) {
            const auto &row = rows[v];
            uint64_t *dst = keys.data() + offset[v];
            for (size_t i = 0; i + 1 < row.size(); ++i)
                dst[i] = ((uint64_t)(uint32_t)row[i] << 32) | (uint32_t)row[i + 1];
        }
        __gnu_parallel::sort(keys.begin(), keys.end());
        cand_key.clear();
        cand_count.clear();
        for (size_t i = 0; i < keys.size();) {
            size_t j = i + 1;
            while (j < keys.size() && keys[j] == keys[i]) ++j;
            if ((int64_t)(j - i) >= min_frequency) {
                cand_key.push_back(keys[i]);
                cand_count.push_back((int32_t)std::min<size_t>(j - i, INT32_MAX));
            }
            i = j;
        }
        if (cand_key.empty()) break;
        const int64_t base = n + (int64_t)rules.size();
        if (base + (int64_t)cand_key.size() >= INT32_MAX) return fail("rule ids exceed int32 capacity");
        // rule id of a pair = base + its rank among the candidates (ascending key): deterministic
        auto find = [&](uint64_t key) -> int64_t {
            auto it = std::lower_bound(cand_key.begin(), cand_key.end(), key);
            return (it != cand_key.end() && *it == key) ? (int64_t)(it - cand_key.begin()) : -1;
        };
        std::vector<int32_t> uses(cand_key.size(), 0);
#pragma omp parallel
        {
            std::vector<int32_t> rid, tmp;  // candidate rule at each position of the row, or -1
            std::vector<uint64_t> weight;   // (pair count, rule id): the parse prefers heavier pairs
            std::vector<char> take;
#pragma omp for schedule(dynamic, 1024)
            for (int64_t v = 0; v < n; ++v) {
                auto &row = rows[v];
                if (row.size() < 2) continue;
                const size_t m = row.size() - 1;
                rid.assign(m, -1);
                weight.assign(m, 0);
                bool any = false;
                for (size_t i = 0; i < m; ++i) {
                    const int64_t k = find(((uint64_t)(uint32_t)row[i] << 32) | (uint32_t)row[i + 1]);
                    if (k >= 0) {
                        rid[i] = (int32_t)(base + k);
                        weight[i] = ((uint64_t)(uint32_t)cand_count[(size_t)k] << 32) | (uint32_t)rid[i];
                        any = true;
                    }
                }
                if (!any) continue;
                // A pair is substituted where it outweighs both overlapping neighbours, so rows
                // that share a run of symbols parse it the same way wherever the run starts;
                // what this leaves is then taken greedily from the left.
                take.assign(m, 0);
                for (size_t i = 0; i < m; ++i)
                    if (rid[i] >= 0 && (i == 0 || weight[i] > weight[i - 1]) &&
                        (i + 1 == m || weight[i] >= weight[i + 1]))
                        take[i] = 1;
                for (size_t i = 0; i < m; ++i)
                    if (!take[i] && rid[i] >= 0 && (i == 0 || !take[i - 1]) && (i + 1 == m || !take[i + 1]))
                        take[i] = 1;
                tmp.clear();
                size_t i = 0;
                while (i < row.size()) {
                    if (i < m && take[i]) {
                        tmp.push_back(rid[i]);
#pragma omp atomic
                        ++uses[(size_t)(rid[i] - base)];
                        i += 2;
                    } else {
                        tmp.push_back(row[i++]);
                    }
                }
                row.assign(tmp.begin(), tmp.end());
            }
        }
        // Drop rules the parse never used and close the gaps in the numbering.
        std::vector<int32_t> remap(cand_key.size(), -1);
        int32_t next = (int32_t)base;
        for (size_t k = 0; k < cand_key.size(); ++k)
            if (uses[k] > 0) {
                remap[k] = next++;
                rules.emplace_back((int32_t)(cand_key[k] >> 32), (int32_t)(cand_key[k] & 0xffffffffu));
            }
        if (next != (int32_t)(base + (int64_t)cand_key.size())) {
#pragma omp parallel for schedule(static)
            for (int64_t v = 0; v < n; ++v)
                for (auto &sym : rows[v])
                    if (sym >= base) sym = remap[(size_t)(sym - base)];
        }
    }
    auto *res = new Result();
    std::vector<int64_t> vl{0}, el;
    for (const auto &row : rows) {
        el.insert(el.end(), row.begin(), row.end());
        vl.push_back((int64_t)el.size());
    }
    for (const auto &rule : rules) {
        el.push_back(rule.first);
        el.push_back(rule.second);
        vl.push_back((int64_t)el.size());
    }
    res->i64 = {std::move(vl), std::move(el)};
    res->scalars[0] = n;
    res->scalars[1] = (int64_t)rules.size();
    *out = res;
    return 0;
}

// ---------------------------------------------------------------------------------------
// Rule filters
// ---------------------------------------------------------------------------------------

// Inline every rule whose saving (freq-1)*(len-1)-1 does not exceed `threshold`, visiting
// rules in id order with len/freq updated as neighbours are inlined
// (ref: filter_csr, src/offline/csrc/filter.h:26-118).
CGNN_HOST_API int cgnn_host_filter_csr(const int64_t *vlist, const int64_t *elist, int64_t n, int64_t r,
                                       int threshold, Result **out) {
    const int64_t total = n + r;
    Rows graph = rows_from_csr(vlist, elist, total);
    Rows graphT = referencing_rows(vlist, elist, total, n);
    std::vector<int> len((size_t)r), freq((size_t)r);
    std::vector<char> removed((size_t)r);
    auto not_worth_keeping = [&](int l, int f) { return (f - 1) * (l - 1) - 1 <= threshold; };
    for (int64_t i = 0; i < r; ++i) {
        freq[i] = (int)graphT[i + n].size();
        len[i] = (int)graph[i + n].size();
        removed[i] = not_worth_keeping(len[i], freq[i]);
    }
    for (int64_t i = 0; i < r; ++i) {
        if (!removed[i]) continue;
        inline_rule(
            i + n, n, graph, graphT,
            [&](int64_t node, int64_t body) {
                if (node >= n) {
                    len[node - n] += (int)(body - 1);
                    removed[node - n] = not_worth_keeping(len[node - n], freq[node - n]);
                }
            },
            [&](int64_t child) {
                if (child >= n) {
                    // The reference adds the whole new reference count, not the delta.
                    freq[child - n] += (int)graphT[child].size();
                    removed[child - n] = not_worth_keeping(len[child - n], freq[child - n]);
                }
            });
    }
    auto *res = new Result();
    emit_filtered(graph, removed, n, r, res);
    *out = res;
    return 0;
}

// Inline the deepest rule levels while they hold fewer than `min_edge` entries, down to
// `max_depth` (ref: depth_filter / depth_filter_csr, src/offline/csrc/depth_filter.h:42-116).
CGNN_HOST_API int cgnn_host_depth_filter_csr(const int64_t *vlist, const int64_t *elist, int64_t n,
                                             int64_t r, int max_depth, int min_edge, Result **out) {
    const int64_t total = n + r;
    Rows graph = rows_from_csr(vlist, elist, total);
    Rows graphT = referencing_rows(vlist, elist, total, n);
    std::vector<int> depth;
    int m_depth = rule_depths(vlist, elist, n, r, depth);
    for (int64_t i = 0; i < r; ++i)
        if (depth[n + i] > m_depth) return fail("depth_filter: a rule is referenced by no row");
    std::vector<char> removed((size_t)r, 0);
    std::vector<int64_t> depth_count((size_t)m_depth + 1, 0);
    for (int64_t i = 0; i < r; ++i) depth_count[depth[n + i]] += (int64_t)graph[n + i].size();
    while (m_depth >= max_depth && m_depth >= 0) {
        if (depth_count[m_depth] >= min_edge) {
            --m_depth;
            continue;
        }
        for (int64_t i = 0; i < r; ++i)
            if (depth[n + i] == m_depth) {
                inline_rule(i + n, n, graph, graphT, [](int64_t, int64_t) {}, [](int64_t) {});
                removed[i] = 1;
            }
        --m_depth;
        for (int d = 0; d <= m_depth; ++d) depth_count[d] = 0;
        for (int64_t i = 0; i < r; ++i)
            if (depth[n + i] <= m_depth && !removed[i])
                depth_count[depth[n + i]] += (int64_t)graph[n + i].size();
    }
    auto *res = new Result();
    emit_filtered(graph, removed, n, r, res);
    *out = res;
    return 0;
}

// ---------------------------------------------------------------------------------------
// Partition into v2v / v2r / r2v / r2r and rule levels
// ---------------------------------------------------------------------------------------

// Split every row of the (transposed) compressed graph at column `n`; rows and columns
// >= n are rules and are re-based to 0.  Rows must have ascending columns
// (ref: hybird_partition, src/offline/csrc/partition.h:14-110).
// Result: i64 = {v2v_v, v2v_e, v2r_v, v2r_e, r2v_v, r2v_e, r2r_v, r2r_e}, f32 = 4 value arrays.
CGNN_HOST_API int cgnn_host_hybrid_partition(const int64_t *vlist, const int64_t *elist, const float *val,
                                             int64_t total, int64_t n, Result **out) {
    auto *res = new Result();
    res->i64.assign(8, {});
    res->f32.assign(4, {});
    for (int b = 0; b < 4; ++b) res->i64[2 * b].push_back(0);
    for (int64_t v = 0; v < total; ++v) {
        const int lo = v < n ? 0 : 2, hi = lo + 1;
        int64_t e = vlist[v];
        const int64_t end = vlist[v + 1];
        for (; e < end && elist[e] < n; ++e) {
            res->i64[2 * lo + 1].push_back(elist[e]);
            res->f32[lo].push_back(val[e]);
        }
        for (; e < end; ++e) {
            res->i64[2 * hi + 1].push_back(elist[e] - n);
            res->f32[hi].push_back(val[e]);
        }
        res->i64[2 * lo].push_back((int64_t)res->i64[2 * lo + 1].size());
        res->i64[2 * hi].push_back((int64_t)res->i64[2 * hi + 1].size());
    }
    *out = res;
    return 0;
}

// Peel the rule-to-rule block into levels: a row with no entries needs no pass; a row joins
// level k once every row it reads has a level, rows visited in ascending order inside a
// pass.  Each level is a full-height CSR whose other rows are empty
// (ref: topo_partition, src/offline/csrc/partition.h:112-216).
// Result: scalars[0] = levels; i64 = {v_0, e_0, v_1, e_1, ...}, f32 = {val_0, val_1, ...}.
CGNN_HOST_API int cgnn_host_topo_partition(const int64_t *vlist, const int64_t *elist, const float *val,
                                           int64_t r, Result **out) {
    std::vector<int> order((size_t)r, -1);
    int64_t left = r;
    for (int64_t v = 0; v < r; ++v)
        if (vlist[v + 1] == vlist[v]) {
            order[v] = 0;
            --left;
        }
    int step = 1;
    while (left > 0) {
        int64_t placed = 0;
        for (int64_t v = 0; v < r; ++v) {
            if (order[v] != -1) continue;
            bool ready = true;
            for (int64_t e = vlist[v]; e < vlist[v + 1] && ready; ++e) ready = order[elist[e]] != -1;
            if (ready) {
                order[v] = step;
                --left;
                ++placed;
            }
        }
        if (placed == 0) return fail("topo_partition: the rule graph has a cycle");
        ++step;
    }
    const int levels = step - 1;
    auto *res = new Result();
    res->scalars[0] = levels;
    res->i64.assign((size_t)2 * levels, {});
    res->f32.assign((size_t)levels, {});
    for (int l = 0; l < levels; ++l) res->i64[2 * l].push_back(0);
    for (int64_t v = 0; v < r; ++v) {
        const int l = order[v] - 1;
        if (l >= 0)
            for (int64_t e = vlist[v]; e < vlist[v + 1]; ++e) {
                res->i64[2 * l + 1].push_back(elist[e]);
                res->f32[l].push_back(val[e]);
            }
        for (int k = 0; k < levels; ++k) res->i64[2 * k].push_back((int64_t)res->i64[2 * k + 1].size());
    }
    *out = res;
    return 0;
}

// Expanded degrees: entries a vertex / rule stands for once every rule is unfolded
// (ref: gen_degree, src/offline/csrc/gen_degree.h:10-85).  Levels are visited last to first.
CGNN_HOST_API int cgnn_host_gen_degree(const int64_t *v2v_v, const int64_t *v2r_v, const int64_t *v2r_e,
                                       const int64_t *r2v_v, int64_t n, int64_t r, int levels,
                                       const int64_t *const *lvl_v, const int64_t *const *lvl_e,
                                       int64_t *v_deg, int64_t *r_deg) {
    for (int64_t v = 0; v < n; ++v) v_deg[v] = v2v_v[v + 1] - v2v_v[v];
    for (int64_t q = 0; q < r; ++q) r_deg[q] = r2v_v[q + 1] - r2v_v[q];
    for (int l = levels - 1; l >= 0; --l)
        for (int64_t q = 0; q < r; ++q)
            for (int64_t e = lvl_v[l][q]; e < lvl_v[l][q + 1]; ++e) r_deg[q] += r_deg[lvl_e[l][e]];
    for (int64_t v = 0; v < n; ++v)
        for (int64_t e = v2r_v[v]; e < v2r_v[v + 1]; ++e) v_deg[v] += r_deg[v2r_e[e]];
    return 0;
}

// Number of phases the reference reports as data.step for a CSR-loaded graph: rules with no
// rule inside them first, then rules all of whose inner rules are placed, counted from 1 and
// including the final empty round (ref: gen_vertex_order_csc, src/offline/csrc/gen_mask.h:129-181).
CGNN_HOST_API int64_t cgnn_host_phase_count(const int64_t *vlist, const int64_t *elist, int64_t n, int64_t r) {
    std::vector<int64_t> indeg((size_t)r, 0);
    for (int64_t q = 0; q < r; ++q)
        for (int64_t e = vlist[n + q]; e < vlist[n + q + 1]; ++e)
            if (elist[e] >= n) ++indeg[elist[e] - n];
    std::vector<char> placed((size_t)(n + r), 0);
    std::vector<int64_t> work, next;
    for (int64_t q = 0; q < r; ++q)
        if (indeg[q] == 0) {
            placed[n + q] = 1;
            work.push_back(n + q);
        }
    int64_t step = 1;
    while (!work.empty()) {
        for (int64_t src : work)
            for (int64_t e = vlist[src]; e < vlist[src + 1]; ++e) {
                const int64_t dst = elist[e];
                if (dst >= n && !placed[dst] && --indeg[dst - n] == 0) {
                    placed[dst] = 1;
                    next.push_back(dst);
                }
            }
        ++step;
        std::swap(work, next);
        next.clear();
    }
    return step;
}

// ---------------------------------------------------------------------------------------
// Seeded synthetic graphs (stand-ins for the public web / citation graphs the reference's
// scripts load; sizes and parameters are the caller's).
// ---------------------------------------------------------------------------------------

// Directed copying-model web graph: node i draws an out-degree from a Pareto(alpha) law
// (scale x_min, clipped to [1, max_degree]) and picks a prototype among the `window`
// preceding ids: `candidates` ids are drawn uniformly from the window and the one that has
// been copied most often so far wins (candidates == 1 is the plain uniform choice; larger
// values model link templates shared by many pages of one site).  A contiguous run of the
// prototype's targets makes up `copy_prob` of the node's list (less if the prototype's list
// is shorter); the remainder is drawn half from the +-window neighbourhood of i and half
// uniformly from all nodes.
// Rows are sorted and de-duplicated.
CGNN_HOST_API int cgnn_host_generate_copy_graph(int64_t n, double alpha, double x_min, int64_t max_degree,
                                                double copy_prob, int64_t window, int candidates,
                                                uint64_t seed, Result **out) {
    if (n <= 0 || alpha <= 1.0 || x_min <= 0 || window < 1 || candidates < 1)
        return fail("generate_copy_graph: bad parameter");
    std::mt19937_64 rng(seed);
    std::uniform_real_distribution<double> uni(0.0, 1.0);
    std::vector<int64_t> vl{0}, el;
    std::vector<int64_t> row;
    std::vector<int32_t> copied((size_t)n, 0);
    for (int64_t i = 0; i < n; ++i) {
        const double u = 1.0 - uni(rng);
        int64_t deg = (int64_t)std::floor(x_min / std::pow(u, 1.0 / alpha));
        deg = std::max<int64_t>(1, std::min<int64_t>(deg, std::min<int64_t>(max_degree, n)));
        row.clear();
        if (i > 0) {
            const int64_t lo = std::max<int64_t>(0, i - window);
            int64_t proto = lo + (int64_t)(uni(rng) * (double)(i - lo));
            for (int c = 1; c < candidates; ++c) {
                const int64_t other = lo + (int64_t)(uni(rng) * (double)(i - lo));
                if (copied[other] > copied[proto]) proto = other;
            }
            ++copied[proto];
            // A contiguous run of the prototype's list, copy_prob of this node's degree long.
            const int64_t plen = vl[proto + 1] - vl[proto];
            const int64_t want = std::min<int64_t>(plen, (int64_t)std::llround(copy_prob * (double)deg));
            const int64_t start = vl[proto] + (int64_t)(uni(rng) * (double)(plen - want + 1));
            for (int64_t e = start; e < start + want; ++e) row.push_back(el[e]);
        }
        while ((int64_t)row.size() < deg) {
            int64_t t;
            if (uni(rng) < 0.5) {
                t = i + (int64_t)std::floor((uni(rng) * 2.0 - 1.0) * (double)window);
                t = std::max<int64_t>(0, std::min<int64_t>(n - 1, t));
            } else {
                t = (int64_t)(uni(rng) * (double)n);
                t = std::min<int64_t>(n - 1, t);
            }
            row.push_back(t);
        }
        std::sort(row.begin(), row.end());
        row.erase(std::unique(row.begin(), row.end()), row.end());
        el.insert(el.end(), row.begin(), row.end());
        vl.push_back((int64_t)el.size());
    }
    auto *res = new Result();
    res->i64 = {std::move(vl), std::move(el)};
    *out = res;
    return 0;
}

// Undirected preferential-attachment graph with list copying: node i >= 1 attaches to 1..3
// earlier nodes chosen in proportion to degree, then copies `copy_frac` of the neighbour
// list of a random earlier node.  The edge set is symmetrised, de-duplicated and trimmed or
// padded (with random pairs) to exactly `undirected_edges`.
CGNN_HOST_API int cgnn_host_generate_pa_graph(int64_t n, int64_t undirected_edges, double copy_frac,
                                              uint64_t seed, Result **out) {
    if (n < 2 || undirected_edges < 1) return fail("generate_pa_graph: bad parameter");
    std::mt19937_64 rng(seed);
    std::uniform_real_distribution<double> uni(0.0, 1.0);
    std::vector<std::vector<int64_t>> adj((size_t)n);
    std::vector<int64_t> ends;  // every edge endpoint once: sampling it is degree-proportional
    std::vector<std::pair<int64_t, int64_t>> edges;
    auto add = [&](int64_t a, int64_t b) {
        if (a == b) return;
        edges.emplace_back(std::min(a, b), std::max(a, b));
        adj[a].push_back(b);
        adj[b].push_back(a);
        ends.push_back(a);
        ends.push_back(b);
    };
    add(0, 1);
    for (int64_t i = 2; i < n; ++i) {
        const int m = 1 + (int)(uni(rng) * 3.0);
        for (int k = 0; k < m; ++k) add(i, ends[(size_t)(uni(rng) * (double)ends.size())]);
        const int64_t proto = (int64_t)(uni(rng) * (double)i);
        const std::vector<int64_t> list = adj[proto];
        for (int64_t t : list)
            if (t != i && uni(rng) < copy_frac) add(i, t);
    }
    std::sort(edges.begin(), edges.end());
    edges.erase(std::unique(edges.begin(), edges.end()), edges.end());
    std::shuffle(edges.begin(), edges.end(), rng);
    if ((int64_t)edges.size() > undirected_edges) edges.resize((size_t)undirected_edges);
    std::sort(edges.begin(), edges.end());
    while ((int64_t)edges.size() < undirected_edges) {
        const int64_t a = (int64_t)(uni(rng) * (double)n), b = (int64_t)(uni(rng) * (double)n);
        if (a == b) continue;
        const auto e = std::make_pair(std::min(a, b), std::max(a, b));
        auto it = std::lower_bound(edges.begin(), edges.end(), e);
        if (it == edges.end() || *it != e) edges.insert(it, e);
    }
    std::vector<int64_t> vl((size_t)n + 1, 0), el((size_t)edges.size() * 2);
    for (const auto &e : edges) {
        ++vl[e.first + 1];
        ++vl[e.second + 1];
    }
    for (int64_t v = 0; v < n; ++v) vl[v + 1] += vl[v];
    std::vector<int64_t> cur(vl.begin(), vl.end() - 1);
    for (const auto &e : edges) {
        el[cur[e.first]++] = e.second;
        el[cur[e.second]++] = e.first;
    }
    for (int64_t v = 0; v < n; ++v) std::sort(el.begin() + vl[v], el.begin() + vl[v + 1]);
    auto *res = new Result();
    res->i64 = {std::move(vl), std::move(el)};
    *out = res;
    return 0;
}
