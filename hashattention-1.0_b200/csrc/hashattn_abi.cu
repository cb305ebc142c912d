// extern "C" entry points of libhashattn.so (declared in include/hashattn.h): argument checks,
// workspace carving and kernel launches. No device memory is allocated, nothing synchronises with
// the host (except where ha_decode_step_host is asked to), nothing throws, and the library creates no
// streams, events or other CUDA resources of its own.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "hash_decode.cuh"
#include "hash_prefill_tc.cuh"
#include "lsh.cuh"
#include "score_select.cuh"
#include "select_attend.cuh"
#include "sparse_decode.cuh"

namespace ha {
namespace {

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// Process-wide dispatch options (ha_set_option); -1 / 0 = the library decides.
std::atomic<int> g_options[HA_OPT_COUNT_] = {};
bool g_options_ready = [] {
    g_options[HA_OPT_CLUSTER_GATHER] = -1;
    g_options[HA_OPT_CLUSTER_SELECT] = -1;
    g_options[HA_OPT_PLAN_HANDOVER] = -1;
    return true;
}();
inline int option(int key) { return g_options[key].load(std::memory_order_relaxed); }

int check_shape(const ha_shape_t* s) {
    if (s == nullptr) return HA_ERR_BAD_ARG;
    if (s->gqa_group != kGroup || s->head_dim != kHeadDim || s->page_size != kPage)
        return HA_ERR_UNSUPPORTED_DIM;
    if (s->batch < 1 || s->num_kv_heads < 1 || s->max_pages < 1 || s->num_pages < 1 ||
        s->sel_stride < 1)
        return HA_ERR_BAD_ARG;
    if (s->batch > 65535 || s->num_kv_heads * kGroup > 65535 || s->max_pages > 65535)
        return HA_ERR_UNSUPPORTED_DIM;
    return HA_OK;
}

int check_budget(const ha_budget_t* b) {
    if (b == nullptr) return HA_ERR_BAD_ARG;
    if (b->init_budget < 0 || b->recent_budget < 0) return HA_ERR_BAD_ARG;
    if (!(b->heavy_budget >= 0.0) || !std::isfinite(b->heavy_budget)) return HA_ERR_BAD_ARG;
    if (b->eval_mode != HA_EVAL_SIMPLE && b->eval_mode != HA_EVAL_DEPTH) return HA_ERR_BAD_ARG;
    if (b->eval_mode == HA_EVAL_DEPTH && (b->retrieve_depth < -64 || b->retrieve_depth > 64)) return HA_ERR_BAD_ARG;
    return HA_OK;
}

int check_weights(const ha_hash_weights_t* w, bool need_q, bool need_k) {
    if (w == nullptr) return HA_ERR_BAD_ARG;
    if (w->dtype != HA_WEIGHTS_BF16 && w->dtype != HA_WEIGHTS_F32) return HA_ERR_BAD_ARG;
    if (w->num_layers != HA_HASH_LSH && (w->num_layers < 0 || w->num_layers > 3)) return HA_ERR_BAD_ARG;
    if (w->num_layers == HA_HASH_LSH && w->lsh_state == nullptr) return HA_ERR_BAD_ARG;
    if (need_q && (w->wq == nullptr || w->bq == nullptr)) return HA_ERR_BAD_ARG;
    if (need_k && (w->wk == nullptr || w->bk == nullptr)) return HA_ERR_BAD_ARG;
    return HA_OK;
}

// How the attended rows of one (sequence, query head) are cut into CTAs: never more rows than
// init + recent + sel_stride, nor than the longest sequence the page table can describe; rounds
// grows with the total so that big problems do not drown in partials.
struct AttSplit {
    int rounds, nsplits;
    bool cluster;  // the splits of a (sequence, head) are the 8 CTAs of a cluster that merge among themselves
};

AttSplit att_split(const ha_shape_t* s, const ha_budget_t* b) {
    long long rows = (long long)s->sel_stride + b->init_budget + b->recent_budget;
    const long long cap = (long long)s->max_pages * kPage;
    if (rows > cap) rows = cap;
    const long long total = rows * s->batch * s->num_kv_heads * kGroup;
    long long rounds = (total + kAttRoundRows * 4096LL - 1) / (kAttRoundRows * 4096LL);
    if (rounds < 1) rounds = 1;
    if (rounds > kAttMaxRounds) rounds = kAttMaxRounds;
    AttSplit a;
    a.rounds = (int)rounds;
    a.nsplits = (int)((rows + kAttRoundRows * rounds - 1) / (kAttRoundRows * rounds));
    a.cluster = false;
    return a;
}

// Small steps (config-1-like: the gather of 41 K rows takes about as long as the hand-over to a merge kernel
// and the merge together) run the gather as clusters of 8 CTAs x 256 threads per (sequence, head), which merge
// through distributed shared memory: no partials, no merge kernel.
AttSplit att_split_launch(const ha_shape_t* s, const ha_budget_t* b) {
    AttSplit a = att_split(s, b);
    long long rows = (long long)s->sel_stride + b->init_budget + b->recent_budget;
    const long long cap = (long long)s->max_pages * kPage;
    if (rows > cap) rows = cap;
    const long long total = rows * s->batch * s->num_kv_heads * kGroup;
    const int cluster_round_rows = kAttClusterThreads / 16 * kAttRowsPerWorker;  // 64
    const long long per_cta = (rows + kAttClusterCtas - 1) / kAttClusterCtas;
    const long long rounds = (per_cta + cluster_round_rows - 1) / cluster_round_rows;
    const int forced = option(HA_OPT_CLUSTER_GATHER);  // 0 / 1 force the choice (experiments, tests)
    const bool fits = rounds <= kAttMaxRounds && a.nsplits > 1;
    const bool want = forced >= 0 ? forced == 1 : total <= 65536;
    if (fits && want) {
        a.cluster = true;
        a.rounds = (int)(rounds < 1 ? 1 : rounds);
        a.nsplits = kAttClusterCtas;
    }
    return a;
}

// How a sequence is cut into chunks for scoring and selection: 4, 8 or 16 pages per chunk (the kernels are
// compiled for these), about 32 chunks per sequence; small problems take smaller chunks (up to 64 per
// sequence) until the scoring grid has two CTAs per SM.
struct Geometry {
    int chunk_pages, nchunks;
    int nslots;  // CTAs per (sequence, head) of select_attend_kernel: the chunks plus the two edge CTAs
};

Geometry geometry(const ha_shape_t* s) {
    Geometry g;
    const int want = (s->max_pages + 31) / 32;
    g.chunk_pages = want <= 4 ? 4 : (want <= 8 ? 8 : kMaxChunkPages);
    const long long units = (long long)s->batch * s->num_kv_heads;
    auto chunks = [&](int cp) { return (s->max_pages + cp - 1) / cp; };
    while (g.chunk_pages > 4 && units * chunks(g.chunk_pages) < 2 * 148 && chunks(g.chunk_pages / 2) <= 64)
        g.chunk_pages /= 2;
    g.nchunks = chunks(g.chunk_pages);
    g.nslots = g.nchunks + kSaEdgeSlots;
    return g;
}

struct Workspace {
    uint32_t* hist;     // [B][Hkv][4*33][nchunks] per-chunk score histograms
    int32_t* sel_rows;  // [B][Hq][sel_stride] physical rows of the selected tokens (single-pass cluster selection)
    float* partials;    // [B][Hq][max(nsplits, nslots)][130] attention partials
    int32_t* plan;      // [B][Hkv][8 + 8 * nchunks] thresholds, tie quotas and per-chunk output bases
    uint8_t* scores;    // [B][Hq][nchunks * chunk tokens] one score byte per token and query head
    uint32_t* arrive;   // [B][Hkv][kArriveStride] arrival counter and histogram totals of the scoring kernel (zero between calls)
    size_t bytes;
};

size_t scores_bytes(const ha_shape_t* s, const Geometry& g) {
    return (size_t)s->batch * s->num_kv_heads * kGroup * g.nchunks * g.chunk_pages * kPage;
}

Workspace carve(const ha_shape_t* s, const ha_budget_t* b, void* base) {
    const Geometry g = geometry(s);
    const size_t Hq = (size_t)s->num_kv_heads * kGroup, units = (size_t)s->batch * s->num_kv_heads;
    char* p = static_cast<char*>(base);
    Workspace w;
    size_t off = 0;
    w.hist = reinterpret_cast<uint32_t*>(p + off);
    off += align_up(units * g.nchunks * kGroup * kBins * sizeof(uint32_t));
    w.sel_rows = reinterpret_cast<int32_t*>(p + off);
    off += align_up((size_t)s->batch * Hq * s->sel_stride * sizeof(int32_t));
    w.partials = reinterpret_cast<float*>(p + off);
    off += align_up((size_t)s->batch * Hq * std::max(att_split(s, b).nsplits, g.nslots) * kPartStride * sizeof(float));
    w.plan = reinterpret_cast<int32_t*>(p + off);
    off += align_up(units * (8 + 8 * (size_t)g.nchunks) * sizeof(int32_t));
    w.scores = reinterpret_cast<uint8_t*>(p + off);
    off += align_up(scores_bytes(s, g));
    w.arrive = reinterpret_cast<uint32_t*>(p + off);
    off += align_up(units * kArriveStride * sizeof(uint32_t));
    w.bytes = off;
    return w;
}

// Every kernel is launched with programmatic stream serialization (it may start while its
// predecessor drains and synchronises itself with griddepcontrol.wait); cluster_x > 1 adds a
// thread-block cluster along x.
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, int cluster_x,
                   Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
    if (cluster_x > 1) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
        attr[cfg.numAttrs].val.clusterDim.x = cluster_x;
        attr[cfg.numAttrs].val.clusterDim.y = 1;
        attr[cfg.numAttrs].val.clusterDim.z = 1;
        ++cfg.numAttrs;
    }
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Kernels that keep more than a few KB of shared memory per CTA ask for a carve-out that holds a full SM's worth
// of their CTAs (the default split may size it for fewer); set once per device and kernel.
std::atomic<unsigned> g_carveout_set[64] = {};

template <typename K>
void prefer_carveout(K kernel, int kernel_id, int percent) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    const unsigned bit = 1u << kernel_id;
    if (g_carveout_set[dev].load(std::memory_order_relaxed) & bit) return;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, percent) != cudaSuccess)
        (void)cudaGetLastError();  // only a hint
    g_carveout_set[dev].fetch_or(bit, std::memory_order_relaxed);
}

// Scoring, histograms and the plan (score_hist_kernel) on the kv-heads [p.kvh0, p.kvh0 + nkvh).
cudaError_t launch_score_hist(const ha_shape_t* shape, const SelectParams& p, int nkvh, cudaStream_t s) {
    const dim3 grid(p.nchunks, nkvh, shape->batch);
    prefer_carveout(score_hist_kernel<1>, 0, 40);  // 5 CTAs x 13 KB
    prefer_carveout(score_hist_kernel<2>, 1, 40);
    prefer_carveout(score_hist_kernel<4>, 2, 40);
    switch (geometry(shape).chunk_pages) {
        case 4: return launch(score_hist_kernel<1>, grid, dim3(kSelThreads), s, 1, p);
        case 8: return launch(score_hist_kernel<2>, grid, dim3(kSelThreads), s, 1, p);
        default: return launch(score_hist_kernel<4>, grid, dim3(kSelThreads), s, 1, p);
    }
}

// Selection + attention (select_attend_kernel and the merge of its partials), or the selection alone, on the
// query heads [p.h0, p.h0 + nheads).
cudaError_t launch_select_attend(const ha_shape_t* shape, const SelectAttendParams& p, int nheads, bool gather,
                                 cudaStream_t s) {
    const dim3 grid(p.nslots, nheads, shape->batch);
    const int chunk_pages = geometry(shape).chunk_pages;
    if (!gather) {
        switch (chunk_pages) {
            case 4: return launch(select_attend_kernel<1, false, 8>, grid, dim3(kSaThreads), s, 1, p);
            case 8: return launch(select_attend_kernel<2, false, 8>, grid, dim3(kSaThreads), s, 1, p);
            default: return launch(select_attend_kernel<4, false, 8>, grid, dim3(kSaThreads), s, 1, p);
        }
    }
    // a grid that fits the GPU at 8 CTAs per SM runs as one wave of the 64-register build; larger grids run faster
    // on the 72-register build at 7 CTAs per SM
    const bool one_wave = (long long)p.nslots * nheads * shape->batch <= 8LL * 148;
    cudaError_t e;
    if (one_wave) {
        prefer_carveout(select_attend_kernel<1, true, 8>, 3, 75);  // 8 CTAs x 6 - 18.5 KB
        prefer_carveout(select_attend_kernel<2, true, 8>, 4, 75);
        prefer_carveout(select_attend_kernel<4, true, 8>, 5, 75);
        switch (chunk_pages) {
            case 4: e = launch(select_attend_kernel<1, true, 8>, grid, dim3(kSaThreads), s, 1, p); break;
            case 8: e = launch(select_attend_kernel<2, true, 8>, grid, dim3(kSaThreads), s, 1, p); break;
            default: e = launch(select_attend_kernel<4, true, 8>, grid, dim3(kSaThreads), s, 1, p); break;
        }
    } else {
        prefer_carveout(select_attend_kernel<1, true, 7>, 6, 75);
        prefer_carveout(select_attend_kernel<2, true, 7>, 7, 75);
        prefer_carveout(select_attend_kernel<4, true, 7>, 8, 75);
        switch (chunk_pages) {
            case 4: e = launch(select_attend_kernel<1, true, 7>, grid, dim3(kSaThreads), s, 1, p); break;
            case 8: e = launch(select_attend_kernel<2, true, 7>, grid, dim3(kSaThreads), s, 1, p); break;
            default: e = launch(select_attend_kernel<4, true, 7>, grid, dim3(kSaThreads), s, 1, p); break;
        }
    }
    if (e != cudaSuccess) return e;
    return launch(select_attend_merge_kernel, dim3(nheads, shape->batch), dim3(kMergeThreads), s, 1, p, chunk_pages * kPage);
}

// One cluster kernel scores and selects in a single pass when the sequences are short and there are at
// most 8 (sequence, kv-head) units, one cluster of 8 CTAs x 1024 threads per GPC: at most two rounds each
// (measured 6.9 us against 9.4 us for the two-pass kernels at B=1, S=32K). With 16 units the clusters no
// longer run side by side (13.7 us against 11.6 us for the two-pass kernels at B=2), and longer sequences
// are bandwidth- rather than latency-bound (45 us against 62 us at B=4, S=128K).
bool use_cluster_select(const ha_shape_t* shape) {
    const long long max_tokens = (long long)shape->max_pages * kPage;
    const long long units = (long long)shape->batch * shape->num_kv_heads;
    const int forced = option(HA_OPT_CLUSTER_SELECT);  // 0 never, 1 whenever the sequences fit the kernel
    if (forced == 0 || max_tokens > 2LL * kClRoundTokens) return false;
    return forced == 1 || units <= 8;
}

}  // namespace
}  // namespace ha

namespace ha {
namespace {

SelectParams select_params(const ha_shape_t* shape, const ha_budget_t* budget, const uint32_t* q_codes,
                           const uint32_t* hash_pages, const int32_t* page_table, const int32_t* seq_lens,
                           int32_t* sel_idx, int32_t* sel_cnt, uint8_t* scores_dbg, int32_t* status,
                           uint32_t* hist, int32_t* plan, uint8_t* scores, uint32_t* arrive, int32_t* sel_rows,
                           const int32_t* budget_lens = nullptr) {
    SelectParams p;
    p.q_codes = q_codes;
    p.hash_pages = reinterpret_cast<const uint4*>(hash_pages);
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.budget_lens = budget_lens;
    p.hist = hist;
    p.arrive = arrive;
    p.plan = plan;
    p.scores = scores;
    p.sel_idx = sel_idx;
    p.sel_rows = sel_rows;
    p.sel_cnt = sel_cnt;
    p.scores_dbg = scores_dbg;
    p.status = status;
    p.B = shape->batch;
    p.Hkv = shape->num_kv_heads;
    p.max_pages = shape->max_pages;
    p.num_pages = shape->num_pages;
    p.sel_stride = shape->sel_stride;
    p.nchunks = geometry(shape).nchunks;
    p.kvh0 = 0;
    p.init_budget = budget->init_budget;
    p.recent_budget = budget->recent_budget;
    p.heavy_budget = budget->heavy_budget;
    p.eval_mode = budget->eval_mode;
    p.depth = budget->retrieve_depth;
    p.signal = 0;
    return p;
}

// The attention side (q, pools, out) may be null when only the selection is run.
SelectAttendParams select_attend_params(const ha_shape_t* shape, const ha_budget_t* budget, const int32_t* plan,
                                        const uint8_t* scores, float* partials, int32_t* sel_idx, const void* q,
                                        const void* k_pages, const void* v_pages, const int32_t* page_table,
                                        const int32_t* seq_lens, const int32_t* budget_lens, float sm_scale, void* out,
                                        int32_t* status, int32_t* status_out) {
    const Geometry g = geometry(shape);
    SelectAttendParams p;
    p.plan = plan;
    p.scores = scores;
    p.sel_idx = sel_idx;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
    p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.budget_lens = budget_lens;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.partials = partials;
    p.status = status;
    p.status_out = status_out;
    p.ready = nullptr;
    p.B = shape->batch;
    p.Hkv = shape->num_kv_heads;
    p.max_pages = shape->max_pages;
    p.num_pages = shape->num_pages;
    p.sel_stride = shape->sel_stride;
    p.nchunks = g.nchunks;
    p.nslots = g.nslots;
    p.h0 = 0;
    p.init_budget = budget->init_budget;
    p.recent_budget = budget->recent_budget;
    p.heavy_budget = budget->heavy_budget;
    p.scale_log2e = sm_scale * 1.4426950408889634f;
    return p;
}

// sel == nullptr with physical == true: use the physical rows select_kernel left in the workspace.
int sparse_decode_impl(const ha_shape_t* shape, const ha_budget_t* budget,
                       const void* q, const void* k_pages, const void* v_pages,
                       const int32_t* page_table, const int32_t* seq_lens,
                       const int32_t* sel, const int32_t* sel_cnt, bool physical, float sm_scale,
                       void* out, void* workspace, size_t workspace_bytes,
                       int32_t* status, void* stream, const int32_t* budget_lens = nullptr,
                       int32_t* status_out = nullptr) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (q == nullptr || k_pages == nullptr || v_pages == nullptr || page_table == nullptr ||
        seq_lens == nullptr || out == nullptr || status == nullptr || !std::isfinite(sm_scale))
        return HA_ERR_BAD_ARG;
    if (budget->eval_mode != HA_EVAL_SIMPLE && sel_cnt == nullptr) return HA_ERR_BAD_ARG;  // variable-size sets
    const int nheads = shape->num_kv_heads * kGroup;
    if (workspace == nullptr) return HA_ERR_WORKSPACE;
    const Workspace w = carve(shape, budget, workspace);
    if (workspace_bytes < w.bytes) return HA_ERR_WORKSPACE;

    SparseDecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
    p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.budget_lens = budget_lens;
    p.sel = physical ? w.sel_rows : sel;
    p.sel_cnt = budget->eval_mode == HA_EVAL_SIMPLE ? nullptr : sel_cnt;  // simple: the count follows from the budget
    p.out = static_cast<__nv_bfloat16*>(out);
    p.status = status;
    p.status_out = nullptr;
    p.B = shape->batch;
    p.Hkv = shape->num_kv_heads;
    p.max_pages = shape->max_pages;
    p.num_pages = shape->num_pages;
    p.sel_stride = shape->sel_stride;
    p.init_budget = budget->init_budget;
    p.recent_budget = budget->recent_budget;
    p.heavy_budget = budget->heavy_budget;
    p.scale_log2e = sm_scale * 1.4426950408889634f;
    const AttSplit split = att_split_launch(shape, budget);
    p.partials = w.partials;
    p.nsplits = split.nsplits;
    p.rounds = split.rounds;
    p.round_rows = split.cluster ? kAttClusterThreads / 16 * kAttRowsPerWorker : kAttRoundRows;
    p.h0 = 0;
    const dim3 grid(split.nsplits, nheads, shape->batch);
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (split.cluster) {
        p.status_out = status_out;
        const cudaError_t ec = physical ? launch(sparse_gather_kernel<true, kAttClusterThreads, true>, grid,
                                                 dim3(kAttClusterThreads), s, kAttClusterCtas, p)
                                        : launch(sparse_gather_kernel<false, kAttClusterThreads, true>, grid,
                                                 dim3(kAttClusterThreads), s, kAttClusterCtas, p);
        return ec == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    const bool merge_follows = split.nsplits > 1;
    p.status_out = merge_follows ? nullptr : status_out;  // the status is published by the last kernel
    cudaError_t e = physical ? launch(sparse_gather_kernel<true, kAttThreads, false>, grid, dim3(kAttThreads), s, 1, p)
                             : launch(sparse_gather_kernel<false, kAttThreads, false>, grid, dim3(kAttThreads), s, 1, p);
    if (e == cudaSuccess && merge_follows) {
        p.status_out = status_out;
        e = launch(sparse_merge_kernel, dim3(nheads, shape->batch), dim3(kHeadDim), s, 1, p);
    }
    return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

}  // namespace
}  // namespace ha

namespace ha {
namespace {

constexpr int kMaxDevices = 64;

// The device-side address of a page-locked, device-addressable host buffer; null for anything else
// (pageable memory, device memory).
void* mapped_host_pointer(const void* host) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        (void)cudaGetLastError();  // an unregistered pointer is not an error of this library
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

}  // namespace
}  // namespace ha

using namespace ha;

extern "C" {

int ha_abi_version(void) { return HA_ABI_VERSION; }

int ha_set_option(int option_key, int value) {
    if (option_key < 0 || option_key >= HA_OPT_COUNT_) return HA_ERR_BAD_ARG;
    g_options[option_key].store(value, std::memory_order_relaxed);
    return HA_OK;
}

int ha_get_option(int option_key) {
    return option_key < 0 || option_key >= HA_OPT_COUNT_ ? 0 : option(option_key);
}

const char* ha_status_str(int status) {
    switch (status) {
        case HA_OK: return "ok";
        case HA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or inconsistent shape)";
        case HA_ERR_UNSUPPORTED_DIM: return "unsupported dimension (needs head_dim 128, gqa_group 4, page_size 256)";
        case HA_ERR_WORKSPACE: return "workspace missing or too small";
        case HA_ERR_LAUNCH: return "CUDA launch or copy failed";
        case HA_ERR_TIMEOUT: return "bounded device-side wait ran out";
        case HA_ERR_BAD_PAGE: return "page id outside the page pool";
        case HA_ERR_BAD_SEQ_LEN: return "sequence length < 1 or beyond the page table";
        case HA_ERR_SEL_OVERFLOW: return "heavy budget exceeds sel_stride";
        case HA_ERR_SCRATCH_LIMIT: return "shape needs more scratch than the library's built-in buffer (HA_STATIC_SCRATCH_BYTES)";
        default: return "unknown status";
    }
}

size_t ha_workspace_bytes(const ha_shape_t* shape, const ha_budget_t* budget) {
    if (check_shape(shape) != HA_OK || check_budget(budget) != HA_OK) return 0;
    return carve(shape, budget, nullptr).bytes;
}

int ha_workspace_init(const ha_shape_t* shape, const ha_budget_t* budget, void* workspace,
                      size_t workspace_bytes, void* stream) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (workspace == nullptr) return HA_ERR_WORKSPACE;
    const Workspace w = carve(shape, budget, workspace);
    if (workspace_bytes < w.bytes) return HA_ERR_WORKSPACE;
    // the arrival counters of the scoring kernel must start at zero (the kernel leaves them at zero);
    // nothing else in the workspace carries state between calls
    if (cudaMemsetAsync(workspace, 0, w.bytes, static_cast<cudaStream_t>(stream)) != cudaSuccess)
        return HA_ERR_LAUNCH;
    return HA_OK;
}

static LshParams lsh_params(const ha_shape_t* shape, const ha_hash_weights_t* weights, const void* q, const void* k_new,
                            const void* v_new, void* k_pages, void* v_pages, uint32_t* hash_pages,
                            const int32_t* page_table, const int32_t* seq_lens, uint32_t* q_codes, float* preact_dbg,
                            void* q_stage, int32_t* status) {
    LshParams l;
    l.q = static_cast<const __nv_bfloat16*>(q);
    l.k_new = static_cast<const __nv_bfloat16*>(k_new);
    l.v_new = static_cast<const __nv_bfloat16*>(v_new);
    l.w = weights->wk != nullptr ? weights->wk : weights->wq;  // one function for both sides
    l.bias = weights->bk != nullptr ? weights->bk : weights->bq;
    l.k_pages = static_cast<__nv_bfloat16*>(k_pages);
    l.v_pages = static_cast<__nv_bfloat16*>(v_pages);
    l.hash_pages = hash_pages;
    l.page_table = page_table;
    l.seq_lens = seq_lens;
    l.q_codes = q_codes;
    l.preact_dbg = preact_dbg;
    l.q_stage = static_cast<__nv_bfloat16*>(q_stage);
    l.m = static_cast<float*>(weights->lsh_state);
    l.stale = static_cast<int32_t*>(weights->lsh_state) + shape->num_kv_heads;
    l.status = status;
    l.B = shape->batch;
    l.Hkv = shape->num_kv_heads;
    l.max_pages = shape->max_pages;
    l.num_pages = shape->num_pages;
    l.only_if_stale = 0;
    return l;
}

static cudaError_t launch_lsh_hash_keys(const ha_shape_t* shape, const LshParams& l, bool bf16, cudaStream_t st) {
    cudaError_t e = bf16 ? cudaFuncSetAttribute(lsh_hash_keys_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)kLshSmemBytes)
                         : cudaFuncSetAttribute(lsh_hash_keys_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)kLshSmemBytes);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(shape->max_pages, shape->num_kv_heads, shape->batch);
    cfg.blockDim = dim3(kLshThreads);
    cfg.dynamicSmemBytes = kLshSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr1[1];
    attr1[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr1[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr1;
    cfg.numAttrs = 1;
    return bf16 ? cudaLaunchKernelEx(&cfg, lsh_hash_keys_kernel<__nv_bfloat16>, l)
                : cudaLaunchKernelEx(&cfg, lsh_hash_keys_kernel<float>, l);
}

// ha_hash_decode with an optional device copy of q (q_stage) for the kernels that follow.
static int hash_decode_impl(const ha_shape_t* shape, const ha_hash_weights_t* weights,
                            const void* q, const void* k_new, const void* v_new,
                            void* k_pages, void* v_pages, uint32_t* hash_pages,
                            const int32_t* page_table, const int32_t* seq_lens,
                            uint32_t* q_codes, float* preact_dbg, void* q_stage, int32_t* status, void* stream) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    const bool key_side = k_new != nullptr;
    rc = check_weights(weights, true, key_side);
    if (rc != HA_OK) return rc;
    if (q == nullptr || q_codes == nullptr || status == nullptr) return HA_ERR_BAD_ARG;
    if (key_side && (hash_pages == nullptr || page_table == nullptr || seq_lens == nullptr))
        return HA_ERR_BAD_ARG;
    if (key_side && v_new != nullptr && (k_pages == nullptr || v_pages == nullptr)) return HA_ERR_BAD_ARG;

    if (weights->num_layers == HA_HASH_LSH) {
        // the LSH baseline: encode (and, key side, append); then re-hash the kv-heads whose largest key norm the new
        // keys raised (a launch that returns at once otherwise)
        LshParams l = lsh_params(shape, weights, q, k_new, v_new, k_pages, v_pages, hash_pages, page_table, seq_lens, q_codes,
                                 preact_dbg, q_stage, status);
        const cudaStream_t st = static_cast<cudaStream_t>(stream);
        const bool bf16 = weights->dtype == HA_WEIGHTS_BF16;
        const dim3 grid(shape->num_kv_heads, shape->batch);
        cudaError_t e = bf16 ? launch(lsh_encode_kernel<__nv_bfloat16>, grid, dim3(kLshThreads), st, 1, l)
                             : launch(lsh_encode_kernel<float>, grid, dim3(kLshThreads), st, 1, l);
        if (e != cudaSuccess) return HA_ERR_LAUNCH;
        if (!key_side) return HA_OK;
        l.only_if_stale = 1;
        return launch_lsh_hash_keys(shape, l, bf16, st) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }

    HashDecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k_new = static_cast<const __nv_bfloat16*>(k_new);
    p.v_new = static_cast<const __nv_bfloat16*>(v_new);
    p.w[0] = weights->wq;
    p.w[1] = weights->wk;
    p.bias[0] = weights->bq;
    p.bias[1] = weights->bk;
    p.k_pages = static_cast<__nv_bfloat16*>(k_pages);
    p.v_pages = static_cast<__nv_bfloat16*>(v_pages);
    p.hash_pages = hash_pages;
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.q_codes = q_codes;
    p.preact_dbg = preact_dbg;
    p.q_stage = static_cast<__nv_bfloat16*>(q_stage);
    p.layers = weights->num_layers == 0 ? 3 : weights->num_layers;
    p.status = status;
    p.B = shape->batch;
    p.Hkv = shape->num_kv_heads;
    p.max_pages = shape->max_pages;
    p.num_pages = shape->num_pages;
    // One CTA (512 threads, the head's weights in registers) fits per SM: give each CTA as many
    // sequences as it takes for the whole grid to be resident at once, instead of a second wave
    // that would fetch the weights again.
    {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
            return HA_ERR_LAUNCH;
        const long long nets = (long long)shape->num_kv_heads * kGroup * (key_side ? 2 : 1);
        const long long slices = sms / nets > 0 ? sms / nets : 1;  // batch slices that fit in one wave
        p.batch_per_cta = (int)((shape->batch + slices - 1) / slices);
    }
    const dim3 grid(shape->num_kv_heads * kGroup, key_side ? 2 : 1,
                    (shape->batch + p.batch_per_cta - 1) / p.batch_per_cta);
    cudaError_t e;
    if (p.batch_per_cta >= kHdbMinRows) {
        // several sequences per CTA: evaluate them together from shared-memory weights
        const bool bf16 = weights->dtype == HA_WEIGHTS_BF16;
        e = bf16 ? cudaFuncSetAttribute(hash_decode_batched_kernel<__nv_bfloat16>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHdbSmemBytes)
                 : cudaFuncSetAttribute(hash_decode_batched_kernel<float>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHdbSmemBytes);
        if (e != cudaSuccess) return HA_ERR_LAUNCH;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kHashDecodeThreads);
        cfg.dynamicSmemBytes = kHdbSmemBytes;
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr1[1];
        attr1[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr1[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr1;
        cfg.numAttrs = 1;
        e = bf16 ? cudaLaunchKernelEx(&cfg, hash_decode_batched_kernel<__nv_bfloat16>, p)
                 : cudaLaunchKernelEx(&cfg, hash_decode_batched_kernel<float>, p);
        return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool pairs = p.batch_per_cta >= 2;  // two sequences of a CTA are evaluated together
    if (weights->dtype == HA_WEIGHTS_BF16)
        e = pairs ? launch(hash_decode_kernel<__nv_bfloat16, true>, grid, dim3(kHashDecodeThreads), st, 1, p)
                  : launch(hash_decode_kernel<__nv_bfloat16, false>, grid, dim3(kHashDecodeThreads), st, 1, p);
    else
        e = pairs ? launch(hash_decode_kernel<float, true>, grid, dim3(kHashDecodeThreads), st, 1, p)
                  : launch(hash_decode_kernel<float, false>, grid, dim3(kHashDecodeThreads), st, 1, p);
    return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

int ha_hash_decode(const ha_shape_t* shape, const ha_hash_weights_t* weights,
                   const void* q, const void* k_new, const void* v_new,
                   void* k_pages, void* v_pages, uint32_t* hash_pages,
                   const int32_t* page_table, const int32_t* seq_lens,
                   uint32_t* q_codes, float* preact_dbg, int32_t* status, void* stream) {
    return hash_decode_impl(shape, weights, q, k_new, v_new, k_pages, v_pages, hash_pages, page_table, seq_lens,
                            q_codes, preact_dbg, nullptr, status, stream);
}

// cuTensorMapEncodeTiled, looked up once through the runtime (the library does not link against libcuda).
static bool encode_key_map(CUtensorMap* map, const void* k_pages, uint64_t rows) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::atomic<encode_fn> cached{nullptr};
    encode_fn fn = cached.load();
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || sym == nullptr)
            return false;
        fn = reinterpret_cast<encode_fn>(sym);
        cached.store(fn);
    }
    const cuuint64_t dims[2] = {(cuuint64_t)kHeadDim, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)kHeadDim * sizeof(__nv_bfloat16)};
    const cuuint32_t box[2] = {64, (cuuint32_t)kTcTile}, elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(k_pages), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int ha_hash_prefill(const ha_shape_t* shape, const ha_hash_weights_t* weights,
                    const void* k_pages, uint32_t* hash_pages,
                    const int32_t* page_table, const int32_t* seq_lens,
                    const int32_t* first_token, int32_t* status, void* stream) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_weights(weights, false, true);
    if (rc != HA_OK) return rc;
    if (k_pages == nullptr || hash_pages == nullptr || page_table == nullptr || seq_lens == nullptr ||
        status == nullptr)
        return HA_ERR_BAD_ARG;

    if (weights->num_layers == HA_HASH_LSH) {
        // the LSH baseline: the largest key norm per kv-head over the whole cache first, then every key's code (the whole
        // cache, whatever first_token says: a longer key changes the code of every other key)
        const LshParams l = lsh_params(shape, weights, nullptr, nullptr, nullptr, const_cast<void*>(k_pages), nullptr, hash_pages,
                                       page_table, seq_lens, nullptr, nullptr, nullptr, status);
        const cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (cudaMemsetAsync(weights->lsh_state, 0, 2 * sizeof(int32_t) * shape->num_kv_heads, st) != cudaSuccess)
            return HA_ERR_LAUNCH;
        const dim3 grid(shape->max_pages, shape->num_kv_heads, shape->batch);
        // (after a memset the first kernel is launched without the programmatic attribute's early start: plain order)
        if (launch(lsh_norm_max_kernel, grid, dim3(kLshThreads), st, 1, l) != cudaSuccess) return HA_ERR_LAUNCH;
        return launch_lsh_hash_keys(shape, l, weights->dtype == HA_WEIGHTS_BF16, st) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    const int layers = weights->num_layers == 0 ? 3 : weights->num_layers;
    if (layers == 3) {
        // the 3-layer MLP: tcgen05 GEMM chain, for bf16 weights and for fp32 weights (split into hi and lo bf16 copies in
        // shared memory). One CTA per SM (its shared memory holds a head's weights).
        // (a per-device function attribute: set at every call, so that a process driving several GPUs is served)
        const bool f32 = weights->dtype != HA_WEIGHTS_BF16;
        const size_t smem_bytes = f32 ? TcLayout<true>::kSmemBytes : TcLayout<false>::kSmemBytes;
        if ((f32 ? cudaFuncSetAttribute(hash_prefill_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes)
                 : cudaFuncSetAttribute(hash_prefill_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem_bytes)) != cudaSuccess)
            return HA_ERR_LAUNCH;
        HashPrefillTcParams t;
        t.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
        t.hash_pages = hash_pages;
        t.wk = weights->wk;
        t.bk = weights->bk;
        t.page_table = page_table;
        t.seq_lens = seq_lens;
        t.first_token = first_token;
        t.status = status;
        t.B = shape->batch;
        t.Hkv = shape->num_kv_heads;
        t.max_pages = shape->max_pages;
        t.num_pages = shape->num_pages;
        // the key cache as a 2-d tensor [rows = pages x kv heads x page size][128] for the kernel's TMA loads: boxes of
        // 64 elements x 128 rows, 128-byte swizzle
        CUtensorMap k_map;
        if (!encode_key_map(&k_map, k_pages, (uint64_t)shape->num_pages * shape->num_kv_heads * kPage)) return HA_ERR_LAUNCH;
        // one CTA per SM; the kernel cuts the (head, tile) pairs into that many equal ranges
        const int Hq = shape->num_kv_heads * kGroup;
        const long long tiles = (long long)Hq * shape->batch * shape->max_pages * (kPage / kTcTile);
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
            return HA_ERR_LAUNCH;
        long long gx = sms;
        if (gx > tiles) gx = tiles;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)gx, 1, 1);
        cfg.blockDim = dim3(kTcThreads);
        cfg.dynamicSmemBytes = smem_bytes;
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr1[1];
        attr1[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr1[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr1;
        cfg.numAttrs = 1;
        const cudaError_t e = f32 ? cudaLaunchKernelEx(&cfg, hash_prefill_tc_kernel<float>, t, k_map)
                                  : cudaLaunchKernelEx(&cfg, hash_prefill_tc_kernel<__nv_bfloat16>, t, k_map);
        return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    // the 1- and 2-layer hash functions: fp32 arithmetic on the CUDA cores
    HashPrefillParams p;
    p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
    p.hash_pages = hash_pages;
    p.wk = weights->wk;
    p.bk = weights->bk;
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.first_token = first_token;
    p.status = status;
    p.B = shape->batch;
    p.Hkv = shape->num_kv_heads;
    p.max_pages = shape->max_pages;
    p.num_pages = shape->num_pages;
    const dim3 grid(shape->num_kv_heads * kGroup, shape->max_pages, shape->batch);
    p.layers = layers;
    const cudaError_t e = weights->dtype == HA_WEIGHTS_BF16
        ? launch(hash_prefill_simt_kernel<__nv_bfloat16>, grid, dim3(kHashDecodeThreads),
                 static_cast<cudaStream_t>(stream), 1, p)
        : launch(hash_prefill_simt_kernel<float>, grid, dim3(kHashDecodeThreads),
                 static_cast<cudaStream_t>(stream), 1, p);
    return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

static int score_select_impl(const ha_shape_t* shape, const ha_budget_t* budget,
                             const uint32_t* q_codes, const uint32_t* hash_pages,
                             const int32_t* page_table, const int32_t* seq_lens, const int32_t* budget_lens,
                             int32_t* sel_idx, int32_t* sel_cnt, uint8_t* scores_dbg,
                             void* workspace, size_t workspace_bytes, int32_t* status, void* stream,
                             bool plan_only = false, bool handover = false) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (q_codes == nullptr || hash_pages == nullptr || page_table == nullptr || seq_lens == nullptr ||
        (sel_idx == nullptr && !plan_only) || sel_cnt == nullptr || status == nullptr)
        return HA_ERR_BAD_ARG;
    if (workspace == nullptr) return HA_ERR_WORKSPACE;
    const Workspace w = carve(shape, budget, workspace);
    if (workspace_bytes < w.bytes) return HA_ERR_WORKSPACE;

    SelectParams p = select_params(shape, budget, q_codes, hash_pages, page_table, seq_lens, sel_idx, sel_cnt,
                                   scores_dbg, status, w.hist, w.plan, w.scores, w.arrive, w.sel_rows, budget_lens);
    // handover: the caller launches the selection right behind this call; it then takes each unit's plan as soon as
    // that unit is ready instead of waiting for the whole scoring grid
    const int ho = option(HA_OPT_PLAN_HANDOVER);  // 0: off; 2: the selection waits for an announcement that is not made
    p.signal = ((!plan_only || handover) && ho != 0 && ho != 2) ? 1 : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long max_tokens = (long long)shape->max_pages * kPage;
    if (!plan_only && use_cluster_select(shape)) {
        const dim3 cgrid(kClCtas, shape->num_kv_heads, shape->batch);
        const cudaError_t e = max_tokens <= kClRoundTokens
            ? launch(score_select_cluster_kernel<1>, cgrid, dim3(kClThreads), s, kClCtas, p)
            : launch(score_select_cluster_kernel<2>, cgrid, dim3(kClThreads), s, kClCtas, p);
        return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    if (launch_score_hist(shape, p, shape->num_kv_heads, s) != cudaSuccess) return HA_ERR_LAUNCH;
    if (plan_only) return HA_OK;
    SelectAttendParams sa = select_attend_params(shape, budget, w.plan, w.scores, w.partials, sel_idx, nullptr,
                                                 nullptr, nullptr, page_table, seq_lens, budget_lens, 1.0f,
                                                 nullptr, status, nullptr);
    if (ho != 0) sa.ready = reinterpret_cast<int32_t*>(w.arrive);
    return launch_select_attend(shape, sa, shape->num_kv_heads * kGroup, false, s) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

// The selection + attention stage on the plan and score bytes a scoring call left in the workspace.
static int select_attend_impl(const ha_shape_t* shape, const ha_budget_t* budget, const void* q, const void* k_pages,
                              const void* v_pages, const int32_t* page_table, const int32_t* seq_lens,
                              const int32_t* budget_lens, int32_t* sel_idx, float sm_scale, void* out, void* workspace,
                              size_t workspace_bytes, int32_t* status, void* stream, int32_t* status_out,
                              bool handover = false) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (q == nullptr || k_pages == nullptr || v_pages == nullptr || page_table == nullptr || seq_lens == nullptr ||
        sel_idx == nullptr || out == nullptr || status == nullptr || !std::isfinite(sm_scale))
        return HA_ERR_BAD_ARG;
    if (workspace == nullptr) return HA_ERR_WORKSPACE;
    const Workspace w = carve(shape, budget, workspace);
    if (workspace_bytes < w.bytes) return HA_ERR_WORKSPACE;
    SelectAttendParams sa = select_attend_params(shape, budget, w.plan, w.scores, w.partials, sel_idx, q, k_pages,
                                                 v_pages, page_table, seq_lens, budget_lens, sm_scale, out,
                                                 status, status_out);
    if (handover) sa.ready = reinterpret_cast<int32_t*>(w.arrive);  // (the scoring call in front was told the same)
    return launch_select_attend(shape, sa, shape->num_kv_heads * kGroup, true, static_cast<cudaStream_t>(stream)) ==
                   cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

int ha_score_plan(const ha_shape_t* shape, const ha_budget_t* budget,
                  const uint32_t* q_codes, const uint32_t* hash_pages,
                  const int32_t* page_table, const int32_t* seq_lens, int32_t* sel_cnt,
                  void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
    return score_select_impl(shape, budget, q_codes, hash_pages, page_table, seq_lens, nullptr, nullptr, sel_cnt,
                             nullptr, workspace, workspace_bytes, status, stream, true);
}

int ha_select_attend(const ha_shape_t* shape, const ha_budget_t* budget,
                     const void* q, const void* k_pages, const void* v_pages,
                     const int32_t* page_table, const int32_t* seq_lens,
                     int32_t* sel_idx, float sm_scale, void* out,
                     void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
    return select_attend_impl(shape, budget, q, k_pages, v_pages, page_table, seq_lens, nullptr, sel_idx, sm_scale, out,
                              workspace, workspace_bytes, status, stream, nullptr);
}

int ha_score_select(const ha_shape_t* shape, const ha_budget_t* budget,
                    const uint32_t* q_codes, const uint32_t* hash_pages,
                    const int32_t* page_table, const int32_t* seq_lens,
                    int32_t* sel_idx, int32_t* sel_cnt, uint8_t* scores_dbg,
                    void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
    return score_select_impl(shape, budget, q_codes, hash_pages, page_table, seq_lens, nullptr, sel_idx, sel_cnt,
                             scores_dbg, workspace, workspace_bytes, status, stream);
}

int ha_sparse_decode(const ha_shape_t* shape, const ha_budget_t* budget,
                     const void* q, const void* k_pages, const void* v_pages,
                     const int32_t* page_table, const int32_t* seq_lens,
                     const int32_t* sel_idx, const int32_t* sel_cnt, float sm_scale,
                     void* out, void* workspace, size_t workspace_bytes,
                     int32_t* status, void* stream) {
    if (sel_idx == nullptr || sel_cnt == nullptr) return check_shape(shape) != HA_OK ? check_shape(shape) : HA_ERR_BAD_ARG;
    return sparse_decode_impl(shape, budget, q, k_pages, v_pages, page_table, seq_lens, sel_idx, sel_cnt, false,
                              sm_scale, out, workspace, workspace_bytes, status, stream);
}

// The step; q_stage, if given, receives a device copy of q from the encoder kernel and the
// attention kernels read that copy instead of q (used when q is mapped host memory).
static int decode_step_impl(const ha_shape_t* shape, const ha_budget_t* budget,
                            const ha_hash_weights_t* weights,
                            const void* q, const void* k_new, const void* v_new, void* q_stage,
                            void* k_pages, void* v_pages, uint32_t* hash_pages,
                            const int32_t* page_table, const int32_t* seq_lens, const int32_t* budget_lens,
                            uint32_t* q_codes, int32_t* sel_idx, int32_t* sel_cnt, float sm_scale,
                            void* out, void* workspace, size_t workspace_bytes,
                            int32_t* status, void* stream, int32_t* status_out = nullptr,
                            bool* status_delivered = nullptr) {
    if (status_delivered != nullptr) *status_delivered = false;
    int rc = hash_decode_impl(shape, weights, q, k_new, v_new, k_pages, v_pages, hash_pages, page_table,
                              seq_lens, q_codes, nullptr, q_stage, status, stream);
    if (rc != HA_OK) return rc;
    const void* q_att = q_stage != nullptr ? q_stage : q;
    if (!use_cluster_select(shape)) {
        const bool handover = option(HA_OPT_PLAN_HANDOVER) != 0;
        // scoring + plan, then selection + attention; the merge kernel, last of the step, also leaves the status
        // word in status_out, if given
        rc = score_select_impl(shape, budget, q_codes, hash_pages, page_table, seq_lens, budget_lens, sel_idx, sel_cnt,
                               nullptr, workspace, workspace_bytes, status, stream, true, handover);
        if (rc != HA_OK) return rc;
        if (status_delivered != nullptr) *status_delivered = status_out != nullptr;
        return select_attend_impl(shape, budget, q_att, k_pages, v_pages, page_table, seq_lens, budget_lens, sel_idx,
                                  sm_scale, out, workspace, workspace_bytes, status, stream, status_out, handover);
    }
    rc = score_select_impl(shape, budget, q_codes, hash_pages, page_table, seq_lens, budget_lens, sel_idx, sel_cnt,
                           nullptr, workspace, workspace_bytes, status, stream);
    if (rc != HA_OK) return rc;
    // the cluster selection left the physical rows of the heavy tokens in the workspace; the step's last kernel
    // also leaves the status word in status_out, if given
    if (status_delivered != nullptr) *status_delivered = status_out != nullptr;
    return sparse_decode_impl(shape, budget, q_att, k_pages, v_pages, page_table, seq_lens, nullptr, sel_cnt, true,
                              sm_scale, out, workspace, workspace_bytes, status, stream, budget_lens, status_out);
}

int ha_decode_step(const ha_shape_t* shape, const ha_budget_t* budget,
                   const ha_hash_weights_t* weights,
                   const void* q, const void* k_new, const void* v_new,
                   void* k_pages, void* v_pages, uint32_t* hash_pages,
                   const int32_t* page_table, const int32_t* seq_lens,
                   uint32_t* q_codes, int32_t* sel_idx, int32_t* sel_cnt, float sm_scale,
                   void* out, void* workspace, size_t workspace_bytes,
                   int32_t* status, void* stream) {
    return decode_step_impl(shape, budget, weights, q, k_new, v_new, nullptr, k_pages, v_pages, hash_pages,
                            page_table, seq_lens, nullptr, q_codes, sel_idx, sel_cnt, sm_scale, out, workspace,
                            workspace_bytes, status, stream);
}

int ha_decode_step_rows(const ha_shape_t* shape, const ha_budget_t* budget,
                        const ha_hash_weights_t* weights,
                        const void* q, const void* k_new, const void* v_new,
                        void* k_pages, void* v_pages, uint32_t* hash_pages,
                        const int32_t* page_table, const int32_t* seq_lens, const int32_t* budget_lens,
                        uint32_t* q_codes, int32_t* sel_idx, int32_t* sel_cnt, float sm_scale,
                        void* out, void* workspace, size_t workspace_bytes,
                        int32_t* status, void* stream) {
    if (budget_lens == nullptr) return check_shape(shape) != HA_OK ? check_shape(shape) : HA_ERR_BAD_ARG;
    // (the LSH baseline takes its norm bound over the vectors of a call; rows of one chunk would have to share it)
    if (weights != nullptr && weights->num_layers == HA_HASH_LSH) return HA_ERR_BAD_ARG;
    return decode_step_impl(shape, budget, weights, q, k_new, v_new, nullptr, k_pages, v_pages, hash_pages,
                            page_table, seq_lens, budget_lens, q_codes, sel_idx, sel_cnt, sm_scale, out, workspace,
                            workspace_bytes, status, stream);
}

int ha_decode_step_launches(const ha_shape_t* shape, const ha_budget_t* budget) {
    if (check_shape(shape) != HA_OK || check_budget(budget) != HA_OK) return 0;
    if (use_cluster_select(shape)) {  // encoder, cluster selection, gather (+ merge)
        const AttSplit as = att_split_launch(shape, budget);
        return 3 + (as.nsplits > 1 && !as.cluster ? 1 : 0);
    }
    return 4;  // encoder, scoring + plan, selection + attention, merge
}

const char* ha_decode_step_path(const ha_shape_t* shape, const ha_budget_t* budget) {
    if (check_shape(shape) != HA_OK || check_budget(budget) != HA_OK) return "invalid";
    if (use_cluster_select(shape))
        return att_split_launch(shape, budget).cluster
            ? "hash_decode | score_select_cluster | sparse_gather (cluster)"
            : "hash_decode | score_select_cluster | sparse_gather | sparse_merge";
    return "hash_decode | score_hist | select_attend | select_attend_merge";
}

int ha_decode_step_host(const ha_shape_t* shape, const ha_budget_t* budget,
                        const ha_hash_weights_t* weights,
                        const void* q_host, const void* k_new_host, const void* v_new_host,
                        void* out_host, int32_t* status_host,
                        void* q_dev, void* k_new_dev, void* v_new_dev, void* out_dev,
                        void* k_pages, void* v_pages, uint32_t* hash_pages,
                        const int32_t* page_table, const int32_t* seq_lens,
                        uint32_t* q_codes, int32_t* sel_idx, int32_t* sel_cnt, float sm_scale,
                        void* workspace, size_t workspace_bytes,
                        int32_t* status, void* stream, int synchronize) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    if (q_host == nullptr || out_host == nullptr || status_host == nullptr || q_dev == nullptr ||
        out_dev == nullptr || status == nullptr)
        return HA_ERR_BAD_ARG;
    if ((k_new_host == nullptr) != (k_new_dev == nullptr) || (v_new_host == nullptr) != (v_new_dev == nullptr))
        return HA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t q_bytes = (size_t)shape->batch * shape->num_kv_heads * kGroup * kHeadDim * sizeof(__nv_bfloat16);
    const size_t kv_bytes = (size_t)shape->batch * shape->num_kv_heads * kHeadDim * sizeof(__nv_bfloat16);
    // Page-locked host buffers that the device can address are used in place: the encoder kernel
    // reads q / k_new / v_new over the bus exactly once (and leaves a device copy of q in q_dev for
    // the attention kernels), the last kernel stores the result straight into out_host. That removes
    // four copy operations and their launch gaps from the step. Pageable buffers are staged.
    void* q_map = mapped_host_pointer(q_host);
    void* k_map = k_new_host != nullptr ? mapped_host_pointer(k_new_host) : nullptr;
    void* v_map = v_new_host != nullptr ? mapped_host_pointer(v_new_host) : nullptr;
    void* out_map = mapped_host_pointer(out_host);
    const bool in_place = q_map != nullptr && out_map != nullptr && (k_new_host == nullptr || k_map != nullptr) &&
                          (v_new_host == nullptr || v_map != nullptr);
    bool status_delivered = false;
    if (in_place) {
        // the status word, too, is stored into the caller's page-locked word by the step's last kernel when a
        // single kernel ends the step: a copy operation after the kernels costs 5-8 us on a 19 us step
        rc = decode_step_impl(shape, budget, weights, q_map, k_map, v_map, q_dev, k_pages, v_pages, hash_pages,
                              page_table, seq_lens, nullptr, q_codes, sel_idx, sel_cnt, sm_scale, out_map, workspace,
                              workspace_bytes, status, stream,
                              static_cast<int32_t*>(mapped_host_pointer(status_host)), &status_delivered);
        if (rc != HA_OK) return rc;
    } else {
        if (cudaMemcpyAsync(q_dev, q_host, q_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) return HA_ERR_LAUNCH;
        if (k_new_host != nullptr &&
            cudaMemcpyAsync(k_new_dev, k_new_host, kv_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
            return HA_ERR_LAUNCH;
        if (v_new_host != nullptr &&
            cudaMemcpyAsync(v_new_dev, v_new_host, kv_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
            return HA_ERR_LAUNCH;
        rc = ha_decode_step(shape, budget, weights, q_dev, k_new_dev, v_new_dev, k_pages, v_pages, hash_pages,
                            page_table, seq_lens, q_codes, sel_idx, sel_cnt, sm_scale, out_dev, workspace,
                            workspace_bytes, status, stream);
        if (rc != HA_OK) return rc;
        if (cudaMemcpyAsync(out_host, out_dev, q_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess) return HA_ERR_LAUNCH;
    }
    if (!status_delivered &&
        cudaMemcpyAsync(status_host, status, sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess)
        return HA_ERR_LAUNCH;
    if (synchronize) {
        if (cudaStreamSynchronize(s) != cudaSuccess) return HA_ERR_LAUNCH;
        return *status_host;
    }
    return HA_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// ha_rope_split: helper of a host model's decode step - splits the fused q|k|v projection of one new token per
// sequence into the contiguous q, k_new, v_new tensors the decode step takes and applies the rotary position
// embedding to q and k on the way (one launch instead of a dozen elementwise ones).
// ------------------------------------------------------------------------------------------
namespace ha {
namespace {

// grid (heads, B), 64 threads: thread t owns dimensions t and t + 64 of one head (the rotate-half pair).
__global__ void __launch_bounds__(64) rope_split_kernel(const __nv_bfloat16* __restrict__ qkv, const long long* __restrict__ pos,
                                                        __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                                        __nv_bfloat16* __restrict__ v, int hq, int hkv, float log2_theta) {
    const int head = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
    const int heads = hq + 2 * hkv;
    const __nv_bfloat16* src = qkv + ((size_t)b * heads + head) * kHeadDim;
    const float x1 = __bfloat162float(src[t]), x2 = __bfloat162float(src[t + 64]);
    __nv_bfloat16* dst;
    if (head < hq) dst = q + ((size_t)b * hq + head) * kHeadDim;
    else if (head < hq + hkv) dst = k + ((size_t)b * hkv + (head - hq)) * kHeadDim;
    else {  // a value head: copied as it is
        dst = v + ((size_t)b * hkv + (head - hq - hkv)) * kHeadDim;
        dst[t] = src[t];
        dst[t + 64] = src[t + 64];
        return;
    }
    // angle = position * theta^(-2 t / 128), cos / sin in fp32 as the reference's rotary tables are
    const float inv_freq = exp2f(-log2_theta * (float)(2 * t) / (float)kHeadDim);
    float sn, cs;
    sincosf((float)pos[b] * inv_freq, &sn, &cs);
    dst[t] = __float2bfloat16_rn(x1 * cs - x2 * sn);
    dst[t + 64] = __float2bfloat16_rn(x2 * cs + x1 * sn);
}

}  // namespace
}  // namespace ha

extern "C" int ha_rope_split(const void* qkv, const int64_t* positions, int32_t batch, int32_t num_q_heads,
                             int32_t num_kv_heads, float rope_theta, void* q, void* k_new, void* v_new, void* stream) {
    if (qkv == nullptr || positions == nullptr || q == nullptr || k_new == nullptr || v_new == nullptr) return HA_ERR_BAD_ARG;
    if (batch < 1 || batch > 65535 || num_q_heads < 1 || num_kv_heads < 1 || !(rope_theta > 1.0f)) return HA_ERR_BAD_ARG;
    rope_split_kernel<<<dim3(num_q_heads + 2 * num_kv_heads, batch), 64, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<const long long*>(positions),
        static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k_new), static_cast<__nv_bfloat16*>(v_new),
        num_q_heads, num_kv_heads, log2f(rope_theta));
    return cudaGetLastError() == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------
// ha_score_select_static: the selection kernels on scratch memory that is part of the library
// image, for callers that may not allocate (see include/hashattn.h).
// ------------------------------------------------------------------------------------------
namespace {

// Lives in every GPU context that loads the library, until the process ends. In host code this
// name is only a handle for cudaGetSymbolAddress: it is not a device address and must never be
// passed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[HA_STATIC_SCRATCH_BYTES];

std::mutex g_static_scratch_mutex;
void* g_static_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device

struct StaticScratch {
    uint32_t* hist;     // [B][Hkv][4*33][nchunks]
    int32_t* plan;      // [B][Hkv][8 + 8 * nchunks]
    uint8_t* scores;    // [B][Hq][nchunks * chunk tokens]
    uint32_t* arrive;   // [B][Hkv][kArriveStride]
    size_t arrive_bytes, bytes;
};

StaticScratch carve_static(const ha_shape_t* s, void* base) {
    const ha::Geometry g = ha::geometry(s);
    const size_t units = (size_t)s->batch * s->num_kv_heads;
    char* p = static_cast<char*>(base);
    StaticScratch w;
    size_t off = 0;
    w.hist = reinterpret_cast<uint32_t*>(p + off);
    off += align_up(units * g.nchunks * kGroup * kBins * sizeof(uint32_t));
    w.plan = reinterpret_cast<int32_t*>(p + off);
    off += align_up(units * (8 + 8 * (size_t)g.nchunks) * sizeof(int32_t));
    w.scores = reinterpret_cast<uint8_t*>(p + off);
    off += align_up(ha::scores_bytes(s, g));
    w.arrive = reinterpret_cast<uint32_t*>(p + off);
    w.arrive_bytes = units * ha::kArriveStride * sizeof(uint32_t);
    off += align_up(w.arrive_bytes);
    w.bytes = off;
    return w;
}

// Device address of the static buffer on the current device; looked up once per device.
int static_scratch_address(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return HA_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return HA_ERR_LAUNCH;
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return HA_OK;
}

}  // namespace

extern "C" {

size_t ha_static_scratch_needed(const ha_shape_t* shape) {
    if (check_shape(shape) != HA_OK) return 0;
    return carve_static(shape, nullptr).bytes;
}

int ha_score_select_static(const ha_shape_t* shape, const ha_budget_t* budget,
                           const uint32_t* q_codes, const uint32_t* hash_pages,
                           const int32_t* page_table, const int32_t* seq_lens,
                           int32_t* sel_idx, int32_t* sel_cnt, int32_t* status, void* stream) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (q_codes == nullptr || hash_pages == nullptr || page_table == nullptr || seq_lens == nullptr ||
        sel_idx == nullptr || sel_cnt == nullptr || status == nullptr)
        return HA_ERR_BAD_ARG;
    if (carve_static(shape, nullptr).bytes > HA_STATIC_SCRATCH_BYTES) return HA_ERR_SCRATCH_LIMIT;
    void* base = nullptr;
    rc = static_scratch_address(&base);
    if (rc != HA_OK) return rc;
    const StaticScratch w = carve_static(shape, base);

    // The arrival counters must be zero when the scoring kernel starts; the buffer keeps whatever the last call
    // (possibly one of another shape, with the counters elsewhere) left, so they are cleared on the stream first.
    // Every other word a kernel reads was written earlier in the same call.
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(w.arrive, 0, w.arrive_bytes, s) != cudaSuccess) return HA_ERR_LAUNCH;
    const SelectParams p = select_params(shape, budget, q_codes, hash_pages, page_table, seq_lens, sel_idx, sel_cnt,
                                         nullptr, status, w.hist, w.plan, w.scores, w.arrive, nullptr);
    if (launch_score_hist(shape, p, shape->num_kv_heads, s) != cudaSuccess) return HA_ERR_LAUNCH;
    const SelectAttendParams sa = select_attend_params(shape, budget, w.plan, w.scores, nullptr, sel_idx, nullptr,
                                                       nullptr, nullptr, page_table, seq_lens, nullptr, 1.0f, nullptr,
                                                       status, nullptr);
    return launch_select_attend(shape, sa, shape->num_kv_heads * kGroup, false, s) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

}  // extern "C"
