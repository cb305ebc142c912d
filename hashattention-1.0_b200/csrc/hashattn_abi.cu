// extern "C" entry points of libhashattn.so (declared in include/hashattn.h): argument checks,
// workspace carving and kernel launches. No device memory is allocated, nothing synchronises with
// the host (except where ha_decode_step_host is asked to), nothing throws. The only resources the
// library creates are a stream and events per device for the staggered decode step, at its first use.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "hash_decode.cuh"
#include "hash_prefill_tc.cuh"
#include "score_select.cuh"
#include "sparse_decode.cuh"

#ifndef HA_USE_PDL
#define HA_USE_PDL 1
#endif

namespace ha {
namespace {

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

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
    if (w->num_layers < 0 || w->num_layers > 3) return HA_ERR_BAD_ARG;
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
    const char* env = std::getenv("HA_CLUSTER_GATHER");  // "0" / "1" force the choice (experiments, tests)
    const bool fits = rounds <= kAttMaxRounds && a.nsplits > 1;
    const bool want = env != nullptr ? env[0] == '1' : total <= 65536;
    if (fits && want) {
        a.cluster = true;
        a.rounds = (int)(rounds < 1 ? 1 : rounds);
        a.nsplits = kAttClusterCtas;
    }
    return a;
}

struct Workspace {
    uint32_t* hist;     // [B][Hkv][4*33][nchunks] per-chunk score histograms
    int32_t* sel_rows;  // [B][Hq][sel_stride] physical rows of the selected tokens
    float* partials;    // [B][Hq][nsplits][130] attention partials
    int32_t* plan;      // [B][Hkv][8 + 8 * nchunks] thresholds, tie quotas and per-chunk output bases
    uint32_t* scores;   // [B][Hkv][nchunks * chunk tokens] packed scores of the 4 heads of a group, one byte each
    size_t bytes;
};

size_t scores_bytes(const ha_shape_t* s) {
    return (size_t)s->batch * s->num_kv_heads * num_chunks_for(s->max_pages) * chunk_pages_for(s->max_pages) * kPage *
           sizeof(uint32_t);
}

Workspace carve(const ha_shape_t* s, const ha_budget_t* b, void* base) {
    const size_t Hq = (size_t)s->num_kv_heads * kGroup;
    const size_t n_hist = (size_t)s->batch * s->num_kv_heads * num_chunks_for(s->max_pages) * kGroup * kBins;
    char* p = static_cast<char*>(base);
    Workspace w;
    size_t off = 0;
    w.hist = reinterpret_cast<uint32_t*>(p + off);
    off += align_up(n_hist * sizeof(uint32_t));
    w.sel_rows = reinterpret_cast<int32_t*>(p + off);
    off += align_up((size_t)s->batch * Hq * s->sel_stride * sizeof(int32_t));
    w.partials = reinterpret_cast<float*>(p + off);
    off += align_up((size_t)s->batch * Hq * att_split(s, b).nsplits * kPartStride * sizeof(float));
    w.plan = reinterpret_cast<int32_t*>(p + off);
    off += align_up((size_t)s->batch * s->num_kv_heads * (8 + 8 * (size_t)num_chunks_for(s->max_pages)) * sizeof(int32_t));
    w.scores = reinterpret_cast<uint32_t*>(p + off);
    off += align_up(scores_bytes(s));
    w.bytes = off;
    return w;
}

// Priority given to the kernels launched inside a PriorityScope (0 = the stream's own). Used only
// by the staggered decode step, where the short latency-bound kernels of one half must get SM
// slots ahead of the queued CTAs of the other half's streaming kernels.
thread_local int t_launch_priority = 0;
struct PriorityScope {
    int saved;
    explicit PriorityScope(int p) : saved(t_launch_priority) { t_launch_priority = p; }
    ~PriorityScope() { t_launch_priority = saved; }
};

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
    cudaLaunchAttribute attr[3];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = HA_USE_PDL;
    cfg.numAttrs = 1;
    if (cluster_x > 1) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
        attr[cfg.numAttrs].val.clusterDim.x = cluster_x;
        attr[cfg.numAttrs].val.clusterDim.y = 1;
        attr[cfg.numAttrs].val.clusterDim.z = 1;
        ++cfg.numAttrs;
    }
    if (t_launch_priority != 0) {
        attr[cfg.numAttrs].id = cudaLaunchAttributePriority;
        attr[cfg.numAttrs].val.priority = t_launch_priority;
        ++cfg.numAttrs;
    }
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The two-pass selection on the kv-heads [p.kvh0, p.kvh0 + nkvh): chunk histograms and packed
// scores (launch_score_hist), then the plan (thresholds and output bases, derived from the
// histograms once per (sequence, kv-head)) and the compaction (launch_plan_select).
cudaError_t launch_score_hist(const ha_shape_t* shape, const SelectParams& p, int nkvh, cudaStream_t s) {
    const dim3 grid(p.nchunks, nkvh, shape->batch);
    switch (chunk_pages_for(shape->max_pages)) {
        case 4: return launch(score_hist_kernel<1>, grid, dim3(kSelThreads), s, 1, p);
        case 8: return launch(score_hist_kernel<2>, grid, dim3(kSelThreads), s, 1, p);
        default: return launch(score_hist_kernel<4>, grid, dim3(kSelThreads), s, 1, p);
    }
}

cudaError_t launch_plan_select(const ha_shape_t* shape, const SelectParams& p, int nkvh, cudaStream_t s,
                               int priority = 0) {
    const dim3 grid(p.nchunks, nkvh, shape->batch);
    const int chunk_pages = chunk_pages_for(shape->max_pages);
    PriorityScope scope(priority);
    const cudaError_t e = launch(select_plan_kernel, dim3(nkvh, shape->batch), dim3(kSelThreads), s, 1, p,
                                 chunk_pages * kPage);
    if (e != cudaSuccess) return e;
    switch (chunk_pages) {
        case 4: return launch(select_kernel<1>, grid, dim3(kSelBThreads), s, 1, p);
        case 8: return launch(select_kernel<2>, grid, dim3(kSelBThreads), s, 1, p);
        default: return launch(select_kernel<4>, grid, dim3(kSelBThreads), s, 1, p);
    }
}

cudaError_t launch_two_pass_select(const ha_shape_t* shape, const SelectParams& p, int nkvh, cudaStream_t s) {
    const cudaError_t e = launch_score_hist(shape, p, nkvh, s);
    return e != cudaSuccess ? e : launch_plan_select(shape, p, nkvh, s);
}

// One cluster kernel scores and selects in a single pass when the sequences are short and there are at
// most 8 (sequence, kv-head) units, one cluster of 8 CTAs x 1024 threads per GPC: at most two rounds each
// (measured 6.9 us against 9.4 us for the two-pass kernels at B=1, S=32K). With 16 units the clusters no
// longer run side by side (13.7 us against 11.6 us for the two-pass kernels at B=2), and longer sequences
// are bandwidth- rather than latency-bound (45 us against 62 us at B=4, S=128K).
bool use_cluster_select(const ha_shape_t* shape) {
    const long long max_tokens = (long long)shape->max_pages * kPage;
    const long long units = (long long)shape->batch * shape->num_kv_heads;
    return max_tokens <= 2LL * kClRoundTokens && units <= 8;
}

}  // namespace
}  // namespace ha

namespace ha {
namespace {

SelectParams select_params(const ha_shape_t* shape, const ha_budget_t* budget, const uint32_t* q_codes,
                           const uint32_t* hash_pages, const int32_t* page_table, const int32_t* seq_lens,
                           int32_t* sel_idx, int32_t* sel_cnt, uint8_t* scores_dbg, int32_t* status,
                           uint32_t* hist, int32_t* plan, uint32_t* scores, int32_t* sel_rows,
                           const int32_t* budget_lens = nullptr) {
    SelectParams p;
    p.q_codes = q_codes;
    p.hash_pages = reinterpret_cast<const uint4*>(hash_pages);
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.budget_lens = budget_lens;
    p.hist = hist;
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
    p.nchunks = num_chunks_for(shape->max_pages);
    p.kvh0 = 0;
    p.init_budget = budget->init_budget;
    p.recent_budget = budget->recent_budget;
    p.heavy_budget = budget->heavy_budget;
    p.eval_mode = budget->eval_mode;
    p.depth = budget->retrieve_depth;
    return p;
}

// sel == nullptr with physical == true: use the physical rows select_kernel left in the workspace.
int sparse_decode_impl(const ha_shape_t* shape, const ha_budget_t* budget,
                       const void* q, const void* k_pages, const void* v_pages,
                       const int32_t* page_table, const int32_t* seq_lens,
                       const int32_t* sel, const int32_t* sel_cnt, bool physical, float sm_scale,
                       void* out, void* workspace, size_t workspace_bytes,
                       int32_t* status, void* stream, int kvh0 = 0, int nkvh = -1, int merge_priority = 0,
                       const int32_t* budget_lens = nullptr, int32_t* status_out = nullptr) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (q == nullptr || k_pages == nullptr || v_pages == nullptr || page_table == nullptr ||
        seq_lens == nullptr || out == nullptr || status == nullptr || !std::isfinite(sm_scale))
        return HA_ERR_BAD_ARG;
    if (budget->eval_mode != HA_EVAL_SIMPLE && sel_cnt == nullptr) return HA_ERR_BAD_ARG;  // variable-size sets
    const int nheads = (nkvh < 0 ? shape->num_kv_heads : nkvh) * kGroup;  // heads [4 kvh0, 4 kvh0 + nheads)
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
    p.h0 = kvh0 * kGroup;
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
        PriorityScope light(merge_priority);
        e = launch(sparse_merge_kernel, dim3(nheads, shape->batch), dim3(kHeadDim), s, 1, p);
    }
    return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

}  // namespace
}  // namespace ha

// ------------------------------------------------------------------------------------------
// Staggered decode step. Between the histogram pass and the gather of one set of kv-heads lie
// the plan and the compaction, short kernels that leave HBM idle. For large problems the step is
// therefore run as two halves of the kv-heads, the second one a histogram pass behind the
// first, so that one half's short kernels overlap the other half's streaming kernels. The second
// half runs on a stream that belongs to the library (one per device, created at the first such
// call) and is forked from / joined to the caller's stream with events, which also works under
// stream capture. Every (sequence, kv-head) is independent, so the result is bit-identical.
// ------------------------------------------------------------------------------------------
namespace ha {
namespace {

constexpr int kMaxDevices = 64;

constexpr int kMaxParts = 4;

struct StaggerResources {
    cudaStream_t aux[kMaxParts - 1] = {};           // parts 1.. run here; part 0 on the caller's stream
    cudaEvent_t fork[kMaxParts - 1] = {}, join[kMaxParts - 1] = {};
    int light_priority = 0;  // for the short kernels: the most urgent priority the device offers
    bool ready = false;
};
std::mutex g_stagger_mutex;  // held while a staggered step is enqueued: the events are shared
StaggerResources g_stagger[kMaxDevices];

// Environment override HA_STAGGER: "0" never, "1" whenever the two-pass selection runs on at
// least two kv-heads; otherwise only when the hash pages of the step exceed 32 MB.
bool use_stagger(const ha_shape_t* shape) {
    if (use_cluster_select(shape) || shape->num_kv_heads < 2) return false;
    const char* env = std::getenv("HA_STAGGER");
    if (env != nullptr && env[0] == '0') return false;
    if (env != nullptr && env[0] == '1') return true;
    const long long hash_bytes = (long long)shape->batch * shape->num_kv_heads * shape->max_pages * kPage * 16;
    return hash_bytes >= (32LL << 20);
}

// Two parts measured best (B=4, S=128K: 82.9 us per step against 83.8 with three and 91.5 with four
// parts, 88.2 without staggering); HA_STAGGER_PARTS is an experiment knob.
int stagger_parts(const ha_shape_t* shape) {
    int parts = 2;
    if (const char* env = std::getenv("HA_STAGGER_PARTS")) parts = std::atoi(env);
    return std::max(2, std::min(parts, std::min(kMaxParts, shape->num_kv_heads)));
}

// Caller holds g_stagger_mutex.
StaggerResources* stagger_resources() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    StaggerResources& r = g_stagger[dev];
    if (!r.ready) {
        int least = 0, greatest = 0;
        if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) return nullptr;
        bool ok = true;
        for (int i = 0; i < kMaxParts - 1 && ok; ++i)
            ok = cudaStreamCreateWithFlags(&r.aux[i], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&r.fork[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&r.join[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {  // give back whatever was created, so that a later call starts from nothing
            for (int i = 0; i < kMaxParts - 1; ++i) {
                if (r.aux[i] != nullptr) cudaStreamDestroy(r.aux[i]);
                if (r.fork[i] != nullptr) cudaEventDestroy(r.fork[i]);
                if (r.join[i] != nullptr) cudaEventDestroy(r.join[i]);
                r.aux[i] = nullptr;
                r.fork[i] = r.join[i] = nullptr;
            }
            return nullptr;
        }
        r.light_priority = greatest;
        r.ready = true;
    }
    return &r;
}

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

int staggered_select_attend(const ha_shape_t* shape, const ha_budget_t* budget, const void* q,
                            const void* k_pages, const void* v_pages, const uint32_t* hash_pages,
                            const int32_t* page_table, const int32_t* seq_lens, const uint32_t* q_codes,
                            int32_t* sel_idx, int32_t* sel_cnt, float sm_scale, void* out, void* workspace,
                            size_t workspace_bytes, int32_t* status, cudaStream_t s, const int32_t* budget_lens) {
    int rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (q_codes == nullptr || hash_pages == nullptr || page_table == nullptr || seq_lens == nullptr ||
        sel_idx == nullptr || sel_cnt == nullptr || status == nullptr)
        return HA_ERR_BAD_ARG;
    if (workspace == nullptr) return HA_ERR_WORKSPACE;
    const Workspace w = carve(shape, budget, workspace);
    if (workspace_bytes < w.bytes) return HA_ERR_WORKSPACE;
    const int parts = stagger_parts(shape);
    const SelectParams base = select_params(shape, budget, q_codes, hash_pages, page_table, seq_lens, sel_idx,
                                            sel_cnt, nullptr, status, w.hist, w.plan, w.scores, w.sel_rows,
                                            budget_lens);

    std::lock_guard<std::mutex> lock(g_stagger_mutex);
    StaggerResources* r = stagger_resources();
    if (r == nullptr) return HA_ERR_LAUNCH;
    const int light = r->light_priority;
    // Part i covers kv-heads [first, first + n) (the larger parts first) on stream i (0 = the caller's) and
    // starts when the histogram pass of part i - 1 is done.
    bool ok = true;
    int first = 0;
    for (int i = 0; i < parts; ++i) {
        const int n = shape->num_kv_heads / parts + (i < shape->num_kv_heads % parts ? 1 : 0);
        cudaStream_t si = i == 0 ? s : r->aux[i - 1];
        SelectParams p = base;
        p.kvh0 = first;
        ok = ok && launch_score_hist(shape, p, n, si) == cudaSuccess;
        if (i + 1 < parts) {  // even after a failed launch: every stream that forks is also joined below
            if (cudaEventRecord(r->fork[i], si) != cudaSuccess ||
                cudaStreamWaitEvent(r->aux[i], r->fork[i], 0) != cudaSuccess)
                return HA_ERR_LAUNCH;
        }
        ok = ok && launch_plan_select(shape, p, n, si, light) == cudaSuccess;
        ok = ok && sparse_decode_impl(shape, budget, q, k_pages, v_pages, page_table, seq_lens, nullptr, sel_cnt, true,
                                      sm_scale, out, workspace, workspace_bytes, status, si, first, n, light,
                                      budget_lens) == HA_OK;
        first += n;
    }
    for (int i = 1; i < parts; ++i)
        if (cudaEventRecord(r->join[i - 1], r->aux[i - 1]) != cudaSuccess ||
            cudaStreamWaitEvent(s, r->join[i - 1], 0) != cudaSuccess)
            return HA_ERR_LAUNCH;
    return ok ? HA_OK : HA_ERR_LAUNCH;
}

}  // namespace
}  // namespace ha

using namespace ha;

extern "C" {

#ifdef HA_TIMELINE
// Debug builds only: where the kernels stamp their timeline (device buffer of
// kTlKernels * kTlEvents * 2 unsigned 64-bit words, minima preset to ~0, maxima to 0).
int ha_debug_set_timeline(unsigned long long* buffer) {
    return cudaMemcpyToSymbol(g_timeline, &buffer, sizeof(buffer)) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}
#endif

int ha_abi_version(void) { return HA_ABI_VERSION; }

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
    // the kernels keep no state in the workspace between calls; clearing it only makes runs
    // that read it before writing (a misuse) reproducible
    if (cudaMemsetAsync(workspace, 0, w.bytes, static_cast<cudaStream_t>(stream)) != cudaSuccess)
        return HA_ERR_LAUNCH;
    return HA_OK;
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
        attr1[0].val.programmaticStreamSerializationAllowed = HA_USE_PDL;
        cfg.attrs = attr1;
        cfg.numAttrs = 1;
        e = bf16 ? cudaLaunchKernelEx(&cfg, hash_decode_batched_kernel<__nv_bfloat16>, p)
                 : cudaLaunchKernelEx(&cfg, hash_decode_batched_kernel<float>, p);
        return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    if (weights->dtype == HA_WEIGHTS_BF16)
        e = launch(hash_decode_kernel<__nv_bfloat16>, grid, dim3(kHashDecodeThreads),
                   static_cast<cudaStream_t>(stream), 1, p);
    else
        e = launch(hash_decode_kernel<float>, grid, dim3(kHashDecodeThreads),
                   static_cast<cudaStream_t>(stream), 1, p);
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

    const int layers = weights->num_layers == 0 ? 3 : weights->num_layers;
    if (weights->dtype == HA_WEIGHTS_BF16 && layers == 3) {
        // bf16 weights, the 3-layer MLP: tcgen05 GEMM chain. One CTA per SM (its shared memory holds a head's weights).
        // (a per-device function attribute: set at every call, so that a process driving several GPUs is served)
        if (cudaFuncSetAttribute(hash_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kTcSmemBytes) != cudaSuccess)
            return HA_ERR_LAUNCH;
        HashPrefillTcParams t;
        t.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
        t.hash_pages = hash_pages;
        t.wk = static_cast<const __nv_bfloat16*>(weights->wk);
        t.bk = weights->bk;
        t.page_table = page_table;
        t.seq_lens = seq_lens;
        t.first_token = first_token;
        t.status = status;
        t.B = shape->batch;
        t.Hkv = shape->num_kv_heads;
        t.max_pages = shape->max_pages;
        t.num_pages = shape->num_pages;
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
        cfg.dynamicSmemBytes = kTcSmemBytes;
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr1[1];
        attr1[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr1[0].val.programmaticStreamSerializationAllowed = HA_USE_PDL;
        cfg.attrs = attr1;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, hash_prefill_tc_kernel, t) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    // fp32 weights, or the 1- and 2-layer hash functions: fp32 arithmetic on the CUDA cores
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
                             void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
    int rc = check_shape(shape);
    if (rc != HA_OK) return rc;
    rc = check_budget(budget);
    if (rc != HA_OK) return rc;
    if (q_codes == nullptr || hash_pages == nullptr || page_table == nullptr || seq_lens == nullptr ||
        sel_idx == nullptr || sel_cnt == nullptr || status == nullptr)
        return HA_ERR_BAD_ARG;
    if (workspace == nullptr) return HA_ERR_WORKSPACE;
    const Workspace w = carve(shape, budget, workspace);
    if (workspace_bytes < w.bytes) return HA_ERR_WORKSPACE;

    const SelectParams p = select_params(shape, budget, q_codes, hash_pages, page_table, seq_lens, sel_idx, sel_cnt,
                                         scores_dbg, status, w.hist, w.plan, w.scores, w.sel_rows, budget_lens);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long max_tokens = (long long)shape->max_pages * kPage;
    if (use_cluster_select(shape)) {
        const dim3 cgrid(kClCtas, shape->num_kv_heads, shape->batch);
        const cudaError_t e = max_tokens <= kClRoundTokens
            ? launch(score_select_cluster_kernel<1>, cgrid, dim3(kClThreads), s, kClCtas, p)
            : launch(score_select_cluster_kernel<2>, cgrid, dim3(kClThreads), s, kClCtas, p);
        return e == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
    }
    return launch_two_pass_select(shape, p, shape->num_kv_heads, s) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
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
    if (use_stagger(shape)) {
        rc = staggered_select_attend(shape, budget, q_att, k_pages, v_pages, hash_pages, page_table, seq_lens,
                                     q_codes, sel_idx, sel_cnt, sm_scale, out, workspace, workspace_bytes, status,
                                     static_cast<cudaStream_t>(stream), budget_lens);
        if (rc == HA_OK && status_out != nullptr) {
            // the step ended on several streams, all joined by now: a one-warp kernel stores the status word
            // (cheaper than a copy operation between the last kernel and the end of the step)
            publish_status_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, status_out);
            if (cudaGetLastError() != cudaSuccess) return HA_ERR_LAUNCH;
            if (status_delivered != nullptr) *status_delivered = true;
        }
        return rc;
    }
    rc = score_select_impl(shape, budget, q_codes, hash_pages, page_table, seq_lens, budget_lens, sel_idx, sel_cnt,
                           nullptr, workspace, workspace_bytes, status, stream);
    if (rc != HA_OK) return rc;
    // the selection kernel left the physical rows of the heavy tokens in the workspace; the step's last kernel
    // also leaves the status word in status_out, if given
    if (status_delivered != nullptr) *status_delivered = status_out != nullptr;
    return sparse_decode_impl(shape, budget, q_att, k_pages, v_pages, page_table, seq_lens, nullptr, sel_cnt, true,
                              sm_scale, out, workspace, workspace_bytes, status, stream, 0, -1, 0, budget_lens,
                              status_out);
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
    return decode_step_impl(shape, budget, weights, q, k_new, v_new, nullptr, k_pages, v_pages, hash_pages,
                            page_table, seq_lens, budget_lens, q_codes, sel_idx, sel_cnt, sm_scale, out, workspace,
                            workspace_bytes, status, stream);
}

int ha_decode_step_launches(const ha_shape_t* shape, const ha_budget_t* budget) {
    if (check_shape(shape) != HA_OK || check_budget(budget) != HA_OK) return 0;
    const AttSplit as = att_split_launch(shape, budget);
    const int merge = as.nsplits > 1 && !as.cluster ? 1 : 0;
    if (use_cluster_select(shape)) return 3 + merge;  // encoder, cluster selection, gather (+ merge)
    const int parts = use_stagger(shape) ? stagger_parts(shape) : 1;
    return 1 + parts * (4 + merge);  // encoder; per part: histograms, plan, compaction, gather (+ merge)
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
    int32_t* sel_rows;  // [B][Hq][sel_stride]
    int32_t* plan;      // [B][Hkv][8 + 8 * nchunks]
    uint32_t* scores;   // [B][Hkv][nchunks * chunk tokens]
    size_t bytes;
};

StaticScratch carve_static(const ha_shape_t* s, void* base) {
    const size_t n_hist = (size_t)s->batch * s->num_kv_heads * num_chunks_for(s->max_pages) * kGroup * kBins;
    const size_t n_rows = (size_t)s->batch * s->num_kv_heads * kGroup * s->sel_stride;
    char* p = static_cast<char*>(base);
    StaticScratch w;
    w.hist = reinterpret_cast<uint32_t*>(p);
    const size_t off = align_up(n_hist * sizeof(uint32_t));
    w.sel_rows = reinterpret_cast<int32_t*>(p + off);
    const size_t off2 = off + align_up(n_rows * sizeof(int32_t));
    w.plan = reinterpret_cast<int32_t*>(p + off2);
    const size_t off3 = off2 + align_up((size_t)s->batch * s->num_kv_heads * (8 + 8 * (size_t)num_chunks_for(s->max_pages)) * sizeof(int32_t));
    w.scores = reinterpret_cast<uint32_t*>(p + off3);
    w.bytes = off3 + align_up(ha::scores_bytes(s));
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

    // Every word of hist / plan / scores / sel_rows that a kernel reads was written earlier in the same
    // call, so nothing left over from the previous call needs clearing.
    const SelectParams p = select_params(shape, budget, q_codes, hash_pages, page_table, seq_lens, sel_idx, sel_cnt,
                                         nullptr, status, w.hist, w.plan, w.scores, w.sel_rows);
    return launch_two_pass_select(shape, p, shape->num_kv_heads, static_cast<cudaStream_t>(stream)) == cudaSuccess ? HA_OK : HA_ERR_LAUNCH;
}

}  // extern "C"
