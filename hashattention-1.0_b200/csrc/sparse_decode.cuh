// Sparse GQA flash-decode over the selected rows of the paged K / V cache.
//
// For query head h of sequence b the attended rows are, in this order, the sink tokens
// [0, lo), the heavy tokens selected for (b, h) and the recent tokens [hi, S). The rows are cut
// into splits of 32 * rounds rows. Gathering random 256-byte rows is latency bound unless the
// SM is full of threads that each keep only a few loads in flight, so the gather kernel is
// built from many light CTAs: 128 threads = 8 half-warps, a half-warp owning four rows per
// round (lane = 8 of the 128 dimensions, eight 16-byte loads in flight per lane), dot products
// by shuffles, online softmax in registers, CTA reduction by shuffle and shared memory, one
// (max, sum, acc[128]) partial per CTA. A second, tiny kernel merges the partials of each
// (b, h) with a log-sum-exp and writes the bf16 output; a (b, h) that fits one split is
// finished by the gather kernel itself. Small steps use a cluster variant of the gather instead
// (8 CTAs of 256 threads per (b, h) that merge through distributed shared memory; see the kernel).
//
// Replaces hashattention/hashattention_llama.py:578-623: there every masked position is set
// to finfo.min before an fp32 softmax, i.e. contributes exactly 0, so the softmax runs
// over the selected rows only. Accumulation is fp32 throughout.
//
// Before waiting for the selection kernel, a CTA already resolves the page of every sink /
// recent row of its first round (they do not depend on the selection). All loads of a phase
// are issued together without branches between them; out-of-range positions are clamped to a
// valid row and masked afterwards.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace ha {

constexpr int kAttClusterCtas = 8;      // splits of one (b, h) in the cluster variant of the gather (portable cluster size)
constexpr int kAttClusterThreads = 256;

struct SparseDecodeParams {
    const __nv_bfloat16* q;        // [B][Hq][128]
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* budget_lens;    // [B] or null: the length the heavy budget is a fraction of, if not seq_lens
    const int32_t* sel;            // [B][Hq][sel_stride]: token indices, or physical rows (kPhysical)
    const int32_t* sel_cnt;        // [B][Hq] entries of `sel` in use, or null: min(heavy budget, candidates),
                                   // which needs no load (HA_EVAL_SIMPLE always selects exactly that many)
    __nv_bfloat16* out;            // [B][Hq][128]
    float* partials;               // workspace: [B][Hq][nsplits][130]
    int32_t* status;
    int32_t* status_out;           // null, or where the step's last kernel leaves a copy of *status once every kernel
                                   // before it has completed (a word of mapped host memory: saves a copy operation)
    int B, Hkv, max_pages, num_pages, sel_stride, nsplits, rounds;
    int round_rows;                // rows a CTA takes per round: 2 per thread / 16 (32 for 128 threads, 64 for 256)
    int h0;                        // first query head of this launch (a launch may cover a slice of the heads)
    int init_budget, recent_budget;
    double heavy_budget;
    float scale_log2e;             // sm_scale * log2(e)
};

// Called after the dependency wait of the step's last kernel: every earlier kernel of the step has completed, so
// the status word holds whatever they reported (a bad page this kernel itself may meet was already reported by the
// selection, which visits every page of the sequence).
__device__ __forceinline__ void publish_status(const SparseDecodeParams& p) {
    if (p.status_out != nullptr && (blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x) == 0)
        *p.status_out = __ldcg(p.status);
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
    x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x);
    x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
    x[4] = bf16_lo(raw.z); x[5] = bf16_hi(raw.z);
    x[6] = bf16_lo(raw.w); x[7] = bf16_hi(raw.w);
}

__device__ __forceinline__ float dot8(const uint4& raw, const float (&x)[8]) {
    float s = bf16_lo(raw.x) * x[0];
    s = fmaf(bf16_hi(raw.x), x[1], s);
    s = fmaf(bf16_lo(raw.y), x[2], s);
    s = fmaf(bf16_hi(raw.y), x[3], s);
    s = fmaf(bf16_lo(raw.z), x[4], s);
    s = fmaf(bf16_hi(raw.z), x[5], s);
    s = fmaf(bf16_lo(raw.w), x[6], s);
    s = fmaf(bf16_hi(raw.w), x[7], s);
    return s;
}

// 2^x on the special-function unit (relative error 2^-22; 2^-inf = 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Rows attended by (b, h) and how they are cut; the same arithmetic in both kernels.
struct AttPlan {
    SeqRange r;
    int cnt;      // heavy rows (what select_kernel emitted)
    int n_total;  // sink + heavy + recent
    int nsplits;  // CTAs with work
    bool ok;
};

// listed: number of entries in the heavy list as read from sel_cnt, or -1 if it follows from the budget
__device__ __forceinline__ AttPlan att_plan(const SparseDecodeParams& p, int b, int listed = -1) {
    AttPlan a;
    const int S = p.seq_lens[b];
    a.ok = S >= 1 && S <= p.max_pages * kPage;  // a bad length was reported by the selection kernels
    a.r = seq_range(a.ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget,
                    p.budget_lens != nullptr ? p.budget_lens[b] : -1);
    a.cnt = listed >= 0 ? min(listed, min(a.r.hi - a.r.lo, p.sel_stride)) : min(a.r.hb, p.sel_stride);
    a.n_total = a.ok ? a.r.lo + a.cnt + (a.r.S - a.r.hi) : 0;
    const int rows_per_cta = p.round_rows * p.rounds;
    a.nsplits = (a.n_total + rows_per_cta - 1) / rows_per_cta;
    return a;
}

// kPhysical: `sel` holds page * 256 + slot of each heavy token (written by select_kernel), so a
// heavy row needs no page-table lookup; otherwise it holds token indices.
//
// kCluster: the splits of one (b, h) are the 8 CTAs (256 threads each) of a thread-block cluster, which merge
// their partials through distributed shared memory and write the output themselves - no partials in global
// memory, no merge kernel, one kernel hand-over less. Used when the whole step is small (latency-bound).
template <bool kPhysical, int kThreads, bool kCluster>
__global__ void __launch_bounds__(kThreads, kCluster ? 2 : 6) sparse_gather_kernel(const SparseDecodeParams p) {
    static_assert(kCluster ? kThreads == kAttClusterThreads : kThreads == kHeadDim, "flat CTAs: thread = output dimension");
    constexpr int kWorkers = kThreads / 16;                          // half-warps
    constexpr int kRoundRows = kWorkers * kAttRowsPerWorker;      // rows per CTA and round
    const int split = blockIdx.x, h = p.h0 + blockIdx.y, b = blockIdx.z;
    const int Hq = p.Hkv * kGroup, kvh = h / kGroup;
    const int tid = threadIdx.x;
    const int worker = tid >> 4, sl = tid & 15, warp = tid >> 5;
    constexpr int kWarps = kThreads / 32;

    __shared__ float s_m[kWarps], s_l[kWarps];
    __shared__ __align__(16) float s_acc[kWarps][kHeadDim];

    // inputs of the step, not products of the preceding kernel: q, seq_lens, the page table
    AttPlan a = att_plan(p, b);
    const int lo = a.r.lo;
    int cnt = a.cnt;
    int edge_shift = a.r.hi - lo - cnt;  // recent token = position + edge_shift
    const int32_t* sel = p.sel + ((size_t)b * Hq + h) * p.sel_stride;
    const int32_t* pt = p.page_table + (size_t)b * p.max_pages;
    const int base = split * kRoundRows * p.rounds + worker;
    const unsigned pool_rows = (unsigned)p.num_pages * kPage;

    // page lookups of the first round's sink / recent rows, issued before the dependency wait
    int pre_page[kAttRowsPerWorker];
    auto first_round_pages = [&] {
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const int pos = base + i * kWorkers;
            const bool edge = pos < a.n_total && (unsigned)(pos - lo) >= (unsigned)cnt;
            const int tok = edge ? (pos < lo ? pos : pos + edge_shift) : 0;
            pre_page[i] = __ldg(pt + tok / kPage);
        }
    };
    if (p.sel_cnt == nullptr) first_round_pages();
    float qf[8];
    {
        const uint4 raw = *reinterpret_cast<const uint4*>(p.q + ((size_t)b * Hq + h) * kHeadDim + sl * 8);
        unpack8(raw, qf);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] *= p.scale_log2e;
    }

    pdl_wait();
    pdl_launch_dependents();
    publish_status(p);
    if (p.sel_cnt != nullptr) {  // the length of the heavy list is a product of the selection kernels
        a = att_plan(p, b, __ldcg(p.sel_cnt + (size_t)b * Hq + h));
        cnt = a.cnt;
        edge_shift = a.r.hi - lo - cnt;
        first_round_pages();
    }
    if (!kCluster && split >= a.nsplits) return;  // (a cluster CTA without rows still takes part in the merge)

    const __nv_bfloat16* kbase = p.k_pages + (size_t)kvh * kPage * kHeadDim + sl * 8;
    const __nv_bfloat16* vbase = p.v_pages + (size_t)kvh * kPage * kHeadDim + sl * 8;
    float m = -INFINITY, l = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool bad = false;

    // gather + online softmax over the rows of one round (row ids resolved, invalid ones masked)
    auto attend = [&](const unsigned (&row)[kAttRowsPerWorker], uint32_t valid) {
        uint4 kraw[kAttRowsPerWorker], vraw[kAttRowsPerWorker];
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {  // K and V loads all issued before any use
            const size_t off = ((size_t)(row[i] / kPage) * p.Hkv * kPage + row[i] % kPage) * kHeadDim;
            kraw[i] = __ldg(reinterpret_cast<const uint4*>(kbase + off));
            vraw[i] = __ldg(reinterpret_cast<const uint4*>(vbase + off));
        }
        float sc[kAttRowsPerWorker];  // scores in log2 units
        float m_new = m;
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            float s = dot8(kraw[i], qf);
            s += __shfl_xor_sync(0xffffffffu, s, 8);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            sc[i] = ((valid >> i) & 1u) ? s : -INFINITY;
            m_new = fmaxf(m_new, sc[i]);
        }
        // guards instead of branches: a worker may have seen no valid row yet (m_new == -inf)
        const float rescale = m == -INFINITY ? 0.f : fast_exp2(m - m_new);
        m = m_new;
        l *= rescale;
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[d] *= rescale;
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const float w = ((valid >> i) & 1u) ? fast_exp2(sc[i] - m) : 0.f;
            l += w;
            float v[8];
            unpack8(vraw[i], v);
#pragma unroll
            for (int d = 0; d < 8; ++d) acc[d] = fmaf(w, v[d], acc[d]);
        }
    };

    // A round whose rows are all heavy rows takes their physical ids straight from the list. In the cluster
    // variant, where a CTA's rounds are the critical path of the step, the ids of the next such round are
    // requested before this round's K / V rows are waited for (a round then costs one memory round trip, not
    // two). The flat variant does not: the extra registers cost it a CTA per SM and, measured, the overlap of
    // the staggered halves.
    auto all_heavy = [&](int cta_first) { return kPhysical && cta_first >= lo && cta_first + kRoundRows <= lo + cnt; };
    unsigned next_row[kAttRowsPerWorker];
    bool have_next = false;
    for (int round = 0; round < p.rounds; ++round) {
        const int rbase = base + round * kRoundRows;
        const int cta_first = rbase - worker;  // first position of the CTA in this round
        if (cta_first >= a.n_total) break;
        unsigned row[kAttRowsPerWorker];
        if (all_heavy(cta_first)) {
            uint32_t valid = (1u << kAttRowsPerWorker) - 1u;
#pragma unroll
            for (int i = 0; i < kAttRowsPerWorker; ++i)
                row[i] = (kCluster && have_next) ? next_row[i] : (unsigned)__ldcg(sel + (rbase + i * kWorkers - lo));
            if constexpr (kCluster) {
                have_next = round + 1 < p.rounds && all_heavy(cta_first + kRoundRows);
                if (have_next) {
#pragma unroll
                    for (int i = 0; i < kAttRowsPerWorker; ++i)
                        next_row[i] = (unsigned)__ldcg(sel + (rbase + kRoundRows + i * kWorkers - lo));
                }
            }
#pragma unroll
            for (int i = 0; i < kAttRowsPerWorker; ++i) {
                if (row[i] >= pool_rows) {
                    bad = true;
                    valid &= ~(1u << i);
                    row[i] = 0;
                }
            }
            attend(row, valid);
            continue;
        }
        // ---- mixed round: one lookup per row, the heavy list entry or the page of a sink / recent token
        have_next = false;
        int look[kAttRowsPerWorker], tokv[kAttRowsPerWorker];
        uint32_t valid = 0, heavy = 0;
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const int pos = rbase + i * kWorkers;
            const bool ok = pos < a.n_total;
            const bool is_heavy = ok && (unsigned)(pos - lo) < (unsigned)cnt;
            const int tok = (ok && !is_heavy) ? (pos < lo ? pos : pos + edge_shift) : 0;
            tokv[i] = tok;
            valid |= (ok ? 1u : 0u) << i;
            heavy |= (is_heavy ? 1u : 0u) << i;
            if (is_heavy) look[i] = __ldcg(sel + (pos - lo));
            else look[i] = round == 0 ? pre_page[i] : __ldg(pt + tok / kPage);
        }
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const bool is_heavy = (heavy >> i) & 1u;
            unsigned rr;
            if (kPhysical || !is_heavy) {  // look = physical row (heavy) or page id (sink / recent)
                rr = is_heavy ? (unsigned)look[i] : (unsigned)look[i] * kPage + (unsigned)(tokv[i] % kPage);
                if (!is_heavy && (unsigned)look[i] >= (unsigned)p.num_pages) rr = ~0u;
            } else {  // look = token index of a heavy row: translate through the page table
                const unsigned tok = (unsigned)look[i];
                const bool tok_ok = tok - (unsigned)lo < (unsigned)(a.r.hi - lo);
                const unsigned page = (unsigned)__ldg(pt + (tok_ok ? tok : 0u) / kPage);
                rr = (tok_ok && page < (unsigned)p.num_pages) ? page * kPage + tok % kPage : ~0u;
            }
            if (rr >= pool_rows) {
                if ((valid >> i) & 1u) bad = true;
                valid &= ~(1u << i);
                rr = 0;
            }
            row[i] = rr;
        }
        attend(row, valid);
    }
    if (bad) report(p.status, HA_ERR_BAD_PAGE);

    // ---- merge the two half-warps of each warp by shuffle, then the warps in shared memory ----
    {
        const float mo = __shfl_xor_sync(0xffffffffu, m, 16);
        const float lo_ = __shfl_xor_sync(0xffffffffu, l, 16);
        const float M2 = fmaxf(m, mo);
        const float f = M2 == -INFINITY ? 0.f : exp2f(m - M2);
        const float fo = M2 == -INFINITY ? 0.f : exp2f(mo - M2);
        l = l * f + lo_ * fo;
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[d] = acc[d] * f + __shfl_xor_sync(0xffffffffu, acc[d], 16) * fo;
        m = M2;
    }
    if ((tid & 31) == 0) {
        s_m[warp] = m;
        s_l[warp] = l;
    }
    if ((tid & 16) == 0) {
        *reinterpret_cast<float4*>(&s_acc[warp][sl * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(&s_acc[warp][sl * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    __syncthreads();
    const int dim = tid & (kHeadDim - 1);  // threads beyond 128 (256-thread CTAs) repeat the first 128
    float M = -INFINITY, L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w]);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const float f = s_m[w] == -INFINITY ? 0.f : exp2f(s_m[w] - M);
        L = fmaf(s_l[w], f, L);
        A = fmaf(s_acc[w][dim], f, A);
    }
    if constexpr (kCluster) {
        // ---- the 8 CTAs of the cluster hold the 8 partials of (b, h): CTA r finishes dimensions [16 r, 16 r + 16)
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        __shared__ float c_part[2 + kHeadDim];
        if (tid < kHeadDim) c_part[2 + tid] = A;
        if (tid == 0) {
            c_part[0] = M;
            c_part[1] = L;
        }
        cluster.sync();
        if (tid < kHeadDim / kAttClusterCtas) {
            const int d = split * (kHeadDim / kAttClusterCtas) + tid;
            float mk[kAttClusterCtas], lk[kAttClusterCtas], ak[kAttClusterCtas];
#pragma unroll
            for (int k = 0; k < kAttClusterCtas; ++k) {  // all remote loads issued together
                const float* rp = cluster.map_shared_rank(c_part, k);
                mk[k] = rp[0];
                lk[k] = rp[1];
                ak[k] = rp[2 + d];
            }
            float Mg = -INFINITY, Lg = 0.f, Ag = 0.f;
#pragma unroll
            for (int k = 0; k < kAttClusterCtas; ++k) Mg = fmaxf(Mg, mk[k]);
#pragma unroll
            for (int k = 0; k < kAttClusterCtas; ++k) {
                const float f = mk[k] == -INFINITY ? 0.f : exp2f(mk[k] - Mg);
                Lg = fmaf(lk[k], f, Lg);
                Ag = fmaf(ak[k], f, Ag);
            }
            if (Lg > 0.f) p.out[((size_t)b * Hq + h) * kHeadDim + d] = __float2bfloat16_rn(Ag / Lg);
        }
        cluster.sync();  // the partial of this CTA may be read by the others until they are done
        return;
    }
    if (a.nsplits == 1) {  // nothing to merge with
        p.out[((size_t)b * Hq + h) * kHeadDim + tid] = __float2bfloat16_rn(A / L);
        return;
    }
    float* part = p.partials + (((size_t)b * Hq + h) * p.nsplits + split) * kPartStride;
    part[2 + tid] = A;
    if (tid == 0) {
        part[0] = M;
        part[1] = L;
    }
}

// Log-sum-exp merge of the partials of one (b, h): 128 threads, thread = output dimension. Warp w
// takes the splits s = w, w + 4, ... (so the dependent accumulate chain is a quarter as long),
// lane = split for the (max, sum) pairs, all loads of a pass issued together; the four warps'
// results are combined in shared memory.
__global__ void __launch_bounds__(kHeadDim) sparse_merge_kernel(const SparseDecodeParams p) {
    const int h = p.h0 + blockIdx.x, b = blockIdx.y;
    const int Hq = p.Hkv * kGroup;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int kWarps = kHeadDim / 32;
    AttPlan a = att_plan(p, b);
    __shared__ float s_m[kWarps], s_l[kWarps];
    __shared__ float s_a[kWarps][kHeadDim];

    pdl_wait();
    pdl_launch_dependents();
    publish_status(p);
    if (p.sel_cnt != nullptr) a = att_plan(p, b, __ldcg(p.sel_cnt + (size_t)b * Hq + h));
    if (a.nsplits <= 1) return;  // written by the gather kernel (or nothing to write)

    const float* base = p.partials + ((size_t)b * Hq + h) * p.nsplits * kPartStride;
    // this warp's splits: s = warp + 4 * i; it accumulates all 128 dimensions (4 per lane)
    const int mine = (a.nsplits - warp + kWarps - 1) / kWarps;
    float Mg = -INFINITY, Lg = 0.f, Ag[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i0 = 0; i0 < mine; i0 += 8) {
        const int n = min(8, mine - i0);
        float ms[8], ls[8];
        float4 av[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float* ps = base + (size_t)(warp + kWarps * (i0 + min(j, n - 1))) * kPartStride;
            ms[j] = __ldcg(ps);
            ls[j] = __ldcg(ps + 1);
            av[j] = make_float4(__ldcg(ps + 2 + lane), __ldcg(ps + 34 + lane), __ldcg(ps + 66 + lane), __ldcg(ps + 98 + lane));
        }
        float mb = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) mb = fmaxf(mb, j < n ? ms[j] : -INFINITY);
        const float Mn = fmaxf(Mg, mb);
        const float rescale = Mg == -INFINITY ? 0.f : exp2f(Mg - Mn);
        Mg = Mn;
        Lg *= rescale;
#pragma unroll
        for (int d = 0; d < 4; ++d) Ag[d] *= rescale;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float f = (j < n && ms[j] != -INFINITY) ? exp2f(ms[j] - Mg) : 0.f;
            Lg = fmaf(ls[j], f, Lg);
            Ag[0] = fmaf(av[j].x, f, Ag[0]);
            Ag[1] = fmaf(av[j].y, f, Ag[1]);
            Ag[2] = fmaf(av[j].z, f, Ag[2]);
            Ag[3] = fmaf(av[j].w, f, Ag[3]);
        }
    }
    if (lane == 0) {
        s_m[warp] = Mg;
        s_l[warp] = Lg;
    }
#pragma unroll
    for (int d = 0; d < 4; ++d) s_a[warp][d * 32 + lane] = Ag[d];
    __syncthreads();
    float M = -INFINITY, L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w]);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const float f = s_m[w] == -INFINITY ? 0.f : exp2f(s_m[w] - M);
        L = fmaf(s_l[w], f, L);
        A = fmaf(s_a[w][tid], f, A);
    }
    p.out[((size_t)b * Hq + h) * kHeadDim + tid] = __float2bfloat16_rn(A / L);
}

}  // namespace ha
