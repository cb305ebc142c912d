// Sparse GQA flash-decode over the selected rows of the paged K / V cache.
//
// For query head h of sequence b the attended rows are, in this order, the sink tokens
// [0, lo), the heavy tokens selected for (b, h) and the recent tokens [hi, S). One thread-block
// cluster of 8 CTAs owns one (b, h); row position pos goes to CTA (pos / 16) % 8, half-warp
// pos % 16, so the rows spread evenly over the cluster whatever their number. Each half-warp
// gathers 8 rows of K and V per round straight into registers (sixteen 16-byte loads in flight
// per lane), computes the scaled dot products with shuffles and keeps an online softmax. The CTA
// reduces its 16 half-warps in shared memory; the cluster then merges the 8 CTA partials
// through distributed shared memory (each CTA finishes 16 of the 128 output dimensions) and
// writes the bf16 output. Nothing goes through global memory but the rows and the result.
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

namespace cg = cooperative_groups;

struct SparseDecodeParams {
    const __nv_bfloat16* q;        // [B][Hq][128]
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* sel;            // [B][Hq][sel_stride]: token indices, or physical rows (kPhysical)
    __nv_bfloat16* out;            // [B][Hq][128]
    int32_t* status;
    int B, Hkv, max_pages, num_pages, sel_stride;
    int init_budget, recent_budget;
    double heavy_budget;
    float scale_log2e;             // sm_scale * log2(e)
};

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

struct AttPartial {  // one CTA's softmax state, read by the other CTAs of the cluster
    float m, l;
    __align__(16) float acc[kHeadDim];
};

// kPhysical: `sel` holds page * 256 + slot of each heavy token (written by select_kernel), so a
// heavy row needs no page-table lookup; otherwise it holds token indices.
template <bool kPhysical>
__global__ void __launch_bounds__(kAttThreads) sparse_decode_kernel(const SparseDecodeParams p) {
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();  // 0..7 within the (b, h) cluster
    const int h = blockIdx.y, b = blockIdx.z;
    const int Hq = p.Hkv * kGroup, kvh = h / kGroup;
    const int tid = threadIdx.x;
    const int worker = tid >> 4, sl = tid & 15;

    __shared__ float s_m[kAttWorkers], s_l[kAttWorkers];
    __shared__ __align__(16) float s_acc[kAttWorkers][kHeadDim];
    __shared__ AttPartial s_part;

    // inputs of the step, not products of the preceding kernel: q, seq_lens, the page table
    float qf[8];
    {
        const uint4 raw = *reinterpret_cast<const uint4*>(p.q + ((size_t)b * Hq + h) * kHeadDim + sl * 8);
        unpack8(raw, qf);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] *= p.scale_log2e;
    }
    const int S_raw = p.seq_lens[b];
    const bool s_ok = S_raw >= 1 && S_raw <= p.max_pages * kPage;  // else reported by the selection kernels
    const SeqRange r = seq_range(s_ok ? S_raw : 1, p.init_budget, p.recent_budget, p.heavy_budget);
    const int S = r.S;
    const int cnt = min(r.hb, p.sel_stride);  // what select_kernel emitted for this head
    const int n_total = s_ok ? r.lo + cnt + (S - r.hi) : 0;
    const int32_t* sel = p.sel + ((size_t)b * Hq + h) * p.sel_stride;
    const int32_t* pt = p.page_table + (size_t)b * p.max_pages;

    // position of row i of round `round` of this half-warp
    auto position = [&](int round, int i) {
        return (round * kAttRowsPerWorker + i) * kAttClusterRows + rank * kAttWorkers + worker;
    };
    // page lookups of the first round's sink / recent rows, issued before the dependency wait
    int pre_page[kAttRowsPerWorker];
#pragma unroll
    for (int i = 0; i < kAttRowsPerWorker; ++i) {
        const int pos = position(0, i);
        const bool edge = pos < n_total && (pos < r.lo || pos >= r.lo + cnt);
        const int tok = edge ? (pos < r.lo ? pos : r.hi + (pos - r.lo - cnt)) : 0;
        pre_page[i] = __ldg(pt + tok / kPage);
    }

    pdl_wait();
    pdl_launch_dependents();

    float m = -INFINITY, l = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool bad = false;
    const int rounds = (n_total + kAttRowsPerWorker * kAttClusterRows - 1) / (kAttRowsPerWorker * kAttClusterRows);
    for (int round = 0; round < rounds; ++round) {
        // ---- phase 1: one lookup per row: the heavy list entry, or the page of an edge token ----
        int look[kAttRowsPerWorker], tokv[kAttRowsPerWorker];
        uint32_t valid = 0, heavy = 0;
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const int pos = position(round, i);
            const bool ok = pos < n_total;
            const bool is_heavy = ok && pos >= r.lo && pos < r.lo + cnt;
            const int tok = (ok && !is_heavy) ? (pos < r.lo ? pos : r.hi + (pos - r.lo - cnt)) : 0;
            tokv[i] = tok;
            valid |= (ok ? 1u : 0u) << i;
            heavy |= (is_heavy ? 1u : 0u) << i;
            if (is_heavy) look[i] = __ldcg(sel + (pos - r.lo));
            else look[i] = round == 0 ? pre_page[i] : __ldg(pt + tok / kPage);
        }
        // ---- phase 2 (token-index lists only): translate heavy token indices through the page table
        int row[kAttRowsPerWorker];
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const bool is_heavy = (heavy >> i) & 1u;
            int rr;
            bool ok_row;
            if (kPhysical || !is_heavy) {
                // look = physical row (heavy) or page id (edge token)
                const bool page_ok = is_heavy || (look[i] >= 0 && look[i] < p.num_pages);
                rr = is_heavy ? look[i] : (page_ok ? look[i] : 0) * kPage + tokv[i] % kPage;
                ok_row = page_ok;
            } else {
                const int tok = look[i];
                const bool tok_ok = tok >= r.lo && tok < r.hi;
                const int page = __ldg(pt + (tok_ok ? tok : 0) / kPage);
                const bool page_ok = page >= 0 && page < p.num_pages;
                rr = (page_ok ? page : 0) * kPage + (tok_ok ? tok : 0) % kPage;
                ok_row = tok_ok && page_ok;
            }
            ok_row = ok_row && rr >= 0 && rr < p.num_pages * kPage;
            if (((valid >> i) & 1u) && !ok_row) {
                bad = true;
                valid &= ~(1u << i);
            }
            row[i] = ok_row ? rr : 0;
        }
        // ---- phase 3: gather, K and V loads all issued before any use -------------------------
        uint4 kraw[kAttRowsPerWorker], vraw[kAttRowsPerWorker];
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const size_t off =
                (((size_t)(row[i] / kPage) * p.Hkv + kvh) * kPage + row[i] % kPage) * kHeadDim + sl * 8;
            kraw[i] = __ldg(reinterpret_cast<const uint4*>(p.k_pages + off));
            vraw[i] = __ldg(reinterpret_cast<const uint4*>(p.v_pages + off));
        }
        // ---- scores (in log2 units), online softmax, weighted V sum ---------------------------
        float sc[kAttRowsPerWorker];
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
        const float rescale = m == -INFINITY ? 0.f : exp2f(m - m_new);
        m = m_new;
        l *= rescale;
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[d] *= rescale;
#pragma unroll
        for (int i = 0; i < kAttRowsPerWorker; ++i) {
            const float w = ((valid >> i) & 1u) ? exp2f(sc[i] - m) : 0.f;
            l += w;
            float v[8];
            unpack8(vraw[i], v);
#pragma unroll
            for (int d = 0; d < 8; ++d) acc[d] = fmaf(w, v[d], acc[d]);
        }
    }
    if (bad) report(p.status, HA_ERR_BAD_PAGE);

    // ---- reduce the 16 half-warps of the CTA -------------------------------------------------
    if (sl == 0) {
        s_m[worker] = m;
        s_l[worker] = l;
    }
    *reinterpret_cast<float4*>(&s_acc[worker][sl * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(&s_acc[worker][sl * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    __syncthreads();
    if (tid < kHeadDim) {
        float M = -INFINITY, L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < kAttWorkers; ++w) M = fmaxf(M, s_m[w]);
#pragma unroll
        for (int w = 0; w < kAttWorkers; ++w) {
            const float f = s_m[w] == -INFINITY ? 0.f : exp2f(s_m[w] - M);
            L = fmaf(s_l[w], f, L);
            A = fmaf(s_acc[w][tid], f, A);
        }
        s_part.acc[tid] = A;
        if (tid == 0) {
            s_part.m = M;
            s_part.l = L;
        }
    }

    // ---- merge the 8 CTA partials through distributed shared memory ----------------------------
    cluster.sync();
    if (tid < kHeadDim / kAttCluster && n_total > 0) {
        const int d = rank * (kHeadDim / kAttCluster) + tid;
        float mc[kAttCluster], lc[kAttCluster], ac[kAttCluster];
#pragma unroll
        for (int c = 0; c < kAttCluster; ++c) {
            const AttPartial* rp = cluster.map_shared_rank(&s_part, c);
            mc[c] = rp->m;
            lc[c] = rp->l;
            ac[c] = rp->acc[d];
        }
        float M = -INFINITY, L = 0.f, A = 0.f;
#pragma unroll
        for (int c = 0; c < kAttCluster; ++c) M = fmaxf(M, mc[c]);
#pragma unroll
        for (int c = 0; c < kAttCluster; ++c) {
            const float f = mc[c] == -INFINITY ? 0.f : exp2f(mc[c] - M);
            L = fmaf(lc[c], f, L);
            A = fmaf(ac[c], f, A);
        }
        p.out[((size_t)b * Hq + h) * kHeadDim + d] = __float2bfloat16_rn(A / L);
    }
    cluster.sync();  // no CTA may exit while another still reads its shared memory
}

}  // namespace ha
