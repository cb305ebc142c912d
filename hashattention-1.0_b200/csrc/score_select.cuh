// Hamming scoring and budget selection.
//
// Pass A (score_hist_kernel) streams the key-hash pages once: one 16-byte word per token per
// kv-head carries the codes of all 4 query heads of the group, so one coalesced pass scores
// the 4 heads together; score = popcount(~(q_code ^ k_code)) in 0..32. Each CTA publishes a
// 4 x 33 histogram of the scores of the candidate tokens of its chunk, stored bin-major
// ([bin][chunk]) so that pass B reads the counts of one bin over all chunks as one line.
//
// Pass B (select_kernel) re-reads its chunk (L2-resident by then), derives from the chunk
// histograms the global threshold T of each head, how many tokens tied at T still fit and
// how many selected tokens precede the chunk, and writes the selected token indices in
// ascending order with ballot-based compaction - no sort, no atomics, nothing to reset.
//
// Together they replace the +-1 dot product of USA.forward and the sort/scatter of
// compute_mask_multi in 'simple' mode (hashattention/hashattention_llama.py:171-187, 423-438).
// A stable descending sort picks, among tokens tied at the threshold, the lowest indices;
// the tie fill below reproduces exactly that set.
//
// All global loads of a phase are issued together and without branches between them (indices
// are clamped into range instead of guarded), so a CTA pays one memory round trip per phase.
#pragma once

#include "common.cuh"

namespace ha {

struct SelectParams {
    const uint32_t* q_codes;   // [B][Hq]
    const uint4* hash_pages;   // [num_pages][Hkv][256] x 16 B
    const int32_t* page_table;
    const int32_t* seq_lens;
    uint32_t* hist;            // workspace: [B][Hkv][4*33][nchunks]
    int32_t* sel_idx;          // [B][Hq][sel_stride] token indices
    int32_t* sel_rows;         // workspace: [B][Hq][sel_stride] page * 256 + slot of the same tokens
    int32_t* sel_cnt;          // [B][Hq]
    uint8_t* scores_dbg;       // [B][Hq][max_pages*256] or null
    int32_t* status;
    int B, Hkv, max_pages, num_pages, sel_stride, nchunks;
    int init_budget, recent_budget;
    double heavy_budget;
};

// Scores of this lane's tokens. Token `it` of the lane is warp_base + it*32 + lane; all 32
// lanes of an iteration lie in one page. Returns per token the four scores packed in one u32
// (byte g = score against query head g of the group) and the token's physical row
// (page * 256 + slot); bit `it` of `valid` marks existing tokens, of `cand` selection candidates.
template <int CP>
struct ChunkScores {
    uint4 words[CP];
    uint32_t sc[CP];
    int32_t row[CP];
    uint32_t valid, cand;
    bool bad_page;

    // Issues every load that does not depend on the preceding kernel: page ids, then the hash
    // words of the chunk. Only the word of the newest token (S - 1) may still be in flight from
    // the encoder kernel; finish() re-reads that one.
    __device__ __forceinline__ void prefetch(const SelectParams& p, int b, int kvh, int warp_base, int lane,
                                             const SeqRange& r) {
        int page[CP];
        const int32_t* pt = p.page_table + (size_t)b * p.max_pages;
#pragma unroll
        for (int it = 0; it < CP; ++it) {
            const int pidx = min((warp_base + it * 32) / kPage, p.max_pages - 1);
            page[it] = __ldg(pt + pidx);
        }
        valid = 0;
        cand = 0;
        bad_page = false;
#pragma unroll
        for (int it = 0; it < CP; ++it) {
            const int t = warp_base + it * 32 + lane;
            const bool ok = t < r.S;
            const bool page_ok = page[it] >= 0 && page[it] < p.num_pages;
            bad_page |= ok && !page_ok;
            const int pg = page_ok ? page[it] : 0;
            const int tc = ok ? t : r.S - 1;  // clamp: the load below is always in range
            row[it] = pg * kPage + tc % kPage;
            words[it] = __ldg(p.hash_pages + ((size_t)pg * p.Hkv + kvh) * kPage + tc % kPage);
            if (ok && page_ok) {
                valid |= 1u << it;
                if (t >= r.lo && t < r.hi) cand |= 1u << it;
            }
        }
    }

    // After the grid dependency wait: refresh the newest token's word, then score.
    __device__ __forceinline__ void finish(const SelectParams& p, int kvh, int warp_base, int lane,
                                           const SeqRange& r, const uint4 qc) {
#pragma unroll
        for (int it = 0; it < CP; ++it) {
            if (warp_base + it * 32 + lane == r.S - 1 && ((valid >> it) & 1u))
                words[it] = __ldcg(p.hash_pages + ((size_t)(row[it] / kPage) * p.Hkv + kvh) * kPage + row[it] % kPage);
        }
#pragma unroll
        for (int it = 0; it < CP; ++it) {
            const uint32_t s0 = __popc(~(qc.x ^ words[it].x));
            const uint32_t s1 = __popc(~(qc.y ^ words[it].y));
            const uint32_t s2 = __popc(~(qc.z ^ words[it].z));
            const uint32_t s3 = __popc(~(qc.w ^ words[it].w));
            sc[it] = s0 | (s1 << 8) | (s2 << 16) | (s3 << 24);
        }
    }
};

template <int CP>
__global__ void __launch_bounds__(kSelThreads) score_hist_kernel(const SelectParams p) {
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    constexpr int chunk_tokens = CP * kPage;

    __shared__ uint32_t s_hist[kSelWarps][kGroup * kBins];
    for (int i = tid; i < kSelWarps * kGroup * kBins; i += kSelThreads) (&s_hist[0][0])[i] = 0;

    // seq_lens, the page table and all hash words but the newest token's are not written by the
    // kernel before this one, so they are fetched while that kernel is still running
    const int S = p.seq_lens[b];
    const bool s_ok = S >= 1 && S <= p.max_pages * kPage;
    const bool active = s_ok && c * chunk_tokens < S;
    const SeqRange r = seq_range(s_ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget);
    const int warp_base = c * chunk_tokens + warp * 32 * CP;
    ChunkScores<CP> cs;
    if (active) cs.prefetch(p, b, kvh, warp_base, lane, r);

    pdl_wait();
    pdl_launch_dependents();

    if (!s_ok) {
        if (tid == 0 && c == 0 && kvh == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
        return;
    }
    if (!active) return;
    const uint4 qc = __ldcg(reinterpret_cast<const uint4*>(p.q_codes + (size_t)b * Hq + kvh * kGroup));
    cs.finish(p, kvh, warp_base, lane, r, qc);
    if (cs.bad_page) report(p.status, HA_ERR_BAD_PAGE);
    __syncthreads();

#pragma unroll
    for (int it = 0; it < CP; ++it) {
        if ((cs.cand >> it) & 1u) {
#pragma unroll
            for (int g = 0; g < kGroup; ++g)
                atomicAdd(&s_hist[warp][g * kBins + ((cs.sc[it] >> (8 * g)) & 0xffu)], 1u);
        }
    }
    if (p.scores_dbg != nullptr) {
        const size_t pitch = (size_t)p.max_pages * kPage;
#pragma unroll
        for (int it = 0; it < CP; ++it) {
            if ((cs.valid >> it) & 1u) {
                const int t = warp_base + it * 32 + lane;
#pragma unroll
                for (int g = 0; g < kGroup; ++g)
                    p.scores_dbg[((size_t)b * Hq + kvh * kGroup + g) * pitch + t] =
                        (uint8_t)((cs.sc[it] >> (8 * g)) & 0xffu);
            }
        }
    }
    __syncthreads();
    if (tid < kGroup * kBins) {
        uint32_t v = 0;
#pragma unroll
        for (int w = 0; w < kSelWarps; ++w) v += s_hist[w][tid];
        p.hist[(((size_t)b * p.Hkv + kvh) * (kGroup * kBins) + tid) * p.nchunks + c] = v;
    }
}

template <int CP>
__global__ void __launch_bounds__(kSelThreads) select_kernel(const SelectParams p) {
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    constexpr int chunk_tokens = CP * kPage;
    constexpr int kBinsPerWarp = (kGroup * kBins + kSelWarps - 1) / kSelWarps;  // 17

    __shared__ int s_tot[kGroup * kBins + kSelWarps];  // padded: warp 7 owns bins up to 135
    __shared__ int s_bef[kGroup * kBins + kSelWarps];
    __shared__ int s_T[kGroup], s_need[kGroup], s_base[kGroup], s_eqb[kGroup];
    __shared__ int s_wgt[kSelWarps][kGroup], s_weq[kSelWarps][kGroup];

    const int S = p.seq_lens[b];
    const bool s_ok = S >= 1 && S <= p.max_pages * kPage;  // a bad length was reported by pass A
    const bool active = s_ok && c * chunk_tokens < S;
    const SeqRange r = seq_range(s_ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget);
    const int nchunks_b = (r.S + chunk_tokens - 1) / chunk_tokens;
    const int warp_base = c * chunk_tokens + warp * 32 * CP;
    ChunkScores<CP> cs;
    if (active) cs.prefetch(p, b, kvh, warp_base, lane, r);

    pdl_wait();
    pdl_launch_dependents();
    if (!active) return;

    // --- histogram lines of this warp's bins: warp w reduces bins [17w, 17w+17), lane = chunk;
    //     the 17 loads of a round are independent and issued together
    const uint4 qc = __ldcg(reinterpret_cast<const uint4*>(p.q_codes + (size_t)b * Hq + kvh * kGroup));
    const uint32_t* hbase = p.hist + ((size_t)b * p.Hkv + kvh) * (kGroup * kBins) * p.nchunks;
    int tot[kBinsPerWarp], bef[kBinsPerWarp];
#pragma unroll
    for (int k = 0; k < kBinsPerWarp; ++k) tot[k] = bef[k] = 0;
    for (int cc0 = 0; cc0 < nchunks_b; cc0 += 32) {
        const int cc = cc0 + lane;
        const int ccl = min(cc, nchunks_b - 1);
        int v[kBinsPerWarp];
#pragma unroll
        for (int k = 0; k < kBinsPerWarp; ++k) {
            const int bin = min(warp * kBinsPerWarp + k, kGroup * kBins - 1);
            v[k] = (int)__ldcg(hbase + (size_t)bin * p.nchunks + ccl);
        }
#pragma unroll
        for (int k = 0; k < kBinsPerWarp; ++k) {
            tot[k] += cc < nchunks_b ? v[k] : 0;
            bef[k] += cc < c ? v[k] : 0;
        }
    }
    cs.finish(p, kvh, warp_base, lane, r, qc);

#pragma unroll
    for (int k = 0; k < kBinsPerWarp; ++k) {
        const int t = __reduce_add_sync(0xffffffffu, tot[k]);
        const int f = __reduce_add_sync(0xffffffffu, bef[k]);
        if (lane == 0) {
            s_tot[warp * kBinsPerWarp + k] = t;
            s_bef[warp * kBinsPerWarp + k] = f;
        }
    }
    __syncthreads();

    // --- threshold, tie quota and output base per head: warp g scans the 33 bins downwards ---
    if (warp < kGroup) {
        const int g = warp;
        int hbe = r.hb;
        if (hbe > p.sel_stride) {
            if (lane == 0) report(p.status, HA_ERR_SEL_OVERFLOW);
            hbe = p.sel_stride;
        }
        // lane l holds bin 32 - l (bins 32..1); bin 0 is the remainder
        const int n = s_tot[g * kBins + 32 - lane], nb = s_bef[g * kBins + 32 - lane];
        int cum = n, cumb = nb;  // inclusive scans over lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, cum, d);
            const int ub = __shfl_up_sync(0xffffffffu, cumb, d);
            if (lane >= d) {
                cum += u;
                cumb += ub;
            }
        }
        const uint32_t reached = __ballot_sync(0xffffffffu, cum >= hbe);
        int T, need, gt_before, eq_before;
        if (hbe <= 0) {
            T = kBins; need = 0; gt_before = 0; eq_before = 0;  // T = 33: nothing qualifies
        } else if (reached != 0) {
            const int l = __ffs(reached) - 1;  // first lane whose cumulative count reaches the budget
            T = 32 - l;
            const int above = __shfl_sync(0xffffffffu, cum - n, l);
            need = hbe - above;
            gt_before = __shfl_sync(0xffffffffu, cumb - nb, l);
            eq_before = __shfl_sync(0xffffffffu, nb, l);
        } else {  // bins 32..1 together hold fewer than the budget: the threshold is 0
            T = 0;
            need = hbe - __shfl_sync(0xffffffffu, cum, 31);
            gt_before = __shfl_sync(0xffffffffu, cumb, 31);
            eq_before = s_bef[g * kBins];
        }
        if (lane == 0) {
            s_T[g] = T;
            s_need[g] = need;
            s_eqb[g] = eq_before;
            s_base[g] = gt_before + min(eq_before, need);
            if (c == 0) p.sel_cnt[(size_t)b * Hq + kvh * kGroup + g] = hbe;
        }
    }
    __syncthreads();

    int T[kGroup], need[kGroup];
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
        T[g] = s_T[g];
        need[g] = s_need[g];
    }

    // --- per-warp counts of (score > T) and (score == T), then a scan over the 8 warps -----
    int cgt[kGroup] = {0, 0, 0, 0}, ceq[kGroup] = {0, 0, 0, 0};
#pragma unroll
    for (int it = 0; it < CP; ++it) {
        const bool is_cand = (cs.cand >> it) & 1u;
#pragma unroll
        for (int g = 0; g < kGroup; ++g) {
            const int v = (int)((cs.sc[it] >> (8 * g)) & 0xffu);
            cgt[g] += is_cand && v > T[g];
            ceq[g] += is_cand && v == T[g];
        }
    }
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
        cgt[g] = __reduce_add_sync(0xffffffffu, cgt[g]);
        ceq[g] = __reduce_add_sync(0xffffffffu, ceq[g]);
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < kGroup; ++g) {
            s_wgt[warp][g] = cgt[g];
            s_weq[warp][g] = ceq[g];
        }
    }
    __syncthreads();

    // --- ordered emission --------------------------------------------------------------
    const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
        if (cgt[g] + ceq[g] == 0) continue;  // nothing of this head in this warp's tokens
        int gt_run = 0, eq_run = s_eqb[g];
        for (int w = 0; w < warp; ++w) {
            gt_run += s_wgt[w][g];
            eq_run += s_weq[w][g];
        }
        // selected tokens of this head that precede this warp's first token
        int out_run = s_base[g] + gt_run + (min(eq_run, need[g]) - min(s_eqb[g], need[g]));
        const size_t off = ((size_t)b * Hq + kvh * kGroup + g) * p.sel_stride;
#pragma unroll
        for (int it = 0; it < CP; ++it) {
            const int v = (int)((cs.sc[it] >> (8 * g)) & 0xffu);
            const bool is_cand = (cs.cand >> it) & 1u;
            const bool gt = is_cand && v > T[g];
            const bool eq = is_cand && v == T[g];
            const uint32_t m_eq = __ballot_sync(0xffffffffu, eq);
            const bool sel = gt || (eq && eq_run + __popc(m_eq & lt_mask) < need[g]);
            const uint32_t m_sel = __ballot_sync(0xffffffffu, sel);
            if (sel) {
                const int pos = out_run + __popc(m_sel & lt_mask);
                if (pos < p.sel_stride) {
                    p.sel_idx[off + pos] = warp_base + it * 32 + lane;
                    p.sel_rows[off + pos] = cs.row[it];
                }
            }
            out_run += __popc(m_sel);
            eq_run += __popc(m_eq);
        }
    }
}

}  // namespace ha
