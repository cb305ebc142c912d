// Hamming scoring and budget selection.
//
// Pass A (score_hist_kernel) streams the key-hash pages once: one 16-byte word per token per
// kv-head carries the codes of all 4 query heads of the group, so one coalesced pass scores
// the 4 heads together; score = popcount(~(q_code ^ k_code)) in 0..32. Each CTA publishes a
// 4 x 33 histogram of the scores of the candidate tokens of its chunk.
//
// Pass B (select_kernel) re-reads its chunk (L2-resident by then), derives from the chunk
// histograms the global threshold T of each head, how many tokens tied at T still fit and
// how many selected tokens precede the chunk, and writes the selected token indices in
// ascending order with ballot-based compaction - no sort, no atomics on the output.
//
// Together they replace the +-1 dot product of USA.forward and the sort/scatter of
// compute_mask_multi in 'simple' mode (hashattention/hashattention_llama.py:171-187, 423-438).
// A stable descending sort picks, among tokens tied at the threshold, the lowest indices;
// the tie fill below reproduces exactly that set.
#pragma once

#include "common.cuh"

namespace ha {

struct SelectParams {
    const uint32_t* q_codes;   // [B][Hq]
    const uint4* hash_pages;   // [num_pages][Hkv][256] x 16 B
    const int32_t* page_table;
    const int32_t* seq_lens;
    uint32_t* hist;            // workspace: [B][Hkv][nchunks][4][33]
    int32_t* sel_idx;          // [B][Hq][sel_stride]
    int32_t* sel_cnt;          // [B][Hq]
    uint8_t* scores_dbg;       // [B][Hq][max_pages*256] or null
    int32_t* status;
    int B, Hkv, max_pages, num_pages, sel_stride, chunk_pages, nchunks;
    int init_budget, recent_budget;
    double heavy_budget;
};

// Loads the hash words of this lane's tokens (token = warp_base + it*32 + lane) and returns the
// four scores of each packed into one u32 (byte g = score against query head g of the group).
// valid bit `it` is set when the token exists; cand bit `it` when it is a selection candidate.
__device__ __forceinline__ void load_scores(const SelectParams& p, int b, int kvh, int warp_base,
                                            int lane, const SeqRange& r, const uint32_t (&qc)[4],
                                            uint32_t (&sc)[kMaxChunkPages], uint32_t& valid,
                                            uint32_t& cand, bool& bad_page) {
    uint4 words[kMaxChunkPages];
    valid = 0;
    cand = 0;
    bad_page = false;
#pragma unroll
    for (int it = 0; it < kMaxChunkPages; ++it) {
        words[it] = make_uint4(0, 0, 0, 0);
        if (it < p.chunk_pages) {
            const int t = warp_base + it * 32 + lane;
            if (t < r.S) {
                const int page = __ldg(p.page_table + (size_t)b * p.max_pages + t / kPage);
                if (page < 0 || page >= p.num_pages) {
                    bad_page = true;
                } else {
                    words[it] = __ldg(p.hash_pages + ((size_t)page * p.Hkv + kvh) * kPage + t % kPage);
                    valid |= 1u << it;
                    if (t >= r.lo && t < r.hi) cand |= 1u << it;
                }
            }
        }
    }
#pragma unroll
    for (int it = 0; it < kMaxChunkPages; ++it) {
        const uint32_t s0 = __popc(~(qc[0] ^ words[it].x));
        const uint32_t s1 = __popc(~(qc[1] ^ words[it].y));
        const uint32_t s2 = __popc(~(qc[2] ^ words[it].z));
        const uint32_t s3 = __popc(~(qc[3] ^ words[it].w));
        sc[it] = s0 | (s1 << 8) | (s2 << 16) | (s3 << 24);
    }
}

__global__ void __launch_bounds__(kSelThreads) score_hist_kernel(const SelectParams p) {
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    const int chunk_tokens = p.chunk_pages * kPage;

    __shared__ uint32_t s_hist[kSelWarps][kGroup * kBins];
    for (int i = tid; i < kSelWarps * kGroup * kBins; i += kSelThreads) (&s_hist[0][0])[i] = 0;

    pdl_wait();
    pdl_launch_dependents();

    const int S = p.seq_lens[b];
    if (S < 1 || S > p.max_pages * kPage) {
        if (tid == 0 && c == 0 && kvh == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
        return;
    }
    if (c * chunk_tokens >= S) return;
    const SeqRange r = seq_range(S, p.init_budget, p.recent_budget, p.heavy_budget);

    uint32_t qc[4];
#pragma unroll
    for (int g = 0; g < kGroup; ++g) qc[g] = p.q_codes[(size_t)b * Hq + kvh * kGroup + g];

    const int warp_base = c * chunk_tokens + warp * 32 * p.chunk_pages;
    uint32_t sc[kMaxChunkPages], valid, cand;
    bool bad_page;
    load_scores(p, b, kvh, warp_base, lane, r, qc, sc, valid, cand, bad_page);
    if (bad_page) report(p.status, HA_ERR_BAD_PAGE);
    __syncthreads();

#pragma unroll
    for (int it = 0; it < kMaxChunkPages; ++it) {
        if ((cand >> it) & 1u) {
#pragma unroll
            for (int g = 0; g < kGroup; ++g)
                atomicAdd(&s_hist[warp][g * kBins + ((sc[it] >> (8 * g)) & 0xffu)], 1u);
        }
        if (p.scores_dbg != nullptr && ((valid >> it) & 1u)) {
            const int t = warp_base + it * 32 + lane;
            const size_t pitch = (size_t)p.max_pages * kPage;
#pragma unroll
            for (int g = 0; g < kGroup; ++g)
                p.scores_dbg[((size_t)b * Hq + kvh * kGroup + g) * pitch + t] =
                    (uint8_t)((sc[it] >> (8 * g)) & 0xffu);
        }
    }
    __syncthreads();
    if (tid < kGroup * kBins) {
        uint32_t v = 0;
#pragma unroll
        for (int w = 0; w < kSelWarps; ++w) v += s_hist[w][tid];
        p.hist[(((size_t)b * p.Hkv + kvh) * p.nchunks + c) * (kGroup * kBins) + tid] = v;
    }
}

__global__ void __launch_bounds__(kSelThreads) select_kernel(const SelectParams p) {
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    const int chunk_tokens = p.chunk_pages * kPage;

    __shared__ int s_tot[kGroup * kBins];
    __shared__ int s_bef[kGroup * kBins];
    __shared__ int s_T[kGroup], s_need[kGroup], s_base[kGroup], s_eqb[kGroup];
    __shared__ int s_wgt[kSelWarps][kGroup], s_weq[kSelWarps][kGroup];

    pdl_wait();
    pdl_launch_dependents();

    const int S = p.seq_lens[b];
    if (S < 1 || S > p.max_pages * kPage) return;  // reported by pass A
    if (c * chunk_tokens >= S) return;
    const SeqRange r = seq_range(S, p.init_budget, p.recent_budget, p.heavy_budget);
    const int nchunks_b = (S + chunk_tokens - 1) / chunk_tokens;

    // --- threshold, tie quota and output base of this chunk, per head -------------------
    if (tid < kGroup * kBins) {
        const uint32_t* hp = p.hist + ((size_t)b * p.Hkv + kvh) * p.nchunks * (kGroup * kBins) + tid;
        int tot = 0, bef = 0;
        for (int cc = 0; cc < nchunks_b; ++cc) {
            const int v = (int)hp[(size_t)cc * (kGroup * kBins)];
            tot += v;
            if (cc < c) bef += v;
        }
        s_tot[tid] = tot;
        s_bef[tid] = bef;
    }
    __syncthreads();
    if (tid < kGroup) {
        const int g = tid;
        int hbe = r.hb;
        if (hbe > p.sel_stride) {
            report(p.status, HA_ERR_SEL_OVERFLOW);
            hbe = p.sel_stride;
        }
        int T = kBins, need = 0, gt_before = 0, eq_before = 0;  // T = 33: nothing qualifies
        if (hbe > 0) {
            int above = 0;  // candidates with score > s
            for (int s = kCodeBits; s >= 0; --s) {
                const int n = s_tot[g * kBins + s];
                if (above + n >= hbe) {
                    T = s;
                    need = hbe - above;
                    break;
                }
                above += n;
                gt_before += s_bef[g * kBins + s];
            }
            if (T < kBins) eq_before = s_bef[g * kBins + T];
        }
        s_T[g] = T;
        s_need[g] = need;
        s_eqb[g] = eq_before;
        s_base[g] = gt_before + min(eq_before, need);
        if (c == 0) p.sel_cnt[(size_t)b * Hq + kvh * kGroup + g] = hbe;
    }

    // --- this chunk's scores -------------------------------------------------------------
    uint32_t qc[4];
#pragma unroll
    for (int g = 0; g < kGroup; ++g) qc[g] = p.q_codes[(size_t)b * Hq + kvh * kGroup + g];
    const int warp_base = c * chunk_tokens + warp * 32 * p.chunk_pages;
    uint32_t sc[kMaxChunkPages], valid, cand;
    bool bad_page;
    load_scores(p, b, kvh, warp_base, lane, r, qc, sc, valid, cand, bad_page);
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
    for (int it = 0; it < kMaxChunkPages; ++it) {
        if ((cand >> it) & 1u) {
#pragma unroll
            for (int g = 0; g < kGroup; ++g) {
                const int v = (int)((sc[it] >> (8 * g)) & 0xffu);
                cgt[g] += v > T[g];
                ceq[g] += v == T[g];
            }
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
        int gt_run = 0, eq_run = s_eqb[g];
        for (int w = 0; w < warp; ++w) {
            gt_run += s_wgt[w][g];
            eq_run += s_weq[w][g];
        }
        // selected tokens of this head that precede this warp's first token
        int out_run = s_base[g] + gt_run + (min(eq_run, need[g]) - min(s_eqb[g], need[g]));
        int32_t* dst = p.sel_idx + ((size_t)b * Hq + kvh * kGroup + g) * p.sel_stride;
#pragma unroll
        for (int it = 0; it < kMaxChunkPages; ++it) {
            if (it < p.chunk_pages) {
                const int v = (int)((sc[it] >> (8 * g)) & 0xffu);
                const bool is_cand = (cand >> it) & 1u;
                const bool gt = is_cand && v > T[g];
                const bool eq = is_cand && v == T[g];
                const uint32_t m_eq = __ballot_sync(0xffffffffu, eq);
                const bool sel = gt || (eq && eq_run + __popc(m_eq & lt_mask) < need[g]);
                const uint32_t m_sel = __ballot_sync(0xffffffffu, sel);
                if (sel) {
                    const int pos = out_run + __popc(m_sel & lt_mask);
                    if (pos < p.sel_stride) dst[pos] = warp_base + it * 32 + lane;
                }
                out_run += __popc(m_sel);
                eq_run += __popc(m_eq);
            }
        }
    }
}

}  // namespace ha
