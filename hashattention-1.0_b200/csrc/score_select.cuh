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
// Tiling: a CTA of 256 threads owns a chunk of 4 * ROUNDS pages of one (sequence, kv-head) and
// walks it in rounds of 1024 tokens; in a round warp w owns tokens [128 w, 128 w + 128) (half a
// page), four per lane. Only four 16-byte loads are in flight per lane, so many CTAs fit on an
// SM; the loads of a round are issued together without branches between them (indices are
// clamped into range instead of guarded). Everything that does not depend on the preceding
// kernel - the sequence length, page ids and the first round's hash words - is fetched before
// the grid-dependency wait.
#pragma once

#include "common.cuh"

namespace ha {

constexpr int kRoundPages = 4;                        // pages per round
constexpr int kRoundTokens = kRoundPages * kPage;     // 1024
constexpr int kLaneTokens = kRoundTokens / kSelThreads;  // 4 tokens per lane and round

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

// One round of one warp: 128 consecutive tokens of one page, token it*32 + lane for it = 0..3.
struct RoundWords {
    uint4 w[kLaneTokens];
    int page;          // page id of the warp's half page (clamped into the pool)
    uint32_t valid;    // bit it: token exists
    uint32_t cand;     // bit it: token is a selection candidate
    bool bad_page;

    // first token of this warp in round `rd` of chunk starting at `chunk_start`
    static __device__ __forceinline__ int first_token(int chunk_start, int rd, int warp) {
        return chunk_start + rd * kRoundTokens + warp * (kLaneTokens * 32);
    }

    __device__ __forceinline__ void load(const SelectParams& p, int b, int kvh, int t0, int lane, const SeqRange& r) {
        const int pidx = min(t0 / kPage, p.max_pages - 1);
        const int pg = __ldg(p.page_table + (size_t)b * p.max_pages + pidx);
        const bool page_ok = pg >= 0 && pg < p.num_pages;
        page = page_ok ? pg : 0;
        valid = 0;
        cand = 0;
        bad_page = false;
        const uint4* src = p.hash_pages + ((size_t)page * p.Hkv + kvh) * kPage;
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) {
            const int t = t0 + it * 32 + lane;
            const bool ok = t < r.S;
            bad_page |= ok && !page_ok;
            w[it] = __ldg(src + (ok ? t : r.S - 1) % kPage);  // clamp: always an in-range slot
            if (ok && page_ok) {
                valid |= 1u << it;
                if (t >= r.lo && t < r.hi) cand |= 1u << it;
            }
        }
    }

    // Re-reads the newest token's word, which the encoder kernel may have written after load().
    __device__ __forceinline__ void refresh_newest(const SelectParams& p, int kvh, int t0, int lane, const SeqRange& r) {
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it)
            if (t0 + it * 32 + lane == r.S - 1 && ((valid >> it) & 1u))
                w[it] = __ldcg(p.hash_pages + ((size_t)page * p.Hkv + kvh) * kPage + (r.S - 1) % kPage);
    }

    // byte g of the result = score of token `it` against query head g of the group
    __device__ __forceinline__ uint32_t scores(int it, const uint4 qc) const {
        return __popc(~(qc.x ^ w[it].x)) | (__popc(~(qc.y ^ w[it].y)) << 8) | (__popc(~(qc.z ^ w[it].z)) << 16) |
               (__popc(~(qc.w ^ w[it].w)) << 24);
    }
};

template <int ROUNDS>
__global__ void __launch_bounds__(kSelThreads) score_hist_kernel(const SelectParams p) {
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    constexpr int chunk_tokens = ROUNDS * kRoundTokens;

    __shared__ uint32_t s_hist[kSelWarps][kGroup * kBins];
    for (int i = tid; i < kSelWarps * kGroup * kBins; i += kSelThreads) (&s_hist[0][0])[i] = 0;

    const int S = p.seq_lens[b];
    const bool s_ok = S >= 1 && S <= p.max_pages * kPage;
    const int chunk_start = c * chunk_tokens;
    const bool active = s_ok && chunk_start < S;
    const SeqRange r = seq_range(s_ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget);
    RoundWords rw;
    if (active) rw.load(p, b, kvh, RoundWords::first_token(chunk_start, 0, warp), lane, r);

    pdl_wait();
    pdl_launch_dependents();

    if (!s_ok) {
        if (tid == 0 && c == 0 && kvh == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
        return;
    }
    if (!active) return;
    const uint4 qc = __ldcg(reinterpret_cast<const uint4*>(p.q_codes + (size_t)b * Hq + kvh * kGroup));
    __syncthreads();  // s_hist is zero

    bool bad_page = false;
#pragma unroll 1
    for (int rd = 0; rd < ROUNDS; ++rd) {
        const int t0 = RoundWords::first_token(chunk_start, rd, warp);
        if (rd > 0) {
            if (chunk_start + rd * kRoundTokens >= S) break;
            rw.load(p, b, kvh, t0, lane, r);
        }
        rw.refresh_newest(p, kvh, t0, lane, r);
        bad_page |= rw.bad_page;
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) {
            const uint32_t sc = rw.scores(it, qc);
            if ((rw.cand >> it) & 1u) {
#pragma unroll
                for (int g = 0; g < kGroup; ++g) atomicAdd(&s_hist[warp][g * kBins + ((sc >> (8 * g)) & 0xffu)], 1u);
            }
            if (p.scores_dbg != nullptr && ((rw.valid >> it) & 1u)) {
                const size_t pitch = (size_t)p.max_pages * kPage;
#pragma unroll
                for (int g = 0; g < kGroup; ++g)
                    p.scores_dbg[((size_t)b * Hq + kvh * kGroup + g) * pitch + t0 + it * 32 + lane] =
                        (uint8_t)((sc >> (8 * g)) & 0xffu);
            }
        }
    }
    if (bad_page) report(p.status, HA_ERR_BAD_PAGE);
    __syncthreads();
    if (tid < kGroup * kBins) {
        uint32_t v = 0;
#pragma unroll
        for (int w = 0; w < kSelWarps; ++w) v += s_hist[w][tid];
        p.hist[(((size_t)b * p.Hkv + kvh) * (kGroup * kBins) + tid) * p.nchunks + c] = v;
    }
}

template <int ROUNDS>
__global__ void __launch_bounds__(kSelThreads, 4) select_kernel(const SelectParams p) {
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    constexpr int chunk_tokens = ROUNDS * kRoundTokens;
    constexpr int kBinsPerWarp = (kGroup * kBins + kSelWarps - 1) / kSelWarps;  // 17
    constexpr int kSlots = ROUNDS * kSelWarps;  // (round, warp) pairs in token order

    __shared__ int s_tot[kGroup * kBins + kSelWarps];  // padded: warp 7 owns bins up to 135
    __shared__ int s_bef[kGroup * kBins + kSelWarps];
    __shared__ int s_T[kGroup], s_need[kGroup], s_base[kGroup], s_eqb[kGroup];
    __shared__ int s_wgt[kSlots][kGroup], s_weq[kSlots][kGroup];

    const int S = p.seq_lens[b];
    const bool s_ok = S >= 1 && S <= p.max_pages * kPage;  // a bad length was reported by pass A
    const int chunk_start = c * chunk_tokens;
    const bool active = s_ok && chunk_start < S;
    const SeqRange r = seq_range(s_ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget);
    const int nchunks_b = (r.S + chunk_tokens - 1) / chunk_tokens;
    RoundWords rw;
    if (active) rw.load(p, b, kvh, RoundWords::first_token(chunk_start, 0, warp), lane, r);

    pdl_wait();
    pdl_launch_dependents();
    if (!active) return;

    // --- histogram lines of this warp's bins: warp w reduces bins [17w, 17w+17), lane = chunk;
    //     the 17 loads of a pass are independent and issued together
    const uint4 qc = __ldcg(reinterpret_cast<const uint4*>(p.q_codes + (size_t)b * Hq + kvh * kGroup));
    const uint32_t* hbase = p.hist + ((size_t)b * p.Hkv + kvh) * (kGroup * kBins) * p.nchunks;
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
            const int t = __reduce_add_sync(0xffffffffu, cc < nchunks_b ? v[k] : 0);
            const int f = __reduce_add_sync(0xffffffffu, cc < c ? v[k] : 0);
            if (lane == 0) {  // only this warp touches these entries: no barrier needed between passes
                s_tot[warp * kBinsPerWarp + k] = cc0 == 0 ? t : s_tot[warp * kBinsPerWarp + k] + t;
                s_bef[warp * kBinsPerWarp + k] = cc0 == 0 ? f : s_bef[warp * kBinsPerWarp + k] + f;
            }
        }
    }

    // --- this chunk's scores, kept packed in registers (one u32 per token) ------------------------
    uint32_t sc[ROUNDS][kLaneTokens];
    int page[ROUNDS];
    uint32_t cand = 0;  // bit rd * 4 + it
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
        const int t0 = RoundWords::first_token(chunk_start, rd, warp);
        if (rd > 0) rw.load(p, b, kvh, min(t0, S - 1), lane, r);  // beyond S: clamped, nothing valid
        rw.refresh_newest(p, kvh, t0, lane, r);
        page[rd] = rw.page;
        const uint32_t cmask = (rd > 0 && t0 >= S) ? 0u : rw.cand;
        cand |= cmask << (rd * kLaneTokens);
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) sc[rd][it] = rw.scores(it, qc);
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

    // --- counts of (score > T) and (score == T) per (round, warp) slot ---------------------------
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
        int cgt[kGroup] = {0, 0, 0, 0}, ceq[kGroup] = {0, 0, 0, 0};
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) {
            const bool is_cand = (cand >> (rd * kLaneTokens + it)) & 1u;
#pragma unroll
            for (int g = 0; g < kGroup; ++g) {
                const int v = (int)((sc[rd][it] >> (8 * g)) & 0xffu);
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
                s_wgt[rd * kSelWarps + warp][g] = cgt[g];
                s_weq[rd * kSelWarps + warp][g] = ceq[g];
            }
        }
    }
    __syncthreads();

    // --- ordered emission: slots in token order are (round, warp), then it, then lane -------------
    const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
        // running counts over all slots before this warp's first slot (round 0)
        int gt_run = 0, eq_run = s_eqb[g];
        const size_t off = ((size_t)b * Hq + kvh * kGroup + g) * p.sel_stride;
        int slot_done = 0;
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) {
            const int slot = rd * kSelWarps + warp;
            for (; slot_done < slot; ++slot_done) {
                gt_run += s_wgt[slot_done][g];
                eq_run += s_weq[slot_done][g];
            }
            const int mine_gt = s_wgt[slot][g], mine_eq = s_weq[slot][g];
            if (mine_gt + mine_eq != 0) {  // something of this head in this warp's 128 tokens
                int out_run = s_base[g] + gt_run + (min(eq_run, need[g]) - min(s_eqb[g], need[g]));
                int eq_here = eq_run;
                const int t0 = RoundWords::first_token(chunk_start, rd, warp);
#pragma unroll
                for (int it = 0; it < kLaneTokens; ++it) {
                    const int v = (int)((sc[rd][it] >> (8 * g)) & 0xffu);
                    const bool is_cand = (cand >> (rd * kLaneTokens + it)) & 1u;
                    const bool gt = is_cand && v > T[g];
                    const bool eq = is_cand && v == T[g];
                    const uint32_t m_eq = __ballot_sync(0xffffffffu, eq);
                    const bool sel = gt || (eq && eq_here + __popc(m_eq & lt_mask) < need[g]);
                    const uint32_t m_sel = __ballot_sync(0xffffffffu, sel);
                    if (sel) {
                        const int pos = out_run + __popc(m_sel & lt_mask);
                        if (pos < p.sel_stride) {
                            const int t = t0 + it * 32 + lane;
                            p.sel_idx[off + pos] = t;
                            p.sel_rows[off + pos] = page[rd] * kPage + t % kPage;
                        }
                    }
                    out_run += __popc(m_sel);
                    eq_here += __popc(m_eq);
                }
            }
            gt_run += mine_gt;
            eq_run += mine_eq;
            slot_done = slot + 1;
        }
    }
}

}  // namespace ha
