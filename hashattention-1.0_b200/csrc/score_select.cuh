// Hamming scoring and the selection plan.
//
// score_hist_kernel streams the key-hash pages once: one 16-byte word per token per kv-head carries
// the four 32-bit codes of the kv-head's query heads, so a lane scores 4 heads per load,
// score = popcount(~(q_code ^ k_code)) in 0..32. Each CTA builds the 4 x 33 histogram of the scores
// of the candidate tokens of its chunk, adds it to the totals of its (sequence, kv-head) with atomic
// adds, and publishes per score the number of its tokens AT OR ABOVE that score, bin-major
// ([bin][chunk]); it also writes the scores of its tokens, one byte per token and query head
// (score + 1, 0 = not a candidate), in one plane per head.
//
// The CTA that finishes last for a (sequence, kv-head) - an arrival counter, no waiting - derives
// the plan of that unit (select_plan): the threshold T of each head and how many tokens tied at T still
// fit from the totals (pick_threshold: both selection rules of the reference), then how many selected /
// tied tokens precede each chunk from two published counts per chunk and head.
//
// select_attend_kernel (select_attend.cuh) then classifies each chunk's score bytes against T, compacts
// the selected tokens and attends them - no sort, no atomics in the output path.
//
// score_select_cluster_kernel does scoring and selection in one kernel for short sequences.
//
// Together they replace the +-1 dot product of USA.forward and the sort/scatter (or threshold) of
// compute_mask_multi (hashattention/hashattention_llama.py:171-187, 423-443).
// A stable descending sort picks, among tokens tied at the threshold, the lowest indices;
// the tie fill reproduces exactly that set.
//
// Tiling of score_hist_kernel: a CTA of 256 threads owns a chunk of 4 * ROUNDS pages of one (sequence,
// kv-head) and walks it in rounds of 1024 tokens; in a round warp w owns tokens [128 w, 128 w + 128)
// (half a page), four per lane. Only four 16-byte loads are in flight per lane, so many CTAs fit on
// an SM; the loads of a round are issued together without branches between them (indices are
// clamped into range instead of guarded). Everything that does not depend on the preceding
// kernel - the sequence length, page ids and the first round's hash words - is fetched before
// the grid-dependency wait.
//
// Layout of a score plane: inside every block of 128 tokens the byte of token 32 it + lane (the it-th
// token of a lane in the warp's round) sits at offset 4 lane + it, so that a lane stores its four
// tokens of one head as one 32-bit word and a warp 128 contiguous bytes per head.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace ha {

namespace cg = cooperative_groups;

constexpr int kShMinCtas = 4;                         // CTAs of score_hist_kernel per SM (64 registers per thread)
constexpr int kRoundPages = 4;                        // pages per round
constexpr int kRoundTokens = kRoundPages * kPage;     // 1024
constexpr int kLaneTokens = kRoundTokens / kSelThreads;  // 4 tokens per lane and round

struct SelectParams {
    const uint32_t* q_codes;   // [B][Hq]
    const uint4* hash_pages;   // [num_pages][Hkv][256] x 16 B
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* budget_lens;  // [B] or null: the length the heavy budget is a fraction of, if not seq_lens
    uint32_t* hist;            // workspace: [B][Hkv][4*33][nchunks] per chunk: tokens at or above each score
    uint32_t* arrive;          // workspace: [B][Hkv][kArriveStride] chunks of the unit that have published, the unit's
                               // histogram totals, and the unit's ready word (all 0 between calls)
    int32_t* sel_idx;          // [B][Hq][sel_stride] token indices
    int32_t* sel_rows;         // workspace: [B][Hq][sel_stride] page * 256 + slot of the same tokens
    int32_t* sel_cnt;          // [B][Hq]
    int32_t* plan;             // workspace: [B][Hkv][8 + 8 * nchunks]: T[4], need[4], then per chunk base[4], eqb[4]
    uint8_t* scores;           // workspace: [B][Hq][nchunks * chunk tokens]: score + 1, 0 = not a candidate (layout above)
    uint8_t* scores_dbg;       // [B][Hq][max_pages*256] or null
    int32_t* status;
    int B, Hkv, max_pages, num_pages, sel_stride, nchunks;
    int kvh0;                  // first kv-head of this launch (a launch may cover a slice of the kv-heads)
    int init_budget, recent_budget;
    double heavy_budget;
    int eval_mode, depth;      // HA_EVAL_*; usa_retrieve_depth (HA_EVAL_DEPTH only)
    int signal;                // 1: the selection kernel launched right behind consumes the plan unit by unit (ready word)
};

// One round of one warp: 128 consecutive tokens of one page, token it*32 + lane for it = 0..3.
// A round whose 128 tokens are all selection candidates (and do not include the newest token,
// whose hash word the encoder kernel may still be writing) is "interior": no per-token masks.
struct RoundWords {
    uint4 w[kLaneTokens];
    int page;          // page id of the warp's half page (clamped into the pool)
    uint32_t cand;     // bit it: token is a selection candidate
    uint32_t valid;    // bit it: token exists
    bool interior;     // warp-uniform: all 128 tokens are candidates, none is the newest token
    bool bad_page;

    // first token of this warp in round `rd` of chunk starting at `chunk_start`
    static __device__ __forceinline__ int first_token(int chunk_start, int rd, int warp) {
        return chunk_start + rd * kRoundTokens + warp * (kLaneTokens * 32);
    }

    // page id (unchecked) of the page that holds token t0
    static __device__ __forceinline__ int page_of(const SelectParams& p, int b, int t0) {
        return __ldg(p.page_table + (size_t)b * p.max_pages + min(t0 / kPage, p.max_pages - 1));
    }

    __device__ __forceinline__ void load(const SelectParams& p, int b, int kvh, int t0, int lane, const SeqRange& r) {
        load(p, kvh, t0, lane, r, page_of(p, b, t0));
    }

    // pg: what page_of() returned for t0 (fetched ahead of time, so that the hash words are the only loads on the way)
    __device__ __forceinline__ void load(const SelectParams& p, int kvh, int t0, int lane, const SeqRange& r, int pg) {
        const bool page_ok = pg >= 0 && pg < p.num_pages;
        page = page_ok ? pg : 0;
        const uint4* src = p.hash_pages + ((size_t)page * p.Hkv + kvh) * kPage;
        interior = page_ok && t0 >= r.lo && t0 + kLaneTokens * 32 <= r.hi &&
                   (unsigned)(r.S - 1 - t0) >= (unsigned)(kLaneTokens * 32);
        bad_page = false;
        if (interior) {
            const uint4* s0 = src + t0 % kPage + lane;
#pragma unroll
            for (int it = 0; it < kLaneTokens; ++it) w[it] = __ldg(s0 + it * 32);
            cand = valid = (1u << kLaneTokens) - 1u;
            return;
        }
        valid = 0;
        cand = 0;
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
        if (interior) return;
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it)
            if (t0 + it * 32 + lane == r.S - 1 && ((valid >> it) & 1u))
                w[it] = __ldcg(p.hash_pages + ((size_t)page * p.Hkv + kvh) * kPage + (r.S - 1) % kPage);
    }
};

// qn = ~q_code per head, so that popcount(qn ^ k) = popcount(~(q ^ k)) = number of agreeing bits
__device__ __forceinline__ uint4 load_qn(const SelectParams& p, int b, int kvh) {
    const uint4 qc = __ldcg(reinterpret_cast<const uint4*>(p.q_codes + ((size_t)b * p.Hkv + kvh) * kGroup));
    return make_uint4(~qc.x, ~qc.y, ~qc.z, ~qc.w);
}

// Per-byte flags (bit 7 of each byte) for packed scores a (bytes <= 32) against packed thresholds.
// gt_add = 0x7F7F7F7F - T4: byte sum a + 127 - T carries into bit 7 iff a > T (no carry across bytes).
__device__ __forceinline__ uint32_t bytes_gt(uint32_t a, uint32_t gt_add) { return (a + gt_add) & 0x80808080u; }
__device__ __forceinline__ uint32_t bytes_eq(uint32_t a, uint32_t t4) {
    return ~((a ^ t4) + 0x7F7F7F7Fu) & 0x80808080u;  // (x + 127) has bit 7 iff x != 0
}
// bit 7 of byte g -> bit g
__device__ __forceinline__ uint32_t flags_to_nibble(uint32_t f) { return (((f >> 7) * 0x01020408u) >> 24) & 0xFu; }

// What is kept of one head's candidates, worked out from the totals per score bin by one full
// warp: lane l passes n = total of bin 32 - l and cum = the inclusive prefix of n over the lanes
// (candidates scoring >= 32 - l); tot0 = total of bin 0; hb = min(budget, candidates).
//   T      tokens scoring above T are kept, of those scoring T the first `need` by token index;
//          T = 33 keeps nothing
//   count  tokens kept in all, cut to sel_stride (`overflow` says whether it had to be)
// HA_EVAL_SIMPLE: the hb best (hashattention/hashattention_llama.py:436-438). HA_EVAL_DEPTH: every
// candidate scoring at least max(best - depth, score of the hb-th best) (:439-443; one score step
// is a span step of 2).
struct Threshold {
    int T, need, count;
};

__device__ __forceinline__ Threshold pick_threshold(const SelectParams& p, int n, int cum, int tot0, int hb,
                                                    bool& overflow) {
    Threshold t;
    t.T = kBins; t.need = 0; t.count = 0;
    overflow = false;
    int hbe = hb;
    if (p.eval_mode == HA_EVAL_SIMPLE && hbe > p.sel_stride) {
        overflow = true;
        hbe = p.sel_stride;
    }
    if (hbe <= 0) return t;
    // the score of the hbe-th best candidate and the number of candidates above it
    const uint32_t reached = __ballot_sync(0xffffffffu, cum >= hbe);
    const int l = reached != 0 ? __ffs(reached) - 1 : 31;  // first lane whose cumulative count reaches the budget
    const int cum31 = __shfl_sync(0xffffffffu, cum, 31);
    const int above_l = __shfl_sync(0xffffffffu, cum - n, l);
    const int T_num = reached != 0 ? 32 - l : 0;  // bins 32..1 hold fewer than the budget: the threshold is 0
    const int above = reached != 0 ? above_l : cum31;
    if (p.eval_mode == HA_EVAL_SIMPLE) {
        t.T = T_num;
        t.need = hbe - above;
        t.count = hbe;
        return t;
    }
    const uint32_t nonzero = __ballot_sync(0xffffffffu, n > 0);
    const int top = nonzero != 0 ? 32 - (__ffs(nonzero) - 1) : 0;  // hbe >= 1: some candidate exists
    const int T = min(max(top - p.depth, T_num), kBins);
    const int at_least = __shfl_sync(0xffffffffu, cum, min(max(32 - T, 0), 31));
    t.T = T;
    t.need = 0x3fffffff;  // every tied token
    t.count = T >= kBins ? 0 : (T >= 1 ? at_least : cum31 + tot0);
    if (t.count > p.sel_stride) {
        overflow = true;
        t.count = p.sel_stride;
    }
    return t;
}

// byte g of each of the 4 words, gathered into one word (byte w of the result = byte g of a[w])
template <int NW>
__device__ __forceinline__ uint32_t gather_byte(const uint32_t (&a)[NW], int g) {
    static_assert(NW == 4, "four words");
    const uint32_t sel = 0x0040u + 0x11u * g;  // bytes g of x (index g) and of y (index 4 + g)
    return __byte_perm(__byte_perm(a[0], a[1], sel), __byte_perm(a[2], a[3], sel), 0x5410u);
}

// The plan of one (sequence, kv-head), worked out by one CTA of 256 threads (the one that published the unit's
// last histogram). The scoring CTAs have added their histograms up in the unit's totals (33 bins x 4 heads, behind
// the arrival counter) and stored, per chunk, the counts of tokens at or above every score: warp g picks head g's
// threshold T and tie quota from the totals, thread (head, chunk) reads what its chunk holds at or above T and
// above T, and a scan over the chunks gives the number of selected and of tied tokens that precede each chunk.
// The totals are left at zero for the next call.
constexpr int kPlanChunks = 64;            // chunks per sweep (sequences of more than 64 chunks take several)
constexpr int kPlanRows = kGroup * kBins;  // 132 (head, bin) rows
constexpr int kArriveStride = 136;         // words per unit behind p.arrive: the arrival counter, then the 132 totals
constexpr int kReadyWord = 133;            // ... and the ready word: > 0 while the unit's plan waits for consumers

struct PlanSmem {
    int tot[kPlanRows];
    int T[kGroup], need[kGroup];
    int warp_gt[kSelWarps], warp_eq[kSelWarps];
};

__device__ __forceinline__ void select_plan(const SelectParams& p, int b, int kvh, const SeqRange& r, int nchunks_b,
                                            PlanSmem& sm, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    const uint32_t* hbase = p.hist + ((size_t)b * p.Hkv + kvh) * kPlanRows * p.nchunks;
    int32_t* plan = p.plan + ((size_t)b * p.Hkv + kvh) * (8 + 8 * p.nchunks);
    uint32_t* totals = p.arrive + ((size_t)b * p.Hkv + kvh) * kArriveStride + 1;
    const int pc_shift = nchunks_b <= 32 ? 5 : 6, pc = 1 << pc_shift;  // chunks per sweep: 32 or 64

    // ---- totals per (head, bin) over all chunks
    if (tid < kPlanRows) {
        sm.tot[tid] = (int)__ldcg(totals + tid);
        totals[tid] = 0u;
    }
    __syncthreads();

    // ---- T and the tie quota: warp g for head g, lane l holds bin 32 - l
    if (warp < kGroup) {
        const int g = warp;
        const int n = sm.tot[g * kBins + 32 - lane];
        int cum = n;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, cum, d);
            if (lane >= d) cum += u;
        }
        bool overflow;
        const Threshold th = pick_threshold(p, n, cum, sm.tot[g * kBins], r.hb, overflow);
        if (lane == 0) {
            if (overflow) report(p.status, HA_ERR_SEL_OVERFLOW);
            sm.T[g] = th.T;
            sm.need[g] = th.need;
            plan[g] = th.T;
            plan[4 + g] = th.need;
            p.sel_cnt[(size_t)b * Hq + kvh * kGroup + g] = th.count;
        }
    }
    __syncthreads();

    // ---- per chunk: tokens above T and tokens at T, then exclusive prefixes over the chunks.
    //      thread = (head g, chunk cl of the sweep): 4 x pc threads, a head's chunks are pc / 32 warps
    const int g = (tid >> pc_shift) & (kGroup - 1), cl = tid & (pc - 1);
    const bool works = tid < kGroup * pc;  // warp-uniform
    const int T = sm.T[g], need = sm.need[g];
    const int wpg = pc >> 5;  // warps per head: 1 or 2
    int gt_carry = 0, eq_carry = 0;
    for (int c0 = 0; c0 < nchunks_b; c0 += pc) {
        if (c0 > 0) __syncthreads();  // (warp_gt / warp_eq of the previous sweep have been read)
        int gt = 0, eq = 0;
        if (works && c0 + cl < nchunks_b) {
            const uint32_t* col = hbase + (size_t)(g * kBins) * p.nchunks + c0 + cl;
            const int ge = T < kBins ? (int)__ldcg(col + (size_t)T * p.nchunks) : 0;  // at or above T
            gt = T + 1 < kBins ? (int)__ldcg(col + (size_t)(T + 1) * p.nchunks) : 0;
            eq = ge - gt;
        }
        int pg = gt, pe = eq;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u0 = __shfl_up_sync(0xffffffffu, pg, d), u1 = __shfl_up_sync(0xffffffffu, pe, d);
            if (lane >= d) {
                pg += u0;
                pe += u1;
            }
        }
        if (lane == 31) {
            sm.warp_gt[warp] = pg;
            sm.warp_eq[warp] = pe;
        }
        __syncthreads();
        if (works) {
            // with two warps per head the upper one adds the lower one's total
            const int w0 = g * wpg;
            const bool upper = wpg == 2 && warp == w0 + 1;
            const int gt_before = gt_carry + (upper ? sm.warp_gt[w0] : 0) + pg - gt;
            const int eq_before = eq_carry + (upper ? sm.warp_eq[w0] : 0) + pe - eq;
            const int cc = c0 + cl;
            if (cc < nchunks_b) {
                plan[8 + 8 * cc + g] = gt_before + min(eq_before, need);
                plan[8 + 8 * cc + 4 + g] = eq_before;
            }
            gt_carry += sm.warp_gt[w0] + (wpg == 2 ? sm.warp_gt[w0 + 1] : 0);
            eq_carry += sm.warp_eq[w0] + (wpg == 2 ? sm.warp_eq[w0 + 1] : 0);
        }
    }
}

template <int ROUNDS>
__global__ void __launch_bounds__(kSelThreads, kShMinCtas) score_hist_kernel(const SelectParams p) {
    const int c = blockIdx.x, kvh = p.kvh0 + blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    constexpr int chunk_tokens = ROUNDS * kRoundTokens;

    __shared__ uint32_t s_hist[kSelWarps][kGroup * kBins];
    __shared__ PlanSmem s_plan;  // the plan's staging area (last CTA of the unit only)
    __shared__ int s_last;
    for (int i = tid; i < kSelWarps * kGroup * kBins; i += kSelThreads) (&s_hist[0][0])[i] = 0;

    const int S = p.seq_lens[b];
    const bool s_ok = S >= 1 && S <= p.max_pages * kPage;
    const int chunk_start = c * chunk_tokens;
    const bool active = s_ok && chunk_start < S;
    const SeqRange r = seq_range(s_ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget,
                                 p.budget_lens != nullptr ? p.budget_lens[b] : -1);
    // two rounds of hash words are kept in flight: while one is scored the next is on its way
    RoundWords rw[2];
    int pgs[ROUNDS];  // page ids of this warp's half pages, all requested up front
    if (active) {
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) pgs[rd] = RoundWords::page_of(p, b, RoundWords::first_token(chunk_start, rd, warp));
        rw[0].load(p, kvh, RoundWords::first_token(chunk_start, 0, warp), lane, r, pgs[0]);
        if (ROUNDS > 1 && chunk_start + kRoundTokens < S)
            rw[1].load(p, kvh, RoundWords::first_token(chunk_start, 1, warp), lane, r, pgs[1]);
    }

    pdl_wait();
    pdl_launch_dependents();

    if (!s_ok) {
        if (tid == 0 && c == 0 && blockIdx.y == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
        return;
    }
    if (!active) return;
    const uint4 qn = load_qn(p, b, kvh);
    __syncthreads();  // s_hist is zero

    uint32_t* h0 = &s_hist[warp][0];
    const size_t pitch = (size_t)p.nchunks * chunk_tokens;
    uint8_t* plane0 = p.scores + ((size_t)b * Hq + kvh * kGroup) * pitch;
    bool bad_page = false;
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
        if (chunk_start + rd * kRoundTokens >= S) break;
        RoundWords& cur = rw[rd & 1];
        const int t0 = RoundWords::first_token(chunk_start, rd, warp);
        cur.refresh_newest(p, kvh, t0, lane, r);
        bad_page |= cur.bad_page;
        uint32_t plane[kGroup] = {0u, 0u, 0u, 0u};  // per head: byte it = score + 1 of this lane's it-th token
        if (cur.interior && p.scores_dbg == nullptr) {
            // the common round: every token is a candidate. The four scores of a token are packed with byte
            // permutes and the 4 x 4 bytes of the lane's tokens transposed at the end.
            uint32_t tok[kLaneTokens];
#pragma unroll
            for (int it = 0; it < kLaneTokens; ++it) {
                const uint32_t s0 = __popc(qn.x ^ cur.w[it].x), s1 = __popc(qn.y ^ cur.w[it].y);
                const uint32_t s2 = __popc(qn.z ^ cur.w[it].z), s3 = __popc(qn.w ^ cur.w[it].w);
                atomicAdd(h0 + s0, 1u);
                atomicAdd(h0 + kBins + s1, 1u);
                atomicAdd(h0 + 2 * kBins + s2, 1u);
                atomicAdd(h0 + 3 * kBins + s3, 1u);
                // bytes (s0, s1, s2, s3): byte 1 of a score register is zero and fills the unused positions
                tok[it] = __byte_perm(__byte_perm(s0, s1, 0x1140u), __byte_perm(s2, s3, 0x1140u), 0x5410u) + 0x01010101u;
            }
#pragma unroll
            for (int g = 0; g < kGroup; ++g) plane[g] = gather_byte<kLaneTokens>(tok, g);
        } else {
#pragma unroll
            for (int it = 0; it < kLaneTokens; ++it) {
                const uint32_t s0 = __popc(qn.x ^ cur.w[it].x), s1 = __popc(qn.y ^ cur.w[it].y);
                const uint32_t s2 = __popc(qn.z ^ cur.w[it].z), s3 = __popc(qn.w ^ cur.w[it].w);
                const bool is_cand = cur.interior || ((cur.cand >> it) & 1u);
                if (is_cand) {
                    atomicAdd(h0 + s0, 1u);
                    atomicAdd(h0 + kBins + s1, 1u);
                    atomicAdd(h0 + 2 * kBins + s2, 1u);
                    atomicAdd(h0 + 3 * kBins + s3, 1u);
                    plane[0] |= (s0 + 1u) << (8 * it);
                    plane[1] |= (s1 + 1u) << (8 * it);
                    plane[2] |= (s2 + 1u) << (8 * it);
                    plane[3] |= (s3 + 1u) << (8 * it);
                }
                if (p.scores_dbg != nullptr && ((cur.valid >> it) & 1u)) {
                    const size_t dpitch = (size_t)p.max_pages * kPage;
                    uint8_t* d = p.scores_dbg + ((size_t)b * Hq + kvh * kGroup) * dpitch + t0 + it * 32 + lane;
                    d[0] = (uint8_t)s0;
                    d[dpitch] = (uint8_t)s1;
                    d[2 * dpitch] = (uint8_t)s2;
                    d[3 * dpitch] = (uint8_t)s3;
                }
            }
        }
        // the round after next takes this round's registers
        if (rd + 2 < ROUNDS && chunk_start + (rd + 2) * kRoundTokens < S)
            cur.load(p, kvh, RoundWords::first_token(chunk_start, rd + 2, warp), lane, r, pgs[rd + 2 < ROUNDS ? rd + 2 : 0]);
        // the selection works from these bytes instead of the 16-byte hash words
#pragma unroll
        for (int g = 0; g < kGroup; ++g)
            *reinterpret_cast<uint32_t*>(plane0 + g * pitch + t0 + lane * 4) = plane[g];
    }
    if (bad_page) report(p.status, HA_ERR_BAD_PAGE);
    __syncthreads();
    // the chunk's histogram: added to the unit's totals, and stored as counts of tokens at or above each score.
    // Warp g takes head g, lane l the score 32 - l (a scan over the lanes gives "at or above"); lane 0 also score 0.
    uint32_t* unit = p.arrive + ((size_t)b * p.Hkv + kvh) * kArriveStride;
    if (warp < kGroup) {
        const int row0 = warp * kBins;
        uint32_t v = 0, v0 = 0;
#pragma unroll
        for (int w = 0; w < kSelWarps; ++w) {
            v += s_hist[w][row0 + 32 - lane];
            v0 += s_hist[w][row0];
        }
        if (v != 0u) atomicAdd(unit + 1 + row0 + 32 - lane, v);
        if (lane == 0 && v0 != 0u) atomicAdd(unit + 1 + row0, v0);
        uint32_t ge = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t u = __shfl_up_sync(0xffffffffu, ge, d);
            if (lane >= d) ge += u;
        }
        uint32_t* dst = p.hist + (((size_t)b * p.Hkv + kvh) * (kGroup * kBins) + row0) * p.nchunks + c;
        dst[(size_t)(32 - lane) * p.nchunks] = ge;
        if (lane == 31) dst[0] = ge + v0;
    }

    // ---- the CTA that publishes last for this (sequence, kv-head) works the unit's plan out. Nobody waits:
    //      every CTA makes its histogram visible, then counts itself in; the one that finds all the others
    //      counted reads their histograms and leaves the counter at zero for the next call.
    __syncthreads();
    const int nchunks_b = (S + chunk_tokens - 1) / chunk_tokens;
    if (tid == 0) {
        __threadfence();  // what the CTA has written (ordered before this thread by the barrier) is visible device-wide
        uint32_t* counter = unit;
        const uint32_t before = atomicAdd(counter, 1u);
        s_last = before + 1u == (uint32_t)nchunks_b;
        if (s_last) *counter = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    select_plan(p, b, kvh, r, nchunks_b, s_plan, tid);
    // ---- hand the unit over: one count per CTA of select_attend_kernel that will take this plan (a chunk of one
    //      query head each). Those CTAs run while other units are still being scored; each takes its count back,
    //      so the word is zero again when the step is over.
    if (p.signal != 0) {
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            atomicAdd(reinterpret_cast<int*>(unit + kReadyWord), nchunks_b * kGroup);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Single-kernel variant for short sequences (up to ROUNDS * 32768 tokens): one cluster of 8 CTAs
// x 1024 threads owns one (sequence, kv-head). A CTA scores 4096 tokens per round (4 per lane),
// keeps the packed scores in registers, and the 8 CTAs exchange their 4 x 33 histograms through
// distributed shared memory instead of global memory - so the hash pages are read once, there
// is no second pass, no histogram traffic and no kernel hand-over between scoring and
// selection. Token order is (round, CTA rank, warp, it, lane); results are identical to
// score_hist_kernel + select_kernel.
// ------------------------------------------------------------------------------------------
constexpr int kClThreads = 1024;
constexpr int kClWarps = kClThreads / 32;                     // 32 = slots per CTA and round
constexpr int kClCtas = 8;                                    // portable cluster size
constexpr int kClCtaTokens = kClThreads * kLaneTokens;        // 4096 tokens per CTA and round
constexpr int kClRoundTokens = kClCtas * kClCtaTokens;        // 32768 tokens per cluster and round
constexpr int kClHistCopies = 8;                              // warp w updates copy w % 8

template <int ROUNDS>
__global__ void __launch_bounds__(kClThreads, 1) score_select_cluster_kernel(const SelectParams p) {
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int kvh = p.kvh0 + blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    constexpr int kHist = kGroup * kBins;  // 132

    __shared__ uint32_t s_hist[ROUNDS][kClHistCopies][kHist];
    __shared__ uint32_t s_cta_hist[ROUNDS][kHist];   // read by the other CTAs of the cluster
    __shared__ int s_tot[kHist];
    __shared__ int s_bef[ROUNDS][kHist];             // counts in (round, rank) pairs before (rd, this CTA)
    __shared__ int s_T[kGroup], s_need[kGroup], s_base[ROUNDS][kGroup], s_eqb[ROUNDS][kGroup];
    __shared__ uint32_t s_sgt[ROUNDS][kClWarps], s_seq[ROUNDS][kClWarps];
    for (int i = tid; i < ROUNDS * kClHistCopies * kHist; i += kClThreads) (&s_hist[0][0][0])[i] = 0;

    const int S = p.seq_lens[b];
    const bool s_ok = S >= 1 && S <= p.max_pages * kPage && S <= ROUNDS * kClRoundTokens;
    const SeqRange r = seq_range(s_ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget,
                                 p.budget_lens != nullptr ? p.budget_lens[b] : -1);
    auto first_token = [&](int rd) { return rd * kClRoundTokens + rank * kClCtaTokens + warp * (kLaneTokens * 32); };
    RoundWords rw;
    const bool active0 = s_ok && first_token(0) < S;  // warp-uniform
    if (active0) rw.load(p, b, kvh, first_token(0), lane, r);

    pdl_wait();
    pdl_launch_dependents();
    if (!s_ok && tid == 0 && rank == 0 && blockIdx.y == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);

    // --- scores of this thread's tokens (packed, byte g = head g) and the CTA's histograms ---------
    uint32_t sc[ROUNDS][kLaneTokens];
    int page[ROUNDS];
    uint32_t cand = 0;  // bit rd * 4 + it
    bool bad_page = false;
    const uint4 qn = load_qn(p, b, kvh);
    __syncthreads();  // s_hist is zero
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
        const int t0 = first_token(rd);
        const bool act = s_ok && t0 < S;  // warp-uniform
        page[rd] = 0;
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) sc[rd][it] = 0;
        if (!act) continue;
        if (rd > 0) rw.load(p, b, kvh, t0, lane, r);
        rw.refresh_newest(p, kvh, t0, lane, r);
        bad_page |= rw.bad_page;
        page[rd] = rw.page;
        cand |= rw.cand << (rd * kLaneTokens);
        uint32_t* h0 = &s_hist[rd][warp % kClHistCopies][0];
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) {
            const uint32_t s0 = __popc(qn.x ^ rw.w[it].x), s1 = __popc(qn.y ^ rw.w[it].y);
            const uint32_t s2 = __popc(qn.z ^ rw.w[it].z), s3 = __popc(qn.w ^ rw.w[it].w);
            sc[rd][it] = s0 | (s1 << 8) | (s2 << 16) | (s3 << 24);
            if (rw.interior || ((rw.cand >> it) & 1u)) {
                atomicAdd(h0 + s0, 1u);
                atomicAdd(h0 + kBins + s1, 1u);
                atomicAdd(h0 + 2 * kBins + s2, 1u);
                atomicAdd(h0 + 3 * kBins + s3, 1u);
            }
            if (p.scores_dbg != nullptr && ((rw.valid >> it) & 1u)) {
                const size_t pitch = (size_t)p.max_pages * kPage;
                uint8_t* d = p.scores_dbg + ((size_t)b * Hq + kvh * kGroup) * pitch + t0 + it * 32 + lane;
                d[0] = (uint8_t)s0;
                d[pitch] = (uint8_t)s1;
                d[2 * pitch] = (uint8_t)s2;
                d[3 * pitch] = (uint8_t)s3;
            }
        }
    }
    if (bad_page) report(p.status, HA_ERR_BAD_PAGE);
    __syncthreads();
    for (int i = tid; i < ROUNDS * kHist; i += kClThreads) {
        const int rd = i / kHist, bin = i % kHist;
        uint32_t v = 0;
#pragma unroll
        for (int k = 0; k < kClHistCopies; ++k) v += s_hist[rd][k][bin];
        s_cta_hist[rd][bin] = v;
    }

    // --- exchange: every CTA sums the histograms of all (round, rank) pairs, and of those before its own
    cluster.sync();
    if (tid < kHist) {
        int tot = 0, run = 0;
        int bef[ROUNDS];
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) {
#pragma unroll
            for (int rk = 0; rk < kClCtas; ++rk) {
                if (rk == rank) bef[rd] = run;
                run += (int)*cluster.map_shared_rank(&s_cta_hist[rd][tid], rk);
            }
        }
        tot = run;
        s_tot[tid] = tot;
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) s_bef[rd][tid] = bef[rd];
    }
    __syncthreads();  // s_tot / s_bef complete (the other CTAs may still be reading s_cta_hist)

    // --- threshold, tie quota and output bases per head: warp g scans the 33 bins downwards --------
    if (warp < kGroup) {
        const int g = warp;
        const int n = s_tot[g * kBins + 32 - lane];  // lane l holds bin 32 - l; bin 0 apart
        int cum = n;
        // tokens per bin in the (round, rank) pairs before (rd, this CTA); scanned together with the totals
        // (independent shuffle chains interleave, this section being a serial stretch of the kernel)
        int nbv[ROUNDS], cumbv[ROUNDS];
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) nbv[rd] = cumbv[rd] = s_bef[rd][g * kBins + 32 - lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, cum, d);
            int ub[ROUNDS];
#pragma unroll
            for (int rd = 0; rd < ROUNDS; ++rd) ub[rd] = __shfl_up_sync(0xffffffffu, cumbv[rd], d);
            if (lane >= d) {
                cum += u;
#pragma unroll
                for (int rd = 0; rd < ROUNDS; ++rd) cumbv[rd] += ub[rd];
            }
        }
        bool overflow;
        const Threshold th = pick_threshold(p, n, cum, s_tot[g * kBins], s_ok ? r.hb : 0, overflow);
        const int T = th.T;
        if (overflow && lane == 0 && rank == 0) report(p.status, HA_ERR_SEL_OVERFLOW);
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) {
            const int nb = nbv[rd], cumb = cumbv[rd];
            const int lt = min(max(32 - T, 0), 31);
            const int gt_l = __shfl_sync(0xffffffffu, cumb - nb, lt), eq_l = __shfl_sync(0xffffffffu, nb, lt);
            const int all31 = __shfl_sync(0xffffffffu, cumb, 31);
            int gt_before = 0, eq_before = 0;
            if (T >= 1 && T <= 32) {
                gt_before = gt_l;
                eq_before = eq_l;
            } else if (T == 0) {
                gt_before = all31;
                eq_before = s_bef[rd][g * kBins];
            }
            if (lane == 0) {
                s_eqb[rd][g] = eq_before;
                s_base[rd][g] = gt_before + min(eq_before, th.need);
            }
        }
        if (lane == 0) {
            s_T[g] = T;
            s_need[g] = th.need;
            if (rank == 0 && s_ok) p.sel_cnt[(size_t)b * Hq + kvh * kGroup + g] = th.count;
        }
    }
    __syncthreads();

    // --- classify and count per (round, warp) slot -------------------------------------------------
    const uint32_t t4 = (uint32_t)s_T[0] | ((uint32_t)s_T[1] << 8) | ((uint32_t)s_T[2] << 16) | ((uint32_t)s_T[3] << 24);
    const uint32_t gt_add = 0x7F7F7F7Fu - t4;
    auto flags_gt = [&](int rd, int it) {
        const uint32_t cm = 0u - ((cand >> (rd * kLaneTokens + it)) & 1u);
        return bytes_gt(sc[rd][it], gt_add) & cm;
    };
    auto flags_eq = [&](int rd, int it) {
        const uint32_t cm = 0u - ((cand >> (rd * kLaneTokens + it)) & 1u);
        return bytes_eq(sc[rd][it], t4) & cm;
    };
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
        uint32_t cg_ = 0, ce_ = 0;
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) {
            cg_ += flags_gt(rd, it) >> 7;
            ce_ += flags_eq(rd, it) >> 7;
        }
        cg_ = __reduce_add_sync(0xffffffffu, cg_);  // <= 128 per byte: no carry between heads
        ce_ = __reduce_add_sync(0xffffffffu, ce_);
        if (lane == 0) {
            s_sgt[rd][warp] = cg_;
            s_seq[rd][warp] = ce_;
        }
    }
    __syncthreads();

    // --- per round: prefix over the CTA's 32 warps, then emission as in select_kernel ---------------
    const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
        // lane = warp index of this round: exclusive prefix sums of the packed counts
        const uint32_t g4 = s_sgt[rd][lane], e4 = s_seq[rd][lane];
        const uint32_t g01 = (g4 & 0xffu) | ((g4 & 0xff00u) << 8), g23 = ((g4 >> 16) & 0xffu) | ((g4 >> 24) << 16);
        const uint32_t e01 = (e4 & 0xffu) | ((e4 & 0xff00u) << 8), e23 = ((e4 >> 16) & 0xffu) | ((e4 >> 24) << 16);
        uint32_t pg01 = g01, pg23 = g23, pe01 = e01, pe23 = e23;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t a0 = __shfl_up_sync(0xffffffffu, pg01, d), a1 = __shfl_up_sync(0xffffffffu, pg23, d);
            const uint32_t a2 = __shfl_up_sync(0xffffffffu, pe01, d), a3 = __shfl_up_sync(0xffffffffu, pe23, d);
            if (lane >= d) {
                pg01 += a0; pg23 += a1; pe01 += a2; pe23 += a3;
            }
        }
        pg01 -= g01; pg23 -= g23; pe01 -= e01; pe23 -= e23;
        const uint32_t sg01 = __shfl_sync(0xffffffffu, pg01, warp), sg23 = __shfl_sync(0xffffffffu, pg23, warp);
        const uint32_t se01 = __shfl_sync(0xffffffffu, pe01, warp), se23 = __shfl_sync(0xffffffffu, pe23, warp);
        const uint32_t mine_g = s_sgt[rd][warp], mine_e = s_seq[rd][warp];
        if ((mine_g | mine_e) == 0) continue;  // nothing of any head in this warp's 128 tokens
        int base_pos[kGroup], eqb[kGroup];
        uint32_t full4 = 0, straddle = 0;
#pragma unroll
        for (int g = 0; g < kGroup; ++g) {
            const int gt_b = (int)(((g < 2 ? sg01 : sg23) >> ((g & 1) * 16)) & 0xffffu);
            const int need = s_need[g];
            eqb[g] = s_eqb[rd][g] + (int)(((g < 2 ? se01 : se23) >> ((g & 1) * 16)) & 0xffffu);
            const int eq_in = (int)((mine_e >> (8 * g)) & 0xffu);
            base_pos[g] = s_base[rd][g] + gt_b + (min(eqb[g], need) - min(s_eqb[rd][g], need));
            if (eqb[g] + eq_in <= need) full4 |= 0x80u << (8 * g);
            else if (eqb[g] < need) straddle |= 1u << g;
        }
        uint32_t selm[kLaneTokens];
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) selm[it] = flags_gt(rd, it) | (flags_eq(rd, it) & full4);
        if (straddle != 0) {  // warp-uniform, at most once per (sequence, head): rank ties by token index
#pragma unroll
            for (int g = 0; g < kGroup; ++g) {
                if (!((straddle >> g) & 1u)) continue;
                int eq_run = eqb[g];
#pragma unroll
                for (int it = 0; it < kLaneTokens; ++it) {
                    const bool eq = (flags_eq(rd, it) >> (8 * g + 7)) & 1u;
                    const uint32_t m_eq = __ballot_sync(0xffffffffu, eq);
                    if (eq && eq_run + __popc(m_eq & lt_mask) < s_need[g]) selm[it] |= 0x80u << (8 * g);
                    eq_run += __popc(m_eq);
                }
            }
        }
        uint32_t cnt4 = 0, bits = 0;
#pragma unroll
        for (int it = 0; it < kLaneTokens; ++it) {
            cnt4 += selm[it] >> 7;
            bits |= flags_to_nibble(selm[it]) << (4 * it);
        }
        uint32_t excl = cnt4;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t u = __shfl_up_sync(0xffffffffu, excl, d);
            if (lane >= d) excl += u;
        }
        excl -= cnt4;
        const int t_lane = first_token(rd) + lane;
        const int prow0 = page[rd] * kPage + t_lane % kPage;
        while (bits != 0) {
            const int i = __ffs(bits) - 1;
            bits &= bits - 1;
            const int it = i >> 2, g = i & 3;
            const int bp = g == 0 ? base_pos[0] : (g == 1 ? base_pos[1] : (g == 2 ? base_pos[2] : base_pos[3]));
            const int pos = bp + (int)((excl >> (8 * g)) & 0xffu);
            excl += 1u << (8 * g);
            if (pos < p.sel_stride) {
                const size_t o = ((size_t)b * Hq + kvh * kGroup + g) * p.sel_stride + pos;
                p.sel_idx[o] = t_lane + it * 32;
                p.sel_rows[o] = prow0 + it * 32;
            }
        }
    }
    cluster.sync();  // s_cta_hist may be read by the other CTAs until they, too, are past the exchange
}

}  // namespace ha
