// Selection and sparse attention in one kernel.
//
// score_hist_kernel (score_select.cuh) leaves, per (sequence, kv-head), the plan - the threshold T of
// each query head, its tie quota and, per chunk, how many selected / tied tokens precede the chunk -
// and one byte of score per token and query head. Here a CTA of 128 threads owns one chunk of one
// (sequence, query head): it compares the chunk's score bytes with T (SWAR, 4 tokens per instruction),
// compacts the selected tokens into a row list in shared memory (and into sel_idx, the caller's copy of
// the selection), and attends exactly those rows: gather of the K / V rows, dot products by shuffles,
// online softmax in registers, one (max, sum, acc[128]) partial per CTA. Two more CTAs per (sequence,
// head) attend the sink and the recent tokens; they depend on nothing the selection produces and do
// their work before the grid-dependency wait, i.e. while the scoring kernel is still running. A small
// kernel merges the partials of a head with a log-sum-exp.
//
// Compared with a separate compaction kernel followed by a gather kernel this saves a kernel hand-over
// and the trip of the row lists through global memory, and the memory system is idle only while a CTA
// classifies its 1 - 4 KB of score bytes.
//
// Inside a decode step the chunk CTAs do not wait for the whole scoring grid: the CTA that finishes the
// plan of a (sequence, kv-head) announces it in a ready word, a chunk CTA of that unit polls the word
// (bounded) and goes on, while other units are still being scored. Rows are asked for in L2 as soon as
// they are known to be attended, so that only the first round of a gather waits for DRAM.
//
// Replaces the sort / scatter of compute_mask_multi and the masked softmax . V of the decode branch
// (hashattention/hashattention_llama.py:430-443, 578-623). Ties at T go to the lowest token indices, as
// a stable descending sort would pick them: chunks are ranked by the plan, tokens inside the one chunk
// where the quota ends by their index.
//
// kGather == false is the selection alone (ha_score_select): sel_idx is written, nothing is attended.
#pragma once

#include "common.cuh"
#include "score_select.cuh"
#include "sparse_decode.cuh"

namespace ha {

constexpr int kSaThreads = 128;
constexpr int kSaLanes = 8;                          // lanes that share a row: 16 of the 128 dimensions each
constexpr int kSaWorkers = kSaThreads / kSaLanes;    // 16 rows are worked on side by side
constexpr int kSaRows = 2;                           // rows a worker keeps in flight per round
constexpr int kSaRoundRows = kSaWorkers * kSaRows;   // 32
constexpr int kSaWarps = kSaThreads / 32;
constexpr int kSaReadyPolls = 1 << 20;               // polls of a unit's ready word (200 ns apart) before a CTA gives up
constexpr int kSaEdgeSlots = 2;  // CTA 0 of a head attends the sink tokens, CTA 1 the recent ones, CTA 2 + c chunk c

// bf16 operands of the mixed-precision multiply-add are taken as they are stored (exact products, fp32
// accumulation, no unpacking).
__device__ __forceinline__ f32x2 bf16x2_to_f32x2(uint32_t w) { return pack2(bf16_lo(w), bf16_hi(w)); }
// c + lo(a) * lo(b) + hi(a) * hi(b) for two words of two bf16 each
__device__ __forceinline__ float dot_bf16x2(uint32_t a, uint32_t b, float c) {
    asm("{\n\t.reg .b16 a0, a1, b0, b1;\n\t"
        "mov.b32 {a0, a1}, %1;\n\tmov.b32 {b0, b1}, %2;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %0, a1, b1, %0;\n\t}"
        : "+f"(c) : "r"(a), "r"(b));
    return c;
}

struct SelectAttendParams {
    const int32_t* plan;          // [B][Hkv][8 + 8 * nchunks]: T[4], need[4], then per chunk base[4], eqb[4]
    const uint8_t* scores;        // [B][Hq][nchunks * chunk tokens] (layout: score_select.cuh)
    int32_t* sel_idx;             // [B][Hq][sel_stride] token indices of the heavy tokens (the caller's copy)
    const __nv_bfloat16* q;       // [B][Hq][128]
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* budget_lens;   // [B] or null
    __nv_bfloat16* out;           // [B][Hq][128]
    float* partials;              // workspace: [B][Hq][nslots][130]
    int32_t* status;
    int32_t* status_out;          // see SparseDecodeParams
    int32_t* ready;               // the scoring kernel's per-unit words (stride kArriveStride; word kReadyWord is used), or
                                  // null: the plan and the score bytes are complete when the kernel in front has ended
    int B, Hkv, max_pages, num_pages, sel_stride, nchunks, nslots;
    int h0;                       // first query head of this launch
    int init_budget, recent_budget;
    double heavy_budget;
    float scale_log2e;
};

// kMinCtas: CTAs per SM the register allocation aims at. 7 (72 registers) runs large grids fastest; 8 (64 registers)
// lets a grid of up to 1184 CTAs run as a single wave.
template <int ROUNDS, bool kGather, int kMinCtas>
__global__ void __launch_bounds__(kSaThreads, kMinCtas) select_attend_kernel(const SelectAttendParams p) {
    constexpr int chunk_tokens = ROUNDS * kRoundTokens;
    constexpr int kWords = 2 * ROUNDS;             // 32-bit words of score bytes per thread: 8 ROUNDS tokens
    constexpr int kTpb = 128 / (4 * kWords);       // threads that share a block of 128 tokens: 16, 8 or 4
    constexpr int kChunkPages = kRoundPages * ROUNDS;
    const int slot = blockIdx.x, h = p.h0 + blockIdx.y, b = blockIdx.z;
    const int Hq = p.Hkv * kGroup, kvh = h / kGroup, g = h % kGroup;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int worker = tid / kSaLanes, sl = tid % kSaLanes;

    __shared__ int s_rows[chunk_tokens];      // the rows this CTA attends: (page * Hkv + kv-head) * 256 + slot; -1: not in the pool
    __shared__ int s_pages[kChunkPages + 1];  // ids of the pages from a page-aligned token on; -1: not in the pool
    __shared__ uint32_t s_wtot[kSaWarps];
    __shared__ float s_m[kSaWarps], s_l[kSaWarps];
    __shared__ __align__(16) float s_acc[kSaWarps][kHeadDim];

    // inputs of the step, not products of the preceding kernel: seq_lens, the page table, q
    const int S = p.seq_lens[b];
    const bool ok = S >= 1 && S <= p.max_pages * kPage;  // a bad length was reported by the scoring kernel
    const SeqRange r = seq_range(ok ? S : 1, p.init_budget, p.recent_budget, p.heavy_budget,
                                 p.budget_lens != nullptr ? p.budget_lens[b] : -1);
    const int32_t* pt = p.page_table + (size_t)b * p.max_pages;

    // A row is shared by 8 lanes; lane sl holds dimensions [8 sl, 8 sl + 8) and [64 + 8 sl, 64 + 8 sl + 8), so
    // that each of its two 16-byte loads per row is one of 8 that cover 128 contiguous bytes.
    uint4 qa = make_uint4(0u, 0u, 0u, 0u), qb = qa;  // q as stored (bf16 pairs)
    if constexpr (kGather) {
        const uint4* qrow = reinterpret_cast<const uint4*>(p.q + ((size_t)b * Hq + h) * kHeadDim);
        qa = qrow[sl];
        qb = qrow[8 + sl];
    }
    const uint4* kbase = reinterpret_cast<const uint4*>(p.k_pages) + sl;  // + 16 per row
    const uint4* vbase = reinterpret_cast<const uint4*>(p.v_pages) + sl;
    float m = -INFINITY, l = 0.f;
    f32x2 acc2[8] = {0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull};  // this lane's 16 output dimensions, in pairs
    bool bad = false;

    // gather + online softmax over the first n rows of s_rows, 32 per round: 16 workers of 8 lanes, kSaRows rows
    // each; the K and V loads of a round are all issued before any use. Products of two bf16 values are exact in
    // fp32, so the multiply-add that takes bf16 operands gives the same dot product as unpacking first.
    auto attend_list = [&](int n) {
        for (int i0 = 0; i0 < n; i0 += kSaRoundRows) {
            uint4 ka[kSaRows], kb[kSaRows], va[kSaRows], vb[kSaRows];
            uint32_t valid = 0;
#pragma unroll
            for (int i = 0; i < kSaRows; ++i) {
                const int idx = i0 + worker + i * kSaWorkers;
                const int rr = idx < n ? s_rows[idx] : 0;
                if (rr < 0) bad = true;
                valid |= ((idx < n && rr >= 0) ? 1u : 0u) << i;
                const size_t off = (size_t)max(rr, 0) * (kHeadDim / 8);
                ka[i] = __ldg(kbase + off);
                kb[i] = __ldg(kbase + off + 8);
                va[i] = __ldg(vbase + off);
                vb[i] = __ldg(vbase + off + 8);
            }
            float sc[kSaRows];  // scores in log2 units
            float m_new = m;
#pragma unroll
            for (int i = 0; i < kSaRows; ++i) {
                float s = dot_bf16x2(ka[i].x, qa.x, 0.f);
                float s2 = dot_bf16x2(kb[i].x, qb.x, 0.f);
                s = dot_bf16x2(ka[i].y, qa.y, s);
                s2 = dot_bf16x2(kb[i].y, qb.y, s2);
                s = dot_bf16x2(ka[i].z, qa.z, s);
                s2 = dot_bf16x2(kb[i].z, qb.z, s2);
                s = dot_bf16x2(ka[i].w, qa.w, s);
                s2 = dot_bf16x2(kb[i].w, qb.w, s2);
                s += s2;
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                sc[i] = ((valid >> i) & 1u) ? s * p.scale_log2e : -INFINITY;
                m_new = fmaxf(m_new, sc[i]);
            }
            // guards instead of branches: a worker may have seen no valid row yet (m_new == -inf)
            const float rescale = m == -INFINITY ? 0.f : fast_exp2(m - m_new);
            m = m_new;
            l *= rescale;
            const f32x2 r2 = pack2(rescale, rescale);
#pragma unroll
            for (int d = 0; d < 8; ++d) acc2[d] = mul2(acc2[d], r2);
#pragma unroll
            for (int i = 0; i < kSaRows; ++i) {
                const float w = ((valid >> i) & 1u) ? fast_exp2(sc[i] - m) : 0.f;
                l += w;
                const f32x2 w2 = pack2(w, w);
                acc2[0] = fma2(bf16x2_to_f32x2(va[i].x), w2, acc2[0]);
                acc2[1] = fma2(bf16x2_to_f32x2(va[i].y), w2, acc2[1]);
                acc2[2] = fma2(bf16x2_to_f32x2(va[i].z), w2, acc2[2]);
                acc2[3] = fma2(bf16x2_to_f32x2(va[i].w), w2, acc2[3]);
                acc2[4] = fma2(bf16x2_to_f32x2(vb[i].x), w2, acc2[4]);
                acc2[5] = fma2(bf16x2_to_f32x2(vb[i].y), w2, acc2[5]);
                acc2[6] = fma2(bf16x2_to_f32x2(vb[i].z), w2, acc2[6]);
                acc2[7] = fma2(bf16x2_to_f32x2(vb[i].w), w2, acc2[7]);
            }
        }
    };

    // the CTA's (max, sum, acc[128]) -> its slot of the partials
    auto store_partial = [&] {
        float acc[16];
#pragma unroll
        for (int d = 0; d < 8; ++d) unpack2(acc2[d], acc[2 * d], acc[2 * d + 1]);
        // the 4 workers of a warp (lanes 8 apart hold the same dimensions), then the warps in shared memory
#pragma unroll
        for (int step = 8; step <= 16; step <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, step);
            const float lo_ = __shfl_xor_sync(0xffffffffu, l, step);
            const float M2 = fmaxf(m, mo);
            const float f = M2 == -INFINITY ? 0.f : fast_exp2(m - M2);
            const float fo = M2 == -INFINITY ? 0.f : fast_exp2(mo - M2);
            l = l * f + lo_ * fo;
#pragma unroll
            for (int d = 0; d < 16; ++d) acc[d] = acc[d] * f + __shfl_xor_sync(0xffffffffu, acc[d], step) * fo;
            m = M2;
        }
        if (lane == 0) {
            s_m[warp] = m;
            s_l[warp] = l;
        }
        if (lane < kSaLanes) {
            *reinterpret_cast<float4*>(&s_acc[warp][sl * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4*>(&s_acc[warp][sl * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            *reinterpret_cast<float4*>(&s_acc[warp][64 + sl * 8]) = make_float4(acc[8], acc[9], acc[10], acc[11]);
            *reinterpret_cast<float4*>(&s_acc[warp][64 + sl * 8 + 4]) = make_float4(acc[12], acc[13], acc[14], acc[15]);
        }
        __syncthreads();
        float M = -INFINITY, L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < kSaWarps; ++w) M = fmaxf(M, s_m[w]);
#pragma unroll
        for (int w = 0; w < kSaWarps; ++w) {
            const float f = s_m[w] == -INFINITY ? 0.f : fast_exp2(s_m[w] - M);
            L = fmaf(s_l[w], f, L);
            A = fmaf(s_acc[w][tid], f, A);
        }
        float* part = p.partials + (((size_t)b * Hq + h) * p.nslots + slot) * kPartStride;
        part[2 + tid] = A;
        if (tid == 0) {
            part[0] = M;
            part[1] = L;
        }
        if (bad) report(p.status, HA_ERR_BAD_PAGE);
    };

    // ---- the sink tokens [0, lo) and the recent tokens [hi, S): nothing here is a product of the kernel in front
    //      (the newest token's K / V rows were appended by the encoder, which lies two kernels back), so the
    //      whole gather runs before the dependency wait
    if (slot < kSaEdgeSlots) {
        if constexpr (kGather) {
            const int first = slot == 0 ? 0 : r.hi;
            const int count = !ok ? 0 : (slot == 0 ? r.lo : r.S - r.hi);
            for (int i0 = 0; i0 < count; i0 += chunk_tokens) {
                const int nb = min(chunk_tokens, count - i0);
                const int tbase = (first + i0) / kPage * kPage;
                if (tid <= kChunkPages) {
                    const int v = __ldg(pt + min(tbase / kPage + tid, p.max_pages - 1));
                    s_pages[tid] = v >= 0 && v < p.num_pages ? v : -1;
                }
                __syncthreads();
                for (int i = tid; i < nb; i += kSaThreads) {
                    const int t = first + i0 + i - tbase, pg = s_pages[t / kPage];
                    s_rows[i] = pg >= 0 ? (pg * p.Hkv + kvh) * kPage + t % kPage : -1;
                }
                __syncthreads();
                attend_list(nb);
                __syncthreads();
            }
        }
        pdl_wait();
        pdl_launch_dependents();
        if constexpr (kGather) {
            if (ok) store_partial();  // (written after the wait: the slot may still be read by the step before)
        }
        return;
    }

    // ---- chunk c of the sequence: page ids before the wait, plan and score bytes after it
    const int c = slot - kSaEdgeSlots;
    const int chunk_start = c * chunk_tokens;
    const bool active = ok && chunk_start < S;
    // (the page ids are requested here and used after the ready word has been asked for: one round trip, not two)
    int pgv = -1;
    if (tid < kChunkPages) pgv = __ldg(pt + min(chunk_start / kPage + tid, p.max_pages - 1));
    auto keep_pages = [&] {
        if (tid < kChunkPages) s_pages[tid] = pgv >= 0 && pgv < p.num_pages ? pgv : -1;  // tokens of a bad page are no candidates
    };
    if (p.ready == nullptr) {
        keep_pages();
        pdl_wait();
    } else if (active) {
        // The scoring kernel in front is still running, but all of its CTAs have started (it lets its dependents go
        // only then), so the unit's plan arrives without any help from this grid. The wait is bounded all the same.
        if (tid == 0) {
            int* word = p.ready + ((size_t)b * p.Hkv + kvh) * kArriveStride + kReadyWord;
            int v, polls = 0;
            for (;;) {
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
                if (v > 0 || ++polls > kSaReadyPolls) break;
                __nanosleep(200);
            }
            s_wtot[0] = v > 0 ? 1u : 0u;
            atomicSub(word, 1);  // (also after giving up: the word still returns to zero)
            if (v <= 0) report(p.status, HA_ERR_TIMEOUT);
        }
        keep_pages();
        __syncthreads();
        const bool arrived = s_wtot[0] != 0u;
        __syncthreads();  // (s_wtot is written again below)
        if (!arrived) return;
    }
    pdl_launch_dependents();
    if (!active) return;

    const int32_t* plan = p.plan + ((size_t)b * p.Hkv + kvh) * (8 + 8 * p.nchunks);
    const int T = __ldcg(plan + g), need = __ldcg(plan + 4 + g);
    const int base = __ldcg(plan + 8 + 8 * c + g), eqb = __ldcg(plan + 8 + 8 * c + 4 + g);
    // this thread's 8 ROUNDS score bytes: offsets [8 ROUNDS tid, ...) of the chunk's plane. The scoring kernel
    // wrote whole rounds of 1024 tokens up to the one that contains S - 1; what lies beyond is stale.
    uint32_t w[kWords];
    {
        const size_t pitch = (size_t)p.nchunks * chunk_tokens;
        const uint8_t* src = p.scores + ((size_t)b * Hq + h) * pitch + chunk_start + tid * (4 * kWords);
        if constexpr (kWords == 2) {
            const uint2 v = __ldcg(reinterpret_cast<const uint2*>(src));
            w[0] = v.x; w[1] = v.y;
        } else {
#pragma unroll
            for (int j = 0; j < kWords / 4; ++j) {
                const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src) + j);
                w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
            }
        }
        const int written_end = (S + kRoundTokens - 1) / kRoundTokens * kRoundTokens;
        if (chunk_start + (tid / kTpb) * 128 >= written_end) {
#pragma unroll
            for (int k = 0; k < kWords; ++k) w[k] = 0u;
        }
    }
    // word k holds the 4 tokens (it = 0..3) of lane la0 + k of the scoring warp in block tid / kTpb of the chunk:
    // token = tok00 + k + 32 it
    const int la0 = (tid % kTpb) * kWords;
    const int tok00 = chunk_start + (tid / kTpb) * 128 + la0;

    // ---- classify: stored bytes are score + 1 (0: no candidate) and are compared with T + 1 >= 1, so a token
    //      that is no candidate never matches. a + (127 - T') carries into bit 7 of a byte iff a > T',
    //      a + (128 - T') iff a >= T' (bytes <= 33: no carry between bytes). The flag bits of word k are moved
    //      to bit k of their byte, so the thread's tokens end up in one mask: bit 8 it + k.
    const uint32_t t4 = (uint32_t)(T + 1) * 0x01010101u;
    const uint32_t gt_add = 0x7F7F7F7Fu - t4, ge_add = 0x80808080u - t4;
    uint32_t gtm = 0, gem = 0;
#pragma unroll
    for (int k = 0; k < kWords; ++k) {
        gtm |= ((w[k] + gt_add) & 0x80808080u) >> (7 - k);
        gem |= ((w[k] + ge_add) & 0x80808080u) >> (7 - k);
    }
    const uint32_t eqm = gem & ~gtm;
    // ask L2 for both lines of a K / V row
    auto prefetch_row = [&](int rr) {
        const __nv_bfloat16* kr = p.k_pages + (size_t)rr * kHeadDim;
        const __nv_bfloat16* vr = p.v_pages + (size_t)rr * kHeadDim;
        prefetch_l2(kr);
        prefetch_l2(kr + kHeadDim / 2);
        prefetch_l2(vr);
        prefetch_l2(vr + kHeadDim / 2);
    };
    // Tokens above the threshold are certain to be attended: their rows are asked for right here, before the scan
    // and its barriers (per-unit hand-over only: there the page ids are complete behind the ready word's barrier)
    const bool early = kGather && p.ready != nullptr;
    if constexpr (kGather) {
        if (early) {
            uint32_t mk = gtm;
            while (mk != 0) {
                const int j = __ffs(mk) - 1;
                mk &= mk - 1;
                const int t = tok00 + (j & 7) + 32 * (j >> 3) - chunk_start;
                const int pg = s_pages[t / kPage];
                if (pg >= 0) prefetch_row((pg * p.Hkv + kvh) * kPage + t % kPage);
            }
        }
    }
    // exclusive prefix over the threads (= over the chunk in block order) of the two counts, 16 bits each
    const uint32_t mine = (uint32_t)__popc(gtm) | ((uint32_t)__popc(eqm) << 16);
    uint32_t incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += u;
    }
    if (lane == 31) s_wtot[warp] = incl;
    __syncthreads();  // (also: s_pages is complete)
    uint32_t before = incl - mine, total = 0;
#pragma unroll
    for (int wv = 0; wv < kSaWarps; ++wv) {
        const uint32_t t = s_wtot[wv];
        before += wv < warp ? t : 0u;
        total += t;
    }
    const int gt_before = (int)(before & 0xffffu), eq_before = (int)(before >> 16);
    const int tot_gt = (int)(total & 0xffffu), tot_eq = (int)(total >> 16);
    // ties: the first `need` of the whole sequence by token index are kept; eqb of them lie in earlier chunks
    const int quota = need - eqb > 0 ? need - eqb : 0;
    uint32_t eq_take = quota >= tot_eq ? eqm : 0u;
    const bool straddle = quota > 0 && quota < tot_eq;  // uniform over the CTA; at most one chunk per (sequence, head)
    int blk_before = 0;
    uint32_t lanes_it[4] = {0u, 0u, 0u, 0u};  // per it: the block's tied tokens as a mask over the scoring warp's lanes
    // rank of this thread's tied token j = 8 it + k among the chunk's ties by token index: blocks in order,
    // inside a block by (it, lane)
    auto tie_rank = [&](int j) {
        const int it = j >> 3, k = j & 7;
        int rank = blk_before;
#pragma unroll
        for (int i = 0; i < 4; ++i) rank += i < it ? __popc(lanes_it[i]) : 0;
        const uint32_t mk = it == 0 ? lanes_it[0] : (it == 1 ? lanes_it[1] : (it == 2 ? lanes_it[2] : lanes_it[3]));
        return rank + __popc(mk & ((1u << (la0 + k)) - 1u));
    };
    if (straddle) {
        blk_before = __shfl_sync(0xffffffffu, eq_before, lane & ~(kTpb - 1));
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            uint32_t mk = ((eqm >> (8 * it)) & ((1u << kWords) - 1u)) << la0;
#pragma unroll
            for (int d = 1; d < kTpb; d <<= 1) mk |= __shfl_xor_sync(0xffffffffu, mk, d);
            lanes_it[it] = mk;
        }
        uint32_t mk = eqm;
        while (mk != 0) {
            const int j = __ffs(mk) - 1;
            mk &= mk - 1;
            if (tie_rank(j) < quota) eq_take |= 1u << j;
        }
    }
    const int n_sel = tot_gt + min(quota, tot_eq);
    const int n_list = max(0, min(n_sel, p.sel_stride - base));  // an overflowing list was reported by the plan
    int32_t* idx = p.sel_idx + ((size_t)b * Hq + h) * p.sel_stride + base;
    auto emit = [&](int j, int pos, bool ask) {
        if (pos >= n_list) return;
        const int tok = tok00 + (j & 7) + 32 * (j >> 3);
        idx[pos] = tok;
        if constexpr (kGather) {
            const int pg = s_pages[(tok - chunk_start) / kPage];
            const int rr = pg >= 0 ? (pg * p.Hkv + kvh) * kPage + tok % kPage : -1;
            s_rows[pos] = rr;
            // ask L2 for the row's K and V lines now (both 128-byte lines of each: half a row measured slower than
            // none): the whole list is on its way before the first round of the gather starts, at no cost in
            // registers, and the later rounds find their rows in L2
            if (rr >= 0 && ask) prefetch_row(rr);
        }
    };
    {
        uint32_t mk = gtm;
        int pos = gt_before;
        while (mk != 0) {
            const int j = __ffs(mk) - 1;
            mk &= mk - 1;
            emit(j, pos++, !early);
        }
        mk = eq_take;
        pos = tot_gt + eq_before;
        while (mk != 0) {
            const int j = __ffs(mk) - 1;
            mk &= mk - 1;
            emit(j, straddle ? tot_gt + tie_rank(j) : pos++, true);
        }
    }
    if constexpr (!kGather) return;
    __syncthreads();
    attend_list(n_list);
    store_partial();
}

// Log-sum-exp merge of the partials select_attend_kernel left for one (sequence, head): the partials of the CTAs
// that had a chunk (those below the sequence length) and of the two edge CTAs. 512 threads: thread = (output
// dimension, one of 4 slices of the partials), so that up to 68 partials are fetched in one trip with at most
// 17 x 3 loads per thread in flight; the slices are combined in shared memory.
constexpr int kMergeSlices = 4;
constexpr int kMergeThreads = kHeadDim * kMergeSlices;
constexpr int kMergeBatch = 17;

__global__ void __launch_bounds__(kMergeThreads) select_attend_merge_kernel(const SelectAttendParams p, int chunk_tokens) {
    const int h = p.h0 + blockIdx.x, b = blockIdx.y;
    const int Hq = p.Hkv * kGroup;
    const int tid = threadIdx.x, d = tid % kHeadDim, slice = tid / kHeadDim;
    __shared__ float s_m[kMergeSlices], s_l[kMergeSlices];
    __shared__ float s_a[kMergeSlices][kHeadDim];
    const int S = p.seq_lens[b];
    const bool ok = S >= 1 && S <= p.max_pages * kPage;
    const int nparts = kSaEdgeSlots + (S + chunk_tokens - 1) / chunk_tokens;

    pdl_wait();
    pdl_launch_dependents();
    if (p.status_out != nullptr && (blockIdx.x | blockIdx.y | threadIdx.x) == 0) *p.status_out = __ldcg(p.status);
    if (!ok) return;

    const float* base = p.partials + ((size_t)b * Hq + h) * p.nslots * kPartStride;
    // this slice's partials: j = slice + 4 i
    const int mine = (nparts - slice + kMergeSlices - 1) / kMergeSlices;
    float Mg = -INFINITY, Lg = 0.f, Ag = 0.f;
    for (int i0 = 0; i0 < mine; i0 += kMergeBatch) {
        const int n = min(kMergeBatch, mine - i0);
        float ms[kMergeBatch], ls[kMergeBatch], as[kMergeBatch];
#pragma unroll
        for (int j = 0; j < kMergeBatch; ++j) {
            const float* ps = base + (size_t)(slice + kMergeSlices * (i0 + min(j, n - 1))) * kPartStride;
            ms[j] = __ldcg(ps);
            ls[j] = __ldcg(ps + 1);
            as[j] = __ldcg(ps + 2 + d);
        }
        float mb = Mg;
#pragma unroll
        for (int j = 0; j < kMergeBatch; ++j) mb = fmaxf(mb, j < n ? ms[j] : -INFINITY);
        const float rescale = Mg == -INFINITY ? 0.f : fast_exp2(Mg - mb);
        Mg = mb;
        Lg *= rescale;
        Ag *= rescale;
#pragma unroll
        for (int j = 0; j < kMergeBatch; ++j) {
            const float f = (j < n && ms[j] != -INFINITY) ? fast_exp2(ms[j] - Mg) : 0.f;
            Lg = fmaf(ls[j], f, Lg);
            Ag = fmaf(as[j], f, Ag);
        }
    }
    if (d == 0) {
        s_m[slice] = Mg;
        s_l[slice] = Lg;
    }
    s_a[slice][d] = Ag;
    __syncthreads();
    if (slice != 0) return;
    float M = -INFINITY, L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < kMergeSlices; ++w) M = fmaxf(M, s_m[w]);
#pragma unroll
    for (int w = 0; w < kMergeSlices; ++w) {
        const float f = s_m[w] == -INFINITY ? 0.f : fast_exp2(s_m[w] - M);
        L = fmaf(s_l[w], f, L);
        A = fmaf(s_a[w][d], f, A);
    }
    p.out[((size_t)b * Hq + h) * kHeadDim + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
}

}  // namespace ha
