// Shared constants and device helpers of the HashAttention sparse-decode kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hashattn.h"

namespace ha {

constexpr int kHeadDim = 128;     // elements per K / V / q row
constexpr int kGroup = 4;         // query heads per kv head == u32 codes per 16-byte hash word
constexpr int kPage = 256;        // tokens per cache page
constexpr int kCodeBits = 32;     // hash width
constexpr int kBins = kCodeBits + 1;  // Hamming scores 0..32
constexpr int kHidden = 128;      // width of the two hidden MLP layers
constexpr int kMlpElems = kHidden * kHeadDim + kHidden * kHidden + kCodeBits * kHidden;  // 36864
constexpr int kMlpBias = kHidden + kHidden + kCodeBits;                                  // 288

// score / select tiling: a CTA of 256 threads owns one chunk of chunk_pages pages of one
// (sequence, kv-head); warp w owns the w-th eighth of the chunk (32 * chunk_pages tokens).
constexpr int kSelThreads = 256;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kMaxChunkPages = 16;  // <= 16 tokens per lane live in registers

// sparse decode tiling: a CTA of 128 threads = 8 half-warp workers, 4 rows per worker and round.
constexpr int kAttThreads = 128;
constexpr int kAttWorkers = kAttThreads / 16;
constexpr int kAttRowsPerWorker = 4;
constexpr int kAttRoundRows = kAttWorkers * kAttRowsPerWorker;  // 32 rows per CTA and round
constexpr int kAttMaxRounds = 8;
constexpr int kPartStride = kHeadDim + 2;                        // m, l, acc[128]

struct SeqRange {
    int S;   // cached tokens incl. the current one
    int lo;  // sink tokens are [0, lo)
    int hi;  // recent tokens are [hi, S); candidates are [lo, hi)
    int hb;  // heavy tokens actually selected: min(budget, hi - lo)
};

// Budget arithmetic of compute_mask_multi (hashattention/hashattention_llama.py:423-435):
// candidates exclude the first init and last recent tokens; the heavy budget is
// int(k * heavy_budget) for heavy_budget <= 1.0, int(heavy_budget) otherwise. k is the length of the
// key sequence: S itself for a single query token; for a row of a multi-token chunk the length
// after the whole chunk (budget_len), while S is what the row's own token may see.
__host__ __device__ inline SeqRange seq_range(int S, int init_budget, int recent_budget,
                                              double heavy_budget, int budget_len = -1) {
    SeqRange r;
    r.S = S;
    r.lo = init_budget < S ? init_budget : S;
    int tail = S - recent_budget;
    r.hi = tail > r.lo ? tail : r.lo;
    int hb = heavy_budget > 1.0 ? (int)heavy_budget : (int)((double)(budget_len >= 0 ? budget_len : S) * heavy_budget);
    if (hb < 0) hb = 0;
    int ncand = r.hi - r.lo;
    r.hb = hb < ncand ? hb : ncand;
    return r;
}

// Pages per score/select chunk: 4, 8 or 16 (the kernels are compiled for these), about
// max_pages / 32 so that a sequence is cut into roughly 32 chunks.
__host__ __device__ inline int chunk_pages_for(int max_pages) {
    const int want = (max_pages + 31) / 32;
    return want <= 4 ? 4 : (want <= 8 ? 8 : kMaxChunkPages);
}

__host__ __device__ inline int num_chunks_for(int max_pages) {
    int cp = chunk_pages_for(max_pages);
    return (max_pages + cp - 1) / cp;
}

__device__ __forceinline__ void report(int32_t* status, int code) {
    if (status != nullptr) atomicCAS(status, 0, code);
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Packed pairs of fp32 values (sm_100: two fp32 operations per instruction).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// asks L2 for the 128-byte line that holds p (no register is written, nothing waits)
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Programmatic dependent launch: a kernel launched with the programmatic-serialization
// attribute may start before its predecessor has finished; it must call pdl_wait() before
// it reads anything the predecessor wrote, and pdl_launch_dependents() lets the successor's
// prologue start early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace ha
