// Prefill key-hash build on the 5th-generation tensor cores (tcgen05, sm_100a only).
//
// For every cached key x (128 bf16) and every query head h of its kv-head the hash MLP
//     code = signbits( W2 . silu( W1 . silu( W0 x + b0 ) + b1 ) + b2 )
// is a chain of three GEMMs over a tile of 128 tokens. The (head, tile) pairs of a call, head-major, are cut
// into one contiguous range per CTA (one CTA per SM, equal tile counts); a CTA keeps the three weight
// matrices of its current head (72 KB bf16) in shared memory in the K-major 128-byte-swizzled layout the
// UMMA shared-memory descriptors describe, reloads them where its range crosses into the next head, and
// walks over its token tiles:
//   1. the 128 x 128 key tile is copied into swizzled shared memory (it is contiguous in a page) by
//      cp.async, one tile ahead of the arithmetic (two buffers),
//   2. one thread issues tcgen05.mma (M = 128, N = 128, K = 16 per instruction, bf16 x bf16 -> fp32)
//      into tensor memory and commits to an mbarrier,
//   3. the 16 warps read the accumulator with tcgen05.ld (thread = token row, 16 columns at a time: first the
//      columns 0..63, then 64..127, and the K-half of the next GEMM that reads the first half's activations is
//      issued in between, so that it runs under the second half of the epilogue), add
//      the bias, apply SiLU in fp32 and split the activation into a hi and a lo bf16 (hi + lo
//      carries 16 mantissa bits), written back to swizzled shared memory as the next A operand,
//   4. layer 2 runs two MMAs per k-step (hi and lo against the same weights), layer 3 likewise
//      with N = 32, and the last epilogue packs the 32 sign bits of a token row into its code.
// The hi/lo split keeps the pre-activations within ~3e-6 of fp32 arithmetic, which is what makes
// the packed codes match the reference bit for bit outside the |x| < 1e-5 band.
//
// Follows USA.k_embedding(hard=True) (hashattention/hashattention_llama.py:204-214).
//
// Every wait on the mbarrier is bounded: if a commit never arrives the CTA records
// HA_ERR_TIMEOUT, stops issuing work, frees its tensor memory and returns.
#pragma once

#include "common.cuh"

namespace ha {

constexpr int kTcThreads = 512;
constexpr int kTcTile = 128;                          // tokens per tile = TMEM lanes
constexpr uint32_t kTcBlockBytes = 128 * 128;         // one K-half of a 128-row operand: 128 rows x 128 B
constexpr uint32_t kTcW2BlockBytes = 32 * 128;        // one K-half of W2 (32 rows)
constexpr uint32_t kTcOffW0 = 0;
constexpr uint32_t kTcOffW1 = kTcOffW0 + 2 * kTcBlockBytes;
constexpr uint32_t kTcOffW2 = kTcOffW1 + 2 * kTcBlockBytes;
constexpr uint32_t kTcOffX = kTcOffW2 + 2 * kTcW2BlockBytes;           // two key-tile buffers (double buffering)
constexpr uint32_t kTcOffHi = kTcOffX + 4 * kTcBlockBytes;
constexpr uint32_t kTcOffLo = kTcOffHi + 2 * kTcBlockBytes;
constexpr uint32_t kTcOffBias = kTcOffLo + 2 * kTcBlockBytes;          // 288 floats
constexpr uint32_t kTcOffBar = kTcOffBias + 1280;                      // mbarrier (8 B) + tmem base (4 B)
constexpr uint32_t kTcSmemBytes = kTcOffBar + 64 + 1024;               // + slack to align the base to 1024 B
constexpr uint32_t kTcTmemCols = 512;
constexpr uint32_t kTcColD1 = 0, kTcColD2 = 128, kTcColD3 = 256;
constexpr int kTcSpinLimit = 1 << 22;

struct HashPrefillTcParams {
    const __nv_bfloat16* k_pages;
    uint32_t* hash_pages;
    const __nv_bfloat16* wk;   // [Hq][36864] bf16
    const float* bk;           // [Hq][288]
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* first_token;  // [B] or null
    int32_t* status;
    int B, Hkv, max_pages, num_pages;
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside one K-half block of a K-major
// operand with 128-byte swizzle: rows are 128 B apart, 8-row groups 1024 B apart, and the chunk
// index is XORed with the row's position in its group.
__device__ __forceinline__ uint32_t tc_swizzled(uint32_t row, uint32_t chunk) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

// Shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t tc_idesc(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Bounded wait for phase `parity` of the mbarrier; false if it ran out.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity) {
    for (int spin = 0; spin < kTcSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ uint32_t tc_pack_bf16(float a, float b) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);  // .x = a (low half), .y = b
    return *reinterpret_cast<const uint32_t*>(&t);
}

// Copies `rows` rows of 128 bf16 (row-major, 256 B apart in global memory) into the two K-half
// blocks of a swizzled operand; block_bytes = rows * 128.
__device__ __forceinline__ void tc_load_operand(unsigned char* dst, const __nv_bfloat16* src, int rows,
                                                uint32_t block_bytes, int tid) {
    for (int i = tid; i < rows * 16; i += kTcThreads) {
        const int row = i >> 4, c16 = i & 15;  // c16: 16-byte chunk of the 256-byte row
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (size_t)row * kHeadDim) + c16);
        *reinterpret_cast<uint4*>(dst + (c16 >> 3) * block_bytes + tc_swizzled(row, c16 & 7)) = v;
    }
}

// bias + SiLU + hi/lo split of 16 accumulator columns (chunks chunk0, chunk0 + 1 of one K-half block).
__device__ __forceinline__ void tc_hidden_epilogue(uint32_t taddr, const float* bias, unsigned char* hi_blk,
                                                   unsigned char* lo_blk, uint32_t row, uint32_t chunk0) {
    float v[16];
    tc_ld16(taddr, v);
#pragma unroll
    for (int c = 0; c < 2; ++c) {  // 2 chunks of 8 columns
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float a[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int col = c * 8 + e * 2 + j;
                const float x = v[col] + bias[col];
                // SiLU with the hardware exp2 / reciprocal (relative error ~1e-6, well below the
                // 2^-17 that the hi/lo split itself leaves)
                float e, r;  // exactly one exp2 and one reciprocal instruction per activation
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
                asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
                a[j] = x * r;
            }
            hi[e] = tc_pack_bf16(a[0], a[1]);  // one paired conversion; the rounded values are read back by shifts
            const float h0 = __uint_as_float(hi[e] << 16), h1 = __uint_as_float(hi[e] & 0xffff0000u);
            lo[e] = tc_pack_bf16(a[0] - h0, a[1] - h1);
        }
        const uint32_t off = tc_swizzled(row, chunk0 + c);
        *reinterpret_cast<uint4*>(hi_blk + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(lo_blk + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// Asynchronous copy (cp.async, 16 bytes per request) of a 128-token key tile into a swizzled buffer.
__device__ __forceinline__ void tc_prefetch_tile(unsigned char* dst, const __nv_bfloat16* src, int tid) {
    for (int i = tid; i < kTcTile * 16; i += kTcThreads) {
        const int row = i >> 4, c16 = i & 15;
        const uint32_t d = tc_smem_u32(dst + (c16 >> 3) * kTcBlockBytes + tc_swizzled(row, c16 & 7));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + (size_t)row * kHeadDim + c16 * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(kTcThreads, 1) hash_prefill_tc_kernel(const HashPrefillTcParams p) {
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    float* s_bias = reinterpret_cast<float*>(smem + kTcOffBias);
    unsigned long long* s_bar = reinterpret_cast<unsigned long long*>(smem + kTcOffBar);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kTcOffBar + 16);

    // The (head, token tile) pairs of the whole call, head-major and counting only tiles that hold tokens to
    // encode, are cut into gridDim.x equal contiguous ranges: every SM gets the same number of tiles whatever the
    // number of heads, and a CTA changes head (reloads the 72 KB of weights) at most once per head boundary it
    // spans. The first head of a CTA follows from its index alone, so its weights are fetched before the
    // dependency wait.
    auto load_head = [&](int h) {
        const __nv_bfloat16* W = p.wk + (size_t)h * kMlpElems;
        tc_load_operand(smem + kTcOffW0, W, 128, kTcBlockBytes, tid);
        tc_load_operand(smem + kTcOffW1, W + kHidden * kHeadDim, 128, kTcBlockBytes, tid);
        tc_load_operand(smem + kTcOffW2, W + kHidden * kHeadDim + kHidden * kHidden, 32, kTcW2BlockBytes, tid);
        for (int i = tid; i < kMlpBias; i += kTcThreads) s_bias[i] = p.bk[(size_t)h * kMlpBias + i];
    };
    int loaded_h = (int)(((long long)blockIdx.x * Hq) / gridDim.x);
    load_head(loaded_h);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(s_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(s_tmem)), "r"(kTcTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    const uint32_t bar = tc_smem_u32(s_bar);
    const uint32_t sbase = tc_smem_u32(smem);
    const uint32_t idesc128 = tc_idesc(128), idesc32 = tc_idesc(32);
    // this thread's accumulator slice: TMEM lanes 32 (warp % 4) .. +31, columns 32 (warp / 4) .. +31
    // in each half of a hidden epilogue: TMEM lanes 32 (warp % 4) .. +31, columns 64 half + 16 (warp / 4) .. +15
    const uint32_t row = (warp & 3) * 32 + lane, cq = warp >> 2;  // cq: group of 16 columns inside a half, 0..3
    const uint32_t chunk0 = cq * 2;                                // first 16-byte chunk inside the K-half block
    const uint32_t t_lane = ((warp & 3) * 32u) << 16;
    uint32_t phase = 0;

    // one K = 128 GEMM: 8 k-steps of 16 (32 bytes inside the swizzled 128-byte rows, 4 per K-half)
    auto gemm = [&](uint32_t col_d, uint32_t off_a, uint32_t off_b, uint32_t b_block_bytes, uint32_t idesc, bool first) {
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ++ks) {
            const uint32_t a = sbase + off_a + (ks >> 2) * kTcBlockBytes + (ks & 3) * 32;
            const uint32_t bb = sbase + off_b + (ks >> 2) * b_block_bytes + (ks & 3) * 32;
            tc_mma(tmem + col_d, tc_smem_desc(a), tc_smem_desc(bb), idesc, (first && ks == 0) ? 0u : 1u);
        }
    };
    // the k-steps of one K-half (half = 0: inputs 0..63, 1: inputs 64..127) of such a GEMM
    auto gemm_half = [&](uint32_t col_d, uint32_t off_a, uint32_t off_b, uint32_t b_block_bytes, uint32_t idesc,
                         uint32_t half, bool first) {
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
            const uint32_t a = sbase + off_a + half * kTcBlockBytes + ks * 32;
            const uint32_t bb = sbase + off_b + half * b_block_bytes + ks * 32;
            tc_mma(tmem + col_d, tc_smem_desc(a), tc_smem_desc(bb), idesc, (first && ks == 0) ? 0u : 1u);
        }
    };
    // Waits (bounded) for the commit of the GEMMs just issued, then agrees CTA-wide on the outcome,
    // so that the warp-synchronous tensor-memory loads that follow are never executed by a part of
    // the CTA only. Returns false for every thread if any thread's wait ran out.
    auto wait_commit = [&]() -> bool {
        const bool ok = tc_wait(bar, phase);
        if (!ok) report(p.status, HA_ERR_TIMEOUT);
        phase ^= 1;
        const bool all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        return all_ok;
    };
    bool aborted = false;
    pdl_wait();  // the weights above are constants; everything below may depend on the previous kernel

    // A sequence's tiles to encode: [first_token / 128, ceil(S / 128)); none if its length is out of range.
    struct Item { int valid, h, S, first, t0; size_t slot0; };
    struct Cursor { int h, b, tile, hi, S, first; long long left; };
    auto seq_tiles = [&](int b, int& S, int& first, int& lo, int& hi) {
        S = __ldg(p.seq_lens + b);
        first = p.first_token != nullptr ? max(0, __ldg(p.first_token + b)) : 0;
        if (S < 0 || S > p.max_pages * kPage) {
            if (tid == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
            S = 0;
        }
        lo = first / kTcTile;
        hi = max(lo, (S + kTcTile - 1) / kTcTile);
    };
    Cursor cs;
    {
        long long per_head = 0;  // tiles to encode per head
        for (int b = 0; b < p.B; ++b) {
            int S, first, lo, hi;
            seq_tiles(b, S, first, lo, hi);
            per_head += hi - lo;
        }
        const long long total = per_head * Hq;
        const long long g0 = total * blockIdx.x / gridDim.x, g1 = total * (blockIdx.x + 1) / gridDim.x;
        cs.left = g1 - g0;
        cs.h = per_head > 0 ? (int)(g0 / per_head) : 0;
        long long skip = per_head > 0 ? g0 % per_head : 0;  // tiles of head cs.h in front of this CTA's range
        cs.b = 0;
        cs.tile = cs.hi = cs.S = cs.first = 0;
        for (int b = 0; b < p.B && cs.left > 0; ++b) {
            int S, first, lo, hi;
            seq_tiles(b, S, first, lo, hi);
            if (skip < hi - lo) {
                cs.b = b; cs.S = S; cs.first = first; cs.tile = lo + (int)skip; cs.hi = hi;
                break;
            }
            skip -= hi - lo;
        }
    }
    // The next tile of this CTA's range (all inputs are CTA-uniform). A tile on a bad page is reported and skipped.
    auto next_item = [&]() {
        Item it;
        it.valid = 0; it.h = 0; it.S = 0; it.first = 0; it.t0 = 0; it.slot0 = 0;
        while (cs.left > 0) {
            if (cs.tile >= cs.hi) {  // on to the next sequence, or to the first one of the next head
                if (++cs.b >= p.B) {
                    cs.b = 0;
                    ++cs.h;
                }
                int lo;
                seq_tiles(cs.b, cs.S, cs.first, lo, cs.hi);
                cs.tile = lo;
                continue;
            }
            const int t0 = cs.tile * kTcTile;
            const int page = __ldg(p.page_table + (size_t)cs.b * p.max_pages + t0 / kPage);
            ++cs.tile;
            --cs.left;
            if (page < 0 || page >= p.num_pages) {
                if (tid == 0) report(p.status, HA_ERR_BAD_PAGE);
                continue;
            }
            it.valid = 1; it.h = cs.h; it.S = cs.S; it.first = cs.first; it.t0 = t0;
            it.slot0 = ((size_t)page * p.Hkv + cs.h / kGroup) * kPage + t0 % kPage;
            return it;
        }
        return it;
    };

    // what the epilogue (or cp.async) wrote becomes visible to the tensor core; the accumulator reads are done
    auto publish = [&]() {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    };
    // layer 0 of a tile whose keys sit in key buffer `buf`: D1 = X W0^T (waits for the keys first)
    auto start_tile = [&](uint32_t buf) {
        asm volatile("cp.async.wait_all;" ::: "memory");
        publish();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            gemm(kTcColD1, kTcOffX + buf * 2 * kTcBlockBytes, kTcOffW0, kTcBlockBytes, idesc128, true);
            tc_commit(bar);
        }
    };
    // bias + SiLU + hi/lo split of this thread's 16 columns in half `half` of accumulator col_d
    auto hidden = [&](uint32_t col_d, const float* bias, uint32_t half) {
        const uint32_t c0 = half * 64 + cq * 16;
        tc_hidden_epilogue(tmem + t_lane + col_d + c0, bias + c0, smem + kTcOffHi + half * kTcBlockBytes,
                           smem + kTcOffLo + half * kTcBlockBytes, row, chunk0);
    };
    auto codes = [&](const Item& it) {  // thread = token row: 32 pre-activations -> one packed code
        if (warp >= 4) return;
        float v[32];
        tc_ld32(tmem + t_lane + kTcColD3, v);
        uint32_t code = 0;
#pragma unroll
        for (int i = 0; i < 32; ++i) code |= (v[i] + s_bias[2 * kHidden + i] > 0.0f ? 1u : 0u) << i;
        const int t = it.t0 + (int)row;
        if (t < it.S && t >= it.first) p.hash_pages[(it.slot0 + row) * kGroup + it.h % kGroup] = code;
    };

    Item cur = next_item();
    if (cur.valid) {
        tc_prefetch_tile(smem + kTcOffX, p.k_pages + cur.slot0 * kHeadDim, tid);
        if (cur.h != loaded_h) {  // (cannot happen for the first tile of a range; kept for safety)
            __syncthreads();
            loaded_h = cur.h;
            load_head(loaded_h);
        }
        start_tile(0);
    }
    for (uint32_t n = 0; cur.valid; ++n) {
        // ---- layer 0 is running; meanwhile the next tile's keys start streaming in
        const Item nxt = next_item();
        if (nxt.valid)
            tc_prefetch_tile(smem + kTcOffX + ((n + 1) & 1) * 2 * kTcBlockBytes, p.k_pages + nxt.slot0 * kHeadDim, tid);
        if (!wait_commit()) { aborted = true; break; }
        // ---- hidden layers: the epilogue runs in two halves of 64 columns; the half of the next GEMM that reads
        //      the first half's activations (its K-half 0, hi and lo) is issued before the second half is worked on
        hidden(kTcColD1, s_bias, 0);
        publish();
        if (tid == 0) {  // layer 1, K-half 0: D2 = (Hhi + Hlo) W1^T
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            gemm_half(kTcColD2, kTcOffHi, kTcOffW1, kTcBlockBytes, idesc128, 0, true);
            gemm_half(kTcColD2, kTcOffLo, kTcOffW1, kTcBlockBytes, idesc128, 0, false);
        }
        hidden(kTcColD1, s_bias, 1);
        publish();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            gemm_half(kTcColD2, kTcOffHi, kTcOffW1, kTcBlockBytes, idesc128, 1, false);
            gemm_half(kTcColD2, kTcOffLo, kTcOffW1, kTcBlockBytes, idesc128, 1, false);
            tc_commit(bar);
        }
        if (!wait_commit()) { aborted = true; break; }
        hidden(kTcColD2, s_bias + kHidden, 0);
        publish();
        if (tid == 0) {  // layer 2, K-half 0: D3 = (Hhi + Hlo) W2^T, N = 32
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            gemm_half(kTcColD3, kTcOffHi, kTcOffW2, kTcW2BlockBytes, idesc32, 0, true);
            gemm_half(kTcColD3, kTcOffLo, kTcOffW2, kTcW2BlockBytes, idesc32, 0, false);
        }
        hidden(kTcColD2, s_bias + kHidden, 1);
        publish();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            gemm_half(kTcColD3, kTcOffHi, kTcOffW2, kTcW2BlockBytes, idesc32, 1, false);
            gemm_half(kTcColD3, kTcOffLo, kTcOffW2, kTcW2BlockBytes, idesc32, 1, false);
            tc_commit(bar);
        }
        if (!wait_commit()) { aborted = true; break; }
        // ---- the codes of this tile are packed while layer 0 of the next tile runs (D1 and D3 are different
        //      columns; D3 is written again only after two more barriers). A change of head rewrites the biases the
        //      codes need, so there the codes come first.
        if (nxt.valid && nxt.h != loaded_h) {
            codes(cur);
            __syncthreads();
            loaded_h = nxt.h;
            load_head(loaded_h);
            start_tile((n + 1) & 1);
        } else {
            if (nxt.valid) start_tile((n + 1) & 1);
            codes(cur);
        }
        cur = nxt;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    // ---- release tensor memory (after a time-out: give in-flight MMAs one more bounded wait) -------
    __syncthreads();
    if (aborted && tid == 0) tc_wait(bar, phase ^ 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcTmemCols) : "memory");
    }
}

}  // namespace ha
