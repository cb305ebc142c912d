// Prefill key-hash build on the 5th-generation tensor cores (tcgen05, sm_100a only), warp-specialised.
//
// For every cached key x (128 bf16) and every query head h of its kv-head the hash MLP
//     code = signbits( W2 . silu( W1 . silu( W0 x + b0 ) + b1 ) + b2 )
// is a chain of three GEMMs over a tile of 128 tokens. The (head, tile) pairs of a call, head-major, are cut
// into one contiguous range per CTA (one CTA per SM, equal tile counts); a CTA keeps the three weight
// matrices of its current head (72 KB bf16) in shared memory in the K-major 128-byte-swizzled layout the
// UMMA shared-memory descriptors describe, and reloads them where its range crosses into the next head.
//
// Roles of the 18 warps of a CTA:
//   * warp 1, the loader: one thread copies the 128 x 128 key tile (two TMA box copies, written in the same
//     swizzle) into a ring of four shared-memory buffers, up to four tiles ahead of the arithmetic;
//   * warp 0, the issuer: one thread issues every tcgen05.mma of the CTA and commits to mbarriers;
//   * warps 2-17, the epilogue: a thread owns one token row (its tensor-memory lane) and one 32-column slice of a
//     hidden layer. It reads its accumulator columns (tcgen05.ld), adds the bias, applies SiLU in fp32, splits
//     the activation into a hi and a lo bf16 (hi + lo carries 16 mantissa bits) and writes both back with
//     tcgen05.st over the columns it has just read: the next GEMM takes its A operand from tensor memory (two
//     MMAs per k-step, hi and lo against the same weights), so activations never pass through shared memory.
//     The last epilogue packs the sign bits of a token row into its code.
// Two tiles are in flight, one per slot of 256 tensor-memory columns (two regions of 128 that swap roles from
// tile to tile: layer-0 accumulator and its activations in one, layer-1 accumulator and its activations in the
// other, the 32 layer-2 columns back in the first). The epilogue warps alternate between the slots,
//     layer 0 of a, layer 0 of b, layer 1 of a, layer 1 of b, codes of a, (next pair) layer 0 of a', codes of b, ...
// and the issuer follows the same order, so the GEMM that a phase waits for was issued a whole phase earlier and
// runs under the other tile's arithmetic.
//
// The hi/lo split keeps the pre-activations within ~1e-6 of fp32 arithmetic, which is what makes
// the packed codes match the reference bit for bit outside the |x| < 1e-5 band.
//
// fp32 weights (hash_prefill_tc_kernel<float>) are split the same way when a head is loaded: a hi and a lo bf16 copy
// in shared memory, every GEMM multiplies by both (layer 0: X Whi + X Wlo; hidden layers: hi Whi + lo Whi + hi Wlo),
// and the key-tile ring shrinks from four tiles to two to make room.
//
// Follows USA.k_embedding(hard=True) (hashattention/hashattention_llama.py:204-214).
//
// Every wait is bounded: if a barrier never completes, the waiting thread records HA_ERR_TIMEOUT and raises a
// CTA-wide flag that ends every other wait; the CTA then waits (bounded) for the tensor core and its copies,
// frees its tensor memory and returns.
#pragma once

#include <cuda.h>  // CUtensorMap (the type only: the encoder is looked up at run time)

#include "common.cuh"

namespace ha {

constexpr int kTcEpiWarps = 16;                       // four 32-column slices x four quarters of the 128 tensor-memory lanes
constexpr int kTcEpiThreads = kTcEpiWarps * 32;
constexpr int kTcMmaWarp = 0;
constexpr int kTcLoadWarp = 1;
constexpr int kTcEpiWarp0 = 2;                        // epilogue warps kTcEpiWarp0 .. kTcEpiWarp0 + kTcEpiWarps - 1
constexpr int kTcThreads = (kTcEpiWarps + 2) * 32;
constexpr int kTcTile = 128;                          // tokens per tile = TMEM lanes
constexpr uint32_t kTcBlockBytes = 128 * 128;         // one K-half of a 128-row operand: 128 rows x 128 B
constexpr uint32_t kTcW2BlockBytes = 32 * 128;        // one K-half of W2 (32 rows)
constexpr uint32_t kTcOffW0 = 0;
constexpr uint32_t kTcOffW1 = kTcOffW0 + 2 * kTcBlockBytes;
constexpr uint32_t kTcOffW2 = kTcOffW1 + 2 * kTcBlockBytes;
constexpr uint32_t kTcWBytes = kTcOffW2 + 2 * kTcW2BlockBytes;  // one copy of a head's weights: 72 KB
constexpr int kTcMaxXBufs = 4;
constexpr int kTcInfoRing = 16;  // tile records the loader keeps for the epilogue (it runs at most 6 tiles ahead of their use)
// Where the codes of a tile go: byte offset of row 0's code word in the hash pages, and the rows [row_lo, row_hi) of the
// tile that hold tokens to encode (none for a tile on a bad page). Written by the loader, read by the epilogue warps.
struct TcTileInfo {
    unsigned long long word0;
    int row_lo, row_hi;
};
static_assert(sizeof(TcTileInfo) == 16, "tile record");
// mbarriers (8 bytes each), by index
constexpr int kTcBarXFull = 0;                           // [key-tile ring] the loader's expect-tx arrival + the bytes of the two copies
constexpr int kTcBarXEmpty = kTcBarXFull + kTcMaxXBufs;  // [key-tile ring] commit: layer 0 has read the tile
constexpr int kTcBarAcc = kTcBarXEmpty + kTcMaxXBufs;    // [2 slots][3 layers] commit: accumulator complete
constexpr int kTcBarAct = kTcBarAcc + 6;              // [2 slots] 16 warps: the activations of a hidden layer are written
constexpr int kTcBarDrained = kTcBarAct + 2;          // 16 epilogue warps + issuer: no GEMM reads the old weights any more
constexpr int kTcBarWeights = kTcBarDrained + 1;      // 16 epilogue warps: the next head's weights are in place
constexpr int kTcBarFinal = kTcBarWeights + 1;        // commit: every GEMM of the CTA has completed
constexpr int kTcNumBars = kTcBarFinal + 1;
static_assert(kTcNumBars <= 32, "barrier block");
// Shared memory of a CTA. bf16 weights: one copy of the head's weights and a ring of four key tiles. fp32 weights are
// split into a hi and a lo bf16 copy (W = hi + lo to 16 mantissa bits; every GEMM multiplies by both), and the ring
// holds two tiles.
template <bool kSplitW>
struct TcLayout {
    static constexpr int kXBufs = kSplitW ? 2 : 4;
    static constexpr uint32_t kOffWLo = kTcWBytes;  // the lo copy (split weights only)
    static constexpr uint32_t kOffX = kSplitW ? 2 * kTcWBytes : kTcWBytes;
    static constexpr uint32_t kOffBias = kOffX + kXBufs * 2 * kTcBlockBytes;  // 288 floats
    static constexpr uint32_t kOffBar = kOffBias + 1280;
    static constexpr uint32_t kOffTmem = kOffBar + 8 * 32;   // tmem base (4 B), abort flag (4 B)
    static constexpr uint32_t kOffInfo = kOffTmem + 16;      // ring of kTcInfoRing tile records (16 B each)
    static constexpr uint32_t kSmemBytes = kOffInfo + kTcInfoRing * 16 + 1024;  // + slack to align the base to 1024 B
    static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
};
constexpr uint32_t kTcTmemCols = 512;
constexpr int kTcSpinLimit = 1 << 22;

struct HashPrefillTcParams {
    const __nv_bfloat16* k_pages;
    uint32_t* hash_pages;
    const void* wk;            // [Hq][36864] bf16 or fp32
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

// Shared-memory matrix descriptor (K-major, SWIZZLE_128B, 8-row groups 1024 B apart) in two parts: only the low word
// depends on the address, and the descriptor of a later k-step of the operand follows by adding the k-step's offset in
// 16-byte units (the sum stays inside the address field).
__device__ __forceinline__ uint32_t tc_desc_lo(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ uint64_t tc_desc(uint32_t lo) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(64u | (1u << 14) | (2u << 29)));
    return d;
}
// k-step ks (16 inputs = 32 bytes of the 128-byte rows, four per K-half block) of an operand, in 16-byte units
__host__ __device__ constexpr uint32_t tc_koff(uint32_t ks, uint32_t block_bytes) { return (ks >> 2) * (block_bytes >> 4) + (ks & 3) * 2; }

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t tc_idesc(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// D (tensor memory) (+)= A (shared memory) . B (shared memory)
__device__ __forceinline__ void tc_mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// D (tensor memory) (+)= A (tensor memory: lane = row, two bf16 per column, K = 16 in 8 columns) . B (shared memory)
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Has phase `parity` of the mbarrier completed? (does not block)
__device__ __forceinline__ bool tc_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

// Bounded wait for phase `parity` of the mbarrier; false if it ran out or another thread of the CTA gave up.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
    for (int spin = 0; spin < kTcSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (*abort_flag != 0) return false;
    }
    report(status, HA_ERR_TIMEOUT);
    *abort_flag = 1;
    return false;
}

// 16 accumulator columns of this thread's lane: issue, and the wait that makes the registers readable (it waits for
// every read the thread has issued). The wait takes the registers as operands, so that nothing that reads them can be
// scheduled in front of it.
__device__ __forceinline__ void tc_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_ld16_wait(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :: "memory");
}

// 8 columns of this thread's lane, complete on return.
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
                 :: "memory");
}

// 16 columns of this thread's lane written to tensor memory (complete after tcgen05.wait::st).
__device__ __forceinline__ void tc_st16_issue(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};\n"
        :: "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
           "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
           "r"(taddr)
        : "memory");
}

// TMA: the box at element column x, row y of the key cache -> shared memory, bytes counted on the mbarrier (the
// copy reads this GPU's memory only and has this CTA as its single destination).
__device__ __forceinline__ void tc_tma_load(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// two fp32 -> one word of two bf16 (round to nearest even): a in the low half, b in the high half
__device__ __forceinline__ uint32_t tc_pack_bf16(float a, float b) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
    return d;
}

// Copies `rows` rows of 128 bf16 (row-major, 256 B apart in global memory) into the two K-half
// blocks of a swizzled operand; block_bytes = rows * 128. Thread t of n.
__device__ __forceinline__ void tc_load_operand(unsigned char* dst, const __nv_bfloat16* src, int rows,
                                                uint32_t block_bytes, int t, int n) {
    for (int i = t; i < rows * 16; i += n) {
        const int row = i >> 4, c16 = i & 15;  // c16: 16-byte chunk of the 256-byte row
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (size_t)row * kHeadDim) + c16);
        *reinterpret_cast<uint4*>(dst + (c16 >> 3) * block_bytes + tc_swizzled(row, c16 & 7)) = v;
    }
}

// The same from fp32 weights: every weight becomes a hi and a lo bf16 (hi + lo carries 16 mantissa bits), written to
// two copies of the operand.
__device__ __forceinline__ void tc_load_operand(unsigned char* dst, unsigned char* dst_lo, const float* src, int rows,
                                                uint32_t block_bytes, int t, int n) {
    for (int i = t; i < rows * 16; i += n) {
        const int row = i >> 4, c16 = i & 15;  // c16: 8 weights = one 16-byte chunk of the bf16 row
        const float4 a = __ldg(reinterpret_cast<const float4*>(src + (size_t)row * kHeadDim) + 2 * c16);
        const float4 b = __ldg(reinterpret_cast<const float4*>(src + (size_t)row * kHeadDim) + 2 * c16 + 1);
        const float w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hi[j] = tc_pack_bf16(w[2 * j], w[2 * j + 1]);
            lo[j] = tc_pack_bf16(w[2 * j] - bf16_lo(hi[j]), w[2 * j + 1] - bf16_hi(hi[j]));
        }
        const uint32_t off = (c16 >> 3) * block_bytes + tc_swizzled(row, c16 & 7);
        *reinterpret_cast<uint4*>(dst + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(dst_lo + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// bias + SiLU + hi/lo split of 16 accumulator columns v (bit patterns of fp32) of one row. The 16 words that take their
// place are the A operand of one k-step of the next GEMM: words 0..7 hold the hi halves of the activations (two per
// word, the even one in the low half), words 8..15 their lo halves.
__device__ __forceinline__ void tc_activate16(const uint32_t (&v)[16], const float* bias, uint32_t (&out)[16]) {
    const f32x2 nlog2e = pack2(-1.4426950408889634f, -1.4426950408889634f), one = pack2(1.0f, 1.0f);
#pragma unroll
    for (int pr = 0; pr < 8; ++pr) {
        const float2 bb = *reinterpret_cast<const float2*>(bias + 2 * pr);  // the same address in every lane: a broadcast
        const f32x2 x = add2(pack2(__uint_as_float(v[2 * pr]), __uint_as_float(v[2 * pr + 1])), pack2(bb.x, bb.y));
        float t0, t1;
        unpack2(mul2(x, nlog2e), t0, t1);
        // SiLU x / (1 + e^-x) with the hardware exp2 and ONE reciprocal for the pair: 1 / (a0 a1) times a1 and a0.
        // e is held below 2^60 so that the product stays finite (the activation is below 1e-16 in magnitude there).
        float e0, e1, r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(fminf(t0, 60.0f)));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(fminf(t1, 60.0f)));
        float a0, a1;
        unpack2(add2(pack2(e0, e1), one), a0, a1);
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a0 * a1));
        const f32x2 y = mul2(x, mul2(pack2(a1, a0), pack2(r, r)));
        float y0, y1;
        unpack2(y, y0, y1);
        const uint32_t hi = tc_pack_bf16(y0, y1);
        float l0, l1;  // y - hi, exact: the multiply-add takes the bf16 halves of hi as they are
        asm("{\n\t.reg .b16 h0, h1;\n\tmov.b32 {h0, h1}, %2;\n\t"
            "fma.rn.f32.bf16 %0, h0, %3, %4;\n\tfma.rn.f32.bf16 %1, h1, %3, %5;\n\t}"
            : "=f"(l0), "=f"(l1) : "r"(hi), "h"((unsigned short)0xBF80), "f"(y0), "f"(y1));
        out[pr] = hi;
        out[pr + 8] = tc_pack_bf16(l0, l1);
    }
}

// The (head, token tile) pairs of the whole call, head-major and counting only tiles that hold tokens to encode,
// are cut into gridDim.x equal contiguous ranges: every SM gets the same number of tiles whatever the number of
// heads. A cursor walks over the tiles of this CTA's range; every value is CTA-uniform, so each role runs its own.
struct TcItem {
    int h, S, first, t0, store;
    size_t slot0;  // (page * Hkv + kv head) * page size + offset of the tile's first token
};
struct TcCursor {
    const HashPrefillTcParams& p;
    long long per_head, g0, total;  // tiles to encode per head; this CTA's first tile; its number of tiles
    int h, b, tile, hi, S, first;
    bool reporter;

    // A sequence's tiles to encode: [first_token / 128, ceil(S / 128)); none if its length is out of range.
    __device__ void seq_tiles(int bb, int& S_, int& first_, int& lo, int& hi_) const {
        S_ = __ldg(p.seq_lens + bb);
        first_ = p.first_token != nullptr ? max(0, __ldg(p.first_token + bb)) : 0;
        if (S_ < 0 || S_ > p.max_pages * kPage) {
            if (reporter) report(p.status, HA_ERR_BAD_SEQ_LEN);
            S_ = 0;
        }
        lo = first_ / kTcTile;
        hi_ = max(lo, (S_ + kTcTile - 1) / kTcTile);
    }
    __device__ TcCursor(const HashPrefillTcParams& p_, bool reporter_) : p(p_), reporter(reporter_) {
        const int Hq = p.Hkv * kGroup;
        per_head = 0;
        for (int bb = 0; bb < p.B; ++bb) {
            int S_, first_, lo, hi_;
            seq_tiles(bb, S_, first_, lo, hi_);
            per_head += hi_ - lo;
        }
        const long long all = per_head * Hq;
        g0 = all * blockIdx.x / gridDim.x;
        total = all * (blockIdx.x + 1) / gridDim.x - g0;
        h = per_head > 0 ? (int)(g0 / per_head) : 0;
        long long skip = per_head > 0 ? g0 % per_head : 0;  // tiles of head h in front of this CTA's range
        b = 0;
        tile = hi = S = first = 0;
        for (int bb = 0; bb < p.B && total > 0; ++bb) {
            int S_, first_, lo, hi_;
            seq_tiles(bb, S_, first_, lo, hi_);
            if (skip < hi_ - lo) {
                b = bb; S = S_; first = first_; tile = lo + (int)skip; hi = hi_;
                break;
            }
            skip -= hi_ - lo;
        }
    }
    // Is local tile i the first one of a head (other than the CTA's first tile)? The weights change in front of it.
    __device__ bool head_starts_at(long long i) const { return i > 0 && (g0 + i) % per_head == 0; }
    __device__ int head_of(long long i) const { return (int)((g0 + i) / per_head); }
    // The next tile (to be called `total` times). A tile on a bad page is reported, read from page 0 and not stored.
    __device__ TcItem next() {
        const int Hq = p.Hkv * kGroup;
        for (int guard = 0; tile >= hi && guard <= p.B * Hq; ++guard) {  // on to the next sequence, or the next head
            if (++b >= p.B) {
                b = 0;
                ++h;
            }
            int lo;
            seq_tiles(b, S, first, lo, hi);
            tile = lo;
        }
        TcItem it;
        it.h = min(h, Hq - 1); it.S = S; it.first = first; it.t0 = tile * kTcTile; it.store = tile < hi ? 1 : 0;
        int page = __ldg(p.page_table + (size_t)b * p.max_pages + min(it.t0 / kPage, p.max_pages - 1));
        ++tile;
        if (page < 0 || page >= p.num_pages) {
            if (reporter) report(p.status, HA_ERR_BAD_PAGE);
            page = 0;
            it.store = 0;
        }
        it.slot0 = ((size_t)page * p.Hkv + it.h / kGroup) * kPage + it.t0 % kPage;
        return it;
    }
};

template <typename WT>
__global__ void __launch_bounds__(kTcThreads, 1) hash_prefill_tc_kernel(const HashPrefillTcParams p,
                                                                        const __grid_constant__ CUtensorMap k_map) {
    constexpr bool kSplitW = sizeof(WT) == 4;  // fp32 weights: hi and lo copies, every GEMM multiplies by both
    using L = TcLayout<kSplitW>;
    constexpr int kTcXBufs = L::kXBufs;
    constexpr uint32_t kTcOffX = L::kOffX, kTcOffBias = L::kOffBias, kTcOffBar = L::kOffBar, kTcOffTmem = L::kOffTmem;
    constexpr uint32_t kTcOffInfo = L::kOffInfo;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = p.Hkv * kGroup;
    float* s_bias = reinterpret_cast<float*>(smem + kTcOffBias);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kTcOffTmem);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kTcOffTmem + 4);
    TcTileInfo* s_info = reinterpret_cast<TcTileInfo*>(smem + kTcOffInfo);
    const uint32_t sbase = tc_smem_u32(smem);
    const uint32_t bars = sbase + kTcOffBar;
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

    // The weights of head h, by thread t of n. The first head of a CTA follows from its index alone, so its weights
    // are fetched before the dependency wait.
    auto load_head = [&](int h, int t, int n) {
        const WT* W = static_cast<const WT*>(p.wk) + (size_t)h * kMlpElems;
        if constexpr (kSplitW) {
            unsigned char* lo = smem + L::kOffWLo;
            tc_load_operand(smem + kTcOffW0, lo + kTcOffW0, W, 128, kTcBlockBytes, t, n);
            tc_load_operand(smem + kTcOffW1, lo + kTcOffW1, W + kHidden * kHeadDim, 128, kTcBlockBytes, t, n);
            tc_load_operand(smem + kTcOffW2, lo + kTcOffW2, W + kHidden * kHeadDim + kHidden * kHidden, 32, kTcW2BlockBytes, t, n);
        } else {
            tc_load_operand(smem + kTcOffW0, W, 128, kTcBlockBytes, t, n);
            tc_load_operand(smem + kTcOffW1, W + kHidden * kHeadDim, 128, kTcBlockBytes, t, n);
            tc_load_operand(smem + kTcOffW2, W + kHidden * kHeadDim + kHidden * kHidden, 32, kTcW2BlockBytes, t, n);
        }
        for (int i = t; i < kMlpBias; i += n) s_bias[i] = p.bk[(size_t)h * kMlpBias + i];
    };
    load_head((int)(((long long)blockIdx.x * Hq) / gridDim.x), tid, kTcThreads);
    if (tid == 0) {
        auto init = [&](int first, int n, uint32_t count) {
            for (int i = first; i < first + n; ++i)
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar(i)), "r"(count));
        };
        init(kTcBarXFull, kTcMaxXBufs, 1);
        init(kTcBarXEmpty, kTcMaxXBufs, 1);
        init(kTcBarAcc, 6, 1);
        init(kTcBarAct, 2, kTcEpiWarps);
        init(kTcBarDrained, 1, kTcEpiWarps + 1);
        init(kTcBarWeights, 1, kTcEpiWarps);
        init(kTcBarFinal, 1, 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(s_tmem)), "r"(kTcTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    pdl_wait();  // the weights above are constants; everything below may depend on the previous kernel

    // every lane waits for itself; the warp then agrees, so that the warp-wide instructions that follow are never
    // executed by a part of it
    auto wait = [&](int b, uint32_t parity) {
        const bool ok = tc_wait(bar(b), parity, s_abort, p.status);
        return __all_sync(0xffffffffu, ok) != 0;
    };

    if (warp >= kTcEpiWarp0) {
        // ---- epilogue warps ----------------------------------------------------------------------------------
        // (a warp reaches the tensor-memory lanes 32 (warp % 4) .. + 31; any 16 consecutive warps cover each quarter 4 times)
        const uint32_t sl = (uint32_t)(warp - kTcEpiWarp0) >> 2;  // this warp's 32-column slice of a hidden layer
        const uint32_t row = (uint32_t)(warp & 3) * 32 + lane;    // token row of the tile = tensor-memory lane
        const uint32_t t_base = tmem + (((uint32_t)(warp & 3) * 32u) << 16);
        int total, per_head, first_end, head0;  // this CTA's tiles; tiles per head; end of its first head's tiles; that head
        {
            const TcCursor cur(p, false);
            total = (int)cur.total;
            per_head = (int)cur.per_head;
            first_end = per_head > 0 ? (int)(cur.per_head - cur.g0 % cur.per_head) : 0;
            head0 = cur.h;
        }
        uint32_t cnt_e[2] = {0, 0}, cnt_c[2] = {0, 0}, changes = 0;  // tiles per slot: hidden layers done, codes done; head changes
        bool ok = true;
        // column of this warp's slice in the accumulator of hidden layer `layer` of the slot's tile number `count` (layer 0
        // works in the slot's region count & 1, layer 1 in the other one)
        auto slice_col = [&](uint32_t slot, uint32_t layer, uint32_t count) { return slot * 256u + ((count & 1) ^ layer) * 128u + 32u * sl; };
        // The slice is read and worked on in two halves of 16 columns, rx and ry, and every read is requested one half
        // ahead of its arithmetic: the second half at the start of the phase, the first half of the FOLLOWING phase between
        // the halves (if that phase's accumulator is complete by then; otherwise the phase starts with `acquire`).
        uint32_t rx[16], ry[16];
        auto acquire = [&](uint32_t slot, uint32_t layer) {
            if (!wait(kTcBarAcc + 3 * (int)slot + (int)layer, cnt_e[slot] & 1)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            tc_ld16_issue(t_base + slice_col(slot, layer, cnt_e[slot]), rx);
            return true;
        };
        // next_count: tiles of that slot whose hidden layers will be done when the phase starts
        auto prefetch = [&](uint32_t slot, uint32_t layer, uint32_t next_count) {
            if (__all_sync(0xffffffffu, tc_test(bar(kTcBarAcc + 3 * (int)slot + (int)layer), next_count & 1)) == 0) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            tc_ld16_issue(t_base + slice_col(slot, layer, next_count), rx);
            return true;
        };
        // a hidden layer of the slot's tile (first half requested): accumulator -> hi/lo activations in place
        auto hidden = [&](uint32_t slot, uint32_t layer, bool want_next, uint32_t next_slot, uint32_t next_layer,
                          uint32_t next_count, bool& have_next) {
            const uint32_t col = slice_col(slot, layer, cnt_e[slot]);
            const float* bias = s_bias + layer * kHidden + 32 * sl;
            uint32_t out[16];
            tc_ld16_wait(rx);
            tc_ld16_issue(t_base + col + 16u, ry);
            tc_activate16(rx, bias, out);
            tc_st16_issue(t_base + col, out);
            tc_ld16_wait(ry);
            have_next = want_next && prefetch(next_slot, next_layer, next_count);
            tc_activate16(ry, bias + 16, out);
            tc_st16_issue(t_base + col + 16u, out);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_arrive(bar(kTcBarAct + (int)slot));
            if (layer == 1) ++cnt_e[slot];
        };
        // the codes of tile i in `slot`: thread = token row, each of the row's four warps packs 8 of the 32 sign bits. Where
        // they go is in the tile's record (read behind the wait below, which orders it behind the loader's write).
        auto codes = [&](uint32_t slot, int i) {
            if (!wait(kTcBarAcc + 3 * (int)slot + 2, cnt_c[slot] & 1)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[8];
            tc_ld8(t_base + slot * 256u + (cnt_c[slot] & 1) * 128u + 8u * sl, r);
            uint32_t code = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) code |= (__uint_as_float(r[k]) + s_bias[2 * kHidden + 8 * sl + k] > 0.0f ? 1u : 0u) << k;
            const TcTileInfo info = s_info[i % kTcInfoRing];
            if ((int)row >= info.row_lo && (int)row < info.row_hi)
                reinterpret_cast<uint8_t*>(p.hash_pages)[info.word0 + row * (kGroup * 4) + sl] = (uint8_t)code;
            ++cnt_c[slot];
            return true;
        };
        // The tiles of a head are worked on in pairs, one tile per slot, in the order
        //     layer 0 of a, [codes of the previous pair's b], layer 0 of b, layer 1 of a, layer 1 of b, codes of a
        // so that the GEMM a phase waits for was issued at least one whole phase earlier.
        for (int s0 = 0, seg = 0; s0 < total && ok; ++seg) {
            const int s1 = min(total, s0 == 0 ? first_end : s0 + per_head);  // end of this head's tiles
            if (s0 > 0) {
                // the weights change: the issuer and every epilogue warp meet (all GEMMs of the old head have completed),
                // then the epilogue warps load together
                __syncwarp();
                if (lane == 0) tc_arrive(bar(kTcBarDrained));
                if (!(ok = wait(kTcBarDrained, changes & 1))) break;
                load_head(head0 + seg, tid - kTcEpiWarp0 * 32, kTcEpiThreads);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) tc_arrive(bar(kTcBarWeights));
                if (!(ok = wait(kTcBarWeights, changes & 1))) break;
                ++changes;
            }
            int pend = -1;  // tile in slot 1 whose codes are due
            for (int a = s0; a < s1 && ok; a += 2) {
                const bool has_b = a + 1 < s1;
                bool have_a = false, have_b = false;
#pragma unroll 1
                for (uint32_t layer = 0; layer < 2 && ok; ++layer) {
                    if (!have_a && !(ok = acquire(0, layer))) break;
                    hidden(0, layer, has_b, 1, layer, cnt_e[1], have_b);
                    if (layer == 0 && pend >= 0 && !(ok = codes(1, pend))) break;
                    if (has_b) {
                        if (!have_b && !(ok = acquire(1, layer))) break;
                        hidden(1, layer, layer == 0, 0, 1, cnt_e[0], have_a);
                    } else {
                        have_a = false;
                    }
                    if (layer == 1) ok = codes(0, a);
                }
                pend = has_b ? a + 1 : -1;
            }
            if (ok && pend >= 0) ok = codes(1, pend);
            s0 = s1;
        }
    } else if (warp == kTcMmaWarp) {
        // ---- issuer ------------------------------------------------------------------------------------------
        // One thread issues every tcgen05.mma of the CTA, in the order in which the epilogue warps finish their phases.
        // The whole warp runs the loop with the same values in every lane (the operands of tcgen05.mma are warp-
        // uniform); lane 0 alone issues.
        const TcCursor cur0(p, false);
        const int total = __shfl_sync(0xffffffffu, (int)cur0.total, 0);
        const int per_head = __shfl_sync(0xffffffffu, (int)cur0.per_head, 0);
        const int first_end = __shfl_sync(0xffffffffu, cur0.per_head > 0 ? (int)(cur0.per_head - cur0.g0 % cur0.per_head) : 0, 0);
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
        const bool issue = lane == 0;
        const uint32_t w0_lo = tc_desc_lo(sbase + kTcOffW0), w1_lo = tc_desc_lo(sbase + kTcOffW1);
        const uint32_t w2_lo = tc_desc_lo(sbase + kTcOffW2), x_lo = tc_desc_lo(sbase + kTcOffX);
        constexpr uint32_t kWLo = L::kOffWLo >> 4;  // from a descriptor of the hi copy to the lo copy
        // accumulator regions of a slot's current tile: layer 0 (and layer 2) in d_a, layer 1 in d_b; they swap per tile
        uint32_t d_a[2] = {tmem_u, tmem_u + 256u}, d_b[2] = {tmem_u + 128u, tmem_u + 384u};
        uint32_t changes = 0;
        bool ok = true;
        // layer 0 of tile i into its slot: D1 = X W0^T
        auto layer0 = [&](int i, int slot) {
            const uint32_t buf = (uint32_t)i % kTcXBufs;
            if (!wait(kTcBarXFull + (int)buf, ((uint32_t)i / kTcXBufs) & 1)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (issue) {
                const uint32_t xb = x_lo + buf * (2 * kTcBlockBytes >> 4);
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ++ks) {
                    const uint64_t xdesc = tc_desc(xb + tc_koff(ks, kTcBlockBytes));
                    tc_mma_ss(d_a[slot], xdesc, tc_desc(w0_lo + tc_koff(ks, kTcBlockBytes)), tc_idesc(128), ks == 0 ? 0u : 1u);
                    if constexpr (kSplitW)
                        tc_mma_ss(d_a[slot], xdesc, tc_desc(w0_lo + kWLo + tc_koff(ks, kTcBlockBytes)), tc_idesc(128), 1u);
                }
                tc_commit(bar(kTcBarXEmpty + (int)buf));
                tc_commit(bar(kTcBarAcc + 3 * slot + 0));
            }
            return true;
        };
        // layer 1 (D2 = act(D1) W1^T) or layer 2 (D3 = act(D2) W2^T, 32 columns over D1) of the slot's tile, once all
        // 16 epilogue warps have written their activations
        auto layer12 = [&](int slot, uint32_t layer) {
            if (!wait(kTcBarAct + slot, layer)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (issue) {
                const uint32_t d = layer == 0 ? d_b[slot] : d_a[slot], a = layer == 0 ? d_a[slot] : d_b[slot];
                const uint32_t w_lo = layer == 0 ? w1_lo : w2_lo, blk = layer == 0 ? kTcBlockBytes : kTcW2BlockBytes;
                const uint32_t idesc = layer == 0 ? tc_idesc(128) : tc_idesc(32);
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ++ks) {
                    const uint32_t b_lo = w_lo + (ks >> 2) * (blk >> 4) + (ks & 3) * 2;
                    const uint64_t bdesc = tc_desc(b_lo);
                    tc_mma_ts(d, a + 16 * ks, bdesc, idesc, ks == 0 ? 0u : 1u);
                    tc_mma_ts(d, a + 16 * ks + 8, bdesc, idesc, 1u);
                    if constexpr (kSplitW) tc_mma_ts(d, a + 16 * ks, tc_desc(b_lo + kWLo), idesc, 1u);  // hi activations x lo weights
                }
                tc_commit(bar(kTcBarAcc + 3 * slot + 1 + (int)layer));
            }
            return true;
        };
        for (int s0 = 0; s0 < total && ok;) {
            const int s1 = min(total, s0 == 0 ? first_end : s0 + per_head);
            if (s0 > 0) {  // the next head's weights
                if (issue) tc_arrive(bar(kTcBarDrained));
                if (!(ok = wait(kTcBarWeights, changes & 1))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                ++changes;
            }
            ok = layer0(s0, 0);
            if (ok && s0 + 1 < s1) ok = layer0(s0 + 1, 1);
            for (int a = s0; a < s1 && ok; a += 2) {
                const bool has_b = a + 1 < s1;
                ok = layer12(0, 0);
                if (ok && has_b) ok = layer12(1, 0);
                if (ok) ok = layer12(0, 1);
                if (ok) {  // the slot's next tile swaps the two regions (layer 0 of it follows layer 2 in the tensor core's order)
                    const uint32_t t = d_a[0]; d_a[0] = d_b[0]; d_b[0] = t;
                    if (a + 2 < s1) ok = layer0(a + 2, 0);
                }
                if (ok && has_b) {
                    ok = layer12(1, 1);
                    const uint32_t t = d_a[1]; d_a[1] = d_b[1]; d_b[1] = t;
                    if (ok && a + 3 < s1) ok = layer0(a + 3, 1);
                }
            }
            s0 = s1;
        }
        // the tensor core has finished everything issued above (after a time-out: one more bounded wait)
        if (issue) tc_commit(bar(kTcBarFinal));
        for (int spin = 0; spin < kTcSpinLimit && __all_sync(0xffffffffu, tc_test(bar(kTcBarFinal), 0)) == 0; ++spin) {}
    } else {
        // ---- loader ------------------------------------------------------------------------------------------
        // One thread: a tile is two TMA box copies (the two K-halves, 64 elements x 128 rows each, written in the
        // 128-byte swizzle) that complete on the buffer's mbarrier; the ring runs up to four tiles ahead.
        if (lane == 0) {
            TcCursor cur(p, true);
            asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
            long long i = 0;
            for (; i < cur.total; ++i) {
                const uint32_t buf = (uint32_t)(i % kTcXBufs);
                if (!tc_wait(bar(kTcBarXEmpty + (int)buf), ((uint32_t)(i / kTcXBufs) & 1) ^ 1, s_abort, p.status)) break;
                const TcItem it = cur.next();
                {  // the tile's record for the epilogue, published by the arrival below
                    TcTileInfo info;
                    info.word0 = ((unsigned long long)it.slot0 * kGroup + (unsigned)(it.h % kGroup)) * 4ull;
                    info.row_lo = max(0, it.first - it.t0);
                    info.row_hi = it.store ? min(kTcTile, it.S - it.t0) : 0;
                    s_info[i % kTcInfoRing] = info;
                }
                const uint32_t full = bar(kTcBarXFull + (int)buf), dst = sbase + kTcOffX + buf * 2 * kTcBlockBytes;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(2 * kTcBlockBytes) : "memory");
                tc_tma_load(dst, &k_map, 0, (int)it.slot0, full);
                tc_tma_load(dst + kTcBlockBytes, &k_map, 64, (int)it.slot0, full);
            }
            // no copy is left in flight when the CTA ends (they have all landed unless the CTA gave up early)
            for (long long j = max(0ll, i - kTcXBufs); j < i; ++j)
                for (int spin = 0; spin < kTcSpinLimit && !tc_test(bar(kTcBarXFull + (int)(j % kTcXBufs)), (uint32_t)(j / kTcXBufs) & 1); ++spin) {}
        }
        __syncwarp();
    }

    // ---- release tensor memory ---------------------------------------------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kTcMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcTmemCols) : "memory");
    }
}

}  // namespace ha
