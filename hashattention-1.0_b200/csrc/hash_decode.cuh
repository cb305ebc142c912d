// Decode-time hash encoder: one CTA per (query head, side) evaluates the head's 3-layer MLP
// (128 -> 128 -> 128 -> 32, SiLU between, sign at the end) for the new query / new key of every
// sequence of its batch slice, packs the 32 sign bits with one warp ballot, and appends the
// new key's code (and the K / V rows) to the paged caches.
//
// Follows USA.q_embedding / USA.k_embedding with hard=True
// (hashattention/hashattention_llama.py:204-226) in fp32 arithmetic.
#pragma once

#include "common.cuh"

namespace ha {

constexpr int kHashDecodeThreads = 512;

struct HashDecodeParams {
    const __nv_bfloat16* q;      // [B][Hq][128]
    const __nv_bfloat16* k_new;  // [B][Hkv][128] or null (query side only)
    const __nv_bfloat16* v_new;  // [B][Hkv][128] or null
    const void* w[2];            // side 0 = query MLPs, side 1 = key MLPs
    const float* bias[2];
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    uint32_t* hash_pages;
    const int32_t* page_table;
    const int32_t* seq_lens;
    uint32_t* q_codes;   // [B][Hq]
    float* preact_dbg;   // [B][2][Hq][32] or null
    __nv_bfloat16* q_stage;  // [B][Hq][128] or null: a device copy of q for the attention kernels, written when
                             // q itself lives in mapped host memory (read once here instead of by every gather CTA)
    int32_t* status;
    int B, Hkv, max_pages, num_pages, batch_per_cta;
};

// Eight consecutive weights of one row, as stored, and their dot product with eight inputs.
template <typename WT>
struct Row8;

template <>
struct Row8<__nv_bfloat16> {
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
        raw = __ldg(reinterpret_cast<const uint4*>(p));
    }
    __device__ __forceinline__ float dot(const float (&x)[8]) const {
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
};

template <>
struct Row8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = __ldg(reinterpret_cast<const float4*>(p));
        b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    }
    __device__ __forceinline__ float dot(const float (&x)[8]) const {
        float s = a.x * x[0];
        s = fmaf(a.y, x[1], s);
        s = fmaf(a.z, x[2], s);
        s = fmaf(a.w, x[3], s);
        s = fmaf(b.x, x[4], s);
        s = fmaf(b.y, x[5], s);
        s = fmaf(b.z, x[6], s);
        s = fmaf(b.w, x[7], s);
        return s;
    }
};

__device__ __forceinline__ float half_warp_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

// Thread mapping: 16 warps; a half-warp (16 lanes x 8 columns) covers one 128-wide weight row.
// In the two hidden layers warp w owns output rows [8w, 8w+8): load j of a lane belongs to
// row 8w + 2j + (lane >> 4). In the last layer warp w owns rows 2w and 2w+1.
constexpr int kMlpWarps = kHashDecodeThreads / 32;   // 16
constexpr int kRowLoads = kHidden / kMlpWarps / 2;   // 4 loads per lane and hidden layer

// One head's MLP held in the registers of a 512-thread CTA.
template <typename WT>
struct MlpRegs {
    Row8<WT> w0[kRowLoads], w1[kRowLoads], w2;
    float b0[kRowLoads], b1[kRowLoads], b2;

    // All three layers are fetched back to back so that their DRAM latency is paid once.
    __device__ __forceinline__ void load(const WT* W, const float* bias, int warp, int half, int col) {
#pragma unroll
        for (int j = 0; j < kRowLoads; ++j) {
            const int row = warp * (2 * kRowLoads) + 2 * j + half;
            w0[j].load(W + row * kHeadDim + col);
            w1[j].load(W + kHidden * kHeadDim + row * kHidden + col);
        }
        w2.load(W + kHidden * kHeadDim + kHidden * kHidden + (warp * 2 + half) * kHidden + col);
#pragma unroll
        for (int j = 0; j < kRowLoads; ++j) {
            const int row = warp * (2 * kRowLoads) + 2 * j + half;
            b0[j] = __ldg(bias + row);
            b1[j] = __ldg(bias + kHidden + row);
        }
        b2 = __ldg(bias + 2 * kHidden + warp * 2 + half);
    }
};

struct MlpSmem {
    __align__(16) float h0[kHidden];
    __align__(16) float h1[kHidden];
    float out[kCodeBits];
};

__device__ __forceinline__ void load_x8(const float* s, float (&x)[8]) {
    const float4 lo = *reinterpret_cast<const float4*>(s);
    const float4 hi = *reinterpret_cast<const float4*>(s + 4);
    x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
    x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
}

// One hidden layer: every lane of a half-warp ends up with the kRowLoads row sums of its half;
// lane j of the half then applies bias + SiLU to row j and stores it (one SiLU per lane).
template <typename WT>
__device__ __forceinline__ void hidden_layer(const Row8<WT> (&w)[kRowLoads], const float (&bias)[kRowLoads],
                                             const float (&x)[8], float* dst, int warp, int lane) {
    const int half = lane >> 4, sub = lane & 15;
    float mine = 0.f;
#pragma unroll
    for (int j = 0; j < kRowLoads; ++j) {
        const float s = half_warp_sum(w[j].dot(x)) + bias[j];
        mine = sub == j ? s : mine;
    }
    if (sub < kRowLoads) dst[warp * (2 * kRowLoads) + 2 * sub + half] = silu(mine);
}

// Evaluates the MLP on one 128-element bf16 row, of which `raw` holds this lane's 8 elements
// (load_x_row). Must be called by all threads of the CTA; on
// return (after its last barrier) sm.out[0..32) holds the final-layer pre-activations.
// `between` runs after the first layer (a place to issue loads whose address depends on a value
// that was requested before the call). The caller may call mlp_eval again without a further
// barrier: each buffer is rewritten only after barriers that every reader of the previous
// round has passed.
template <typename WT, typename F>
__device__ __forceinline__ void mlp_eval(const MlpRegs<WT>& r, const uint4 raw,
                                         MlpSmem& sm, int warp, int lane, F&& between) {
    const int half = lane >> 4, col = (lane & 15) * 8;
    float x[8];
    {
        x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x);
        x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
        x[4] = bf16_lo(raw.z); x[5] = bf16_hi(raw.z);
        x[6] = bf16_lo(raw.w); x[7] = bf16_hi(raw.w);
    }
    hidden_layer(r.w0, r.b0, x, sm.h0, warp, lane);
    between();
    __syncthreads();
    load_x8(sm.h0 + col, x);
    hidden_layer(r.w1, r.b1, x, sm.h1, warp, lane);
    __syncthreads();
    load_x8(sm.h1 + col, x);
    {
        const float s = half_warp_sum(r.w2.dot(x)) + r.b2;
        if ((lane & 15) == 0) sm.out[warp * 2 + half] = s;
    }
    __syncthreads();
}

// This lane's 8 consecutive elements (columns 8 * (lane % 16) ...) of a 128-element bf16 row.
__device__ __forceinline__ uint4 load_x_row(const __nv_bfloat16* xrow, int lane) {
    return *reinterpret_cast<const uint4*>(xrow + (lane & 15) * 8);
}

template <typename WT>
__global__ void __launch_bounds__(kHashDecodeThreads)
hash_decode_kernel(const HashDecodeParams p) {
    HA_TL(kTlHashDecode, kTlEntry);
    const int h = blockIdx.x;                // query head whose MLP this CTA evaluates
    const int side = blockIdx.y;             // 0 = query net, 1 = key net
    const int Hq = p.Hkv * kGroup;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    MlpRegs<WT> regs;
    regs.load(static_cast<const WT*>(p.w[side]) + (size_t)h * kMlpElems,
              p.bias[side] + (size_t)h * kMlpBias, warp, lane >> 4, (lane & 15) * 8);
    __shared__ MlpSmem sm;

    pdl_wait();
    HA_TL(kTlHashDecode, kTlAfterWait);
    pdl_launch_dependents();

    const int b_begin = blockIdx.z * p.batch_per_cta;
    const int b_end = min(p.B, b_begin + p.batch_per_cta);
    const int kvh = h / kGroup, g = h % kGroup;

    // The input row and (key side) the sequence length of the next sequence are requested while the
    // current one is evaluated; the page-table entry of the append slot, whose address depends on
    // the length, is fetched underneath the MLP arithmetic.
    auto x_row = [&](int b) {
        return side == 0 ? p.q + ((size_t)b * Hq + h) * kHeadDim : p.k_new + ((size_t)b * p.Hkv + kvh) * kHeadDim;
    };
    uint4 raw_next = make_uint4(0u, 0u, 0u, 0u);
    int S_next = 1;
    if (b_begin < b_end) {
        raw_next = load_x_row(x_row(b_begin), lane);
        if (side == 1) S_next = p.seq_lens[b_begin];
    }
    for (int b = b_begin; b < b_end; ++b) {
        const uint4 raw = raw_next;
        const int S = S_next;
        if (b + 1 < b_end) {
            raw_next = load_x_row(x_row(b + 1), lane);
            if (side == 1) S_next = p.seq_lens[b + 1];
        }
        if (side == 0 && p.q_stage != nullptr && warp == 0 && lane < 16)
            *reinterpret_cast<uint4*>(p.q_stage + ((size_t)b * Hq + h) * kHeadDim + lane * 8) = raw;
        int page = 0;
        mlp_eval(regs, raw, sm, warp, lane, [&] {
            if (side == 1) {
                const int pidx = min(max(S - 1, 0) / kPage, p.max_pages - 1);
                page = p.page_table[(size_t)b * p.max_pages + pidx];
            }
        });
        if (warp != 0) continue;

        const float pre = sm.out[lane];
        // bit i = 1 iff output i > 0 (efficiency/kernels/torchatt.py:35-36: relu(sign(x)))
        const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.0f);
        if (p.preact_dbg != nullptr)
            p.preact_dbg[(((size_t)b * 2 + side) * Hq + h) * kCodeBits + lane] = pre;
        if (side == 0) {
            if (lane == 0) p.q_codes[(size_t)b * Hq + h] = code;
            continue;
        }
        if (S < 1 || S > p.max_pages * kPage) {
            if (lane == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
            continue;
        }
        const int tok = S - 1;
        if (page < 0 || page >= p.num_pages) {
            if (lane == 0) report(p.status, HA_ERR_BAD_PAGE);
            continue;
        }
        const size_t slot = ((size_t)page * p.Hkv + kvh) * kPage + tok % kPage;
        if (lane == 0) p.hash_pages[slot * kGroup + g] = code;
        // the group's first head also appends the K and V rows (256 B each)
        if (g == 0 && p.v_new != nullptr) {
            const size_t src = ((size_t)b * p.Hkv + kvh) * kHeadDim;
            const uint4* s = lane < 16 ? reinterpret_cast<const uint4*>(p.k_new + src) + lane
                                       : reinterpret_cast<const uint4*>(p.v_new + src) + (lane - 16);
            uint4* d = lane < 16 ? reinterpret_cast<uint4*>(p.k_pages + slot * kHeadDim) + lane
                                 : reinterpret_cast<uint4*>(p.v_pages + slot * kHeadDim) + (lane - 16);
            *d = *s;
        }
    }
    HA_TL(kTlHashDecode, kTlExit);
}

// Prefill key-hash build on the CUDA cores, exact fp32 arithmetic: CTA (h, page, b) keeps the
// key MLP of query head h in registers and walks the tokens of one cache page.
// Follows USA.k_embedding(hard=True) over the cached keys
// (hashattention/hashattention_llama.py:204-214).
struct HashPrefillParams {
    const __nv_bfloat16* k_pages;
    uint32_t* hash_pages;
    const void* wk;
    const float* bk;
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* first_token;  // [B] or null
    int32_t* status;
    int B, Hkv, max_pages, num_pages;
};

template <typename WT>
__global__ void __launch_bounds__(kHashDecodeThreads)
hash_prefill_simt_kernel(const HashPrefillParams p) {
    const int h = blockIdx.x, pg = blockIdx.y, b = blockIdx.z;
    const int kvh = h / kGroup, g = h % kGroup;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int S = p.seq_lens[b];  // 0 is legal here: nothing cached yet, nothing to encode
    if (S < 0 || S > p.max_pages * kPage) {
        if (tid == 0 && h == 0 && pg == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
        return;
    }
    const int first = p.first_token != nullptr ? max(0, p.first_token[b]) : 0;
    const int t_begin = max(pg * kPage, first), t_end = min((pg + 1) * kPage, S);
    if (t_begin >= t_end) return;
    const int page = p.page_table[(size_t)b * p.max_pages + pg];
    if (page < 0 || page >= p.num_pages) {
        if (tid == 0) report(p.status, HA_ERR_BAD_PAGE);
        return;
    }

    MlpRegs<WT> regs;
    regs.load(static_cast<const WT*>(p.wk) + (size_t)h * kMlpElems, p.bk + (size_t)h * kMlpBias,
              warp, lane >> 4, (lane & 15) * 8);
    __shared__ MlpSmem sm;
    pdl_wait();  // the keys may have been written by the kernel before this one

    const size_t slot0 = ((size_t)page * p.Hkv + kvh) * kPage;
    uint4 raw_next = load_x_row(p.k_pages + (slot0 + t_begin % kPage) * kHeadDim, lane);
    for (int t = t_begin; t < t_end; ++t) {
        const size_t slot = slot0 + t % kPage;
        const uint4 raw = raw_next;  // the next token's row is requested while this one is evaluated
        if (t + 1 < t_end) raw_next = load_x_row(p.k_pages + (slot + 1) * kHeadDim, lane);
        mlp_eval(regs, raw, sm, warp, lane, [] {});
        if (warp == 0) {
            const float pre = sm.out[lane];
            const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.0f);
            if (lane == 0) p.hash_pages[slot * kGroup + g] = code;
        }
    }
}

}  // namespace ha
