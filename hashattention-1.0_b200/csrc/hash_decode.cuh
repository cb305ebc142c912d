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
    int layers;          // 3, 2 or 1 Linear layers (see ha_hash_weights_t.num_layers)
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
    __device__ __forceinline__ void unpack(float (&e)[8]) const {
        e[0] = bf16_lo(raw.x); e[1] = bf16_hi(raw.x); e[2] = bf16_lo(raw.y); e[3] = bf16_hi(raw.y);
        e[4] = bf16_lo(raw.z); e[5] = bf16_hi(raw.z); e[6] = bf16_lo(raw.w); e[7] = bf16_hi(raw.w);
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
    __device__ __forceinline__ void unpack(float (&e)[8]) const {
        e[0] = a.x; e[1] = a.y; e[2] = a.z; e[3] = a.w;
        e[4] = b.x; e[5] = b.y; e[6] = b.z; e[7] = b.w;
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
//
// layers: 3 = all of W0, W1, W2; 2 = W0 then W2 (Linear-SiLU-Linear, hashattention_llama.py:112-120);
// 1 = W2 alone (:121-127).
template <typename WT, typename F>
__device__ __forceinline__ void mlp_eval(const MlpRegs<WT>& r, const uint4 raw,
                                         MlpSmem& sm, int warp, int lane, F&& between, int layers = 3) {
    const int half = lane >> 4, col = (lane & 15) * 8;
    float x[8];
    {
        x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x);
        x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
        x[4] = bf16_lo(raw.z); x[5] = bf16_hi(raw.z);
        x[6] = bf16_lo(raw.w); x[7] = bf16_hi(raw.w);
    }
    if (layers >= 2) hidden_layer(r.w0, r.b0, x, sm.h0, warp, lane);
    between();
    if (layers >= 2) {
        __syncthreads();
        load_x8(sm.h0 + col, x);
    } else {
        __syncthreads();  // no hidden layer separates this call's write of `out` from the previous call's readers
    }
    if (layers == 3) {
        hidden_layer(r.w1, r.b1, x, sm.h1, warp, lane);
        __syncthreads();
        load_x8(sm.h1 + col, x);
    }
    {
        const float s = half_warp_sum(r.w2.dot(x)) + r.b2;
        if ((lane & 15) == 0) sm.out[warp * 2 + half] = s;
    }
    __syncthreads();
}

// mlp_eval for two rows at once (`sm[0]`, `sm[1]`): the same weights in registers feed both rows, and the two
// dependent chains (dot, shuffle reduction, SiLU, barrier) interleave, so the pair costs little more than one row.
template <typename WT>
__device__ __forceinline__ void hidden_layer2(const Row8<WT> (&w)[kRowLoads], const float (&bias)[kRowLoads],
                                              const float (&xa)[8], const float (&xb)[8], float* da, float* db,
                                              int warp, int lane) {
    const int half = lane >> 4, sub = lane & 15;
    float ma = 0.f, mb = 0.f;
#pragma unroll
    for (int j = 0; j < kRowLoads; ++j) {
        const float sa = half_warp_sum(w[j].dot(xa)) + bias[j];
        const float sb = half_warp_sum(w[j].dot(xb)) + bias[j];
        ma = sub == j ? sa : ma;
        mb = sub == j ? sb : mb;
    }
    if (sub < kRowLoads) {
        da[warp * (2 * kRowLoads) + 2 * sub + half] = silu(ma);
        db[warp * (2 * kRowLoads) + 2 * sub + half] = silu(mb);
    }
}

__device__ __forceinline__ void unpack_x8(const uint4 raw, float (&x)[8]) {
    x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x);
    x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
    x[4] = bf16_lo(raw.z); x[5] = bf16_hi(raw.z);
    x[6] = bf16_lo(raw.w); x[7] = bf16_hi(raw.w);
}

template <typename WT, typename F>
__device__ __forceinline__ void mlp_eval2(const MlpRegs<WT>& r, const uint4 raw_a, const uint4 raw_b,
                                          MlpSmem (&sm)[2], int warp, int lane, F&& between, int layers = 3) {
    const int half = lane >> 4, col = (lane & 15) * 8;
    float xa[8], xb[8];
    unpack_x8(raw_a, xa);
    unpack_x8(raw_b, xb);
    if (layers >= 2) hidden_layer2(r.w0, r.b0, xa, xb, sm[0].h0, sm[1].h0, warp, lane);
    between();
    __syncthreads();
    if (layers >= 2) {
        load_x8(sm[0].h0 + col, xa);
        load_x8(sm[1].h0 + col, xb);
    }
    if (layers == 3) {
        hidden_layer2(r.w1, r.b1, xa, xb, sm[0].h1, sm[1].h1, warp, lane);
        __syncthreads();
        load_x8(sm[0].h1 + col, xa);
        load_x8(sm[1].h1 + col, xb);
    }
    {
        const float sa = half_warp_sum(r.w2.dot(xa)) + r.b2;
        const float sb = half_warp_sum(r.w2.dot(xb)) + r.b2;
        if ((lane & 15) == 0) {
            sm[0].out[warp * 2 + half] = sa;
            sm[1].out[warp * 2 + half] = sb;
        }
    }
    __syncthreads();
}

// This lane's 8 consecutive elements (columns 8 * (lane % 16) ...) of a 128-element bf16 row.
__device__ __forceinline__ uint4 load_x_row(const __nv_bfloat16* xrow, int lane) {
    return *reinterpret_cast<const uint4*>(xrow + (lane & 15) * 8);
}

// kPairs: a CTA with two or more sequences evaluates them two at a time; with one sequence per CTA the
// single-row loop is a little leaner.
template <typename WT, bool kPairs>
__global__ void __launch_bounds__(kHashDecodeThreads)
hash_decode_kernel(const HashDecodeParams p) {
    const int h = blockIdx.x;                // query head whose MLP this CTA evaluates
    const int side = blockIdx.y;             // 0 = query net, 1 = key net
    const int Hq = p.Hkv * kGroup;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    MlpRegs<WT> regs;
    regs.load(static_cast<const WT*>(p.w[side]) + (size_t)h * kMlpElems,
              p.bias[side] + (size_t)h * kMlpBias, warp, lane >> 4, (lane & 15) * 8);
    __shared__ MlpSmem sm[2];

    const int b_begin = blockIdx.z * p.batch_per_cta;
    const int b_end = min(p.B, b_begin + p.batch_per_cta);
    const int kvh = h / kGroup, g = h % kGroup;

    // The input rows may be products of the kernel in front, so they are read after the wait; asking L2 for their
    // lines beforehand is harmless either way (L2 is where that kernel's stores land) and saves the DRAM trip when
    // the rows were written long ago. Not for rows in mapped host memory (q_stage given), which L2 does not hold.
    if (p.q_stage == nullptr) {
        for (int i = tid; i < 2 * (b_end - b_begin); i += kHashDecodeThreads) {
            const int b = b_begin + (i >> 1);
            const __nv_bfloat16* row = side == 0 ? p.q + ((size_t)b * Hq + h) * kHeadDim
                                                 : p.k_new + ((size_t)b * p.Hkv + kvh) * kHeadDim;
            prefetch_l2(row + (i & 1) * (kHeadDim / 2));
            if (side == 1 && g == 0 && p.v_new != nullptr)
                prefetch_l2(p.v_new + ((size_t)b * p.Hkv + kvh) * kHeadDim + (i & 1) * (kHeadDim / 2));
        }
    }

    pdl_wait();
    pdl_launch_dependents();

    if constexpr (kPairs) {
        // The sequences of this CTA are evaluated two at a time (the pair shares every weight register and its two
        // dependent chains interleave); the input rows, the V rows of the append and (key side) the sequence lengths
        // of a pair are requested together, the page-table entries of the append slots underneath the MLP arithmetic.
        auto x_row = [&](int b) {
            return side == 0 ? p.q + ((size_t)b * Hq + h) * kHeadDim : p.k_new + ((size_t)b * p.Hkv + kvh) * kHeadDim;
        };
        // The group's first key head also appends the K and V rows: lanes 0-15 of warp 0 hold the K row already (it
        // is the MLP's input), lanes 16-31 request the V row together with it - the inputs may live in mapped
        // host memory, where a second read at the end of the kernel would cost another trip over the bus.
        const bool appends = side == 1 && g == 0 && p.v_new != nullptr && warp == 0;
        auto v_part = [&](int b) {
            return *(reinterpret_cast<const uint4*>(p.v_new + ((size_t)b * p.Hkv + kvh) * kHeadDim) + (lane - 16));
        };
        // what warp 0 does with a finished row: code out, and (key side) the append
        auto finish = [&](int b, const MlpSmem& m, const uint4 raw, const uint4 v_raw, int S, int page) {
            const float pre = m.out[lane];
            // bit i = 1 iff output i > 0 (efficiency/kernels/torchatt.py:35-36: relu(sign(x)))
            const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.0f);
            if (p.preact_dbg != nullptr)
                p.preact_dbg[(((size_t)b * 2 + side) * Hq + h) * kCodeBits + lane] = pre;
            if (side == 0) {
                if (lane == 0) p.q_codes[(size_t)b * Hq + h] = code;
                return;
            }
            if (S < 1 || S > p.max_pages * kPage) {
                if (lane == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
                return;
            }
            if (page < 0 || page >= p.num_pages) {
                if (lane == 0) report(p.status, HA_ERR_BAD_PAGE);
                return;
            }
            const size_t slot = ((size_t)page * p.Hkv + kvh) * kPage + (S - 1) % kPage;
            if (lane == 0) p.hash_pages[slot * kGroup + g] = code;
            // the group's first head also appends the K and V rows (256 B each)
            if (appends) {
                uint4* d = lane < 16 ? reinterpret_cast<uint4*>(p.k_pages + slot * kHeadDim) + lane
                                     : reinterpret_cast<uint4*>(p.v_pages + slot * kHeadDim) + (lane - 16);
                *d = lane < 16 ? raw : v_raw;
            }
        };
        auto page_of = [&](int b, int S) {
            return p.page_table[(size_t)b * p.max_pages + min(max(S - 1, 0) / kPage, p.max_pages - 1)];
        };
        for (int b = b_begin; b < b_end; b += 2) {
            const bool two = b + 1 < b_end;
            const int b1 = two ? b + 1 : b;
            const uint4 raw0 = load_x_row(x_row(b), lane), raw1 = load_x_row(x_row(b1), lane);
            uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
            if (appends && lane >= 16) {
                v0 = v_part(b);
                v1 = v_part(b1);
            }
            int S0 = 1, S1 = 1, page0 = 0, page1 = 0;
            if (side == 1) {
                S0 = p.seq_lens[b];
                S1 = p.seq_lens[b1];
            }
            if (side == 0 && p.q_stage != nullptr && warp == 0 && lane < 16) {
                *reinterpret_cast<uint4*>(p.q_stage + ((size_t)b * Hq + h) * kHeadDim + lane * 8) = raw0;
                if (two) *reinterpret_cast<uint4*>(p.q_stage + ((size_t)b1 * Hq + h) * kHeadDim + lane * 8) = raw1;
            }
            if (two) {
                mlp_eval2(regs, raw0, raw1, sm, warp, lane, [&] {
                    if (side == 1) {
                        page0 = page_of(b, S0);
                        page1 = page_of(b1, S1);
                    }
                }, p.layers);
            } else {
                mlp_eval(regs, raw0, sm[0], warp, lane, [&] {
                    if (side == 1) page0 = page_of(b, S0);
                }, p.layers);
            }
            if (warp != 0) continue;
            finish(b, sm[0], raw0, v0, S0, page0);
            if (two) finish(b1, sm[1], raw1, v1, S1, page1);
        }
    } else {
        // The input row and (key side) the sequence length of the next sequence are requested while the
        // current one is evaluated; the page-table entry of the append slot, whose address depends on
        // the length, is fetched underneath the MLP arithmetic.
        auto x_row = [&](int b) {
            return side == 0 ? p.q + ((size_t)b * Hq + h) * kHeadDim : p.k_new + ((size_t)b * p.Hkv + kvh) * kHeadDim;
        };
        // The group's first key head also appends the K and V rows: lanes 0-15 of warp 0 hold the K row already (it
        // is the MLP's input), lanes 16-31 request the V row together with it - the inputs may live in mapped
        // host memory, where a second read at the end of the kernel would cost another trip over the bus.
        const bool appends = side == 1 && g == 0 && p.v_new != nullptr && warp == 0;
        auto v_part = [&](int b) {
            return *(reinterpret_cast<const uint4*>(p.v_new + ((size_t)b * p.Hkv + kvh) * kHeadDim) + (lane - 16));
        };
        uint4 raw_next = make_uint4(0u, 0u, 0u, 0u), v_next = make_uint4(0u, 0u, 0u, 0u);
        int S_next = 1;
        if (b_begin < b_end) {
            raw_next = load_x_row(x_row(b_begin), lane);
            if (appends && lane >= 16) v_next = v_part(b_begin);
            if (side == 1) S_next = p.seq_lens[b_begin];
        }
        for (int b = b_begin; b < b_end; ++b) {
            const uint4 raw = raw_next, v_raw = v_next;
            const int S = S_next;
            if (b + 1 < b_end) {
                raw_next = load_x_row(x_row(b + 1), lane);
                if (appends && lane >= 16) v_next = v_part(b + 1);
                if (side == 1) S_next = p.seq_lens[b + 1];
            }
            if (side == 0 && p.q_stage != nullptr && warp == 0 && lane < 16)
                *reinterpret_cast<uint4*>(p.q_stage + ((size_t)b * Hq + h) * kHeadDim + lane * 8) = raw;
            int page = 0;
            mlp_eval(regs, raw, sm[0], warp, lane, [&] {
                if (side == 1) {
                    const int pidx = min(max(S - 1, 0) / kPage, p.max_pages - 1);
                    page = p.page_table[(size_t)b * p.max_pages + pidx];
                }
            }, p.layers);
            if (warp != 0) continue;

            const float pre = sm[0].out[lane];
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
            if (appends) {
                uint4* d = lane < 16 ? reinterpret_cast<uint4*>(p.k_pages + slot * kHeadDim) + lane
                                     : reinterpret_cast<uint4*>(p.v_pages + slot * kHeadDim) + (lane - 16);
                *d = lane < 16 ? raw : v_raw;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Batched variant for large batches: a CTA evaluates up to 16 sequences of its (head, side) at
// once as three small GEMMs instead of one sequence after the other. The head's weights are
// converted to fp32 and stored transposed ([in][out]) in shared memory (144 KB); in a hidden layer
// warp w owns rows 4 (w % 4) .. +3 and the input slice 32 (w / 4) .. +31, lane l the outputs
// 4 l .. 4 l + 3: one 16-byte weight load feeds 16 FMAs (4 rows x 4 outputs). The four partial
// sums of an output are added, biased and passed through SiLU in a second sweep. In the last
// layer warp = row, lane = output bit, and the warp's ballot is the row's code, so the 16 rows
// finish (store / append) in parallel. Same arithmetic type (fp32 FMA) as the kernel above; the
// summation order differs, which only matters inside the |x| < 1e-5 band of the sign.
// ------------------------------------------------------------------------------------------
constexpr int kHdbRows = 16;   // sequences per CTA and pass
constexpr int kHdbKSplit = 4;  // input slices of a hidden layer
// Sequences per CTA from which the batched kernel is used: a pass costs about 8.5 us whatever the number of
// rows (weights to shared memory + three full GEMM sweeps), the register kernel 3.3 us + 1.5 us per further row.
constexpr int kHdbMinRows = 6;
struct HdbSmem {
    float wt0[kHeadDim][kHidden];    // layer 0, [in][out]
    float wt1[kHidden][kHidden];     // layer 1
    float wt2[kHidden][kCodeBits];   // layer 2
    float bias[kMlpBias];
    float x[2][kHdbRows][kHidden];   // activations, ping-pong
    float part[kHdbKSplit][kHdbRows][kHidden];
};
constexpr size_t kHdbSmemBytes = sizeof(HdbSmem);

template <typename WT>
__device__ __forceinline__ void hdb_load_weights(HdbSmem& sm, const WT* W, const float* bias, int tid) {
    // A load is 8 consecutive inputs of one output row; consecutive threads take consecutive output
    // rows of the same input chunk, so a warp's transposed stores hit 32 different banks. All nine
    // loads of a thread are issued before the first store.
    constexpr int kPer = kHidden * (kHeadDim / 8) / kHashDecodeThreads;  // 4 loads per thread and hidden layer
    static_assert(kPer * kHashDecodeThreads == kHidden * (kHeadDim / 8) && kCodeBits * (kHidden / 8) == kHashDecodeThreads,
                  "thread mapping of the weight transposition");
    const WT* W1 = W + kHidden * kHeadDim;
    const WT* W2 = W1 + kHidden * kHidden;
    Row8<WT> r0[kPer], r1[kPer], r2;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int idx = tid + j * kHashDecodeThreads, o = idx % kHidden, chunk = idx / kHidden;
        r0[j].load(W + (size_t)o * kHeadDim + chunk * 8);
        r1[j].load(W1 + (size_t)o * kHidden + chunk * 8);
    }
    r2.load(W2 + (size_t)(tid % kCodeBits) * kHidden + (tid / kCodeBits) * 8);
    for (int i = tid; i < kMlpBias; i += kHashDecodeThreads) sm.bias[i] = __ldg(bias + i);
    float e[8];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int idx = tid + j * kHashDecodeThreads, o = idx % kHidden, chunk = idx / kHidden;
        r0[j].unpack(e);
#pragma unroll
        for (int k = 0; k < 8; ++k) sm.wt0[chunk * 8 + k][o] = e[k];
        r1[j].unpack(e);
#pragma unroll
        for (int k = 0; k < 8; ++k) sm.wt1[chunk * 8 + k][o] = e[k];
    }
    r2.unpack(e);
#pragma unroll
    for (int k = 0; k < 8; ++k) sm.wt2[(tid / kCodeBits) * 8 + k][tid % kCodeBits] = e[k];
}

// One hidden layer for 16 rows: partial sums by (row group, input slice), then bias + SiLU.
__device__ __forceinline__ void hdb_hidden(HdbSmem& sm, const float (*wt)[kHidden], const float* bias, int cur,
                                           int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    const int rg = warp & 3, ks = warp >> 2;
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
#pragma unroll 8
    for (int ii = 0; ii < kHidden / kHdbKSplit; ++ii) {
        const int i = ks * (kHidden / kHdbKSplit) + ii;
        const float4 w4 = *reinterpret_cast<const float4*>(&wt[i][lane * 4]);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float xv = sm.x[cur][rg * 4 + r][i];  // broadcast
            acc[r][0] = fmaf(xv, w4.x, acc[r][0]);
            acc[r][1] = fmaf(xv, w4.y, acc[r][1]);
            acc[r][2] = fmaf(xv, w4.z, acc[r][2]);
            acc[r][3] = fmaf(xv, w4.w, acc[r][3]);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float4*>(&sm.part[ks][rg * 4 + r][lane * 4]) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    __syncthreads();
    {
        const int row = warp;  // 16 warps, 16 rows; lane l finishes outputs 4 l .. 4 l + 3
        float4 sum = *reinterpret_cast<const float4*>(&bias[lane * 4]);
#pragma unroll
        for (int k = 0; k < kHdbKSplit; ++k) {
            const float4 p4 = *reinterpret_cast<const float4*>(&sm.part[k][row][lane * 4]);
            sum.x += p4.x; sum.y += p4.y; sum.z += p4.z; sum.w += p4.w;
        }
        *reinterpret_cast<float4*>(&sm.x[cur ^ 1][row][lane * 4]) = make_float4(silu(sum.x), silu(sum.y), silu(sum.z), silu(sum.w));
    }
    __syncthreads();
}

template <typename WT>
__global__ void __launch_bounds__(kHashDecodeThreads, 1)
hash_decode_batched_kernel(const HashDecodeParams p) {
    extern __shared__ __align__(16) unsigned char hdb_raw[];
    HdbSmem& sm = *reinterpret_cast<HdbSmem*>(hdb_raw);
    const int h = blockIdx.x, side = blockIdx.y;
    const int Hq = p.Hkv * kGroup;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kvh = h / kGroup, g = h % kGroup;

    hdb_load_weights(sm, static_cast<const WT*>(p.w[side]) + (size_t)h * kMlpElems, p.bias[side] + (size_t)h * kMlpBias, tid);

    pdl_wait();
    pdl_launch_dependents();

    const int b_begin = blockIdx.z * p.batch_per_cta;
    const int b_end = min(p.B, b_begin + p.batch_per_cta);
    for (int b0 = b_begin; b0 < b_end; b0 += kHdbRows) {
        // ---- this warp's row: the sequence's input row (4 elements per lane) and, key side, its append slot
        const int b = b0 + warp;
        const bool live = b < b_end;
        int S = 1, page = 0;
        // the rows the group's first key head appends (lanes 0-15: K, 16-31: V), requested with the inputs
        const bool appends = live && side == 1 && g == 0 && p.v_new != nullptr;
        uint4 app = make_uint4(0u, 0u, 0u, 0u);
        if (appends) {
            const size_t src = ((size_t)b * p.Hkv + kvh) * kHeadDim;
            app = lane < 16 ? *(reinterpret_cast<const uint4*>(p.k_new + src) + lane)
                            : *(reinterpret_cast<const uint4*>(p.v_new + src) + (lane - 16));
        }
        {
            float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live) {
                const __nv_bfloat16* xrow = side == 0 ? p.q + ((size_t)b * Hq + h) * kHeadDim
                                                      : p.k_new + ((size_t)b * p.Hkv + kvh) * kHeadDim;
                const uint2 raw = *reinterpret_cast<const uint2*>(xrow + lane * 4);
                xv = make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
                if (side == 0 && p.q_stage != nullptr)
                    *reinterpret_cast<uint2*>(p.q_stage + ((size_t)b * Hq + h) * kHeadDim + lane * 4) = raw;
                if (side == 1) {
                    S = p.seq_lens[b];
                    page = p.page_table[(size_t)b * p.max_pages + min(max(S - 1, 0) / kPage, p.max_pages - 1)];
                }
            }
            *reinterpret_cast<float4*>(&sm.x[0][warp][lane * 4]) = xv;
        }
        __syncthreads();  // inputs (and, in the first pass, the weights) are in shared memory
        int cur = 0;  // which of the two activation buffers holds the input of the next layer
        if (p.layers >= 2) {
            hdb_hidden(sm, sm.wt0, sm.bias, cur, tid);
            cur ^= 1;
        }
        if (p.layers == 3) {
            hdb_hidden(sm, sm.wt1, sm.bias + kHidden, cur, tid);
            cur ^= 1;
        }
        // ---- last layer: warp = row, lane = output bit
        float pre = sm.bias[2 * kHidden + lane];
#pragma unroll 16
        for (int i = 0; i < kHidden; ++i) pre = fmaf(sm.x[cur][warp][i], sm.wt2[i][lane], pre);
        // bit i = 1 iff output i > 0 (efficiency/kernels/torchatt.py:35-36: relu(sign(x)))
        const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.0f);
        __syncthreads();  // the activation buffers are rewritten by the next pass
        if (!live) continue;
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
        if (page < 0 || page >= p.num_pages) {
            if (lane == 0) report(p.status, HA_ERR_BAD_PAGE);
            continue;
        }
        const size_t slot = ((size_t)page * p.Hkv + kvh) * kPage + (S - 1) % kPage;
        if (lane == 0) p.hash_pages[slot * kGroup + g] = code;
        if (appends) {  // 256 B each
            uint4* dp = lane < 16 ? reinterpret_cast<uint4*>(p.k_pages + slot * kHeadDim) + lane
                                  : reinterpret_cast<uint4*>(p.v_pages + slot * kHeadDim) + (lane - 16);
            *dp = app;
        }
    }
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
    int layers;  // 3, 2 or 1 Linear layers
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
        mlp_eval(regs, raw, sm, warp, lane, [] {}, p.layers);
        if (warp == 0) {
            const float pre = sm.out[lane];
            const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.0f);
            if (lane == 0) p.hash_pages[slot * kGroup + g] = code;
        }
    }
}

}  // namespace ha
