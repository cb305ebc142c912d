// The LSH baseline of the reference (lth_num_layers == 0, hashattention/hashattention_llama.py:75-84 and 130-139):
// one random projection per query head, shared by keys and queries,
//     code = signbits( W . [x, sqrt(relu(M^2 - |x|^2))] + b ),   W: 32 x 129,
// where M = 1e-3 + the largest norm among ALL vectors of the call for that head (IpToCS.forward: norm.max() over
// batch and positions). For the keys that is the largest key norm of the kv-head's whole cache, over every
// sequence of the batch - the reference re-hashes all keys on every step, so a key's code changes whenever a
// longer key arrives anywhere in the batch. Here the codes are cached like those of the learned hash functions,
// together with the largest key norm seen per kv-head (m); a step whose new keys raise m re-hashes that kv-head's
// cache (rare: m only grows), every other step encodes the new token alone. For the queries M is taken over the
// batch of the step.
//
// State per cache, behind ha_hash_weights_t.lsh_state: float m[Hkv], then int stale[Hkv] (set by a step that raised
// m, consumed by the re-hash kernel of the same step, rewritten by the next step).
//
// Weight layout (the common one, include/hashattn.h): columns 0..127 of W in the W2 slot ([32][128]), column 128 in
// the first 32 entries of the b0 slot, b in the b2 slot. Plain fp32 arithmetic on the CUDA cores: the mode is a
// baseline, one 129 x 32 product per vector.
#pragma once

#include "common.cuh"

namespace ha {

constexpr int kLshThreads = 128;
constexpr float kLshMargin = 1e-3f;  // IpToCS: M = norm.max() + 1e-3

struct LshParams {
    const __nv_bfloat16* q;      // [B][Hq][128]
    const __nv_bfloat16* k_new;  // [B][Hkv][128] or null (query-only encode)
    const __nv_bfloat16* v_new;  // or null
    const void* w;               // [Hq][36864] (W2 slot used)
    const float* bias;           // [Hq][288]
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    uint32_t* hash_pages;
    const int32_t* page_table;
    const int32_t* seq_lens;
    uint32_t* q_codes;           // [B][Hq]
    float* preact_dbg;           // [B][2][Hq][32] or null
    __nv_bfloat16* q_stage;      // [B][Hq][128] or null
    float* m;                    // [Hkv] largest key norm of the cache
    int32_t* stale;              // [Hkv]
    int32_t* status;
    int B, Hkv, max_pages, num_pages;
    int only_if_stale;           // lsh_hash_keys_kernel: 1 = re-hash pass of a decode step
};

template <typename WT>
__device__ __forceinline__ float lsh_w(const WT* w, int i);
template <>
__device__ __forceinline__ float lsh_w<float>(const float* w, int i) { return __ldg(w + i); }
template <>
__device__ __forceinline__ float lsh_w<__nv_bfloat16>(const __nv_bfloat16* w, int i) {
    return __bfloat162float(w[i]);
}

// |x|^2 of a 128-element bf16 row, all lanes of the warp get the sum; x4: this lane's elements 4 lane .. 4 lane + 3
__device__ __forceinline__ float lsh_row_norm2(const __nv_bfloat16* row, int lane, float (&x4)[4]) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(row) + lane);
    x4[0] = bf16_lo(raw.x); x4[1] = bf16_hi(raw.x); x4[2] = bf16_lo(raw.y); x4[3] = bf16_hi(raw.y);
    float s = x4[0] * x4[0] + x4[1] * x4[1] + x4[2] * x4[2] + x4[3] * x4[3];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    return s;
}

// max of non-negative floats through their bit patterns
__device__ __forceinline__ void lsh_atomic_max(float* addr, float v) { atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v)); }

// Output `lane` of head h for the vector in shared memory xs[0..127] with extra coordinate `extra`.
template <typename WT>
__device__ __forceinline__ float lsh_output(const LshParams& p, int h, int lane, const float* xs, float extra) {
    const WT* W = static_cast<const WT*>(p.w) + (size_t)h * kMlpElems + kHidden * kHeadDim + kHidden * kHidden + lane * kHeadDim;
    const float* bias = p.bias + (size_t)h * kMlpBias;
    float acc = 0.f;
#pragma unroll 8
    for (int d = 0; d < kHeadDim; ++d) acc = fmaf(lsh_w<WT>(W, d), xs[d], acc);
    return acc + bias[lane] * extra + bias[2 * kHidden + lane];
}

// Decode step: query codes of every head, and (key side) the new token's codes, K / V rows and the kv-head's largest
// key norm. Grid (Hkv, B), 128 threads: warp g serves query head 4 kvh + g.
template <typename WT>
__global__ void __launch_bounds__(kLshThreads) lsh_encode_kernel(const LshParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int kvh = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, g = tid >> 5;
    const int Hq = p.Hkv * kGroup, h = kvh * kGroup + g;
    __shared__ float s_x[kGroup][kHeadDim];   // q of head g, later the new key (all warps the same)
    __shared__ float s_qmax[kGroup];          // largest |q| of head g over the batch
    __shared__ float s_kmax;                  // largest |k_new| of the kv-head over the batch
    if (tid < kGroup) s_qmax[tid] = 0.f;
    if (tid == 0) s_kmax = 0.f;
    __syncthreads();
    float x4[4];
    // norms over the batch: IpToCS takes the maximum over every vector of the call
    for (int bb = 0; bb < p.B; ++bb) {
        const float n2 = lsh_row_norm2(p.q + ((size_t)bb * Hq + h) * kHeadDim, lane, x4);
        if (lane == 0) lsh_atomic_max(&s_qmax[g], sqrtf(n2));
    }
    if (p.k_new != nullptr)
        for (int bb = g; bb < p.B; bb += kGroup) {
            const float n2 = lsh_row_norm2(p.k_new + ((size_t)bb * p.Hkv + kvh) * kHeadDim, lane, x4);
            if (lane == 0) lsh_atomic_max(&s_kmax, sqrtf(n2));
        }
    // this warp's query
    const __nv_bfloat16* qrow = p.q + ((size_t)b * Hq + h) * kHeadDim;
    const float qn2 = lsh_row_norm2(qrow, lane, x4);
#pragma unroll
    for (int i = 0; i < 4; ++i) s_x[g][4 * lane + i] = x4[i];
    if (p.q_stage != nullptr)
        reinterpret_cast<uint2*>(p.q_stage + ((size_t)b * Hq + h) * kHeadDim)[lane] = __ldg(reinterpret_cast<const uint2*>(qrow) + lane);
    __syncthreads();
    {
        const float M = s_qmax[g] + kLshMargin;
        const float pre = lsh_output<WT>(p, h, lane, s_x[g], sqrtf(fmaxf(M * M - qn2, 0.f)));
        const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.f);
        if (lane == 0) p.q_codes[(size_t)b * Hq + h] = code;
        if (p.preact_dbg != nullptr) p.preact_dbg[(((size_t)b * 2 + 0) * Hq + h) * kCodeBits + lane] = pre;
    }
    if (p.k_new == nullptr) return;

    // ---- key side: the new token of sequence b
    const int S = p.seq_lens[b];
    if (S < 1 || S > p.max_pages * kPage) {
        if (tid == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
        return;
    }
    const int t = S - 1, page = __ldg(p.page_table + (size_t)b * p.max_pages + t / kPage);
    if (page < 0 || page >= p.num_pages) {
        if (tid == 0) report(p.status, HA_ERR_BAD_PAGE);
        return;
    }
    const float m_old = *reinterpret_cast<volatile float*>(p.m + kvh);  // (a CTA may see this step's value already: same result)
    const float m_new = fmaxf(m_old, s_kmax);
    if (b == 0 && tid == 0) {  // one CTA per kv-head records the step's outcome
        p.stale[kvh] = m_new > m_old ? 1 : 0;
        p.m[kvh] = m_new;
    }
    const size_t slot = ((size_t)page * p.Hkv + kvh) * kPage + t % kPage;
    const __nv_bfloat16* krow = p.k_new + ((size_t)b * p.Hkv + kvh) * kHeadDim;
    __syncthreads();  // the queries in s_x have been read
    const float kn2 = lsh_row_norm2(krow, lane, x4);
#pragma unroll
    for (int i = 0; i < 4; ++i) s_x[g][4 * lane + i] = x4[i];
    if (g == 0) {  // append the rows
        reinterpret_cast<uint2*>(p.k_pages + slot * kHeadDim)[lane] = __ldg(reinterpret_cast<const uint2*>(krow) + lane);
        if (p.v_new != nullptr)
            reinterpret_cast<uint2*>(p.v_pages + slot * kHeadDim)[lane] =
                __ldg(reinterpret_cast<const uint2*>(p.v_new + ((size_t)b * p.Hkv + kvh) * kHeadDim) + lane);
    }
    __syncwarp();
    const float M = m_new + kLshMargin;
    const float pre = lsh_output<WT>(p, h, lane, s_x[g], sqrtf(fmaxf(M * M - kn2, 0.f)));
    const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.f);
    if (lane == 0) p.hash_pages[slot * kGroup + g] = code;
    if (p.preact_dbg != nullptr) p.preact_dbg[(((size_t)b * 2 + 1) * Hq + h) * kCodeBits + lane] = pre;
}

// Largest key norm per kv-head over the whole cache (prefill). Grid (max_pages, Hkv, B), 128 threads; m starts at 0.
__global__ void __launch_bounds__(kLshThreads) lsh_norm_max_kernel(const LshParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int pg = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int S = p.seq_lens[b];
    if (S < 0 || S > p.max_pages * kPage) {
        if (threadIdx.x == 0 && pg == 0 && kvh == 0) report(p.status, HA_ERR_BAD_SEQ_LEN);
        return;
    }
    const int t0 = pg * kPage;
    if (t0 >= S) return;
    const int page = __ldg(p.page_table + (size_t)b * p.max_pages + pg);
    if (page < 0 || page >= p.num_pages) {
        if (threadIdx.x == 0) report(p.status, HA_ERR_BAD_PAGE);
        return;
    }
    const __nv_bfloat16* rows = p.k_pages + ((size_t)page * p.Hkv + kvh) * kPage * kHeadDim;
    float best = 0.f, x4[4];
    for (int r = warp; r < min(kPage, S - t0); r += kLshThreads / 32) best = fmaxf(best, lsh_row_norm2(rows + (size_t)r * kHeadDim, lane, x4));
    if (lane == 0 && best > 0.f) lsh_atomic_max(p.m + kvh, sqrtf(best));
}

// Codes of every cached key of a page (prefill, or the re-hash of a step that raised m). Grid (max_pages, Hkv, B),
// 128 threads: warp g = query head 4 kvh + g walks the page's tokens; its 32 x 128 weights sit transposed in shared
// memory ([input][output]: lane = output, conflict-free), 64 KB per CTA.
constexpr uint32_t kLshSmemBytes = kGroup * kHeadDim * kCodeBits * sizeof(float);

template <typename WT>
__global__ void __launch_bounds__(kLshThreads) lsh_hash_keys_kernel(const LshParams p) {
    extern __shared__ float s_w[];  // [4 heads][128 inputs][32 outputs]
    // No early start for the kernel behind this one: the scoring kernel reads hash words ahead of its dependency wait
    // (it expects only the newest token to change under it), and a re-hash rewrites them all.
    pdl_wait();
    const int pg = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, g = tid >> 5;
    if (p.only_if_stale && *reinterpret_cast<volatile int32_t*>(p.stale + kvh) == 0) return;
    const int S = p.seq_lens[b];
    if (S < 0 || S > p.max_pages * kPage) return;  // (reported by the kernel that ran before)
    const int t0 = pg * kPage;
    if (t0 >= S) return;
    const int page = __ldg(p.page_table + (size_t)b * p.max_pages + pg);
    if (page < 0 || page >= p.num_pages) {
        if (tid == 0) report(p.status, HA_ERR_BAD_PAGE);
        return;
    }
    __shared__ float s_x[kGroup][kHeadDim];
    const int h = kvh * kGroup + g;
    float* w = s_w + g * kHeadDim * kCodeBits;
    {
        const WT* W = static_cast<const WT*>(p.w) + (size_t)h * kMlpElems + kHidden * kHeadDim + kHidden * kHidden;
        for (int i = lane; i < kCodeBits * kHeadDim; i += 32) w[(i % kHeadDim) * kCodeBits + i / kHeadDim] = lsh_w<WT>(W, i);
    }
    const float* bias = p.bias + (size_t)h * kMlpBias;
    const float w_last = bias[lane], b_out = bias[2 * kHidden + lane];
    const float M = *reinterpret_cast<volatile float*>(p.m + kvh) + kLshMargin;
    const size_t slot0 = ((size_t)page * p.Hkv + kvh) * kPage;
    const int n = min(kPage, S - t0);
    for (int r = 0; r < n; ++r) {
        float x4[4];
        const float n2 = lsh_row_norm2(p.k_pages + (slot0 + r) * kHeadDim, lane, x4);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) s_x[g][4 * lane + i] = x4[i];
        __syncwarp();
        float acc = 0.f;  // the same order of additions as lsh_output
#pragma unroll 8
        for (int d = 0; d < kHeadDim; ++d) acc = fmaf(w[d * kCodeBits + lane], s_x[g][d], acc);
        const float pre = acc + w_last * sqrtf(fmaxf(M * M - n2, 0.f)) + b_out;
        const uint32_t code = __ballot_sync(0xffffffffu, pre > 0.f);
        if (lane == 0) p.hash_pages[(slot0 + r) * kGroup + g] = code;
    }
}

}  // namespace ha
