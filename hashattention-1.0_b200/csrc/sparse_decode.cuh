// Sparse GQA flash-decode over the selected rows of the paged K / V cache.
//
// For query head h of sequence b the attended rows are, in this order, the sink tokens
// [0, lo), the heavy tokens sel_idx[b][h][0..cnt) and the recent tokens [hi, S). The rows are
// cut into splits of 128; one CTA handles one (b, h, split): each of its 16 half-warps gathers
// 8 rows of K and V straight into registers (sixteen 16-byte loads in flight per lane),
// computes the scaled dot products with shuffles, and forms a local softmax-weighted sum.
// The CTA reduces its 16 workers in shared memory and publishes (max, sum, acc[128]); the
// CTA that arrives last for a (b, h) merges the partials with a log-sum-exp and writes the
// bf16 output. The arrival counter is left at zero for the next call.
//
// Replaces hashattention/hashattention_llama.py:578-623: there every masked position is set
// to finfo.min before an fp32 softmax, i.e. contributes exactly 0, so the softmax runs
// over the selected rows only. Accumulation is fp32 throughout.
#pragma once

#include "common.cuh"

namespace ha {

struct SparseDecodeParams {
    const __nv_bfloat16* q;        // [B][Hq][128]
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* sel_idx;        // [B][Hq][sel_stride]
    const int32_t* sel_cnt;        // [B][Hq]
    __nv_bfloat16* out;            // [B][Hq][128]
    float* partials;               // workspace: [B][Hq][nsplits][130]
    unsigned int* counters;        // workspace: [B][Hq], zero between calls
    int32_t* status;
    int B, Hkv, max_pages, num_pages, sel_stride, nsplits;
    int init_budget, recent_budget;
    double heavy_budget;
    float scale_log2e;             // sm_scale * log2(e)
};

__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
    x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x);
    x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
    x[4] = bf16_lo(raw.z); x[5] = bf16_hi(raw.z);
    x[6] = bf16_lo(raw.w); x[7] = bf16_hi(raw.w);
}

__device__ __forceinline__ float dot8(const uint4& raw, const float (&x)[8]) {
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

__global__ void __launch_bounds__(kAttThreads) sparse_decode_kernel(const SparseDecodeParams p) {
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int Hq = p.Hkv * kGroup, kvh = h / kGroup;
    const int tid = threadIdx.x, lane = tid & 31;
    const int worker = tid >> 4, sl = tid & 15;

    __shared__ float s_m[kAttWorkers], s_l[kAttWorkers];
    __shared__ __align__(16) float s_acc[kAttWorkers][kHeadDim];
    __shared__ bool s_last;

    // the query is an input of the step, not a product of the preceding kernel
    float qf[8];
    {
        const uint4 raw = *reinterpret_cast<const uint4*>(p.q + ((size_t)b * Hq + h) * kHeadDim + sl * 8);
        unpack8(raw, qf);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] *= p.scale_log2e;
    }

    pdl_wait();
    pdl_launch_dependents();

    const int S = p.seq_lens[b];
    if (S < 1 || S > p.max_pages * kPage) return;  // reported by the selection kernels
    const SeqRange r = seq_range(S, p.init_budget, p.recent_budget, p.heavy_budget);
    int cnt = p.sel_cnt[(size_t)b * Hq + h];
    cnt = max(0, min(cnt, min(r.hb, p.sel_stride)));
    const int n_total = r.lo + cnt + (S - r.hi);
    const int nsplits_b = (n_total + kAttRows - 1) / kAttRows;
    if (split >= nsplits_b) return;

    const int32_t* sel = p.sel_idx + ((size_t)b * Hq + h) * p.sel_stride;
    const int32_t* pt = p.page_table + (size_t)b * p.max_pages;

    // ---- gather: 8 rows per worker, K and V loads all issued before any use ---------------
    uint4 kraw[kAttRowsPerWorker], vraw[kAttRowsPerWorker];
    uint32_t valid = 0;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < kAttRowsPerWorker; ++i) {
        const int pos = split * kAttRows + i * kAttWorkers + worker;
        kraw[i] = make_uint4(0, 0, 0, 0);
        vraw[i] = make_uint4(0, 0, 0, 0);
        if (pos < n_total) {
            int tok;
            if (pos < r.lo) tok = pos;
            else if (pos < r.lo + cnt) tok = __ldg(sel + (pos - r.lo));
            else tok = r.hi + (pos - r.lo - cnt);
            if (tok < 0 || tok >= S) {
                bad = true;
            } else {
                const int page = __ldg(pt + tok / kPage);
                if (page < 0 || page >= p.num_pages) {
                    bad = true;
                } else {
                    const size_t row = (((size_t)page * p.Hkv + kvh) * kPage + tok % kPage) * kHeadDim + sl * 8;
                    kraw[i] = __ldg(reinterpret_cast<const uint4*>(p.k_pages + row));
                    vraw[i] = __ldg(reinterpret_cast<const uint4*>(p.v_pages + row));
                    valid |= 1u << i;
                }
            }
        }
    }
    if (bad) report(p.status, HA_ERR_BAD_PAGE);

    // ---- scores (already in log2 units), local softmax, weighted V sum ---------------------
    float sc[kAttRowsPerWorker];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kAttRowsPerWorker; ++i) {
        float s = dot8(kraw[i], qf);
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        sc[i] = ((valid >> i) & 1u) ? s : -INFINITY;
        m = fmaxf(m, sc[i]);
    }
    float l = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kAttRowsPerWorker; ++i) {
        const float w = ((valid >> i) & 1u) ? exp2f(sc[i] - m) : 0.f;
        l += w;
        float v[8];
        unpack8(vraw[i], v);
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[d] = fmaf(w, v[d], acc[d]);
    }

    // ---- reduce the 16 workers of the CTA --------------------------------------------------
    if (sl == 0) {
        s_m[worker] = m;
        s_l[worker] = l;
    }
    *reinterpret_cast<float4*>(&s_acc[worker][sl * 8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(&s_acc[worker][sl * 8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    __syncthreads();

    float M = -INFINITY, L = 0.f, A = 0.f;
    if (tid < kHeadDim) {
#pragma unroll
        for (int w = 0; w < kAttWorkers; ++w) M = fmaxf(M, s_m[w]);
#pragma unroll
        for (int w = 0; w < kAttWorkers; ++w) {
            const float f = s_m[w] == -INFINITY ? 0.f : exp2f(s_m[w] - M);
            L = fmaf(s_l[w], f, L);
            A = fmaf(s_acc[w][tid], f, A);
        }
    }

    __nv_bfloat16* out = p.out + ((size_t)b * Hq + h) * kHeadDim;
    if (nsplits_b == 1) {  // nothing to merge with
        if (tid < kHeadDim) out[tid] = __float2bfloat16_rn(A / L);
        return;
    }

    float* part = p.partials + (((size_t)b * Hq + h) * p.nsplits + split) * kPartStride;
    if (tid < kHeadDim) {
        part[2 + tid] = A;
        if (tid == 0) {
            part[0] = M;
            part[1] = L;
        }
    }
    // publish, then count arrivals; the last CTA of this (b, h) merges. No CTA waits.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int prev = atomicAdd(p.counters + (size_t)b * Hq + h, 1u);
        s_last = prev == (unsigned int)(nsplits_b - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    if (tid < kHeadDim) {
        const float* base = p.partials + ((size_t)b * Hq + h) * p.nsplits * kPartStride;
        float Mg = -INFINITY;
        for (int s = 0; s < nsplits_b; ++s) Mg = fmaxf(Mg, __ldcg(base + (size_t)s * kPartStride));
        float Lg = 0.f, Ag = 0.f;
        for (int s = 0; s < nsplits_b; ++s) {
            const float* ps = base + (size_t)s * kPartStride;
            const float f = exp2f(__ldcg(ps) - Mg);
            Lg = fmaf(__ldcg(ps + 1), f, Lg);
            Ag = fmaf(__ldcg(ps + 2 + tid), f, Ag);
        }
        out[tid] = __float2bfloat16_rn(Ag / Lg);
    }
    if (tid == 0) p.counters[(size_t)b * Hq + h] = 0u;
    (void)lane;
}

}  // namespace ha
