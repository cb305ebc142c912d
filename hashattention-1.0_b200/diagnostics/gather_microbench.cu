// Microbenchmark: how fast can random 256-byte K/V rows be gathered on B200, as a function of the
// thread mapping and the number of loads in flight?  Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o gather_microbench gather_microbench.cu
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <random>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

constexpr int ROWB = 256;  // bytes per row

// ---- A: register gather. LPR lanes per row (16 -> uint4 per lane; 8 -> 2x uint4 per lane), RPW rows in flight per worker
template <int LPR, int RPW, int THREADS>
__global__ void __launch_bounds__(THREADS) gather_reg(const uint4* __restrict__ K, const uint4* __restrict__ V,
                                                     const int* __restrict__ idx, int total_rows, uint32_t* out) {
    constexpr int VEC = ROWB / 16 / LPR;  // uint4 per lane per row
    const int workers_per_cta = THREADS / LPR;
    const int worker = threadIdx.x / LPR, sl = threadIdx.x % LPR;
    const long base = (long)blockIdx.x * workers_per_cta * RPW;
    int rows[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        long pos = base + (long)i * workers_per_cta + worker;
        rows[i] = idx[pos < total_rows ? pos : total_rows - 1];
    }
    uint4 k[RPW][VEC], v[RPW][VEC];
#pragma unroll
    for (int i = 0; i < RPW; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            k[i][j] = __ldg(K + (size_t)rows[i] * (ROWB / 16) + sl * VEC + j);
            v[i][j] = __ldg(V + (size_t)rows[i] * (ROWB / 16) + sl * VEC + j);
        }
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < RPW; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            acc ^= k[i][j].x ^ k[i][j].y ^ k[i][j].z ^ k[i][j].w ^ v[i][j].x ^ v[i][j].y ^ v[i][j].z ^ v[i][j].w;
    if (acc == 0x12345678u) out[blockIdx.x * THREADS + threadIdx.x] = acc;
}

// ---- B: persistent register gather: grid = SMs * k, each worker loops over rounds
template <int RPW, int THREADS>
__global__ void __launch_bounds__(THREADS) gather_reg_loop(const uint4* __restrict__ K, const uint4* __restrict__ V,
                                                          const int* __restrict__ idx, int total_rows, uint32_t* out) {
    const int workers_per_cta = THREADS / 16;
    const int worker = threadIdx.x / 16, sl = threadIdx.x % 16;
    const long stride = (long)gridDim.x * workers_per_cta * RPW;
    uint32_t acc = 0;
    for (long base = (long)blockIdx.x * workers_per_cta * RPW; base < total_rows; base += stride) {
        int rows[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            long pos = base + (long)i * workers_per_cta + worker;
            rows[i] = idx[pos < total_rows ? pos : total_rows - 1];
        }
        uint4 k[RPW], v[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            k[i] = __ldg(K + (size_t)rows[i] * 16 + sl);
            v[i] = __ldg(V + (size_t)rows[i] * 16 + sl);
        }
#pragma unroll
        for (int i = 0; i < RPW; ++i)
            acc ^= k[i].x ^ k[i].y ^ k[i].z ^ k[i].w ^ v[i].x ^ v[i].y ^ v[i].z ^ v[i].w;
    }
    if (acc == 0x12345678u) out[blockIdx.x * THREADS + threadIdx.x] = acc;
}

// ---- C: bulk-copy gather: one lane per row issues cp.async.bulk (256 B for K, 256 B for V) into shared memory
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int ROWS_PER_CTA, int THREADS>
__global__ void __launch_bounds__(THREADS) gather_bulk(const uint4* __restrict__ K, const uint4* __restrict__ V,
                                                      const int* __restrict__ idx, int total_rows, uint32_t* out) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar;
    uint4* sk = reinterpret_cast<uint4*>(smem);
    uint4* sv = sk + ROWS_PER_CTA * 16;
    const long base = (long)blockIdx.x * ROWS_PER_CTA;
    const int nrows = (int)min((long)ROWS_PER_CTA, (long)total_rows - base);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bar)), "r"(nrows * 2 * ROWB) : "memory");
    __syncthreads();
    for (int r = threadIdx.x; r < nrows; r += THREADS) {
        const int row = idx[base + r];
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(sk + r * 16)), "l"(K + (size_t)row * 16), "r"(ROWB), "r"(smem_u32(&bar)) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(sv + r * 16)), "l"(V + (size_t)row * 16), "r"(ROWB), "r"(smem_u32(&bar)) : "memory");
    }
    // bounded wait on phase 0
    uint32_t done = 0;
    for (int spin = 0; spin < (1 << 22) && !done; ++spin)
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(smem_u32(&bar)) : "memory");
    uint32_t acc = done ? 0 : 0xdeadbeef;
    for (int i = threadIdx.x; i < nrows * 16; i += THREADS) {
        uint4 a = sk[i], b = sv[i];
        acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w;
    }
    if (acc == 0x12345678u || !done) out[blockIdx.x * THREADS + threadIdx.x] = acc;
}

// ---- D: contiguous streaming read of the same number of bytes
template <int THREADS, int PER>
__global__ void __launch_bounds__(THREADS) stream_read(const uint4* __restrict__ K, size_t n_vec, uint32_t* out) {
    size_t i0 = ((size_t)blockIdx.x * THREADS * PER) + threadIdx.x;
    uint4 r[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        size_t i = i0 + (size_t)j * THREADS;
        r[j] = __ldg(K + (i < n_vec ? i : n_vec - 1));
    }
    uint32_t acc = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) acc ^= r[j].x ^ r[j].y ^ r[j].z ^ r[j].w;
    if (acc == 0x12345678u) out[blockIdx.x * THREADS + threadIdx.x] = acc;
}

__global__ void empty_kernel(int* p) { if (p != nullptr && threadIdx.x == 9999) *p = 1; }
__global__ void empty_pdl_kernel(int* p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (p != nullptr && threadIdx.x == 9999) *p = 1;
}

template <typename F>
float time_us(F launch, int reps) {
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int i = 0; i < 3; ++i) launch(i);
    CK(cudaDeviceSynchronize());
    CK(cudaEventRecord(e0));
    for (int i = 0; i < reps; ++i) launch(i);
    CK(cudaEventRecord(e1));
    CK(cudaDeviceSynchronize());
    float ms;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    return ms * 1000.f / reps;
}

int main() {
    const int NPOOL = 12;                    // rotate pools: 12 x (64 + 64 MB) > L2
    const int N_ROWS = 262144;               // rows per pool: 64 MB of K, 64 MB of V
    std::vector<uint4*> K(NPOOL), V(NPOOL);
    for (int i = 0; i < NPOOL; ++i) {
        CK(cudaMalloc(&K[i], (size_t)N_ROWS * ROWB));
        CK(cudaMalloc(&V[i], (size_t)N_ROWS * ROWB));
        CK(cudaMemset(K[i], i + 1, (size_t)N_ROWS * ROWB));
        CK(cudaMemset(V[i], i + 7, (size_t)N_ROWS * ROWB));
    }
    uint32_t* out;
    CK(cudaMalloc(&out, 64 << 20));
    std::mt19937 rng(1);
    for (int total_rows : {40960, 557056}) {
        // index lists: groups of `per` sorted random rows (like one head's ascending selection)
        const int per = total_rows == 40960 ? 1280 : 4352;
        std::vector<int> h(total_rows);
        for (int g = 0; g < total_rows / per; ++g) {
            for (int i = 0; i < per; ++i) h[g * per + i] = rng() % N_ROWS;
            std::sort(h.begin() + g * per, h.begin() + (g + 1) * per);
        }
        int* idx;
        CK(cudaMalloc(&idx, total_rows * sizeof(int)));
        CK(cudaMemcpy(idx, h.data(), total_rows * sizeof(int), cudaMemcpyHostToDevice));
        const double bytes = (double)total_rows * 2 * ROWB;
        printf("== total_rows %d (%.1f MB)\n", total_rows, bytes / 1e6);
        auto report = [&](const char* name, float us) { printf("%-44s %8.2f us  %8.1f GB/s\n", name, us, bytes / us / 1e3); };
        const int reps = 200;
#define RUN_REG(LPR, RPW, THREADS) { \
            int rows_per_cta = THREADS / LPR * RPW; int grid = (total_rows + rows_per_cta - 1) / rows_per_cta; \
            float us = time_us([&](int i) { gather_reg<LPR, RPW, THREADS><<<grid, THREADS>>>(K[i % NPOOL], V[i % NPOOL], idx, total_rows, out); }, reps); \
            char nm[64]; snprintf(nm, 64, "reg lanes/row=%d rows/worker=%d thr=%d grid=%d", LPR, RPW, THREADS, grid); report(nm, us); }
        RUN_REG(16, 1, 256) RUN_REG(16, 2, 256) RUN_REG(16, 4, 256) RUN_REG(16, 8, 256) RUN_REG(16, 8, 128)
        RUN_REG(16, 4, 128) RUN_REG(16, 4, 512) RUN_REG(8, 4, 256) RUN_REG(8, 2, 256) RUN_REG(8, 8, 256) RUN_REG(16, 16, 256)
#define RUN_LOOP(RPW, THREADS, MULT) { \
            int grid = 148 * MULT; \
            float us = time_us([&](int i) { gather_reg_loop<RPW, THREADS><<<grid, THREADS>>>(K[i % NPOOL], V[i % NPOOL], idx, total_rows, out); }, reps); \
            char nm[64]; snprintf(nm, 64, "loop rows/worker=%d thr=%d grid=148x%d", RPW, THREADS, MULT); report(nm, us); }
        RUN_LOOP(4, 256, 2) RUN_LOOP(4, 256, 4) RUN_LOOP(8, 256, 2) RUN_LOOP(2, 256, 8) RUN_LOOP(4, 512, 2) RUN_LOOP(2, 1024, 2) RUN_LOOP(4, 128, 8)
#define RUN_BULK(RPC, THREADS) { \
            int grid = (total_rows + RPC - 1) / RPC; size_t smem = (size_t)RPC * 2 * ROWB; \
            CK(cudaFuncSetAttribute(gather_bulk<RPC, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            float us = time_us([&](int i) { gather_bulk<RPC, THREADS><<<grid, THREADS, smem>>>(K[i % NPOOL], V[i % NPOOL], idx, total_rows, out); }, reps); \
            char nm[64]; snprintf(nm, 64, "bulk rows/cta=%d thr=%d grid=%d", RPC, THREADS, grid); report(nm, us); }
        RUN_BULK(32, 128) RUN_BULK(64, 128) RUN_BULK(128, 128) RUN_BULK(64, 64) RUN_BULK(192, 256)
        {
            size_t n_vec = (size_t)bytes / 16;  // same bytes, contiguous, from the K pool(s)
            if (n_vec > (size_t)N_ROWS * 16) n_vec = (size_t)N_ROWS * 16;
            int grid = (int)((n_vec + 256 * 8 - 1) / (256 * 8));
            float us = time_us([&](int i) { stream_read<256, 8><<<grid, 256>>>(K[i % NPOOL], n_vec, out); }, reps);
            printf("%-44s %8.2f us  %8.1f GB/s\n", "contiguous stream (same bytes, capped 64MB)", us, n_vec * 16.0 / us / 1e3);
        }
        CK(cudaFree(idx));
    }
    // ---- launch overheads
    {
        cudaStream_t s;
        CK(cudaStreamCreate(&s));
        float us = time_us([&](int) { empty_kernel<<<148, 128, 0, s>>>(nullptr); }, 2000);
        printf("empty kernel back-to-back (stream)          %8.2f us per launch\n", us);
        for (int pdl = 0; pdl < 2; ++pdl) {
            cudaGraph_t g; cudaGraphExec_t ge;
            CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeGlobal));
            for (int i = 0; i < 64; ++i) {
                cudaLaunchConfig_t cfg = {}; cfg.gridDim = dim3(148); cfg.blockDim = dim3(128); cfg.stream = s;
                cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                at[0].val.programmaticStreamSerializationAllowed = pdl; cfg.attrs = at; cfg.numAttrs = 1;
                int* np = nullptr;
                if (pdl) CK(cudaLaunchKernelEx(&cfg, empty_pdl_kernel, np)); else CK(cudaLaunchKernelEx(&cfg, empty_kernel, np));
            }
            CK(cudaStreamEndCapture(s, &g));
            CK(cudaGraphInstantiate(&ge, g, 0));
            float usg = time_us([&](int) { CK(cudaGraphLaunch(ge, s)); }, 200);
            printf("graph of 64 empty kernels, pdl=%d            %8.2f us per kernel\n", pdl, usg / 64);
        }
    }
    printf("done\n");
    return 0;
}
