// A read-only stream through the path the weight-streaming GEMMs use: bulk asynchronous copies
// into a ring of shared-memory stages, completed on mbarriers and dropped.  It measures what
// this GPU delivers to kernels that read HBM this way (more than a copy's read + write
// figure, and more than a plain reduction kernel reaches); benchmarks report it beside their
// roofline fractions.  Nothing is computed: no result depends on it.
#include "common.cuh"

namespace se {
namespace rs {

constexpr int kStages = 6;
constexpr int kChunk = 16 * 1024;                 // bytes per copy
constexpr int kStageBytes = 2 * kChunk;
constexpr int kRun = 48;                          // stages a CTA reads in a row before it moves on (1.5 MB, as a GEMM walks K)
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// `stages` stages of kStageBytes in all, dealt to the CTAs in runs of kRun.
__global__ void __launch_bounds__(64, 1)
read_stream_kernel(const char* __restrict__ src, long long stages, int* __restrict__ error) {
    extern __shared__ uint8_t raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * kStages];
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2 * kStages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full0 + 8 * s) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long runs = (stages + kRun - 1) / kRun;
    if (threadIdx.x == 0) {                       // the loader
        long long it = 0;
        bool ok = true;
        for (long long r = blockIdx.x; r < runs && ok; r += gridDim.x) {
            for (long long st = r * kRun; st < min(stages, (r + 1) * kRun); ++st, ++it) {
                const int s = (int)(it % kStages);
                if (!mbar_wait(empty0 + 8 * s, (uint32_t)(((it / kStages) & 1) ^ 1))) {
                    atomicCAS(error, 0, 14);
                    ok = false;
                    break;
                }
                const uint32_t dst = smem_u32(smem + (size_t)s * kStageBytes), bar = full0 + 8 * s;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kStageBytes) : "memory");
                const char* p = src + st * kStageBytes;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst), "l"(p), "r"(kChunk), "r"(bar) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst + kChunk), "l"(p + kChunk), "r"(kChunk), "r"(bar) : "memory");
            }
        }
        // what is still on its way lands before the shared memory goes away
        for (long long k = max(0LL, it - kStages); k < it; ++k) mbar_wait(full0 + 8 * (int)(k % kStages), (uint32_t)((k / kStages) & 1));
    } else if (threadIdx.x == 32) {               // the consumer: hands every stage straight back
        long long it = 0;
        for (long long r = blockIdx.x; r < runs; r += gridDim.x) {
            for (long long st = r * kRun; st < min(stages, (r + 1) * kRun); ++st, ++it) {
                const int s = (int)(it % kStages);
                if (!mbar_wait(full0 + 8 * s, (uint32_t)((it / kStages) & 1))) return;     // the loader has given up or will
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * s) : "memory");
            }
        }
    }
}

}  // namespace rs
}  // namespace se

// Reads `bytes` (rounded down to 32 KB) from `src` (16-byte aligned) once, with one CTA per SM.
extern "C" int se_read_stream(const void* src, long long bytes, int* error, cudaStream_t stream) {
    const long long stages = bytes / se::rs::kStageBytes;
    if (stages <= 0) return 0;
    if (((uintptr_t)src & 15) != 0) return SE_ERR_ARGUMENT;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    const int smem = se::rs::kStages * se::rs::kStageBytes + 1024;
    static bool configured = false;
    if (!configured) {
        e = cudaFuncSetAttribute(se::rs::read_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    se::rs::read_stream_kernel<<<sms, 64, smem, stream>>>((const char*)src, stages, error);
    SE_LAUNCH_CHECK();
}
