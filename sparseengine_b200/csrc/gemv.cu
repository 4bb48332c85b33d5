// Dense projection for a handful of rows (decode): out[t, n] = sum_k x[t, k] w[n, k], bf16
// in, fp32 accumulate, bf16 out, for up to 16 rows of x.
//
// With so few rows the projection is a stream over the weight matrix.  A warp owns 16
// weight rows and walks K in 32-element chunks: every lane loads 16 contiguous bytes of two
// weight rows (and of one x row) straight from global memory into the registers of
// m16n8k16 tensor-core fragments.  The fragment's k slots are filled in a permuted order
// (slot pairs {2t, 2t+1} and {2t+8, 2t+9} of lane t take 4 consecutive elements), which is
// harmless because A and B use the same permutation and the sum over k does not care.  No
// shared memory on the way in; the 8 or 16 warps of a block split K and add their partial
// sums through shared memory at the end.  The weights are read exactly once.
#include "common.cuh"
#include "mma_util.cuh"
#include <cstdlib>

namespace se {
namespace gemv {

// NT: 8-row tiles of x, 1 (up to 8 rows) or 2 (up to 16).  kWarps: warps of a block, which
// split K.  kRowsPerBlock: weight rows of a block, 16 (a full fragment) or 8 (the fragment's
// upper half stays zero): fewer rows make more blocks, which a matrix with few rows needs to
// keep every SM loading.
// Chunks of a warp whose weights are loaded before x is waited for.  They are held in registers,
// and more than 4 chunks cost more in residency than they gain (measured: 8 chunks are slower
// than none, also for the few blocks of 16 warps that the output projection has).
#ifndef SE_GEMV_PRELOAD
#define SE_GEMV_PRELOAD 4
#endif

template <int NT, int kWarps, int kRowsPerBlock>
__global__ void __launch_bounds__(32 * kWarps)
gemv_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
            int rows, int n_out, int k_dim) {
    grid_dependency_trigger();       // the kernel after this one may set itself up meanwhile
    constexpr int kPreload = SE_GEMV_PRELOAD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int n0 = blockIdx.x * kRowsPerBlock;
    const int chunks = k_dim / 32;
    const int c_begin = warp * chunks / kWarps, c_end = (warp + 1) * chunks / kWarps;
    const __nv_bfloat16* w_lo = w + (size_t)min(n0 + g, n_out - 1) * k_dim + 8 * t4;
    const __nv_bfloat16* w_hi = w + (size_t)min(n0 + g + 8, n_out - 1) * k_dim + 8 * t4;
    const __nv_bfloat16* x_row[NT];
    bool x_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        x_ok[nt] = nt * 8 + g < rows;
        x_row[nt] = x + (size_t)min(nt * 8 + g, rows - 1) * k_dim + 8 * t4;
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    auto step = [&](int c, const uint4& a_lo, const uint4& a_hi) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint4 b = make_uint4(0u, 0u, 0u, 0u);
            if (x_ok[nt]) b = *reinterpret_cast<const uint4*>(x_row[nt] + c * 32);
            const uint32_t a0[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};
            const uint32_t a1[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};
            se::mma::mma_bf16(acc[nt], a0, b.x, b.y);
            se::mma::mma_bf16(acc[nt], a1, b.z, b.w);
        }
    };
    // The first chunks' weights are asked for before the kernel that makes x has ended (this
    // kernel is launched as its dependent): the weights are what takes the time, and no kernel
    // writes them.  x is read with ordinary loads through a pointer that is not __restrict__:
    // loads the compiler may take for read-only over the kernel's lifetime could move above the wait.
    uint4 pre_lo[kPreload > 0 ? kPreload : 1], pre_hi[kPreload > 0 ? kPreload : 1];
#pragma unroll
    for (int i = 0; i < kPreload; ++i) {
        pre_lo[i] = pre_hi[i] = make_uint4(0u, 0u, 0u, 0u);
        if (c_begin + i < c_end) {
            pre_lo[i] = __ldcs(reinterpret_cast<const uint4*>(w_lo + (c_begin + i) * 32));     // streamed once
            if (kRowsPerBlock == 16) pre_hi[i] = __ldcs(reinterpret_cast<const uint4*>(w_hi + (c_begin + i) * 32));
        }
    }
    grid_dependency_wait();
#pragma unroll
    for (int i = 0; i < kPreload; ++i)
        if (c_begin + i < c_end) step(c_begin + i, pre_lo[i], pre_hi[i]);
#pragma unroll 4
    for (int c = c_begin + kPreload; c < c_end; ++c) {
        const uint4 a_lo = __ldcs(reinterpret_cast<const uint4*>(w_lo + c * 32));
        uint4 a_hi = make_uint4(0u, 0u, 0u, 0u);
        if (kRowsPerBlock == 16) a_hi = __ldcs(reinterpret_cast<const uint4*>(w_hi + c * 32));
        step(c, a_lo, a_hi);
    }
    __shared__ float part[kWarps][kRowsPerBlock][8 * NT + 1];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        part[warp][g][nt * 8 + 2 * t4] = acc[nt][0];
        part[warp][g][nt * 8 + 2 * t4 + 1] = acc[nt][1];
        if (kRowsPerBlock == 16) {
            part[warp][g + 8][nt * 8 + 2 * t4] = acc[nt][2];
            part[warp][g + 8][nt * 8 + 2 * t4 + 1] = acc[nt][3];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kRowsPerBlock * 8 * NT; i += blockDim.x) {
        const int r = i % kRowsPerBlock, t = i / kRowsPerBlock;      // consecutive threads -> consecutive n
        if (t < rows && n0 + r < n_out) {
            float v = 0.f;
#pragma unroll
            for (int wq = 0; wq < kWarps; ++wq) v += part[wq][r][t];
            out[(size_t)t * n_out + n0 + r] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace gemv
}  // namespace se

extern "C" int se_gemv_supported(int rows, int n_out, int k_dim) {
    return (rows >= 1 && rows <= 16 && n_out >= 1 && k_dim >= 32 && k_dim % 32 == 0) ? 1 : 0;
}

template <int NT, int W, int R>
static void launch_gemv(const void* x, const void* w, void* out, int rows, int n_out, int k_dim, cudaStream_t stream) {
    SE_LAUNCH_DEPENDENT("gemv", se::gemv::gemv_kernel<NT, W, R>, dim3(se::ceil_div(n_out, R)), dim3(32 * W), 0, stream,
                         (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, rows, n_out, k_dim);
}

// x [rows <= 16, k_dim], w [n_out, k_dim], out [rows, n_out]; bf16; k_dim a multiple of 32.
extern "C" int se_gemv(const void* x, const void* w, void* out, int rows, int n_out, int k_dim, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!se_gemv_supported(rows, n_out, k_dim)) return SE_ERR_UNSUPPORTED;
    // Shape = 100 * (warps that split K) + (weight rows per block).  A warp's walk over its
    // share of K is one chain of dependent loads, so a long K takes more warps (measured:
    // K = 6144 runs in 9.4 us with 16 warps, 14.4 us with 8).  SE_GEMV_SHAPE overrides (tuning aid).
    static const int force = [] { const char* v = std::getenv("SE_GEMV_SHAPE"); return v ? atoi(v) : 0; }();
    const int shape = force ? force : (k_dim >= 4096 ? 1616 : 816);
    const int nt = rows <= 8 ? 1 : 2;
#define SE_GEMV_CASE(W, R)                                                       \
    case W * 100 + R:                                                            \
        if (nt == 1) launch_gemv<1, W, R>(x, w, out, rows, n_out, k_dim, stream); \
        else launch_gemv<2, W, R>(x, w, out, rows, n_out, k_dim, stream);         \
        break;
    switch (shape) {
        SE_GEMV_CASE(4, 8) SE_GEMV_CASE(4, 16) SE_GEMV_CASE(8, 8) SE_GEMV_CASE(8, 16) SE_GEMV_CASE(16, 8) SE_GEMV_CASE(16, 16)
        default: return SE_ERR_ARGUMENT;
    }
#undef SE_GEMV_CASE
    SE_LAUNCH_CHECK();
}
