// Routed experts, plain path: routing build (count, rank, scatter, tile list), grouped
// GEMMs on CUDA cores with 32-bit accumulation (float32 or bfloat16 operands), and the
// top-k combine in router slot order.
//
// Reference pipeline: src/sparseengine/kernels/triton/moe.py:336-463 (assignment),
// :466-574,634-739 (routed GEMM, gate/up + SwiGLU), :1098-1210 (sum over k in slot
// order), :1374-1440 (bf16 pipeline); SiLU src/sparseengine/kernels/triton/silu_and_mul.py:41-60.
// Rounding points: gate and up are rounded to the activation type, silu(gate) is
// computed in 32-bit and rounded, the product with up is rounded; the down projection
// times the routing weight (32-bit) is rounded; the sum over slots is 32-bit, rounded once.
#include "common.cuh"

namespace se {

// ---- routing build -------------------------------------------------------------------
// ids: [assignments] expert of flat assignment a = token * top_k + slot.
// Block e walks all assignments in order and ranks those of expert e (stable).
__global__ void moe_count_rank_kernel(const int* __restrict__ ids, int assignments, int* __restrict__ counts,
                                      int* __restrict__ rank) {
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __shared__ int warp_total[32];
    // each warp owns a contiguous chunk (a multiple of 32 assignments)
    const int per = ((assignments + nwarps - 1) / nwarps + 31) & ~31;
    const int a0 = warp * per, a1 = min(assignments, a0 + per);
    int mine = 0;
    for (int base = a0; base < a1; base += 32) {
        const int a = base + lane;
        mine += __popc(__ballot_sync(0xffffffffu, a < a1 && ids[a] == e));
    }
    if (lane == 0) warp_total[warp] = mine;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_total[w];
    for (int base = a0; base < a1; base += 32) {
        const int a = base + lane;
        const bool hit = a < a1 && ids[a] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (hit) rank[a] = before + __popc(ballot & ((1u << lane) - 1u));
        before += __popc(ballot);
    }
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int w = 0; w < nwarps; ++w) tot += warp_total[w];
        counts[e] = tot;
    }
}

// Exclusive scans, by one whole block, of the rows per expert and of the tiles per expert
// (tile_rows rows each) into off[experts + 1] and toff[experts + 1] (shared memory).
__device__ __forceinline__ void scan_counts(const int* counts, int experts, int tile_rows, int* off, int* toff) {
    __shared__ int carry[2];
    __shared__ int wsum[2][32];
    if (threadIdx.x == 0) carry[0] = carry[1] = 0;
    __syncthreads();
    for (int base = 0; base < experts; base += blockDim.x) {
        const int e = base + threadIdx.x;
        const int c = e < experts ? counts[e] : 0;
        const int tl = (c + tile_rows - 1) / tile_rows;
        // inclusive scan within the block: warp scans, then the warp totals
        int vc = c, vt = tl;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int uc = __shfl_up_sync(0xffffffffu, vc, o), ut = __shfl_up_sync(0xffffffffu, vt, o);
            if (lane >= o) { vc += uc; vt += ut; }
        }
        if (lane == 31) { wsum[0][warp] = vc; wsum[1][warp] = vt; }
        __syncthreads();
        int pc = carry[0], pt = carry[1];
        for (int w = 0; w < warp; ++w) { pc += wsum[0][w]; pt += wsum[1][w]; }
        if (e < experts) { off[e] = pc + vc - c; toff[e] = pt + vt - tl; }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) { carry[0] = pc + vc; carry[1] = pt + vt; }
        __syncthreads();
    }
    if (threadIdx.x == 0) { off[experts] = carry[0]; toff[experts] = carry[1]; }
    __syncthreads();
}

// stats[0] += experts that got at least one row, stats[1] += 1 (one block calls this, once per
// routing build): how many experts' weights the steps of a run have to read, counted where
// the counts already are.
__device__ __forceinline__ void count_used_experts(const int* counts, int experts, unsigned long long* stats) {
    if (stats == nullptr) return;
    int mine = 0;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) mine += counts[e] > 0 ? 1 : 0;
    mine = __reduce_add_sync(0xffffffffu, mine);
    if ((threadIdx.x & 31) == 0 && mine > 0) atomicAdd(&stats[0], (unsigned long long)mine);
    if (threadIdx.x == 0) atomicAdd(&stats[1], 1ull);
}

// The tile list and the offsets, from the scans (one block writes them).
__device__ __forceinline__ void write_tiles(const int* off, const int* toff, int experts, int tile_rows,
                                            int* __restrict__ offsets, int* __restrict__ tile_expert,
                                            int* __restrict__ tile_row0, int* __restrict__ num_tiles) {
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int first = toff[e], n = toff[e + 1] - first;
        for (int i = 0; i < n; ++i) {
            tile_expert[first + i] = e;
            tile_row0[first + i] = off[e] + i * tile_rows;
        }
    }
    if (threadIdx.x == 0) num_tiles[0] = toff[experts];
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = off[e];
}

// One block: exclusive scan of counts -> offsets[experts+1], tile list for rows-per-tile
// `tile_rows`: tile_expert[i], tile_row0[i] (first sorted row), num_tiles[0].
// All blocks: scatter sorted[offset[e] + rank[a]] = a, inv_pos[a] = that position.
__global__ void moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ rank,
                                   const int* __restrict__ counts, int assignments, int experts, int tile_rows,
                                   int* __restrict__ offsets, int* __restrict__ sorted, int* __restrict__ inv_pos,
                                   int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                   int* __restrict__ num_tiles, unsigned long long* stats) {
    extern __shared__ int off[];   // experts + 1 row offsets, then experts + 1 tile offsets
    int* toff = off + experts + 1;
    scan_counts(counts, experts, tile_rows, off, toff);
    if (blockIdx.x == 0) {
        write_tiles(off, toff, experts, tile_rows, offsets, tile_expert, tile_row0, num_tiles);
        count_used_experts(counts, experts, stats);
    }
    for (int a = blockIdx.x * blockDim.x + threadIdx.x; a < assignments; a += gridDim.x * blockDim.x) {
        const int e = ids[a];
        if ((unsigned)e >= (unsigned)experts) continue;      // not an expert: no rank was written for it, nothing is indexed with it
        const int p = off[e] + rank[a];
        sorted[p] = a;
        inv_pos[a] = p;
    }
}

// Few assignments (decode steps): the whole routing build in one launch, and with it the
// gather of the activation rows into expert order that the tensor-core GEMM reads.  Every
// block builds the same routing in its shared memory (thread e walks the assignments in
// order and ranks those of expert e, so the order within an expert is the order of the
// assignments, as above); block 0 writes the tables, and block b copies row b.  Beyond a few
// hundred assignments the three kernels above are faster (measured at 512: every block's walk
// over all assignments costs more than the launches it saves).
constexpr int kRouteSmallAssignments = 256;
constexpr int kRouteSmallExperts = 1024;

__global__ void __launch_bounds__(256)
moe_route_small_kernel(const int* __restrict__ ids, int assignments, int experts, int tile_rows, int top_k,
                       int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ sorted,
                       int* __restrict__ inv_pos, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                       int* __restrict__ num_tiles, const uint4* __restrict__ x, uint4* __restrict__ xs,
                       int row_vecs, unsigned long long* stats) {
    extern __shared__ int sm[];
    grid_dependency_trigger();              // the grouped GEMM that follows may set itself up
    int* ids_s = sm;                        // [assignments]
    int* rank_s = ids_s + assignments;      // [assignments]
    int* sorted_s = rank_s + assignments;   // [assignments]
    int* cnt = sorted_s + assignments;      // [experts]
    int* off = cnt + experts;               // [experts + 1]
    int* toff = off + experts + 1;          // [experts + 1]
    for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
        ids_s[a] = ids[a];
        sorted_s[a] = 0;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int c = 0;
        for (int a = 0; a < assignments; ++a)
            if (ids_s[a] == e) rank_s[a] = c++;
        cnt[e] = c;
    }
    __syncthreads();
    scan_counts(cnt, experts, tile_rows, off, toff);
    for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
        const int e = ids_s[a];
        if ((unsigned)e >= (unsigned)experts) continue;      // not an expert: the caller's fault, nothing is read out of range
        const int p = off[e] + rank_s[a];
        sorted_s[p] = a;
        if (blockIdx.x == 0) {
            sorted[p] = a;
            inv_pos[a] = p;
        }
    }
    if (blockIdx.x == 0) {
        write_tiles(off, toff, experts, tile_rows, offsets, tile_expert, tile_row0, num_tiles);
        for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = cnt[e];
        count_used_experts(cnt, experts, stats);
    }
    if (x == nullptr) return;
    __syncthreads();
    for (int p = blockIdx.x; p < assignments; p += gridDim.x) {
        const uint4* src = x + (size_t)(sorted_s[p] / top_k) * row_vecs;
        uint4* dst = xs + (size_t)p * row_vecs;
        for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) dst[i] = src[i];
    }
}

// out[p, :] = x[sorted[p] / top_k, :] in 16-byte words (activation rows gathered into expert order)
__global__ void gather_sorted_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ sorted,
                                          uint4* __restrict__ out, int row_vecs, int top_k) {
    grid_dependency_trigger();              // the grouped GEMM that follows may stream its first weight tiles
    const uint4* src = x + (size_t)(sorted[blockIdx.x] / top_k) * row_vecs;
    uint4* dst = out + (size_t)blockIdx.x * row_vecs;
    for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) dst[i] = src[i];
}

// ---- grouped GEMM on CUDA cores ------------------------------------------------------
constexpr int kBM = 32, kBN = 64, kBK = 16;   // 256 threads, each 2 x 4 outputs

// MODE 0: gate/up + SwiGLU.  A row of sorted position p = x[sorted[p] / top_k];
//         W = w13[e] ([2*n_out, k_dim]: gate rows then up rows); out[p, n] (n_out = I).
// MODE 1: down.  A row = act[p]; W = w2[e] ([n_out, k_dim]); out[p, n] = acc * weight[sorted[p]].
template <typename T, int MODE>
__global__ void grouped_gemm_plain_kernel(const T* __restrict__ a, const T* __restrict__ w,
                                          const int* __restrict__ sorted, const int* __restrict__ offsets,
                                          const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                                          const int* __restrict__ num_tiles, const float* __restrict__ route_w,
                                          T* __restrict__ out, int n_out, int k_dim, int top_k) {
    if ((int)blockIdx.x >= num_tiles[0]) return;
    const int e = tile_expert[blockIdx.x];
    const int row0 = tile_row0[blockIdx.x];
    const int row_end = offsets[e + 1];
    const int n0 = blockIdx.y * kBN;
    constexpr int NW = MODE == 0 ? 2 : 1;
    __shared__ float as[kBK][kBM + 1];
    __shared__ float ws[NW][kBK][kBN + 1];
    __shared__ int src_row[kBM];
    const int tid = threadIdx.x;
    if (tid < kBM) {
        const int p = row0 + tid;
        src_row[tid] = p < row_end ? (MODE == 0 ? sorted[p] / top_k : p) : -1;
    }
    __syncthreads();
    const size_t w_rows = (size_t)(MODE == 0 ? 2 * n_out : n_out);
    const T* we = w + (size_t)e * w_rows * k_dim;
    const int tm = (tid / 16) * 2, tn = (tid % 16) * 4;
    float acc[NW][2][4] = {};
    for (int k0 = 0; k0 < k_dim; k0 += kBK) {
        for (int i = tid; i < kBM * kBK; i += 256) {
            const int r = i / kBK, c = i % kBK;
            const int sr = src_row[r];
            as[c][r] = (sr >= 0 && k0 + c < k_dim) ? to_float(a[(size_t)sr * k_dim + k0 + c]) : 0.f;
        }
        for (int i = tid; i < kBN * kBK; i += 256) {
            const int r = i / kBK, c = i % kBK;
            const bool ok = n0 + r < n_out && k0 + c < k_dim;
#pragma unroll
            for (int h = 0; h < NW; ++h)
                ws[h][c][r] = ok ? to_float(we[((size_t)h * n_out + n0 + r) * k_dim + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < kBK; ++c) {
            float av[2], wv[NW][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) av[i] = as[c][tm + i];
#pragma unroll
            for (int h = 0; h < NW; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[h][j] = ws[h][c][tn + j];
#pragma unroll
            for (int h = 0; h < NW; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[h][i][j] = fmaf(av[i], wv[h][j], acc[h][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int p = row0 + tm + i;
        if (p >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n >= n_out) continue;
            float v;
            if (MODE == 0) {
                const float g = round_act<T>(acc[0][i][j]);
                const float u = round_act<T>(acc[NW - 1][i][j]);
                v = round_act<T>(g / (1.f + expf(-g))) * u;
            } else {
                v = acc[0][i][j] * route_w[sorted[p]];
            }
            out[(size_t)p * n_out + n] = from_float<T>(v);
        }
    }
}

// out[t, :] = cast(sum over slots (32-bit, slot order) of y[inv_pos[t * top_k + slot], :]).
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ inv_pos, T* __restrict__ out,
                                   int hidden, int top_k) {
    grid_dependency_trigger();       // the norm that follows may fetch its weights, and the projection after it its own
    const int t = blockIdx.x;
    if ((hidden & 7) == 0 && aligned8(y) && aligned8(out)) {
        const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
        if (i >= hidden) return;
        float acc[8] = {};
        for (int k = 0; k < top_k; ++k) {
            float v[8];
            load8(y + (size_t)inv_pos[t * top_k + k] * hidden + i, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        store8(out + (size_t)t * hidden + i, acc);
        return;
    }
    for (int i = blockIdx.y * blockDim.x * 8 + threadIdx.x; i < min(hidden, (int)(blockIdx.y + 1) * (int)blockDim.x * 8);
         i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top_k; ++k) s += to_float(y[(size_t)inv_pos[t * top_k + k] * hidden + i]);
        out[(size_t)t * hidden + i] = from_float<T>(s);
    }
}

}  // namespace se

// Most experts the routing build takes: its scans keep two ints per expert in the 48 KB of
// shared memory a kernel has without asking.
extern "C" int se_moe_max_experts() { return (48 * 1024 / (int)sizeof(int) - 2) / 2 - 64; }

static int launch_route_build(const int* ids, int assignments, int experts, int tile_rows, int* counts, int* rank,
                              int* offsets, int* sorted, int* inv_pos, int* tile_expert, int* tile_row0,
                              int* num_tiles, unsigned long long* stats, cudaStream_t stream) {
    se::moe_count_rank_kernel<<<experts, assignments > 2048 ? 1024 : 256, 0, stream>>>(ids, assignments, counts, rank);
    const int blocks = min(se::ceil_div(assignments, 256), 64);
    se::moe_scatter_kernel<<<blocks, 256, (2 * experts + 2) * sizeof(int), stream>>>(
        ids, rank, counts, assignments, experts, tile_rows, offsets, sorted, inv_pos, tile_expert, tile_row0, num_tiles,
        stats);
    SE_LAUNCH_CHECK();
}

// 1 if a routing build of this size is one launch (se_moe_route_gather then gathers the rows in it too).
extern "C" int se_moe_route_is_small(int assignments, int experts) {
    return assignments <= se::kRouteSmallAssignments && experts <= se::kRouteSmallExperts ? 1 : 0;
}

// The routing build and, if x is given, xs[p, :] = x[sorted[p] / top_k, :] (rows of row_bytes
// bytes, a multiple of 16, both 16-byte aligned).  stats (optional, two 64-bit counters):
// [0] += experts with at least one row, [1] += 1.
extern "C" int se_moe_route_gather(const int* ids, int assignments, int experts, int tile_rows, int top_k, int* counts,
                                   int* rank, int* offsets, int* sorted, int* inv_pos, int* tile_expert,
                                   int* tile_row0, int* num_tiles, const void* x, void* xs, int row_bytes,
                                   unsigned long long* stats, cudaStream_t stream) {
    if (assignments <= 0) return 0;
    if (tile_rows <= 0 || experts <= 0 || top_k <= 0) return SE_ERR_ARGUMENT;
    if (experts > se_moe_max_experts()) return SE_ERR_UNSUPPORTED;
    if (x != nullptr && (row_bytes <= 0 || row_bytes % 16 || ((uintptr_t)x & 15) || ((uintptr_t)xs & 15)))
        return SE_ERR_UNSUPPORTED;
    const int row_vecs = x != nullptr ? row_bytes / 16 : 0;
    if (se_moe_route_is_small(assignments, experts)) {
        const size_t smem = (size_t)(3 * assignments + 3 * experts + 2) * sizeof(int);
        const int blocks = x != nullptr ? assignments : 1;
        se::moe_route_small_kernel<<<blocks, 256, smem, stream>>>(
            ids, assignments, experts, tile_rows, top_k, counts, offsets, sorted, inv_pos, tile_expert, tile_row0,
            num_tiles, (const uint4*)x, (uint4*)xs, row_vecs, stats);
        SE_LAUNCH_CHECK();
    }
    const int rc = launch_route_build(ids, assignments, experts, tile_rows, counts, rank, offsets, sorted, inv_pos,
                                      tile_expert, tile_row0, num_tiles, stats, stream);
    if (rc != 0 || x == nullptr) return rc;
    se::gather_sorted_rows_kernel<<<assignments, 128, 0, stream>>>((const uint4*)x, sorted, (uint4*)xs, row_vecs, top_k);
    SE_LAUNCH_CHECK();
}

extern "C" int se_moe_route_build(const int* ids, int assignments, int experts, int tile_rows, int* counts, int* rank,
                                  int* offsets, int* sorted, int* inv_pos, int* tile_expert, int* tile_row0,
                                  int* num_tiles, cudaStream_t stream) {
    return se_moe_route_gather(ids, assignments, experts, tile_rows, 1, counts, rank, offsets, sorted, inv_pos,
                               tile_expert, tile_row0, num_tiles, nullptr, nullptr, 0, nullptr, stream);
}

extern "C" int se_moe_plain_tile_rows() { return se::kBM; }

// mode 0: gate/up + SwiGLU (a = x [tokens, k_dim], w = w13 [E, 2*n_out, k_dim]);
// mode 1: down * routing weight (a = act [assignments, k_dim], w = w2 [E, n_out, k_dim]).
extern "C" int se_moe_grouped_gemm_plain(int mode, const void* a, const void* w, const int* sorted, const int* offsets,
                                         const int* tile_expert, const int* tile_row0, const int* num_tiles,
                                         const float* route_w, void* out, int max_tiles, int n_out, int k_dim,
                                         int top_k, int dtype, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    dim3 grid(max_tiles, se::ceil_div(n_out, se::kBN));
    SE_DISPATCH_DTYPE(dtype, T, {
        if (mode == 0)
            se::grouped_gemm_plain_kernel<T, 0><<<grid, 256, 0, stream>>>(
                (const T*)a, (const T*)w, sorted, offsets, tile_expert, tile_row0, num_tiles, route_w, (T*)out, n_out,
                k_dim, top_k);
        else
            se::grouped_gemm_plain_kernel<T, 1><<<grid, 256, 0, stream>>>(
                (const T*)a, (const T*)w, sorted, offsets, tile_expert, tile_row0, num_tiles, route_w, (T*)out, n_out,
                k_dim, top_k);
    });
    SE_LAUNCH_CHECK();
}

extern "C" int se_moe_combine(const void* y, const int* inv_pos, void* out, int tokens, int hidden, int top_k,
                              int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    SE_DISPATCH_DTYPE(dtype, T,
        se::moe_combine_kernel<T><<<dim3(tokens, se::ceil_div(hidden, 128 * 8)), 128, 0, stream>>>((const T*)y, inv_pos, (T*)out, hidden, top_k));
    SE_LAUNCH_CHECK();
}

// ---- routing build without any allocation (declared in no_alloc.h) -------------------------
// This entry point has no counterpart in CURRENTF/SparseEngine.  It serves callers that may
// not allocate device memory around the call; see no_alloc.h for who they are and for the
// rules of use.  The routing build needs two scratch arrays (per-expert counts, per-
// assignment ranks); here they live in one file-scope device array of fixed size instead
// of coming from the caller.
#include "no_alloc.h"

namespace se {

// counts[SE_NOALLOC_MAX_EXPERTS] followed by rank[SE_NOALLOC_MAX_ASSIGNMENTS]; about 260 KB
// that every GPU which loads this library holds until the process exits.
static __device__ __align__(256) int g_route_scratch[SE_NOALLOC_MAX_EXPERTS + SE_NOALLOC_MAX_ASSIGNMENTS];

// Device address of g_route_scratch per device ordinal.  In host code the array's name is
// only a stand-in for the symbol, not an address a kernel can use, so the address is asked
// for once per device, with that device current.
constexpr int kMaxDevices = 64;
static int* g_route_scratch_ptr[kMaxDevices] = {};

static int route_scratch_for_current_device(int** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return SE_NOALLOC_ERR_DEVICE;
    if (g_route_scratch_ptr[dev] == nullptr) {
        int* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_route_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return SE_NOALLOC_ERR_DEVICE;
        g_route_scratch_ptr[dev] = p;
    }
    *out = g_route_scratch_ptr[dev];
    return 0;
}

}  // namespace se

extern "C" int se_moe_route_build_no_alloc(const int* ids, int assignments, int experts, int tile_rows, int* offsets,
                                           int* sorted, int* inv_pos, int* tile_expert, int* tile_row0,
                                           int* num_tiles, cudaStream_t stream) {
    if (assignments < 0 || experts <= 0 || tile_rows <= 0) return SE_NOALLOC_ERR_ARGUMENT;
    if (assignments > SE_NOALLOC_MAX_ASSIGNMENTS) return SE_NOALLOC_ERR_TOO_MANY_ASSIGNMENTS;
    if (experts > SE_NOALLOC_MAX_EXPERTS) return SE_NOALLOC_ERR_TOO_MANY_EXPERTS;
    if (assignments == 0) return 0;
    int* scratch = nullptr;
    const int rc = se::route_scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
    // Both scratch arrays are written in full by the first kernel before the second reads
    // them (every count, and the rank of every assignment whose expert id is valid), so
    // nothing of the previous call's contents survives into this one and nothing has to be
    // cleared.
    int* counts = scratch;
    int* rank = scratch + SE_NOALLOC_MAX_EXPERTS;
    se::moe_count_rank_kernel<<<experts, assignments > 2048 ? 1024 : 256, 0, stream>>>(ids, assignments, counts, rank);
    const int blocks = min(se::ceil_div(assignments, 256), 64);
    se::moe_scatter_kernel<<<blocks, 256, (2 * experts + 2) * sizeof(int), stream>>>(
        ids, rank, counts, assignments, experts, tile_rows, offsets, sorted, inv_pos, tile_expert, tile_row0, num_tiles,
        nullptr);
    return (int)cudaGetLastError();
}

extern "C" const char* se_no_alloc_strerror(int code) {
    switch (code) {
        case 0: return "success";
        case SE_NOALLOC_ERR_ARGUMENT: return "negative assignments, or experts/tile_rows not positive";
        case SE_NOALLOC_ERR_TOO_MANY_ASSIGNMENTS: return "assignments exceed SE_NOALLOC_MAX_ASSIGNMENTS (65536)";
        case SE_NOALLOC_ERR_TOO_MANY_EXPERTS: return "experts exceed SE_NOALLOC_MAX_EXPERTS (1024)";
        case SE_NOALLOC_ERR_DEVICE: return "no usable device address for the built-in scratch array on the current device";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
    }
}
