// Paged decode attention for bfloat16, split over the keys (flash decoding): one CTA per
// (query token, KV head, key split).  The query heads that share the KV head (the GQA
// group, up to 16) are the 16 rows of m16n8k16 tensor-core tiles, so keys and values are
// read once per group.  K/V rows go from their pages to shared memory with cp.async
// (three 64-key stages), the four warps of the CTA take 16 keys each, keep their own
// running softmax state in 32-bit and are merged at the end; key splits are merged by a
// second kernel through their log-sum-exp.
//
// Arithmetic as in the plain kernel and the reference's split-KV decode
// (src/sparseengine/kernels/triton/gqa_flash_decoding_stage1.py:69-120,
// src/sparseengine/kernels/triton/flash_decoding_stage2.py:27-45): scores and softmax in
// 32-bit, probabilities rounded to bfloat16 before they multiply V, the output rounded once.
//
// Any page size; head sizes 64 and 128 (others use the plain kernel); a window is honoured.
// A block-table entry outside [0, num_pages) is not followed: the rows it stands for are
// zero-filled and a code goes to the error word.
#include "common.cuh"
#include "mma_util.cuh"

namespace se {
namespace dec {

constexpr int kTileKeys = 64;
constexpr int kStages = 3;
constexpr int kWarps = 4;
constexpr int kThreads = 32 * kWarps;

using namespace se::mma;

template <int D>
__global__ void __launch_bounds__(kThreads)
attn_decode_kernel(const __nv_bfloat16* q, const __nv_bfloat16* cache,      // written by the kernel before this one: no __restrict__ (see the wait below)
                   const int* __restrict__ table, int table_stride, const int* __restrict__ seq_rows,
                   const int* __restrict__ token_seq, const int* __restrict__ positions,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int hq,
                   int hkv, int page_size, float scale_log2, int window, int splits, int keys_per_split,
                   int num_pages, int* __restrict__ error) {
    constexpr int kChunks = D / 8;                   // 16-byte chunks per row
    constexpr int kTileBytes = kTileKeys * D * 2;    // one K or V tile
    extern __shared__ __align__(128) uint8_t smem[];

    const int t = blockIdx.x;
    const int group = hq / hkv;
    const int gtiles = (group + 15) / 16;
    const int kvh = blockIdx.y / gtiles, gt = blockIdx.y % gtiles;
    const int split = blockIdx.z;
    const int rows_valid = min(16, group - gt * 16);
    const int head0 = kvh * group + gt * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;

    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int ks = lo + split * keys_per_split;
    const int ke = min(pos + 1, ks + keys_per_split);
    const int* row_table = table + (size_t)seq_rows[token_seq[t]] * table_stride;
    const size_t page_elems = (size_t)2 * hkv * page_size * D;
    const size_t head_off = (size_t)kvh * page_size * D;
    const size_t v_off = (size_t)hkv * page_size * D;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    const int num_tiles = ks < ke ? (ke - ks + kTileKeys - 1) / kTileKeys : 0;

    auto load_tile = [&](int tile, int stage) {
        uint8_t* kbase = smem + (size_t)stage * 2 * kTileBytes;
        uint8_t* vbase = kbase + kTileBytes;
        const int base = ks + tile * kTileKeys;
        // A thread copies chunk (tid % kChunks) of rows tid / kChunks + k * (kThreads / kChunks).  The
        // rows' addresses are looked up first (independent loads), so that no table load sits
        // between the asynchronous copies.
        constexpr int kRowStep = kThreads / kChunks, kIters = kTileKeys / kRowStep;
        static_assert(kThreads % kChunks == 0 && kTileKeys % kRowStep == 0, "tile copy mapping");
        const int c = threadIdx.x % kChunks, r0t = threadIdx.x / kChunks;
        const __nv_bfloat16* srcs[kIters];
        bool page_ok[kIters];
#pragma unroll
        for (int k = 0; k < kIters; ++k) {
            const int j = base + r0t + k * kRowStep;
            const int jj = j < ke ? j : ks;      // any valid key: the copy is zero-filled when out of range
            const int page = row_table[jj / page_size];
            // an entry that names no page of the pool is not followed: its rows are zero-filled
            page_ok[k] = page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_ATTN_DECODE);
            srcs[k] = cache + (size_t)(page_ok[k] ? page : 0) * page_elems + head_off + (size_t)(jj % page_size) * D + c * 8;
        }
#pragma unroll
        for (int k = 0; k < kIters; ++k) {
            const int r = r0t + k * kRowStep;
            const bool ok = base + r < ke && page_ok[k];
            cp_async16(smem_u32(kbase) + tile_off<D>(r, c), srcs[k], ok);
            cp_async16(smem_u32(vbase) + tile_off<D>(r, c), srcs[k] + v_off, ok);
        }
    };

    // Where the step's inputs are older than the kernel before this one (the one that writes the
    // queries and this step's keys), this kernel is launched as its dependent and may have come
    // this far (its place in the block table looked up) while that one runs.  q and the cache
    // are not declared read-only for this kernel's lifetime, or the compiler would be free to
    // move their loads above the wait.
    grid_dependency_wait();
    // Q fragments (A operand, 16 rows x D): rows g and g+8 of this lane
    uint32_t qa[D / 16][4];
    {
        const __nv_bfloat16* q0 = q + ((size_t)t * hq + head0 + g) * D;
        const __nv_bfloat16* q1 = q + ((size_t)t * hq + head0 + g + 8) * D;
        const bool v0 = g < rows_valid, v1 = g + 8 < rows_valid;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int c = kk * 16 + 2 * t4;
            qa[kk][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
            qa[kk][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
            qa[kk][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
            qa[kk][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
        }
    }

    for (int s = 0; s < kStages - 1; ++s) {
        if (s < num_tiles) load_tile(s, s);
        cp_async_commit();
    }

    for (int tile = 0; tile < num_tiles; ++tile) {
        cp_async_wait<kStages - 2>();
        __syncthreads();
        // prefetch the tile that reuses the stage everyone has just finished with
        if (tile + kStages - 1 < num_tiles) load_tile(tile + kStages - 1, (tile + kStages - 1) % kStages);
        cp_async_commit();

        const int stage = tile % kStages;
        const uint32_t kaddr = smem_u32(smem + (size_t)stage * 2 * kTileBytes);
        const uint32_t vaddr = kaddr + kTileBytes;
        const int r0 = warp * 16;                       // this warp's 16 keys of the tile
        const int key0 = ks + tile * kTileKeys + r0;
        if (key0 < ke) {                                // warp-uniform
            float s[2][4] = {};
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t b0, b1, b2, b3;
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4(kaddr + tile_off<D>(r0 + (mat >> 1) * 8 + rr, 2 * kk + (mat & 1)), b0, b1, b2, b3);
                mma_bf16(s[0], qa[kk], b0, b1);
                mma_bf16(s[1], qa[kk], b2, b3);
            }
            // mask keys beyond the range (rows share the token, hence the range)
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + 2 * t4 + (e & 1);
                    if (j >= ke) s[nt][e] = -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);   // finite: key0 < ke, so some key is valid
                corr[h] = exp2f((m_run[h] - m_new) * scale_log2);
                m_run[h] = m_new;
            }
            float psum[2] = {0.f, 0.f};
            uint32_t pa[4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float p0 = exp2f((s[nt][0] - m_run[0]) * scale_log2);
                const float p1 = exp2f((s[nt][1] - m_run[0]) * scale_log2);
                const float p2 = exp2f((s[nt][2] - m_run[1]) * scale_log2);
                const float p3 = exp2f((s[nt][3] - m_run[1]) * scale_log2);
                psum[0] += p0 + p1;
                psum[1] += p2 + p3;
                pa[nt * 2 + 0] = pack_bf16(p0, p1);
                pa[nt * 2 + 1] = pack_bf16(p2, p3);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + psum[h];
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {       // two 8-wide dim tiles per ldmatrix
                uint32_t b0, b1, b2, b3;
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4_trans(vaddr + tile_off<D>(r0 + (mat & 1) * 8 + rr, 2 * n2 + (mat >> 1)), b0, b1, b2, b3);
                mma_bf16(o[2 * n2], pa, b0, b1);
                mma_bf16(o[2 * n2 + 1], pa, b2, b3);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four warps (shared memory is free now) ----------------------------------
    for (int h = 0; h < 2; ++h) {        // row sums live in 4 lanes each
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* sm_m = reinterpret_cast<float*>(smem);                 // [warps][16]
    float* sm_l = sm_m + kWarps * 16;
    float* sm_o = sm_l + kWarps * 16;                             // [warps][16][D]
    if (t4 == 0) {
        sm_m[warp * 16 + g] = m_run[0];
        sm_m[warp * 16 + g + 8] = m_run[1];
        sm_l[warp * 16 + g] = l_run[0];
        sm_l[warp * 16 + g + 8] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + 2 * t4;
        float* r_lo = sm_o + ((size_t)warp * 16 + g) * D + c;
        float* r_hi = sm_o + ((size_t)warp * 16 + g + 8) * D + c;
        r_lo[0] = o[i][0]; r_lo[1] = o[i][1];
        r_hi[0] = o[i][2]; r_hi[1] = o[i][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows_valid * D; i += kThreads) {
        const int r = i / D, d = i % D;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, sm_m[w * 16 + r]);
        float acc = 0.f, lt = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float mw = sm_m[w * 16 + r];
            const float f = mw == -INFINITY ? 0.f : exp2f((mw - mt) * scale_log2);
            acc += sm_o[((size_t)w * 16 + r) * D + d] * f;
            lt += sm_l[w * 16 + r] * f;
        }
        const int head = head0 + r;
        if (splits == 1) {
            out[((size_t)t * hq + head) * D + d] = __float2bfloat16_rn(acc / lt);
        } else {
            const size_t pidx = ((size_t)t * hq + head) * splits + split;
            part_o[pidx * D + d] = acc;
            if (d == 0) {
                part_ml[pidx * 2] = mt == -INFINITY ? -INFINITY : mt * scale_log2;
                part_ml[pidx * 2 + 1] = lt;
            }
        }
    }
}

// out[t, h, :] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int d, int splits) {
    grid_dependency_trigger();       // the output projection that follows may start streaming its weights
    const size_t th = blockIdx.x;
    float mt = -INFINITY;
    for (int s = 0; s < splits; ++s) mt = fmaxf(mt, part_ml[(th * splits + s) * 2]);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.f, lt = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(th * splits + s) * 2];
            if (ms == -INFINITY) continue;
            const float f = exp2f(ms - mt);
            acc += part_o[(th * splits + s) * d + i] * f;
            lt += part_ml[(th * splits + s) * 2 + 1] * f;
        }
        out[th * d + i] = __float2bfloat16_rn(acc / lt);
    }
}

template <int D>
static int launch(const void* q, const void* cache, const int* table, int table_stride, const int* seq_rows,
                  const int* token_seq, const int* positions, void* out, float* part_o, float* part_ml, int tokens,
                  int hq, int hkv, int page_size, float scale, int window, int splits, int keys_per_split,
                  int num_pages, int* error, int settled, cudaStream_t stream) {
    const int group = hq / hkv;
    const int gtiles = (group + 15) / 16;
    const size_t stage_smem = (size_t)kStages * 2 * kTileKeys * D * 2;
    const size_t merge_smem = (size_t)kWarps * 16 * (D + 2) * sizeof(float);
    const size_t smem = stage_smem > merge_smem ? stage_smem : merge_smem;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(tokens, hkv * gtiles, splits);
    cudaError_t e = SE_LAUNCH_DEPENDENT_IF(
        settled != 0, "attn", attn_decode_kernel<D>, grid, dim3(kThreads), smem, stream, (const __nv_bfloat16*)q,
        (const __nv_bfloat16*)cache, table, table_stride, seq_rows, token_seq, positions, (__nv_bfloat16*)out, part_o,
        part_ml, hq, hkv, page_size, scale * 1.4426950408889634f, window, splits, keys_per_split, num_pages, error);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (splits > 1) {
        attn_combine_kernel<<<tokens * hq, 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, D, splits);
        e = cudaGetLastError();
    }
    return (int)e;
}

}  // namespace dec
}  // namespace se

extern "C" int se_attn_decode_supported(int head_dim, int hq, int hkv) {
    return ((head_dim == 64 || head_dim == 128) && hkv > 0 && hq % hkv == 0) ? 1 : 0;
}

// part_o: float [tokens, hq, splits, head_dim]; part_ml: float [tokens, hq, splits, 2] (unused when splits == 1).
// keys_per_split is a multiple of 64; split s of a token covers keys lo + s*keys_per_split ...
// settled: positions, token_seq, seq_rows and the block table were complete before the kernel
// launched just before this one began (they are inputs of the step, and that kernel is the one
// that writes the queries and the step's keys).  The attention kernel is then launched as that
// kernel's dependent and reads them while it may still run; else it is launched the ordinary way.
extern "C" int se_attn_decode(const void* q, const void* cache, const int* table, int table_stride,
                              const int* seq_rows, const int* token_seq, const int* positions, void* out,
                              float* part_o, float* part_ml, int tokens, int hq, int hkv, int head_dim, int page_size,
                              float scale, int window, int splits, int keys_per_split, int num_pages, int* error,
                              int settled, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (!se_attn_decode_supported(head_dim, hq, hkv) || splits < 1 || keys_per_split <= 0 || keys_per_split % 64)
        return SE_ERR_UNSUPPORTED;
    if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return SE_ERR_ARGUMENT;
    if (head_dim == 64)
        return se::dec::launch<64>(q, cache, table, table_stride, seq_rows, token_seq, positions, out, part_o, part_ml,
                                   tokens, hq, hkv, page_size, scale, window, splits, keys_per_split, num_pages, error,
                                   settled, stream);
    return se::dec::launch<128>(q, cache, table, table_stride, seq_rows, token_seq, positions, out, part_o, part_ml,
                                tokens, hq, hkv, page_size, scale, window, splits, keys_per_split, num_pages, error,
                                settled, stream);
}
