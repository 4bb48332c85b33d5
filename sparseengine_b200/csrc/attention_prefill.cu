// Paged attention for prompt portions in bfloat16: one CTA per (batch entry, KV head, tile
// of 64 query rows), where a "row" is one (query token, query head of the GQA group) pair,
// token-major.  A 64-row tile therefore spans a few tokens and all the heads that share the
// KV head, and every K/V tile brought to shared memory is used by all of them.
//
// Flash-attention loop on m16n8k16 tensor-core tiles: each of the four warps owns 16 rows,
// all warps walk the same 64-key tiles (cp.async from the pages, three stages) up to the
// last key the tile's rows may see; scores and the online softmax are 32-bit, P is rounded
// to bfloat16 before P·V, the output is rounded once.  A query at position p sees keys
// max(0, p-window+1)..p of its own request; the portion's own keys were written to the
// cache before this kernel runs.  Reference arithmetic:
// src/sparseengine/kernels/triton/context_flashattention_nopad.py:92-127.
//
// Any page size; head sizes 64 and 128 (others use the plain kernel).  A block-table entry
// outside [0, num_pages) is not followed: its rows are zero-filled and a code goes to the
// error word.
#include "common.cuh"
#include "mma_util.cuh"

namespace se {
namespace pre {

constexpr int kTileKeys = 64;
constexpr int kTileRows = 64;
constexpr int kStages = 3;
constexpr int kWarps = 4;
constexpr int kThreads = 32 * kWarps;

using namespace se::mma;

template <int D>
__global__ void __launch_bounds__(kThreads)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                    const int* __restrict__ table, int table_stride, const int* __restrict__ seq_rows,
                    const int* __restrict__ cu_q, const int* __restrict__ kv_len, __nv_bfloat16* __restrict__ out,
                    int hq, int hkv, int page_size, float scale_log2, int window, int num_pages,
                    int* __restrict__ error) {
    constexpr int kChunks = D / 8;
    constexpr int kTileBytes = kTileKeys * D * 2;
    extern __shared__ __align__(128) uint8_t smem[];

    // Blocks start in the order of their index, x fastest: the KV heads are x, and the row tiles
    // are y taken from the end, so that the tiles with the most keys (the last rows of a causal
    // portion) start first and the short ones fill the tail of the launch.
    const int entry = blockIdx.z, kvh = blockIdx.x;
    const int group = hq / hkv;
    const int tok0 = cu_q[entry];
    const int q_len = cu_q[entry + 1] - tok0;
    const int total_rows = q_len * group;
    const int row_base = (int)(gridDim.y - 1 - blockIdx.y) * kTileRows;
    if (row_base >= total_rows) return;
    const int kv_end = kv_len[entry];                 // keys in the cache after this step's writes
    const int q_start = kv_end - q_len;               // position of the portion's first token
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;

    // rows of this lane: r_lo = warp*16 + g, r_hi = r_lo + 8 (flattened token-major)
    int rows[2], pos[2], tok[2], head[2];
    bool valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        rows[h] = row_base + warp * 16 + g + 8 * h;
        valid[h] = rows[h] < total_rows;
        const int r = valid[h] ? rows[h] : total_rows - 1;
        tok[h] = tok0 + r / group;
        head[h] = kvh * group + r % group;
        pos[h] = q_start + r / group;
    }
    // key range of the CTA: from the first row's window start to the last row's position
    const int last_row = min(row_base + kTileRows, total_rows) - 1;
    const int max_pos = q_start + last_row / group;
    const int first_pos = q_start + row_base / group;
    const int k_lo = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int k_begin = (k_lo / kTileKeys) * kTileKeys;
    const int k_end = max_pos + 1;
    const int num_tiles = (k_end - k_begin + kTileKeys - 1) / kTileKeys;

    const int* row_table = table + (size_t)seq_rows[entry] * table_stride;
    const size_t page_elems = (size_t)2 * hkv * page_size * D;
    const size_t head_off = (size_t)kvh * page_size * D;
    const size_t v_off = (size_t)hkv * page_size * D;

    uint32_t qa[D / 16][4];
    {
        const __nv_bfloat16* q0 = q + ((size_t)tok[0] * hq + head[0]) * D;
        const __nv_bfloat16* q1 = q + ((size_t)tok[1] * hq + head[1]) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int c = kk * 16 + 2 * t4;
            qa[kk][0] = valid[0] ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
            qa[kk][1] = valid[1] ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
            qa[kk][2] = valid[0] ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
            qa[kk][3] = valid[1] ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    int lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) lo[h] = window > 0 ? max(0, pos[h] - window + 1) : 0;

    auto load_tile = [&](int tile, int stage) {
        uint8_t* kbase = smem + (size_t)stage * 2 * kTileBytes;
        uint8_t* vbase = kbase + kTileBytes;
        const int base = k_begin + tile * kTileKeys;
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
            // a key every row of the tile may see (clamped into [k_lo, k_end)): rows outside that range
            // are zero-filled, never read, so a page the window has left behind, which may belong to
            // another request by now, is not touched
            const int jj = min(max(j, k_lo), k_end - 1);
            const int page = row_table[jj / page_size];
            page_ok[k] = page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_ATTN_PREFILL);
            srcs[k] = cache + (size_t)(page_ok[k] ? page : 0) * page_elems + head_off + (size_t)(jj % page_size) * D + c * 8;
        }
#pragma unroll
        for (int k = 0; k < kIters; ++k) {
            const int r = r0t + k * kRowStep;
            const bool ok = base + r < k_end && base + r >= k_lo && page_ok[k];
            cp_async16(smem_u32(kbase) + tile_off<D>(r, c), srcs[k], ok);
            cp_async16(smem_u32(vbase) + tile_off<D>(r, c), srcs[k] + v_off, ok);
        }
    };

    for (int s = 0; s < kStages - 1; ++s) {
        if (s < num_tiles) load_tile(s, s);
        cp_async_commit();
    }
    // the last key any row of this warp may see
    const int warp_last_row = min(row_base + warp * 16 + 15, total_rows - 1);
    const int warp_max_pos = q_start + warp_last_row / group;

    for (int tile = 0; tile < num_tiles; ++tile) {
        cp_async_wait<kStages - 2>();
        __syncthreads();
        if (tile + kStages - 1 < num_tiles) load_tile(tile + kStages - 1, (tile + kStages - 1) % kStages);
        cp_async_commit();

        const int key0 = k_begin + tile * kTileKeys;
        if (key0 > warp_max_pos || row_base + warp * 16 >= total_rows) continue;   // warp-uniform: nothing visible
        const int stage = tile % kStages;
        const uint32_t kaddr = smem_u32(smem + (size_t)stage * 2 * kTileBytes);
        const uint32_t vaddr = kaddr + kTileBytes;

        float s[kTileKeys / 8][4];
#pragma unroll
        for (int n = 0; n < kTileKeys / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < kTileKeys / 16; ++n2) {
                uint32_t b0, b1, b2, b3;
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4(kaddr + tile_off<D>(n2 * 16 + (mat >> 1) * 8 + rr, 2 * kk + (mat & 1)), b0, b1, b2, b3);
                mma_bf16(s[2 * n2], qa[kk], b0, b1);
                mma_bf16(s[2 * n2 + 1], qa[kk], b2, b3);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < kTileKeys / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = key0 + n * 8 + 2 * t4 + (e & 1);
                const int h = e >> 1;
                if (j > pos[h] || j < lo[h]) s[n][e] = -INFINITY;
                mx[h] = fmaxf(mx[h], s[n][e]);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;        // a row that has seen no key yet
            corr[h] = exp2f((m_run[h] - m_use[h]) * scale_log2);
            m_run[h] = m_new;
        }
        float psum[2] = {0.f, 0.f};
        uint32_t pa[kTileKeys / 16][4];
#pragma unroll
        for (int n = 0; n < kTileKeys / 8; ++n) {
            const float p0 = exp2f((s[n][0] - m_use[0]) * scale_log2);
            const float p1 = exp2f((s[n][1] - m_use[0]) * scale_log2);
            const float p2 = exp2f((s[n][2] - m_use[1]) * scale_log2);
            const float p3 = exp2f((s[n][3] - m_use[1]) * scale_log2);
            psum[0] += p0 + p1;
            psum[1] += p2 + p3;
            pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + psum[h];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < kTileKeys / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t b0, b1, b2, b3;
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4_trans(vaddr + tile_off<D>(kk * 16 + (mat & 1) * 8 + rr, 2 * n2 + (mat >> 1)), b0, b1, b2, b3);
                mma_bf16(o[2 * n2], pa[kk], b0, b1);
                mma_bf16(o[2 * n2 + 1], pa[kk], b2, b3);
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!valid[h]) continue;
        const float inv = 1.f / l_run[h];
        __nv_bfloat16* dst = out + ((size_t)tok[h] * hq + head[h]) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
}

template <int D>
static int launch(const void* q, const void* cache, const int* table, int table_stride, const int* seq_rows,
                  const int* cu_q, const int* kv_len, void* out, int entries, int max_q_len, int hq, int hkv,
                  int page_size, float scale, int window, int num_pages, int* error, cudaStream_t stream) {
    const size_t smem = (size_t)kStages * 2 * kTileKeys * D * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group = hq / hkv;
    const int row_tiles = ceil_div(max_q_len * group, kTileRows);
    if (row_tiles > 65535) return SE_ERR_UNSUPPORTED;
    dim3 grid(hkv, row_tiles, entries);
    attn_prefill_kernel<D><<<grid, kThreads, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, table, table_stride, seq_rows, cu_q, kv_len,
        (__nv_bfloat16*)out, hq, hkv, page_size, scale * 1.4426950408889634f, window, num_pages, error);
    return (int)cudaGetLastError();
}

}  // namespace pre
}  // namespace se

// q, out: [tokens, hq, head_dim]; cu_q: [entries + 1] token offsets; kv_len: [entries] keys of each
// request once this step's keys are written; seq_rows: [entries] block-table rows.
extern "C" int se_attn_prefill(const void* q, const void* cache, const int* table, int table_stride,
                               const int* seq_rows, const int* cu_q, const int* kv_len, void* out, int entries,
                               int max_q_len, int hq, int hkv, int head_dim, int page_size, float scale, int window,
                               int num_pages, int* error, cudaStream_t stream) {
    if (entries <= 0 || max_q_len <= 0) return 0;
    if (!(head_dim == 64 || head_dim == 128) || hkv <= 0 || hq % hkv || entries > 65535 || hkv > 65535)
        return SE_ERR_UNSUPPORTED;
    if (head_dim == 64)
        return se::pre::launch<64>(q, cache, table, table_stride, seq_rows, cu_q, kv_len, out, entries, max_q_len, hq,
                                   hkv, page_size, scale, window, num_pages, error, stream);
    return se::pre::launch<128>(q, cache, table, table_stride, seq_rows, cu_q, kv_len, out, entries, max_q_len, hq, hkv,
                                page_size, scale, window, num_pages, error, stream);
}
