// Prompt-portion attention on 5th-generation tensor cores (bfloat16, head size 128).
//
// One CTA per (batch entry, KV head, 256 query rows); a row is one (query token, query head
// of the GQA group) pair, token-major, so 128 rows span ~21 tokens of M2 and all six heads
// that share the KV head.  The CTA holds two query tiles of 128 rows, each with its own four
// softmax warps and its own MMA-issuing warp; the two tiles take turns on the tensor pipe and
// share every 64-key K/V tile that is loaded.  Per query tile and K/V tile:
//
//   S = Q·Kᵀ        tcgen05.mma, M 128 x N 64 x K 128, Q and K K-major in shared memory
//                   (128-byte swizzle), S in tensor memory (two buffers per query tile);
//   softmax         four warps, one thread per row: tcgen05.ld of its row of S, mask
//                   (causal, window, end of keys), running maximum and sum in 32-bit, P
//                   rounded to bfloat16 and written back to tensor memory over the row's
//                   scores (tcgen05.st, two values per column);
//   O += P·V        tcgen05.mma with the A operand (P) in tensor memory, M 128 x N 128 x K 64,
//                   V straight from its pages (dims contiguous: the MN-major B operand), O in
//                   tensor memory.
//
// Tensor memory is used in full: O of the two tiles (2 x 128 columns) and their S buffers
// (2 x 2 x 64), whose first halves hold P between the softmax and P·V; shared memory holds
// the two Q tiles and five K/V stages.  The running maximum only moves when a row's maximum grows by more than 2^8
// (then O and the sum are rescaled), so O is read back from tensor memory rarely; the final
// division by the sum is exact for whatever reference maximum was used.
//
// Warp roles (12 warps): warps 0 and 10 gather K/V tiles from their pages with cp.async into
// five stages, alternately, and tie each tile's barrier to their copies
// (cp.async.mbarrier.arrive.noinc), so a tile is announced the moment it has landed and the
// loaders never wait for data; warp 1 owns tensor memory and issues the MMAs of query tile 0,
// warp 11 those of tile 1 (S(j) first, then P·V of tile j-1 as its P arrives), independently
// of one another; warps 2-5 and 6-9 are the softmax/epilogue warps of tiles 0 and 1.  A K/V
// stage is free again when both issuers have committed its P·V.  Every mbarrier wait is
// bounded and reports through the error word.  Arithmetic as the reference's prefill kernel
// (src/sparseengine/kernels/triton/context_flashattention_nopad.py:92-127).
#include "common.cuh"
#include "mma_util.cuh"

namespace se {
namespace fa {

constexpr int D = 128;
constexpr int kRows = 128;
constexpr int kKeys = 64;
constexpr int kTiles = 2;                            // query tiles per CTA
constexpr int kStages = 5;
constexpr int kLoaderWarp2 = 2 + 4 * kTiles;         // the second loader warp
constexpr int kMmaWarp2 = kLoaderWarp2 + 1;          // the MMA issuer of query tile 1 (tile 0: warp 1)
constexpr int kThreads = 32 * (kMmaWarp2 + 1);       // loader, MMA, 4 softmax warps per query tile, loader, MMA
constexpr int kHalfBytes = 64 * 128;                 // [64 rows][64 dims] bf16: rows of 128 bytes
constexpr int kQBytes = 2 * kRows * 128;             // two dim-halves of [128 rows][64 dims]
constexpr int kKVStageBytes = 4 * kHalfBytes;        // K halves, V halves
constexpr uint32_t kSpin = 1u << 24;
constexpr float kRescaleThreshold = 8.f;             // log2 units

using se::mma::smem_u32;
using se::mma::cp_async16;
using se::mma::cp_async_commit;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpin; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
// rows of 128 bytes, 16-byte chunks XOR-swizzled by (row % 8): the canonical 128-byte-swizzle image
__device__ __forceinline__ uint32_t sw128(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// K-major operand (rows = M or N index, 64 contiguous K elements per 128-byte row)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand: 64 contiguous N elements per 128-byte row, rows = K index; 8-row groups
// 1024 bytes apart (stride offset), 64-element N groups `lbo` bytes apart (leading offset)
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint32_t idesc(int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(id), "r"(acc) : "memory");
}
// the same with the A operand in tensor memory (rows = lanes, two bfloat16 per 32-bit column)
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a_tmem), "l"(b), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Bars {
    uint64_t kv_full[kStages], kv_empty[kStages];
    uint64_t s_full[kTiles][2], s_empty[kTiles][2];      // per query tile: two S buffers
    uint64_t p_full[kTiles][2], p_empty[kTiles];         // per query tile: P of a tile is complete (one per S buffer); its P·V has finished
    uint64_t o_done[kTiles];                             // per query tile: the last P·V has finished (a warp that never had to
                                                         // wait for p_empty may be phases behind it, so the end has a barrier of its own)
};

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                       const int* __restrict__ table, int table_stride, const int* __restrict__ seq_rows,
                       const int* __restrict__ cu_q, const int* __restrict__ kv_len, __nv_bfloat16* __restrict__ out,
                       int* error, int hq, int hkv, int page_size, float scale_log2, int window, int num_pages) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;                               // [2 tiles][2 halves][128 rows][128 B]
    uint8_t* kv_s = q_s + kTiles * kQBytes;            // [stages][K half0, K half1, V half0, V half1]
    __shared__ __align__(8) Bars bars;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;

    // Blocks start in the order of their index, x fastest: the KV heads are x, and the row tiles
    // are y taken from the end, so that the tiles with the most keys (the last rows of a causal
    // portion) start first and the short ones fill the tail of the launch.
    const int entry = blockIdx.z, kvh = blockIdx.x;
    const int group = hq / hkv;
    const int tok0 = cu_q[entry];
    const int q_len = cu_q[entry + 1] - tok0;
    const int total_rows = q_len * group;
    const int row_base = (int)(gridDim.y - 1 - blockIdx.y) * (kTiles * kRows);
    if (row_base >= total_rows) return;
    const int kv_end = kv_len[entry];
    const int q_start = kv_end - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int last_row = min(row_base + kTiles * kRows, total_rows) - 1;
    const int max_pos = q_start + last_row / group;
    const int first_pos = q_start + row_base / group;
    const int k_lo = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int k_begin = (k_lo / kKeys) * kKeys;
    const int k_end = max_pos + 1;
    const int num_tiles = (k_end - k_begin + kKeys - 1) / kKeys;

    auto bar = [&](uint64_t* b) { return smem_u32(b); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bar(&bars.kv_full[s]), 32); mbar_init(bar(&bars.kv_empty[s]), kTiles); }   // full: every lane of the tile's loader warp; empty: both query tiles' MMAs
        for (int x = 0; x < kTiles; ++x) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(bar(&bars.s_full[x][b]), 1);
                mbar_init(bar(&bars.s_empty[x][b]), 4);      // one arrival per softmax warp
            }
            mbar_init(bar(&bars.p_full[x][0]), 4);
            mbar_init(bar(&bars.p_full[x][1]), 4);
            mbar_init(bar(&bars.p_empty[x]), 1);
            mbar_init(bar(&bars.o_done[x]), 1);
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Q tiles: every thread copies chunks; rows beyond the portion's rows are zero-filled
    for (int i = threadIdx.x; i < kTiles * kRows * 16; i += kThreads) {
        const int r = i >> 4, c = i & 15;                  // r: 0..255 over both tiles
        const int row = row_base + r;
        const bool ok = row < total_rows;
        const int rr = ok ? row : total_rows - 1;
        const __nv_bfloat16* src = q + ((size_t)(tok0 + rr / group) * hq + kvh * group + rr % group) * D + c * 8;
        cp_async16(smem_u32(q_s) + (r >> 7) * kQBytes + (c >> 3) * (kRows * 128) + sw128(r & 127, c & 7), src, ok);
    }
    cp_async_commit();
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    // tensor memory: O of tile x in columns 128 x .. 128 x + 127; S buffer b of tile x in 256 + 128 x + 64 b ..
    auto tmem_o = [&](int x) { return tmem + (uint32_t)(128 * x); };
    auto tmem_s = [&](int x, int b) { return tmem + (uint32_t)(256 + 128 * x + 64 * b); };

    const int* row_table = table + (size_t)seq_rows[entry] * table_stride;
    const size_t page_elems = (size_t)2 * hkv * page_size * D;
    const size_t head_off = (size_t)kvh * page_size * D;
    const size_t v_off = (size_t)hkv * page_size * D;

    if (warp == 0 || warp == kLoaderWarp2) {
        // ---- loaders: K/V tiles from their pages ------------------------------------------
        // Lane l looks up where keys base+l and base+32+l live (two independent table loads per
        // lane and tile); the copy loop gets each row's address by shuffle, so no load sits
        // between the asynchronous copies.
        auto issue = [&](int tile) {
            uint8_t* st = kv_s + (size_t)(tile % kStages) * kKVStageBytes;
            const int base = k_begin + tile * kKeys;
            // Keys outside [k_lo, k_end) are zero-filled, never read: a page the window has left
            // behind may belong to another request by now.  An entry that names no page of the pool
            // is not followed either (address 0 marks its row; a code goes to the error word).
            unsigned long long src_row[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int j = min(max(base + 32 * h + lane, k_lo), k_end - 1);
                const int page = row_table[j / page_size];
                const bool in_pool = page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_ATTN_PREFILL_TC);
                src_row[h] = in_pool ? (unsigned long long)(cache + (size_t)page * page_elems + head_off + (size_t)(j % page_size) * D) : 0ull;
            }
            const int c = lane & 15;
#pragma unroll 4
            for (int k = 0; k < kKeys / 2; ++k) {
                const int r = 2 * k + (lane >> 4);
                const unsigned long long a = __shfl_sync(0xffffffffu, src_row[0], r & 31);
                const unsigned long long b = __shfl_sync(0xffffffffu, src_row[1], r & 31);
                const unsigned long long row_addr = r < 32 ? a : b;
                const bool ok = base + r < k_end && base + r >= k_lo && row_addr != 0ull;
                const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(ok ? row_addr : (unsigned long long)cache) + c * 8;
                const uint32_t off = (c >> 3) * kHalfBytes + sw128(r, c & 7);
                cp_async16(smem_u32(st) + off, src, ok);
                cp_async16(smem_u32(st) + 2 * kHalfBytes + off, src + v_off, ok);
            }
        };
        // Two loader warps take alternate tiles and run ahead as far as stages are free.  Each
        // lane ties the tile's barrier to its own copies (cp.async.mbarrier.arrive.noinc: the
        // arrival happens when the lane's earlier copies have landed), so the warp never waits
        // for data and a tile is announced the moment it is complete.
        const int first = warp == 0 ? 0 : 1;
        bool ok = true;
        for (int tile = first; tile < num_tiles && ok; tile += 2) {
            if (tile >= kStages) ok = mbar_wait(bar(&bars.kv_empty[tile % kStages]), ((tile / kStages) - 1) & 1, &abort_s);
            if (!ok) break;
            issue(tile);
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(&bars.kv_full[tile % kStages])) : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (!ok) { abort_s = 1; if (lane == 0) atomicCAS(error, 0, 11); }
    } else if (warp == 1 || warp == kMmaWarp2) {
        // ---- MMA issuers: one warp (one lane) per query tile ---------------------------------------
        // Order for a tile: S(j), then P·V of tile j-1 as its P arrives; S(j+1) is thus issued
        // before the softmax of tile j has finished.  The two issuers share the tensor pipe and
        // do not wait for one another; a K/V stage is free when both have committed its P·V.
        if (lane == 0) {
            const int x = warp == 1 ? 0 : 1;
            const uint32_t id_s = idesc(kKeys, 0), id_o = idesc(D, 1);
            bool ok = true;
            auto issue_pv = [&](int i) {
                if (!mbar_wait(bar(&bars.p_full[x][i & 1]), (i >> 1) & 1, &abort_s)) { ok = false; return; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t va = smem_u32(kv_s) + (i % kStages) * kKVStageBytes + 2 * kHalfBytes;
                const uint32_t pa = tmem_s(x, i & 1);        // P of tile i lies over the first half of its S buffer
#pragma unroll
                for (int kk = 0; kk < kKeys / 16; ++kk)      // 16 keys per MMA: 8 columns of P, two 8-key groups of V
                    umma_ts(tmem_o(x), pa + (uint32_t)(kk * 8), desc_mnmajor(va + kk * 2048, kHalfBytes), id_o,
                            (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(bar(&bars.p_empty[x]));
                umma_commit(bar(&bars.kv_empty[i % kStages]));
            };
            for (int j = 0; j < num_tiles && ok; ++j) {
                const int b = j & 1;
                if (!mbar_wait(bar(&bars.kv_full[j % kStages]), (j / kStages) & 1, &abort_s)) { ok = false; break; }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the copies were generic-proxy writes
                if (j >= 2 && !mbar_wait(bar(&bars.s_empty[x][b]), ((j >> 1) - 1) & 1, &abort_s)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t ka = smem_u32(kv_s) + (j % kStages) * kKVStageBytes;
#pragma unroll
                for (int kb = 0; kb < 2; ++kb)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(tmem_s(x, b), desc_kmajor(smem_u32(q_s) + x * kQBytes + kb * (kRows * 128)) + (uint64_t)(kk * 2),
                             desc_kmajor(ka + kb * kHalfBytes) + (uint64_t)(kk * 2), id_s, (kb > 0 || kk > 0) ? 1u : 0u);
                umma_commit(bar(&bars.s_full[x][b]));
                if (j >= 1) issue_pv(j - 1);
            }
            if (ok) issue_pv(num_tiles - 1);
            if (ok) umma_commit(bar(&bars.o_done[x]));
            if (!ok) { abort_s = 1; atomicCAS(error, 0, 12); }
        }
    } else if (warp < 2 + 4 * kTiles) {
        // ---- softmax and epilogue: warps 2-5 own query tile 0, warps 6-9 tile 1; one thread per row ----
        const int x = (warp - 2) >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                 // row of the tile = TMEM lane
        const int row = row_base + x * kRows + r;
        const bool valid = row < total_rows;
        const int rr = valid ? row : total_rows - 1;
        const int pos = q_start + rr / group;
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        float m_ref = -INFINITY, l = 0.f;                  // reference maximum (log2 units), running sum
        bool ok = true;
        for (int j = 0; j < num_tiles && ok; ++j) {
            const int b = j & 1;
            if (!mbar_wait(bar(&bars.s_full[x][b]), (j >> 1) & 1, &abort_s)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sv[64];
            tmem_ld32(tmem_s(x, b) + lane_addr, sv);
            tmem_ld32(tmem_s(x, b) + 32 + lane_addr, sv + 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(&bars.s_empty[x][b]));
            const int key0 = k_begin + j * kKeys;
            // A tile every row of the warp sees in full needs no masking (rows ascend with the
            // lane: lane 0 has the smallest position, lane 31 the largest window start).
            const bool full = key0 + kKeys - 1 <= __shfl_sync(0xffffffffu, pos, 0) &&
                              key0 >= __shfl_sync(0xffffffffu, lo, 31);
            if (!full) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int key = key0 + c;
                    if (key > pos || key < lo) sv[c] = 0xff800000u;      // -inf
                }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one of 64
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                m4[0] = fmaxf(m4[0], __uint_as_float(sv[c]));
                m4[1] = fmaxf(m4[1], __uint_as_float(sv[c + 1]));
                m4[2] = fmaxf(m4[2], __uint_as_float(sv[c + 2]));
                m4[3] = fmaxf(m4[3], __uint_as_float(sv[c + 3]));
            }
            float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            mx *= scale_log2;                                            // log2 units (scale > 0)
            // move the reference maximum only on the first visible keys or a large jump
            float factor = 1.f;
            bool need = false;
            if (mx > m_ref + kRescaleThreshold || (m_ref == -INFINITY && mx != -INFINITY)) {
                factor = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
                need = m_ref != -INFINITY;
                m_ref = mx;
                l *= factor;
            }
            if (__any_sync(0xffffffffu, need)) {
                // O must be at rest: P·V of the previous tile has finished.  (Only then: a warp whose
                // rows keep their reference maximum runs on, up to a tile ahead of the others, which
                // is why P's barrier exists once per S buffer.)
                if (j >= 1 && !mbar_wait(bar(&bars.p_empty[x]), (j - 1) & 1, &abort_s)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem_o(x) + c0 + lane_addr, ov);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * (need ? factor : 1.f));
                    tmem_st32(tmem_o(x) + c0 + lane_addr, ov);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            const float neg_m = -m_use;
            // P goes back to tensor memory, over the row's own scores (which are in registers now):
            // two bfloat16 per column, the A operand of P·V.
            uint32_t packed[32];
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // p = 2^(s * scale - m): one fused multiply-add and one ex2 per element
                    const float p0 = ex2(fmaf(__uint_as_float(sv[c8 * 8 + 2 * i]), scale_log2, neg_m));
                    const float p1 = ex2(fmaf(__uint_as_float(sv[c8 * 8 + 2 * i + 1]), scale_log2, neg_m));
                    sum4[i] += p0 + p1;
                    packed[c8 * 4 + i] = se::mma::pack_bf16(p0, p1);
                }
            }
            tmem_st32(tmem_s(x, b) + lane_addr, packed);
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(&bars.p_full[x][b]));
        }
        if (ok && mbar_wait(bar(&bars.o_done[x]), 0, &abort_s)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = 1.f / l;
            __nv_bfloat16* dst = out + ((size_t)(tok0 + rr / group) * hq + kvh * group + rr % group) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem_o(x) + c0 + lane_addr, ov);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (valid) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            w[i] = se::mma::pack_bf16(__uint_as_float(ov[c + 2 * i]) * inv, __uint_as_float(ov[c + 2 * i + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        } else {
            abort_s = 1;
            atomicCAS(error, 0, 13);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace fa
}  // namespace se

extern "C" int se_attn_prefill_tc_supported(int head_dim, int hq, int hkv) {
    return (head_dim == 128 && hkv > 0 && hq % hkv == 0) ? 1 : 0;
}

extern "C" int se_attn_prefill_tc(const void* q, const void* cache, const int* table, int table_stride,
                                  const int* seq_rows, const int* cu_q, const int* kv_len, void* out, int* error,
                                  int entries, int max_q_len, int hq, int hkv, int head_dim, int page_size, float scale,
                                  int window, int num_pages, cudaStream_t stream) {
    using namespace se::fa;
    if (entries <= 0 || max_q_len <= 0) return 0;
    if (!se_attn_prefill_tc_supported(head_dim, hq, hkv) || entries > 65535 || hkv > 65535) return SE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)kTiles * kQBytes + kStages * kKVStageBytes + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group = hq / hkv;
    const int row_tiles = se::ceil_div(max_q_len * group, kTiles * kRows);
    if (row_tiles > 65535) return SE_ERR_UNSUPPORTED;
    dim3 grid(hkv, row_tiles, entries);
    attn_prefill_tc_kernel<<<grid, kThreads, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, table, table_stride, seq_rows, cu_q, kv_len,
        (__nv_bfloat16*)out, error, hq, hkv, page_size, scale * 1.4426950408889634f, window, num_pages);
    return (int)cudaGetLastError();
}
