// Grouped expert GEMMs on a pair of SMs: two CTAs (a cluster of 2) share one 256 x 256 tile.
//
// The one-CTA kernel of gemm_tc.cu is at its best where the weights stream from HBM (few rows
// per expert).  With hundreds of rows per expert the tensor cores should bind, and there one
// CTA per tile takes too many bytes per flop from L2 and shared memory.  Here the MMA is
// `tcgen05.mma.cta_group::2`: M = 256 weight rows (128 in each CTA's shared memory and tensor
// memory), N = up to 256 activation rows of which each CTA loads one half, so a CTA brings
// 32 KB per 64-wide K block for 512 tensor-core cycles.  Each CTA loads its own operands with
// plain per-CTA TMA (no multicast); the transaction bytes of both land on the leader's
// barrier.  One elected thread of the leader CTA (cluster rank 0) issues the MMAs of the pair
// and commits them to the barriers of both CTAs.
//
//   MODE_GATE_UP  a CTA's 128 A rows are 64 gate rows and the 64 up rows of the same output
//                 features (two TMA boxes), so one accumulator (256 columns) holds both and the
//                 other 256 columns of tensor memory take the next item: the SwiGLU epilogue of
//                 item j runs while the MMAs of item j + 1 do.  The warps that own the gate lanes and
//                 those that own the up lanes exchange their values through shared memory and share
//                 the SiLU and the stores.
//   MODE_DOWN     128 rows of w2[e] per CTA; epilogue multiplies by the routing weight.
//
// Work items (tile of activation rows x block of output features) are dealt round-robin to
// the pairs; a tile with fewer than 256 rows runs MMAs of its own rows only (N is a field of
// the instruction descriptor; the two CTAs then split the N rows that exist).  Warp roles as
// in gemm_tc.cu: warp 0 loads, warp 1 owns tensor memory and (in the leader) issues the MMAs,
// warps 2-5 run the epilogue.  Every wait is bounded and reports through the error word; the
// CTAs of a pair leave together.  Arithmetic and rounding points are those of gemm_tc.cu
// (src/sparseengine/kernels/triton/moe.py:557-563,726-732,1374-1440).
#include "common.cuh"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace se {
namespace tcp {

constexpr int kBlockK = 64;            // bf16 elements: 128 bytes, one swizzle span
constexpr int kUmmaK = 16;
constexpr int kCtaM = 128;             // weight rows per CTA
constexpr int kHalfN = 128;            // activation rows a CTA loads (half of the pair's 256)
constexpr int kTileN = 2 * kHalfN;
constexpr int kABytes = kCtaM * kBlockK * 2;
constexpr int kBBytes = kHalfN * kBlockK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStages = 6;
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr int kXchCols = 32;           // columns the up warps hand over at a time

enum Mode { MODE_GATE_UP = 0, MODE_DOWN = 1 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// arrive on a barrier anywhere in the cluster (`bar` is a shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
// A tile into this CTA's shared memory; the bytes are counted on `bar`, a shared::cluster
// address (the leader's barrier).  No multicast: every CTA fetches what it needs itself.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16, bf16 x bf16 -> fp32, both operands K-major, M = 256 over the pair
__device__ __forceinline__ uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs when the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
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

struct Params {
    const int* sorted;          // [assignments] flat assignment of each sorted row
    const int* offsets;         // [experts + 1]
    const int* tile_expert;     // [max_tiles]
    const int* tile_row0;       // tiles of up to 256 rows
    const int* num_tiles;
    const float* route_w;       // [assignments] (MODE_DOWN)
    __nv_bfloat16* out;         // [rows, n_out]
    int* error;
    int n_out;                  // output features per expert (I for gate/up, H for down)
    int k_dim;
    int w_rows_per_expert;      // 2I or H
    int up_offset;              // row offset of the up rows inside an expert (MODE_GATE_UP)
};

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
    // output features per item: the pair's 256 A rows are 128 gate + 128 up rows, or 256 rows of w2
    constexpr int kItemFeatures = MODE == MODE_GATE_UP ? 128 : 256;
    constexpr int kCtaFeatures = kItemFeatures / 2;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles = p.num_tiles[0];
    const int n_blocks = (p.n_out + kItemFeatures - 1) / kItemFeatures;
    const int items = tiles * n_blocks;
    const int num_kb = (p.k_dim + kBlockK - 1) / kBlockK;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * kStages + 4];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;
    __shared__ float route_s[2][kTileN];
    // [buffer][gate | up][column][feature] (lanes walk features); only the gate/up epilogue exchanges values
    __shared__ __align__(16) __nv_bfloat16 xch_s[2][2][kXchCols][MODE == MODE_GATE_UP ? kCtaFeatures : 1];
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * kStages]), acc_empty0 = smem_u32(&bars[2 * kStages + 2]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);          // the leader's own arrival with the bytes of both CTAs (used in the leader)
            mbar_init(empty0 + 8 * s, 1);         // the pair's MMA commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);      // the pair's MMA commit
            mbar_init(acc_empty0 + 8 * b, 8);     // four epilogue warps of each CTA (used in the leader)
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {      // the same warp in both CTAs: tensor memory of the pair (two accumulators of 256 columns)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();           // both CTAs' barriers exist before anything of the peer touches them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    // what item `item` is: (tile, block of features) -> expert, first row, rows it holds
    auto item_info = [&](int item, int* expert, int* row0, int* valid, int* nb) {
        const int tile = item / n_blocks;
        *nb = item % n_blocks;
        *expert = p.tile_expert[tile];
        *row0 = p.tile_row0[tile];
        *valid = min(kTileN, p.offsets[*expert + 1] - *row0);
    };

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t leader_full0 = map_to_cta(full0, 0);
            int it = 0;
            bool ok = true;
            for (int item = pair; item < items && ok; item += num_pairs) {
                int expert, row0, valid, nb;
                item_info(item, &expert, &row0, &valid, &nb);
                const int n_mma = max(16, (valid + 15) & ~15);
                const int b_row = row0 + (int)rank * (n_mma / 2);                      // this CTA's half of the rows
                const int w_row = expert * p.w_rows_per_expert + nb * kItemFeatures + (int)rank * kCtaFeatures;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(empty0 + 8 * s, ((it / kStages) & 1) ^ 1, &abort_s)) {
                        abort_s = 1;
                        atomicCAS(p.error, 0, 1);
                        ok = false;
                        break;
                    }
                    const uint32_t a = smem_u32(smem + (size_t)s * kStageBytes);
                    if (leader) mbar_expect_tx(full0 + 8 * s, 2 * kStageBytes);
                    const uint32_t bar = leader_full0 + 8 * s;
                    if (MODE == MODE_GATE_UP) {       // 64 gate rows, then the 64 up rows of the same features
                        tma_load_2d(a, &map_w, bar, kb * kBlockK, w_row);
                        tma_load_2d(a + kABytes / 2, &map_w, bar, kb * kBlockK, w_row + p.up_offset);
                    } else {
                        tma_load_2d(a, &map_w, bar, kb * kBlockK, w_row);
                    }
                    tma_load_2d(a + kABytes, &map_x, bar, kb * kBlockK, b_row);
                }
            }
            if (abort_s && leader) {
                // let what is in flight land before this CTA's shared memory goes away
                for (int k = max(0, it - kStages); k < it; ++k)
                    for (uint32_t i = 0; i < kSpinLimit && !mbar_try_wait(full0 + 8 * (k % kStages), (k / kStages) & 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            int it = 0, used = 0;
            bool ok = true;
            for (int item = pair; item < items && ok; item += num_pairs, ++used) {
                int expert, row0, valid, nb;
                item_info(item, &expert, &row0, &valid, &nb);
                const uint32_t idesc = instr_desc(max(16, (valid + 15) & ~15));
                const int b = used & 1;
                if (!mbar_wait(acc_empty0 + 8 * b, ((used >> 1) & 1) ^ 1, &abort_s)) {     // both CTAs have drained buffer b
                    abort_s = 1;
                    atomicCAS(p.error, 0, 4);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)(b * kTileN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(full0 + 8 * s, (it / kStages) & 1, &abort_s)) {
                        abort_s = 1;
                        atomicCAS(p.error, 0, 2);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a = smem_u32(smem + (size_t)s * kStageBytes);
                    const uint64_t da = smem_desc(a), db = smem_desc(a + kABytes);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                        const uint64_t adv = (uint64_t)((kk * kUmmaK * 2) >> 4);
                        umma_pair(acc, da + adv, db + adv, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty0 + 8 * s);        // frees the stage in both CTAs
                }
                if (!ok) break;
                umma_commit_pair(acc_full0 + 8 * b);         // the accumulator of both CTAs is complete
            }
        }
    } else {
        const int quarter = warp & 3;                 // the TMEM lanes this warp may read: 32 * quarter ..
        const uint32_t leader_acc_empty0 = map_to_cta(acc_empty0, 0);
        const int et = (quarter * 32 + lane);         // 0..127 = TMEM lane = A row of this CTA
        int used = 0, chunk = 0;
        for (int item = pair; item < items; item += num_pairs, ++used) {
            int expert, row0, valid, nb;
            item_info(item, &expert, &row0, &valid, &nb);
            const int b = used & 1;
            if (MODE == MODE_DOWN) {
                for (int e = et; e < kTileN; e += 128) route_s[b][e] = e < valid ? p.route_w[p.sorted[row0 + e]] : 0.f;
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (!mbar_wait(acc_full0 + 8 * b, (used >> 1) & 1, &abort_s)) {
                abort_s = 1;
                atomicCAS(p.error, 0, 3);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * kTileN);
            if (MODE == MODE_GATE_UP) {
                // Lanes 0-63 hold gate rows, lanes 64-127 the up rows of the same features.  Both
                // halves put their values (rounded to bfloat16, as the pipeline rounds them) into
                // shared memory, then every thread takes one feature and half of the chunk's
                // columns, so all four warps share the SiLU and the stores.
                const bool is_up = et >= kCtaFeatures;
                const int f = et & (kCtaFeatures - 1);
                const int n = nb * kItemFeatures + (int)rank * kCtaFeatures + f;
                const int j0 = is_up ? kXchCols / 2 : 0;                     // this thread's columns of a chunk
                // `chunk` runs on across items: the two exchange buffers alternate without a gap
                for (int c0 = 0; c0 < valid; c0 += kXchCols, ++chunk) {      // uniform over the 128 threads
                    uint32_t v[32];
                    tmem_ld32(taddr + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    auto mine = xch_s[chunk & 1][is_up ? 1 : 0];
#pragma unroll
                    for (int j = 0; j < kXchCols; ++j) mine[j][f] = __float2bfloat16_rn(__uint_as_float(v[j]));
                    asm volatile("bar.sync 1, 128;" ::: "memory");           // both halves of this chunk are there
                    if (n < p.n_out) {
                        const auto gs = xch_s[chunk & 1][0];
                        const auto us = xch_s[chunk & 1][1];
#pragma unroll
                        for (int jj = 0; jj < kXchCols / 2; ++jj) {
                            const int j = j0 + jj;
                            if (c0 + j >= valid) break;
                            const float gate = __bfloat162float(gs[j][f]);
                            const float up = __bfloat162float(us[j][f]);
                            // silu in 32-bit (fast exponential and reciprocal: the result is rounded to bfloat16 next)
                            const float silu = __fdividef(gate, 1.f + __expf(-gate));
                            p.out[(size_t)(row0 + c0 + j) * p.n_out + n] =
                                __float2bfloat16_rn(round_act<__nv_bfloat16>(silu) * up);
                        }
                    }
                    // a buffer is written again two chunks on, after the next chunk's barrier
                }
            } else {
                const int n = nb * kItemFeatures + (int)rank * kCtaFeatures + et;
                for (int c0 = 0; c0 < valid; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (n < p.n_out) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (c0 + j >= valid) break;
                            p.out[(size_t)(row0 + c0 + j) * p.n_out + n] =
                                __float2bfloat16_rn(__uint_as_float(v[j]) * route_s[b][c0 + j]);
                        }
                    }
                }
            }
            // this warp has read its lanes of buffer b: tell the leader's MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8 * b);
        }
    }
    // Leave together: the leader's MMAs read the peer's shared memory, and the peer's epilogue
    // arrives on the leader's barriers.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)f;
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    uint64_t rows, cols;
    uint32_t box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (k.rows * 1000003u) ^ (k.cols * 10007u) ^ k.box_rows;
    }
};

// 2-D bf16 row-major [rows, cols] -> map with box [box_rows, 64 cols], 128-byte swizzle.
static int make_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    const MapKey key{ptr, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return SE_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return SE_ERR_ARGUMENT;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

template <int MODE>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int max_items, cudaStream_t stream) {
    const size_t smem = (size_t)kStages * kStageBytes + 1024;
    static int max_pairs = 0;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cfg.gridDim = dim3(sms > 1 ? (sms / 2) * 2 : 2);
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<MODE>, &cfg);
        if (e != cudaSuccess || clusters <= 0) {
            cudaGetLastError();
            clusters = sms / 2;
        }
        max_pairs = clusters > 0 ? clusters : 1;
    }
    const int pairs = max_items < max_pairs ? max_items : max_pairs;
    cfg.gridDim = dim3(2 * (pairs > 0 ? pairs : 1));
    return (int)cudaLaunchKernelEx(&cfg, gemm_pair_kernel<MODE>, mw, mx, p);
}

}  // namespace tcp
}  // namespace se

using namespace se::tcp;

// Rows per activation tile of this kernel: the tile list must have been built with it.
extern "C" int se_moe_pair_tile_rows() { return kTileN; }

// 1 if the pair kernel takes these sizes (bf16; row pitches of 16-byte multiples for TMA).
extern "C" int se_moe_grouped_gemm_pair_supported(int k_dim, int n_out) {
    return (k_dim % 8 == 0 && k_dim >= 8 && n_out >= 1) ? 1 : 0;
}

// Grouped expert GEMM on pairs of SMs (bf16).
//   mode 0: a = x rows in sorted order [assignments, k_dim]; w = w13 [experts, 2*n_out, k_dim]; out [assignments, n_out]
//   mode 1: a = act [assignments, k_dim];                    w = w2 [experts, n_out, k_dim];    out [assignments, n_out]
extern "C" int se_moe_grouped_gemm_pair(int mode, const void* a, const void* w, const int* sorted, const int* offsets,
                                        const int* tile_expert, const int* tile_row0, const int* num_tiles,
                                        const float* route_w, void* out, int* error, int assignments, int experts,
                                        int max_tiles, int n_out, int k_dim, cudaStream_t stream) {
    if (assignments <= 0 || max_tiles <= 0) return 0;
    if (!se_moe_grouped_gemm_pair_supported(k_dim, n_out) || (mode != 0 && mode != 1)) return SE_ERR_UNSUPPORTED;
    const int w_rows = mode == 0 ? 2 * n_out : n_out;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, (uint64_t)experts * w_rows, k_dim, mode == 0 ? kCtaM / 2 : kCtaM);
    if (rc) return rc;
    rc = make_map(&mx, a, assignments, k_dim, kHalfN);
    if (rc) return rc;
    Params p{sorted, offsets, tile_expert, tile_row0, num_tiles, route_w, (__nv_bfloat16*)out, error,
             n_out,  k_dim,   w_rows,      n_out};
    const int item_features = mode == 0 ? 128 : 256;
    const int max_items = max_tiles * ((n_out + item_features - 1) / item_features);
    if (mode == 0) return launch<MODE_GATE_UP>(mw, mx, p, max_items, stream);
    return launch<MODE_DOWN>(mw, mx, p, max_items, stream);
}
