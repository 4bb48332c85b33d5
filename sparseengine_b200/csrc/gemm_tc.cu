// Tensor-core GEMMs for sm_100a: TMA (cp.async.bulk.tensor) -> shared memory (128-byte
// swizzle) -> tcgen05.mma with the accumulator in tensor memory -> tcgen05.ld epilogue.
//
// One kernel, three epilogues, all "weights on the M side" (swap-AB): a CTA owns 128 rows
// of a weight matrix W[n, k] and up to NT activation rows X[t, k] and computes
// D[n, t] = sum_k W[n, k] X[t, k].  Decode and small expert batches have few rows per
// expert and are bound by streaming W, so W takes the 128-wide M side of the MMA and the
// few tokens the N side (16..128); large prefill tiles use NT = 128.
//
//   MODE_GATE_UP  grouped: W = w13[e] (gate rows, then up rows); two accumulators share the
//                 X tile; epilogue rounds gate/up to bf16, SiLU in fp32, product -> act[p, n]
//   MODE_DOWN     grouped: W = w2[e]; epilogue multiplies by the routing weight -> y[p, n]
//   MODE_DENSE    one weight matrix for all rows -> out[t, n]
//
// Rows are "sorted positions" p: the routing build sorts the (token, slot) assignments by
// expert and lists tiles (expert, first row).  X for MODE_GATE_UP is the token rows
// gathered into that order (by the routing build, se_moe_route_gather).  Rounding points follow the reference's
// bf16 pipeline (src/sparseengine/kernels/triton/moe.py:557-563,726-732,1374-1440).
//
// Warp roles (192 threads): warp 0 issues TMA loads, warp 1 allocates tensor memory and
// issues the MMAs (one elected lane), warps 2-5 run the epilogue (one TMEM lane quarter
// each).  Every wait on an mbarrier is bounded; on a timeout the CTA records an error code,
// drains its outstanding copies, frees its tensor memory and returns.
//
// A work item is one block index of the grid: NA blocks of 128 weight rows (the gate and the
// up block of MODE_GATE_UP, one block in the other modes; two neighbouring blocks per item
// were measured there and gained nothing) times one tile of activation rows, which the NA
// accumulators share.
#include "common.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace se {
namespace tc {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;          // bf16 elements: 128 bytes, one swizzle span
constexpr int kUmmaK = 16;
constexpr int kMaxStages = 8;     // the ring's depth is a launch parameter (2..8)
constexpr int kThreads = 192;
constexpr int kTileABytes = kBlockM * kBlockK * 2;
constexpr uint32_t kSpinLimit = 1u << 24;

enum Mode { MODE_GATE_UP = 0, MODE_DOWN = 1, MODE_DENSE = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false on timeout or when another role of the CTA has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart (tile bases are 1024-byte aligned).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset: 1024 bytes between 8-row groups
    d |= (uint64_t)1 << 46;                 // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                 // 128-byte swizzle
    return d;
}

// Instruction descriptor for kind::f16: bf16 x bf16 -> fp32, both operands K-major.
__device__ __forceinline__ uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBlockM >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
}

struct Params {
    const int* sorted;          // [assignments] flat assignment of each sorted row (MODE_DOWN: routing weight index)
    const int* offsets;         // [experts + 1]
    const int* tile_expert;     // null: dense (one weight matrix, tiles are consecutive row blocks)
    const int* tile_row0;
    const int* num_tiles;
    const float* route_w;       // [assignments] (MODE_DOWN)
    __nv_bfloat16* out;         // [rows, n_out]
    int* error;                 // device word: 0 ok, else a code of the first failure
    int n_out;                  // weight rows per expert that are outputs (I for gate/up, H for down)
    int k_dim;
    int w_rows_per_expert;      // rows of the 2-D weight view per expert (2I or H)
    int up_offset;              // row offset of the "up" half (MODE_GATE_UP)
    int total_rows;             // dense: number of activation rows
    int nt;                     // activation rows per tile: 16, 32, 64, 128 or 256
    int stages;                 // depth of the shared-memory ring
    int lists_settled;          // the tile list and offsets were complete before the kernel before this one began
};

// ---- the persistent form ---------------------------------------------------------------------
// The same roles and the same arithmetic, but a CTA does not end with its item (one 128-row
// block of one tile = one block index of the grid).  When it starts an item it asks the
// hardware for another block of this grid that has not started yet
// (clusterlaunchcontrol.try_cancel): that block then never launches and this CTA does its
// work next.  So the SMs that stream faster take more items, as with one CTA per item, but
// without a prologue and an epilogue per item: the loader keeps the shared-memory ring full
// across items, and the accumulator lives in one of two tensor-memory buffers, so that the
// MMAs of item j + 1 fill buffer b ^ 1 while the epilogue warps drain buffer b of item j.
//
// The answer to a request is 16 bytes that land in a shared-memory slot (ring of kSchedSlots)
// and complete an mbarrier; the loader thread, the MMA thread and the four epilogue warps
// each read it (sched_full), the last five arrive on sched_empty before the slot is used
// again.  After the first answer "nothing left" no further request is made.
constexpr int kSchedSlots = 4;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void clc_try_cancel(uint32_t response, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], 16;" ::"r"(bar) : "memory");
    asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
                 ::"r"(response), "r"(bar)
                 : "memory");
}
// The block index in the answer at `response`; false if no block was left to take.
__device__ __forceinline__ bool clc_read(uint32_t response, int* x, int* y) {
    uint32_t got, bx, by;
    asm volatile(
        "{\n\t.reg .b128 r;\n\t.reg .pred p;\n\t.reg .b32 z, w;\n\t"
        "ld.shared.b128 r, [%3];\n\t"
        "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, r;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "mov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\t"
        "@p clusterlaunchcontrol.query_cancel.get_first_ctaid.v4.b32.b128 {%1, %2, z, w}, r;\n\t}"
        : "=r"(got), "=r"(bx), "=r"(by)
        : "r"(response)
        : "memory");
    *x = (int)bx;
    *y = (int)by;
    return got != 0;
}

template <int MODE, int NA>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          const Params p) {
    static_assert(MODE != MODE_GATE_UP || NA == 2, "gate and up are the two blocks of an item");
    // rows of the weight view between the item's blocks, and weight rows (= outputs) per item
    const int second = MODE == MODE_GATE_UP ? p.up_offset : kBlockM;
    constexpr int kItemM = MODE == MODE_GATE_UP ? kBlockM : NA * kBlockM;
    const int nt = p.nt;
    const int num_kb = (p.k_dim + kBlockK - 1) / kBlockK;
    const int kStages = p.stages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t stage_bytes = NA * kTileABytes + nt * kBlockK * 2;
    __shared__ __align__(8) uint64_t bars[2 * kMaxStages + 4 + 2 * kSchedSlots];
    __shared__ __align__(16) uint4 sched_s[kSchedSlots];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;
    __shared__ float route_s[2][256];
    __shared__ int valid_s[kSchedSlots];     // activation rows of the loader's last items (see the MMA thread)
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kMaxStages]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * kMaxStages]), acc_empty0 = smem_u32(&bars[2 * kMaxStages + 2]);
    const uint32_t sched_full0 = smem_u32(&bars[2 * kMaxStages + 4]);
    const uint32_t sched_empty0 = smem_u32(&bars[2 * kMaxStages + 4 + kSchedSlots]);
    const uint32_t sched0 = smem_u32(&sched_s[0]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // two accumulator buffers where tensor memory (512 columns) holds them, else one: the
    // epilogue of an item then ends before the MMAs of the next one begin
    const int bufs = 2 * NA * nt <= 512 ? 2 : 1;
    uint32_t cols = 32;
    while ((int)cols < bufs * NA * nt) cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);       // one arrival per epilogue warp
        }
        for (int q = 0; q < kSchedSlots; ++q) {
            mbar_init(sched_full0 + 8 * q, 1);
            mbar_init(sched_empty0 + 8 * q, 5);     // the MMA thread and the four epilogue warps
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"(cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    // Launched as a dependent, this kernel may have come this far while the kernel before it
    // still runs.  If that kernel writes the tile list, everything waits for it here; if not,
    // only the loader waits, and only before it asks for activation rows.
    if (!p.lists_settled) grid_dependency_wait();
    const int tiles = p.tile_expert != nullptr ? p.num_tiles[0] : (p.total_rows + nt - 1) / nt;

    // Every role walks the same list of items: its own block index first, then the answers in
    // the scheduling ring.  `next_item` waits for answer j (the item after item j).
    int bx = blockIdx.x, by = blockIdx.y;
    // role: 0 the loader (it frees nothing), 1 a single thread, 2 a whole warp
    auto next_item = [&](int j, int role) -> bool {
        const int q = j % kSchedSlots;
        if (!mbar_wait(sched_full0 + 8 * q, (j / kSchedSlots) & 1, &abort_s)) {
            abort_s = 1;
            atomicCAS(p.error, 0, 5);
            return false;
        }
        const bool more = clc_read(sched0 + 16 * q, &bx, &by);
        if (role == 2) __syncwarp();          // every lane has read the slot
        if (role != 0 && lane == 0) mbar_arrive(sched_empty0 + 8 * q);
        return more;
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            int asked = 0;          // requests made so far
            int used = 0;           // items with work so far
            bool waited = !p.lists_settled;    // the kernel before this one has ended
            // From here on the kernel after this one may set itself up and stream its weights; its
            // own tile list is then older than the kernel before it (this one), which has seen the
            // end of everything before itself.
            if (waited) grid_dependency_trigger();
            int expert = 0, row0 = by * nt, row_end = p.total_rows;
            if (p.tile_expert != nullptr && by < tiles) {
                expert = p.tile_expert[by];
                row0 = p.tile_row0[by];
                row_end = p.offsets[expert + 1];
            }
            for (int j = 0; ok; ++j) {
                // ask for the item after this one; the answer comes while this item streams
                {
                    const int q = j % kSchedSlots;
                    if (!mbar_wait(sched_empty0 + 8 * q, ((j / kSchedSlots) & 1) ^ 1, &abort_s)) {
                        abort_s = 1;
                        atomicCAS(p.error, 0, 6);
                        break;
                    }
                    clc_try_cancel(sched0 + 16 * q, sched_full0 + 8 * q);
                    asked = j + 1;
                }
                const int tile = by, n0 = bx * kItemM;
                // The answer is read half-way through this item (it has had time to arrive, and
                // the ring is full), and the next tile's expert and first row are fetched then,
                // so the first copies of the next item do not wait for them.
                bool answered = false, more = false;
                int expert_next = 0, row0_next = 0, row_end_next = p.total_rows;
                auto read_answer = [&]() {
                    answered = true;
                    more = next_item(j, 0);
                    row0_next = by * nt;
                    if (more && p.tile_expert != nullptr && by < tiles) {
                        expert_next = p.tile_expert[by];
                        row0_next = p.tile_row0[by];
                        row_end_next = p.offsets[expert_next + 1];
                    }
                };
                if (tile < tiles) {
                    // the item's activation rows, for the MMA thread: written before this item's first
                    // arrival on a `full` barrier, which the MMA thread waits for before it reads it
                    valid_s[used % kSchedSlots] = min(nt, row_end - row0);
                    ++used;
                    const int wy = expert * p.w_rows_per_expert + n0;
                    int kb_first = 0;
                    if (!waited) {
                        // This kernel may have started before the one that writes the activation rows
                        // has ended.  The first trip round the ring asks for the weight tiles at once
                        // (no kernel writes them; the tile list is older than the kernel before this
                        // one) and for the activation tiles once that kernel has ended.
                        kb_first = min(kStages, num_kb);
                        for (int kb = 0; kb < kb_first; ++kb) {
                            const uint32_t a = smem_u32(smem + (size_t)kb * stage_bytes);
                            mbar_expect_tx(full0 + 8 * kb, stage_bytes);
                            tma_load_2d(a, &map_w, full0 + 8 * kb, kb * kBlockK, wy);
                            if (NA == 2) tma_load_2d(a + kTileABytes, &map_w, full0 + 8 * kb, kb * kBlockK, wy + second);
                        }
                        grid_dependency_wait();
                        grid_dependency_trigger();
                        waited = true;
                        for (int kb = 0; kb < kb_first; ++kb)
                            tma_load_2d(smem_u32(smem + (size_t)kb * stage_bytes) + NA * kTileABytes, &map_x,
                                        full0 + 8 * kb, kb * kBlockK, row0);
                        it = kb_first;
                    }
                    for (int kb = kb_first; kb < num_kb; ++kb, ++it) {
                        if (kb == num_kb / 2) {
                            read_answer();
                            if (abort_s) {
                                ok = false;
                                break;
                            }
                        }
                        const int s = it % kStages;
                        const uint32_t ph = (it / kStages) & 1;
                        if (!mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_s)) {
                            abort_s = 1;
                            atomicCAS(p.error, 0, 1);
                            ok = false;
                            break;
                        }
                        const uint32_t a = smem_u32(smem + (size_t)s * stage_bytes);
                        mbar_expect_tx(full0 + 8 * s, stage_bytes);
                        tma_load_2d(a, &map_w, full0 + 8 * s, kb * kBlockK, wy);
                        if (NA == 2) tma_load_2d(a + kTileABytes, &map_w, full0 + 8 * s, kb * kBlockK, wy + second);
                        tma_load_2d(a + NA * kTileABytes, &map_x, full0 + 8 * s, kb * kBlockK, row0);
                    }
                }
                if (ok && !answered) read_answer();
                if (!ok || !more) break;
                expert = expert_next;
                row0 = row0_next;
                row_end = row_end_next;
            }
            if (abort_s) {
                // let what is still in flight land before the CTA's shared memory goes away:
                // the copies of the ring and the answer to the last request
                for (int k = max(0, it - kStages); k < it; ++k) {
                    const uint32_t bar = full0 + 8 * (k % kStages);
                    const uint32_t ph = (k / kStages) & 1;
                    for (uint32_t i = 0; i < kSpinLimit && !mbar_try_wait(bar, ph); ++i) {}
                }
                if (asked > 0) {
                    const int j = asked - 1;
                    const uint32_t bar = sched_full0 + 8 * (j % kSchedSlots);
                    for (uint32_t i = 0; i < kSpinLimit && !mbar_try_wait(bar, (j / kSchedSlots) & 1); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // An item whose tile holds fewer rows than nt (the last tile of an expert) runs MMAs of
            // just those rows, rounded up to 16: N is a field of the instruction descriptor.
            uint32_t idesc = instr_desc(nt);
            int it = 0, used = 0;       // used: items that took an accumulator buffer
            bool ok = true;
            for (int j = 0; ok; ++j) {
                if (by < tiles) {
                    const int b = used % bufs;
                    if (!mbar_wait(acc_empty0 + 8 * b, ((used / bufs) & 1) ^ 1, &abort_s)) {   // the epilogue has drained buffer b
                        abort_s = 1;
                        atomicCAS(p.error, 0, 4);
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t acc_col = tmem_base + (uint32_t)(b * NA * nt);
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int s = it % kStages;
                        const uint32_t ph = (it / kStages) & 1;
                        if (!mbar_wait(full0 + 8 * s, ph, &abort_s)) {
                            abort_s = 1;
                            atomicCAS(p.error, 0, 2);
                            ok = false;
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        if (kb == 0) idesc = instr_desc(max(16, (valid_s[used % kSchedSlots] + 15) & ~15));
                        const uint32_t a = smem_u32(smem + (size_t)s * stage_bytes);
                        const uint64_t da = smem_desc(a), db = smem_desc(a + NA * kTileABytes);
#pragma unroll
                        for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                            const uint64_t adv = (uint64_t)((kk * kUmmaK * 2) >> 4);      // 32 bytes per K step
                            const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
                            umma(acc_col, da + adv, db + adv, idesc, acc);
                            if (NA == 2) umma(acc_col + (uint32_t)nt, smem_desc(a + kTileABytes) + adv, db + adv, idesc, acc);
                        }
                        umma_commit(empty0 + 8 * s);     // frees the stage when these MMAs have read it
                    }
                    if (!ok) break;
                    umma_commit(acc_full0 + 8 * b);      // arrives when every MMA of this item has finished
                    ++used;
                }
                if (!next_item(j, 1)) break;
            }
        }
    } else {
        const int quarter = warp & 3;            // TMEM lanes this warp may read: 32*quarter ..
        const int et = threadIdx.x - 64;         // 0..127 among the epilogue threads
        int used = 0;
        for (int j = 0;; ++j) {
            if (by < tiles) {
                const int b = used % bufs;
                const int tile = by, n0 = bx * kItemM;
                int row0 = tile * nt, row_end = p.total_rows;
                if (p.tile_expert != nullptr) {
                    row0 = p.tile_row0[tile];
                    row_end = p.offsets[p.tile_expert[tile] + 1];
                }
                const int valid = min(nt, row_end - row0);
                if (MODE == MODE_DOWN) {
                    for (int e = et; e < nt; e += 128) route_s[b][e] = e < valid ? p.route_w[p.sorted[row0 + e]] : 0.f;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
                if (!mbar_wait(acc_full0 + 8 * b, (used / bufs) & 1, &abort_s)) {
                    abort_s = 1;
                    atomicCAS(p.error, 0, 3);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * NA * nt);
                if (MODE == MODE_GATE_UP) {
                    const int n = n0 + quarter * 32 + lane;
                    for (int c0 = 0; c0 < nt; c0 += 16) {
                        if (c0 >= valid) break;          // warp-uniform
                        uint32_t g[16], u[16];
                        tmem_ld16(taddr + c0, g);
                        tmem_ld16(taddr + nt + c0, u);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (n < p.n_out) {
#pragma unroll
                            for (int jj = 0; jj < 16; ++jj) {
                                if (c0 + jj >= valid) break;
                                const float gate = round_act<__nv_bfloat16>(__uint_as_float(g[jj]));
                                const float up = round_act<__nv_bfloat16>(__uint_as_float(u[jj]));
                                const float v = round_act<__nv_bfloat16>(gate / (1.f + expf(-gate))) * up;
                                p.out[(size_t)(row0 + c0 + jj) * p.n_out + n] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int blk = 0; blk < NA; ++blk) {
                        const int n = n0 + blk * kBlockM + quarter * 32 + lane;
                        if (n0 + blk * kBlockM >= p.n_out) break;       // warp-uniform: no such block
                        for (int c0 = 0; c0 < nt; c0 += 16) {
                            if (c0 >= valid) break;      // warp-uniform
                            uint32_t g[16];
                            tmem_ld16(taddr + blk * nt + c0, g);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            if (n < p.n_out) {
#pragma unroll
                                for (int jj = 0; jj < 16; ++jj) {
                                    if (c0 + jj >= valid) break;
                                    float v = __uint_as_float(g[jj]);
                                    if (MODE == MODE_DOWN) v *= route_s[b][c0 + jj];
                                    p.out[(size_t)(row0 + c0 + jj) * p.n_out + n] = __float2bfloat16_rn(v);
                                }
                            }
                        }
                    }
                }
                // this warp has read its lanes of buffer b: hand it back to the MMA thread
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * b);
                ++used;
            }
            if (!next_item(j, 2)) break;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(cols) : "memory");
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
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
    }
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

// NA: blocks of 128 weight rows per work item (2 for gate/up, else 1).
template <int MODE, int NA>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int tiles, cudaStream_t stream) {
    size_t smem = (size_t)p.stages * (NA * kTileABytes + p.nt * kBlockK * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<MODE, NA>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // A CTA takes 2 * NA * nt columns of tensor memory (512 per SM).  Where two CTAs would
    // fit by shared memory but not by columns, ask for more than half of the shared memory, so
    // that no CTA waits for columns behind a persistent neighbour.
    const int bufs = 2 * NA * p.nt <= 512 ? 2 : 1;
    int cols = 32;
    while (cols < bufs * NA * p.nt) cols <<= 1;
    if (2 * cols > 512) smem = std::max<size_t>(smem, 116 * 1024);
    const int item_m = MODE == MODE_GATE_UP ? kBlockM : NA * kBlockM;
    dim3 grid(ceil_div(p.n_out, item_m), tiles);
    // as a dependent of the kernel before it: see the loader's first trip round the ring
    cudaError_t e = SE_LAUNCH_DEPENDENT("gemm", gemm_tc_persistent_kernel<MODE, NA>, grid, dim3(kThreads), smem, stream, mw, mx, p);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

}  // namespace tc
}  // namespace se

using namespace se::tc;

#include <cstdlib>

// Depth of the shared-memory ring.  Small token tiles make small stages: several CTAs then
// fit on an SM (their prologues and epilogues overlap) and each still has several stages in
// flight.  SE_TC_STAGES_GATE_UP / SE_TC_STAGES_OTHER override the choice (tuning aid).
static int pick_stages(int na, int nt) {
    const char* env = std::getenv(na == 2 ? "SE_TC_STAGES_GATE_UP" : "SE_TC_STAGES_OTHER");
    if (env != nullptr) {
        const int v = std::atoi(env);
        if (v >= 2 && v <= kMaxStages) return v;
    }
    const int stage_bytes = na * kTileABytes + nt * kBlockK * 2;
    int stages = na == 2 && nt <= 32 ? 3 : 4;      // measured: three 34 KB stages x two CTAs per SM stream a little faster
    while (stages < kMaxStages && (stages + 1) * stage_bytes + 1024 <= 100 * 1024) ++stages;   // two CTAs per SM
    while (stages > 2 && stages * stage_bytes + 1024 > 224 * 1024) --stages;
    return stages;
}

// 1 if the tensor-core path takes these sizes (bf16 only; row pitches must be 16-byte
// multiples for TMA), else 0.
extern "C" int se_gemm_tc_supported(int k_dim, int n_out, int nt) {
    return (k_dim % 8 == 0 && k_dim >= 8 && n_out >= 1 && (nt == 16 || nt == 32 || nt == 64 || nt == 128 || nt == 256)) ? 1 : 0;
}

// Grouped expert GEMM on tensor cores (bf16).
//   mode 0: a = x rows in sorted order [assignments, k_dim]; w = w13 [experts, 2*n_out, k_dim]; out [assignments, n_out]
//   mode 1: a = act [assignments, k_dim];                    w = w2 [experts, n_out, k_dim];    out [assignments, n_out]
// The tile list must have been built with tile_rows = nt.  lists_settled: the kernel launched
// just before this one on the stream does not write the tile list, the offsets or `sorted`
// (they were complete before it began), so this kernel may read them while that one still runs.
extern "C" int se_moe_grouped_gemm_tc(int mode, const void* a, const void* w, const int* sorted, const int* offsets,
                                      const int* tile_expert, const int* tile_row0, const int* num_tiles,
                                      const float* route_w, void* out, int* error, int assignments, int experts,
                                      int max_tiles, int n_out, int k_dim, int nt, int lists_settled,
                                      cudaStream_t stream) {
    if (assignments <= 0 || max_tiles <= 0) return 0;
    if (!se_gemm_tc_supported(k_dim, n_out, nt) || (mode != 0 && mode != 1)) return SE_ERR_UNSUPPORTED;
    const int w_rows = mode == 0 ? 2 * n_out : n_out;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, (uint64_t)experts * w_rows, k_dim, kBlockM);
    if (rc) return rc;
    rc = make_map(&mx, a, assignments, k_dim, nt);
    if (rc) return rc;
    const int na = mode == 0 ? 2 : 1;
    Params p{sorted, offsets, tile_expert, tile_row0, num_tiles, route_w, (__nv_bfloat16*)out, error,
             n_out,  k_dim,   w_rows,      n_out,     assignments, nt, pick_stages(na, nt), lists_settled ? 1 : 0};
    if (mode == 0) return launch<MODE_GATE_UP, 2>(mw, mx, p, max_tiles, stream);
    // With 128-row tiles the activation tile of the down projection is as large as a weight block
    // (K is the expert width), so two weight blocks share it, which cuts what an SM takes from L2
    // by a quarter (measured: 2,048 tokens 1.251 -> 1.186 ms for the expert layer; no gain at the
    // other tile sizes, and with 256 rows the second accumulator would cost the overlapped epilogue).
    if (nt == 128) {
        p.stages = pick_stages(2, nt);
        return launch<MODE_DOWN, 2>(mw, mx, p, max_tiles, stream);
    }
    return launch<MODE_DOWN, 1>(mw, mx, p, max_tiles, stream);
}

// Dense projection on tensor cores: out[rows, n_out] = x[rows, k_dim] · w[n_out, k_dim]ᵀ (bf16, fp32 accumulate).
extern "C" int se_gemm_tc_dense(const void* x, const void* w, void* out, int* error, int rows, int n_out, int k_dim,
                                int nt, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!se_gemm_tc_supported(k_dim, n_out, nt)) return SE_ERR_UNSUPPORTED;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, n_out, k_dim, kBlockM);
    if (rc) return rc;
    rc = make_map(&mx, x, rows, k_dim, nt);
    if (rc) return rc;
    Params p{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, (__nv_bfloat16*)out, error,
             n_out,   k_dim,   n_out,   0,       rows,    nt, pick_stages(1, nt), 1};
    return launch<MODE_DENSE, 1>(mw, mx, p, se::ceil_div(rows, nt), stream);
}
