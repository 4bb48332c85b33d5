// Router: 32-bit logits, score function, selection bias, top-k and renormalisation in
// one kernel.  Every constant (experts, top-k, score function, bias, scale) is an
// argument.
//
// Reference: logits = float(x)·Wgᵀ with a 32-bit weight (src/sparseengine/models/minimax_m2.py:166);
// p = sigmoid(logits), score = p + bias, NaN scores count as +inf, order of the chosen
// ids = strictly above the k-th value in ascending index, then ties in ascending index
// (src/sparseengine/kernels/triton/moe_biased_sigmoid.py:71-111); weights = unbiased p
// of the chosen, divided by their sum (:202-238, epsilon 0 for M2:
// src/sparseengine/kernels/triton/minimax_m2_router.py:50-63).
#include "common.cuh"
#include "mma_util.cuh"

namespace se {

constexpr int kRouterTokens = 8;   // tokens per block
constexpr int kRouterWarps = 8;
constexpr int kRouterExperts = 4;  // gate rows a warp walks at once in the many-token kernel

// The one order in which a router logit is summed, whatever the batch: the row is cut into
// four quarters; within a quarter lane l takes elements (or 16-byte groups) l, l+32, ... in
// increasing order with fused multiply-adds, the 32 lanes are combined by a butterfly, and
// the quarters are added as (q0 + q1) + (q2 + q3).  Both kernels below use it, so a token's
// logits do not depend on how many tokens share its step.
template <int NTOK, int NEXP>
__device__ __forceinline__ void quarter_dot(const float* __restrict__ xs, int hidden, int ntok,
                                            const float* const* __restrict__ g, int quarter, int lane,
                                            float (&acc)[NTOK][NEXP]) {
#pragma unroll
    for (int j = 0; j < NTOK; ++j)
#pragma unroll
        for (int e = 0; e < NEXP; ++e) acc[j][e] = 0.f;
    if ((hidden & 3) == 0) {
        const int n4 = hidden >> 2;
        const int per = (n4 + 3) / 4, a = quarter * per, b = min(n4, a + per);
#pragma unroll 2
        for (int i = a + lane; i < b; i += 32) {
            float4 gv[NEXP];
#pragma unroll
            for (int e = 0; e < NEXP; ++e) gv[e] = __ldg(reinterpret_cast<const float4*>(g[e]) + i);
#pragma unroll
            for (int j = 0; j < NTOK; ++j) {
                if (j < ntok) {
                    const float4 xv = *reinterpret_cast<const float4*>(xs + j * hidden + 4 * i);
#pragma unroll
                    for (int e = 0; e < NEXP; ++e) {
                        acc[j][e] = fmaf(xv.x, gv[e].x, acc[j][e]);
                        acc[j][e] = fmaf(xv.y, gv[e].y, acc[j][e]);
                        acc[j][e] = fmaf(xv.z, gv[e].z, acc[j][e]);
                        acc[j][e] = fmaf(xv.w, gv[e].w, acc[j][e]);
                    }
                }
            }
        }
    } else {
        const int per = (hidden + 3) / 4, a = quarter * per, b = min(hidden, a + per);
        for (int i = a + lane; i < b; i += 32) {
#pragma unroll
            for (int j = 0; j < NTOK; ++j)
                if (j < ntok)
#pragma unroll
                    for (int e = 0; e < NEXP; ++e) acc[j][e] = fmaf(xs[j * hidden + i], g[e][i], acc[j][e]);
        }
    }
#pragma unroll
    for (int j = 0; j < NTOK; ++j)
#pragma unroll
        for (int e = 0; e < NEXP; ++e) acc[j][e] = warp_sum(acc[j][e]);
}

template <typename T>
__device__ __forceinline__ void load_tokens(const T* xt, float* xs, int n) {
    if ((n & 7) == 0 && aligned8(xt)) {
        for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) load8(xt + i, xs + i);
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) xs[i] = to_float(xt[i]);
    }
}

// Many tokens, a width that is no multiple of 4: block (bx, by) takes tokens bx*8 .. +7 (converted to 32-bit in shared memory)
// and experts by*32 .. +31; each warp walks 4 gate rows at once for the 8 tokens.
template <typename T>
__global__ void router_logits_kernel(const T* __restrict__ x, const float* __restrict__ gate,
                                     float* __restrict__ logits, int tokens, int hidden, int experts) {
    extern __shared__ __align__(16) float xs[];              // [kRouterTokens][hidden]
    const int t0 = blockIdx.x * kRouterTokens;
    const int nt = min(kRouterTokens, tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    load_tokens(x + (size_t)t0 * hidden, xs, nt * hidden);
    __syncthreads();
    const int e0 = (blockIdx.y * kRouterWarps + warp) * kRouterExperts;
    if (e0 >= experts) return;
    const float* g[kRouterExperts];
#pragma unroll
    for (int e = 0; e < kRouterExperts; ++e) g[e] = gate + (size_t)min(e0 + e, experts - 1) * hidden;
    float q[4][kRouterTokens][kRouterExperts];
#pragma unroll
    for (int quarter = 0; quarter < 4; ++quarter) quarter_dot<kRouterTokens, kRouterExperts>(xs, hidden, nt, g, quarter, lane, q[quarter]);
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < kRouterTokens; ++j)
#pragma unroll
            for (int e = 0; e < kRouterExperts; ++e)
                if (j < nt && e0 + e < experts)
                    logits[(size_t)(t0 + j) * experts + e0 + e] = (q[0][j][e] + q[1][j][e]) + (q[2][j][e] + q[3][j][e]);
    }
}

// Many tokens: a block of 8 warps takes 32 tokens x 16 experts; warp w owns the 8 x 8
// sub-tile (tokens 8*(w/2).., experts 8*(w%2)..) with 64 accumulators per lane.  The token
// and gate rows go to shared memory with cp.async in chunks of 32 16-byte groups (three
// chunks in flight, one block barrier per chunk), which are exactly the groups the 32 lanes
// take in one step of the fixed summation order (see quarter_dot), so every (token, expert,
// quarter, lane) partial sum is accumulated in the same order as in the other kernels;
// quarters are reduced by the same butterfly and combined as (q0 + q1) + (q2 + q3).  The
// chunks of the four quarters form one stream, so the copies run ahead across the quarters'
// ends too.  Token rows stay in their own type in shared memory and are widened when they are
// read.  Needs hidden % 4 == 0.
//
// Plain fused multiply-adds: the packed fma.rn.f32x2 of this architecture occupies its pipe
// for twice as long as a scalar one (measured: 3.7 pipe cycles per packed instruction), and the
// scalar ones spread over both multiply-add pipes.
constexpr int kBigTokens = 32, kBigExperts = 16;
constexpr int kBigStages = 3;

__device__ __forceinline__ void cp_async_small(uint32_t dst, const void* src, int bytes, bool valid) {
    const int n = valid ? bytes : 0;           // the rest of the destination is filled with zeros
    if (bytes == 16)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

// the four elements of a staged group as 32-bit values
__device__ __forceinline__ float4 staged4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 staged4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}

template <int N, int M>
__device__ __forceinline__ void halve_over_lanes(float* v, int lane) {
    const bool upper = (lane & M) != 0;
#pragma unroll
    for (int k = 0; k < N / 2; ++k) {
        const float send = upper ? v[k] : v[k + N / 2];
        const float keep = upper ? v[k + N / 2] : v[k];
        v[k] = keep + __shfl_xor_sync(0xffffffffu, send, M);
    }
}

template <typename T>
__global__ void __launch_bounds__(256, 2)
router_logits_tiled_kernel(const T* __restrict__ x, const float* __restrict__ gate, float* __restrict__ logits,
                           int tokens, int hidden, int experts) {
    extern __shared__ __align__(16) uint8_t tiled_smem[];
    constexpr int kXStage = kBigTokens * 128 * (int)sizeof(T), kGStage = kBigExperts * 128 * (int)sizeof(float);
    uint8_t* xs_base = tiled_smem;                                  // [stages][tokens][128] of T
    uint8_t* gs_base = tiled_smem + kBigStages * kXStage;           // [stages][experts][128] float
    float (*qsum)[4][64] = reinterpret_cast<float (*)[4][64]>(tiled_smem + kBigStages * (kXStage + kGStage));
    const int t0 = blockIdx.x * kBigTokens, e0 = blockIdx.y * kBigExperts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wt = (warp >> 1) * 8, we = (warp & 1) * 8;
    const int n4 = hidden >> 2;
    const int per = (n4 + 3) / 4;
    const int cpq = (per + 31) / 32, total = 4 * cpq;      // chunks per quarter (the last of a short quarter are empty)

    // Chunk -> stage: thread (warp, lane) copies group `lane` of tokens warp, warp + 8, .. and of
    // experts 2 warp, 2 warp + 1.  Tokens, experts and groups past the end are read from the last
    // valid one instead (their sums are never used: see the guards below), so no copy has a
    // condition.  The chunk to load next is tracked by (quarter, chunk in quarter), without a division.
    const T* x_src[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) x_src[k] = x + (size_t)min(t0 + warp + 8 * k, tokens - 1) * hidden;
    const float* g_src[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) g_src[k] = gate + (size_t)min(e0 + 2 * warp + k, experts - 1) * hidden;
    const uint32_t xs0 = se::mma::smem_u32(xs_base) + (uint32_t)((warp * 128 + 4 * lane) * sizeof(T));
    const uint32_t gs0 = se::mma::smem_u32(gs_base) + (uint32_t)((2 * warp * 128 + 4 * lane) * sizeof(float));
    int load_q = 0, load_c = 0, load_stage = 0;
    auto load_next = [&]() {
        const int i = min(load_q * per + 32 * load_c + lane, n4 - 1);
#pragma unroll
        for (int k = 0; k < 4; ++k)
            cp_async_small(xs0 + (uint32_t)(load_stage * kXStage + k * 8 * 128 * (int)sizeof(T)), x_src[k] + 4 * i,
                           4 * (int)sizeof(T), true);
#pragma unroll
        for (int k = 0; k < 2; ++k)
            cp_async_small(gs0 + (uint32_t)(load_stage * kGStage + k * 128 * (int)sizeof(float)), g_src[k] + 4 * i, 16, true);
        if (++load_c == cpq) { load_c = 0; ++load_q; }
        if (++load_stage == kBigStages) load_stage = 0;
    };

    float acc[8][8];                          // [token][expert]
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
    for (int g = 0; g < kBigStages - 1; ++g) {
        if (g < total) load_next();
        se::mma::cp_async_commit();
    }
    int stage = 0;
    for (int quarter = 0; quarter < 4; ++quarter) {
        const int a = quarter * per, b = min(n4, a + per);
        for (int c = 0; c < cpq; ++c) {
            se::mma::cp_async_wait<kBigStages - 2>();
            __syncthreads();  // this chunk is there for everyone, and everyone is done with the one before, whose stage is refilled now
            if (load_q < 4) load_next();
            se::mma::cp_async_commit();
            if (a + 32 * c + lane < b) {         // lanes past the quarter's end add nothing (as in quarter_dot)
                const T* xs = reinterpret_cast<const T*>(xs_base + (size_t)stage * kXStage) + wt * 128 + 4 * lane;
                const float* gs = reinterpret_cast<const float*>(gs_base + (size_t)stage * kGStage) + we * 128 + 4 * lane;
                float4 gv[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) gv[e] = *reinterpret_cast<const float4*>(gs + e * 128);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 xv = staged4(xs + i * 128);
                    // every accumulator takes its four products in the order x, y, z, w
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(xv.x, gv[e].x, acc[i][e]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(xv.y, gv[e].y, acc[i][e]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(xv.z, gv[e].z, acc[i][e]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(xv.w, gv[e].w, acc[i][e]);
                }
            }
            if (++stage == kBigStages) stage = 0;
        }
        // The quarter is complete.  64 sums over the lanes at once: each step halves the values a
        // lane holds and adds the partner's copy of the half it keeps.  The pairs are those of
        // warp_sum (lanes l and l ^ 16, then ^ 8, 4, 2, 1) and a + b = b + a, so every total has
        // warp_sum's bits; lane l ends with the totals of values 2l and 2l + 1.
        float* v = &acc[0][0];
        halve_over_lanes<64, 16>(v, lane);
        halve_over_lanes<32, 8>(v, lane);
        halve_over_lanes<16, 4>(v, lane);
        halve_over_lanes<8, 2>(v, lane);
        halve_over_lanes<4, 1>(v, lane);
        qsum[warp][quarter][2 * lane] = v[0];
        qsum[warp][quarter][2 * lane + 1] = v[1];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
    }
    __syncwarp();
    for (int o = lane; o < 64; o += 32) {
        const int t = t0 + wt + o / 8, e = e0 + we + o % 8;
        if (t < tokens && e < experts)
            logits[(size_t)t * experts + e] = (qsum[warp][0][o] + qsum[warp][1][o]) + (qsum[warp][2][o] + qsum[warp][3][o]);
    }
}

// Few tokens (decode): the latency of one warp walking a whole gate row dominates, so a
// block of 8 warps takes 2 experts, 4 warps each on one quarter of the row.  A lane's share
// of the gate row (up to kGatePre 16-byte groups: widths up to 4096) is asked for before the
// tokens are staged, so that the two trips to memory overlap; the sums are formed in the
// order of quarter_dot.
constexpr int kGatePre = 8;

template <typename T>
__global__ void router_logits_small_kernel(const T* x, const float* __restrict__ gate,
                                           float* __restrict__ logits, int tokens, int hidden, int experts) {
    extern __shared__ __align__(16) float xs[];              // [tokens <= kRouterTokens][hidden]
    __shared__ float part[kRouterWarps][kRouterTokens];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.x * 2 + (warp >> 2), quarter = warp & 3;
    const float* g[1] = {gate + (size_t)min(e, experts - 1) * hidden};
    const int n4 = hidden >> 2;
    const int per = (n4 + 3) / 4, a = quarter * per, b = min(n4, a + per);
    const bool pre = (hidden & 3) == 0 && per <= 32 * kGatePre;
    float4 gv[kGatePre];
    if (pre) {
#pragma unroll
        for (int u = 0; u < kGatePre; ++u) {
            const int i = a + lane + 32 * u;
            if (i < b) gv[u] = __ldg(reinterpret_cast<const float4*>(g[0]) + i);
        }
    }
    grid_dependency_wait();      // launched as a dependent: the gate rows are on their way before x is complete (x: no __restrict__)
    load_tokens(x, xs, tokens * hidden);
    __syncthreads();
    float acc[kRouterTokens][1];
    if (pre) {
#pragma unroll
        for (int j = 0; j < kRouterTokens; ++j) acc[j][0] = 0.f;
#pragma unroll
        for (int u = 0; u < kGatePre; ++u) {
            const int i = a + lane + 32 * u;
            if (i < b) {
#pragma unroll
                for (int j = 0; j < kRouterTokens; ++j) {
                    if (j < tokens) {
                        const float4 xv = *reinterpret_cast<const float4*>(xs + j * hidden + 4 * i);
                        acc[j][0] = fmaf(xv.x, gv[u].x, acc[j][0]);
                        acc[j][0] = fmaf(xv.y, gv[u].y, acc[j][0]);
                        acc[j][0] = fmaf(xv.z, gv[u].z, acc[j][0]);
                        acc[j][0] = fmaf(xv.w, gv[u].w, acc[j][0]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kRouterTokens; ++j) acc[j][0] = warp_sum(acc[j][0]);
    } else {
        quarter_dot<kRouterTokens, 1>(xs, hidden, tokens, g, quarter, lane, acc);
    }
    if (lane == 0)
#pragma unroll
        for (int j = 0; j < kRouterTokens; ++j) part[warp][j] = acc[j][0];
    __syncthreads();
    if (threadIdx.x < 2 * kRouterTokens) {
        const int which = threadIdx.x / kRouterTokens, j = threadIdx.x % kRouterTokens;
        const int ee = blockIdx.x * 2 + which;
        if (ee < experts && j < tokens)
            logits[(size_t)j * experts + ee] = (part[which * 4][j] + part[which * 4 + 1][j]) +
                                               (part[which * 4 + 2][j] + part[which * 4 + 3][j]);
    }
}

// A logit may arrive in parts to be added: parts[chunk][token][term][expert] (the partial
// products of a tensor-core router product: K in chunks, the 32-bit gate in terms), summed here
// in one fixed order, chunk by chunk and term by term, instead of by a kernel of its own.
struct LogitParts {
    const float* p;
    int tokens, experts, chunks, terms;
};
__device__ __forceinline__ float logit_at(const LogitParts& s, int t, int e) {
    if (s.chunks * s.terms == 1) return s.p[(size_t)t * s.experts + e];
    // the parts' loads do not wait for one another: they are issued several at a time, the adds
    // follow in order
    float v = 0.f;
    const float* base = s.p + (size_t)t * s.terms * s.experts + e;
    const size_t chunk_stride = (size_t)s.tokens * s.terms * s.experts;
#pragma unroll 2
    for (int c = 0; c < s.chunks; ++c) {
        const float* pc = base + c * chunk_stride;
#pragma unroll 3
        for (int k = 0; k < s.terms; ++k) v += __ldg(pc + (size_t)k * s.experts);
    }
    return v;
}

// One block per token: score function, selection bias, top-k in the reference's order,
// renormalisation.
__global__ void router_select_kernel(const LogitParts src, const float* __restrict__ bias,
                                     int* __restrict__ ids, float* __restrict__ weights, int experts, int top_k,
                                     int score_fn, int renormalize, float routed_scale) {
    extern __shared__ __align__(16) float sel[];
    const int padded = (experts + 3) & ~3;
    float* pj = sel;                     // [experts] probabilities
    float* sj = pj + padded;             // [experts] selection scores (16-byte aligned)
    int* ranks = (int*)(sj + padded);    // [experts]
    float* w_s = (float*)(ranks + padded);   // [top_k] probabilities of the chosen, in slot order
    __shared__ float red[33];
    __shared__ float thr_s;
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const float* lg = src.p + (size_t)t * experts;
    if (src.chunks * src.terms != 1) {       // the sums first, into the array that takes the scores below
        for (int e = threadIdx.x; e < experts; e += blockDim.x) sj[e] = logit_at(src, t, e);
        __syncthreads();
        lg = sj;
    }
    if (score_fn == 1) {   // softmax over experts
        float mx = -INFINITY;
        for (int e = threadIdx.x; e < experts; e += blockDim.x) mx = fmaxf(mx, lg[e]);
        mx = warp_max(mx);
        if (lane == 0) red[warp] = mx;
        __syncthreads();
        mx = -INFINITY;
        for (int w = 0; w < nwarps; ++w) mx = fmaxf(mx, red[w]);
        float sum = 0.f;
        for (int e = threadIdx.x; e < experts; e += blockDim.x) sum += expf(lg[e] - mx);
        sum = block_sum(sum, red);
        for (int e = threadIdx.x; e < experts; e += blockDim.x) {
            const float pe = expf(lg[e] - mx) / sum;
            const float s = pe + (bias ? bias[e] : 0.f);
            pj[e] = pe;
            sj[e] = (s == s) ? s : INFINITY;
        }
    } else {
        for (int e = threadIdx.x; e < experts; e += blockDim.x) {     // logit and bias: one trip to memory
            const float l = lg[e], bv = bias ? bias[e] : 0.f;
            const float pe = 1.f / (1.f + expf(-l));
            const float s = pe + bv;
            pj[e] = pe;
            sj[e] = (s == s) ? s : INFINITY;
        }
    }
    __syncthreads();
    // rank of e = number of experts that precede it in (score descending, index ascending);
    // ranks are a permutation, the chosen are the ranks below top_k and the threshold is
    // the score of rank top_k-1.
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const float s = sj[e];
        int rank = 0;
        int o = 0;
        for (; o + 4 <= experts; o += 4) {           // sj is 16-byte aligned: experts*4 bytes per array
            const float4 v = *reinterpret_cast<const float4*>(sj + o);
            rank += (v.x > s) || (v.x == s && o < e);
            rank += (v.y > s) || (v.y == s && o + 1 < e);
            rank += (v.z > s) || (v.z == s && o + 2 < e);
            rank += (v.w > s) || (v.w == s && o + 3 < e);
        }
        for (; o < experts; ++o) {
            const float so = sj[o];
            rank += (so > s) || (so == s && o < e);
        }
        ranks[e] = rank;
        if (rank == top_k - 1) thr_s = s;
    }
    __syncthreads();
    const float thr = thr_s;
    // Slot order: strictly greater than the threshold by ascending index, then ties with it
    // by ascending index: two prefix counts over the experts in index order.
    float cnt = 0.f;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt += (ranks[e] < top_k && sj[e] > thr) ? 1.f : 0.f;
    const int n_greater = (int)block_sum(cnt, red);
    __shared__ int wcount[2][32];
    __shared__ int run[2];
    if (threadIdx.x == 0) run[0] = run[1] = 0;
    __syncthreads();
    for (int base = 0; base < experts; base += blockDim.x) {
        const int e = base + threadIdx.x;
        const bool chosen = e < experts && ranks[e] < top_k;
        const bool gr = chosen && sj[e] > thr, tie = chosen && !gr;
        const unsigned bg = __ballot_sync(0xffffffffu, gr), bt = __ballot_sync(0xffffffffu, tie);
        if (lane == 0) { wcount[0][warp] = __popc(bg); wcount[1][warp] = __popc(bt); }
        __syncthreads();
        int pg = run[0], pt = run[1];
        for (int w = 0; w < warp; ++w) { pg += wcount[0][w]; pt += wcount[1][w]; }
        pg += __popc(bg & ((1u << lane) - 1u));
        pt += __popc(bt & ((1u << lane) - 1u));
        if (chosen) {
            const int slot = gr ? pg : n_greater + pt;
            ids[(size_t)t * top_k + slot] = e;
            w_s[slot] = pj[e];
        }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int w = 0; w < nwarps; ++w) { run[0] += wcount[0][w]; run[1] += wcount[1][w]; }
        __syncthreads();
    }
    // every writer adds the chosen probabilities in slot order, as one thread would
    for (int k = threadIdx.x; k < top_k; k += blockDim.x) {
        float sum = 0.f;
        for (int s = 0; s < top_k; ++s) sum += w_s[s];
        weights[(size_t)t * top_k + k] = (renormalize ? w_s[k] / sum : w_s[k]) * routed_scale;
    }
}

// The same selection by one warp per token, for sigmoid scores and up to 256 experts (what
// MiniMax M2 has): lane l holds experts l, l + 32, ... in registers; top_k rounds of "best
// remaining" find the chosen set (the warp's best key by one redux.max, the lowest expert
// that has it by one redux.min), then slots and weights as above.  Same values, slot for slot.
constexpr int kSelPer = 8;             // experts per lane

__global__ void __launch_bounds__(256)
router_select_warp_kernel(const LogitParts src, const float* __restrict__ bias, int* __restrict__ ids,
                          float* __restrict__ weights, int tokens, int experts, int top_k, int renormalize,
                          float routed_scale) {
    extern __shared__ float sel_w[];                 // [warps][top_k] probabilities of the chosen, in slot order
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    float* w_s = sel_w + warp * top_k;
    const unsigned below = (1u << lane) - 1u;
    float pj[kSelPer], sj[kSelPer];
    unsigned key[kSelPer];                           // the score as an unsigned key in the same order; 0 = none or taken
    // the lane's logits; parts are added chunk by chunk and term by term, the loads of a step for
    // all of the lane's experts at once
    float lg[kSelPer];
    if (src.chunks * src.terms == 1) {
#pragma unroll
        for (int i = 0; i < kSelPer; ++i) lg[i] = 32 * i + lane < experts ? src.p[(size_t)t * experts + 32 * i + lane] : 0.f;
    } else {
#pragma unroll
        for (int i = 0; i < kSelPer; ++i) lg[i] = 0.f;
        const float* base = src.p + (size_t)t * src.terms * experts + lane;
        const size_t chunk_stride = (size_t)src.tokens * src.terms * experts;
        for (int c = 0; c < src.chunks; ++c) {
#pragma unroll 3
            for (int k = 0; k < src.terms; ++k) {
                const float* pk = base + c * chunk_stride + (size_t)k * experts;
#pragma unroll
                for (int i = 0; i < kSelPer; ++i)
                    if (32 * i + lane < experts) lg[i] += __ldg(pk + 32 * i);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kSelPer; ++i) {
        const int e = 32 * i + lane;
        pj[i] = 0.f;
        sj[i] = 0.f;
        key[i] = 0u;
        if (e < experts) {
            pj[i] = 1.f / (1.f + expf(-lg[i]));
            const float sc = pj[i] + (bias ? bias[e] : 0.f);
            sj[i] = (sc == sc) ? sc : INFINITY;      // a NaN score counts as +inf
            const unsigned u = __float_as_uint(sj[i]);
            key[i] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
            if (key[i] == 0u) key[i] = 1u;
        }
    }
    unsigned chosen = 0;                             // bit i: expert 32 i + lane
    float thr = 0.f;
    for (int r = 0; r < top_k; ++r) {
        unsigned bk = 0u;
        int bi = 0;
#pragma unroll
        for (int i = 0; i < kSelPer; ++i)
            if (key[i] > bk) {                       // ascending i: the lowest index among equals stays
                bk = key[i];
                bi = i;
            }
        const unsigned top = __reduce_max_sync(0xffffffffu, bk);
        const unsigned mine = (bk == top && bk != 0u) ? (unsigned)(32 * bi + lane) : 0xffffffffu;
        const unsigned win = __reduce_min_sync(0xffffffffu, mine);
        if (mine == win) {
            chosen |= 1u << bi;
#pragma unroll
            for (int i = 0; i < kSelPer; ++i)
                if (i == bi) {
                    thr = sj[i];
                    key[i] = 0u;
                }
        }
        thr = __shfl_sync(0xffffffffu, thr, win & 31u);
    }
    // slots: strictly above the threshold by ascending index, then the ties with it
    int n_greater = 0;
#pragma unroll
    for (int i = 0; i < kSelPer; ++i) n_greater += (((chosen >> i) & 1u) && sj[i] > thr) ? 1 : 0;
    n_greater = __reduce_add_sync(0xffffffffu, n_greater);
    int run_g = 0, run_t = 0;
#pragma unroll
    for (int i = 0; i < kSelPer; ++i) {
        const bool c = (chosen >> i) & 1u;
        const bool gr = c && sj[i] > thr, tie = c && !gr;
        const unsigned bg = __ballot_sync(0xffffffffu, gr), bt = __ballot_sync(0xffffffffu, tie);
        if (c) {
            const int slot = gr ? run_g + __popc(bg & below) : n_greater + run_t + __popc(bt & below);
            ids[(size_t)t * top_k + slot] = 32 * i + lane;
            w_s[slot] = pj[i];
        }
        run_g += __popc(bg);
        run_t += __popc(bt);
    }
    __syncwarp();
    float sum = 0.f;
    for (int k = 0; k < top_k; ++k) sum += w_s[k];                  // slot order, as one thread adds them
    for (int k = lane; k < top_k; k += 32)
        weights[(size_t)t * top_k + k] = (renormalize ? w_s[k] / sum : w_s[k]) * routed_scale;
}

}  // namespace se

// impl: 0 = by sizes, 1 = the block-per-token kernel, 2 = the warp-per-token kernel
static int launch_select(const float* logits, int chunks, int terms, const float* bias, int* ids, float* weights,
                         int tokens, int experts, int top_k, int score_fn, int renormalize, float routed_scale, int impl,
                         cudaStream_t stream) {
    const se::LogitParts src{logits, tokens, experts, chunks, terms};
    const size_t smem_sel = (size_t)((experts + 3) & ~3) * 4 * sizeof(float);
    const bool warp_ok = score_fn == 0 && experts <= 32 * se::kSelPer && top_k <= 256;
    if (impl == 2 && !warp_ok) return SE_ERR_UNSUPPORTED;
    if (experts > 200 * 1024 / 16) return SE_ERR_UNSUPPORTED;
    // A warp's selection is one long chain of dependent steps (8 us for a token, against 6.6 us
    // for the block kernel), so it pays when there are tokens enough to fill the SMs with warps.
    if (impl == 2 || (impl == 0 && warp_ok && tokens >= 128)) {
        se::router_select_warp_kernel<<<se::ceil_div(tokens, 8), 256, 8 * top_k * sizeof(float), stream>>>(
            src, bias, ids, weights, tokens, experts, top_k, renormalize, routed_scale);
        SE_LAUNCH_CHECK();
    }
    if (smem_sel > 40 * 1024) {      // static shared memory counts against the 48 KB a kernel has without asking
        cudaError_t e = cudaFuncSetAttribute(se::router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_sel);
        if (e != cudaSuccess) return (int)e;
    }
    se::router_select_kernel<<<tokens, 256, smem_sel, stream>>>(src, bias, ids, weights, experts, top_k, score_fn,
                                                                renormalize, routed_scale);
    SE_LAUNCH_CHECK();
}

// Selection alone, from given logits: float [tokens, experts], or float [chunks, tokens, terms,
// experts] whose sum over chunks and terms (in that order) is the logit.
extern "C" int se_router_select(const float* logits, int chunks, int terms, const float* bias, int* ids, float* weights,
                                int tokens, int experts, int top_k, int score_fn, int renormalize, float routed_scale,
                                int impl, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (top_k <= 0 || top_k > experts || impl < 0 || impl > 2 || chunks < 1 || terms < 1) return SE_ERR_ARGUMENT;
    return launch_select(logits, chunks, terms, bias, ids, weights, tokens, experts, top_k, score_fn, renormalize,
                         routed_scale, impl, stream);
}

// Most experts the selection takes (four floats per expert in 200 KB of shared memory), and the
// widest row whose width is no multiple of 4.
extern "C" int se_router_max_experts() { return 200 * 1024 / 16; }
extern "C" int se_router_max_unaligned_width() { return 200 * 1024 / (se::kRouterTokens * (int)sizeof(float)); }

// logits: float [tokens, experts] workspace (also the logits output for whoever wants them).
extern "C" int se_router(const void* x, const float* gate, const float* bias, int* ids, float* weights,
                         float* logits, int tokens, int hidden, int experts, int top_k, int score_fn,
                         int renormalize, float routed_scale, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (top_k <= 0 || top_k > experts || logits == nullptr) return SE_ERR_ARGUMENT;
    const int tile_tokens = tokens < se::kRouterTokens ? tokens : se::kRouterTokens;
    const size_t smem = (size_t)tile_tokens * hidden * sizeof(float);
    // The kernels that keep a tile of token rows in shared memory take rows up to 200 KB / 8
    // tokens; wider rows go to the tiled kernel (same order of sums), which needs a width that is
    // a multiple of 4.
    const bool rows_fit = smem <= 200 * 1024;
    if (experts > se_router_max_experts() || (!rows_fit && (hidden & 3) != 0)) return SE_ERR_UNSUPPORTED;
    SE_DISPATCH_DTYPE(dtype, T, {
        if (tokens <= se::kRouterTokens && rows_fit) {
            if (smem > 40 * 1024) {      // static shared memory counts against the 48 KB a kernel has without asking
                cudaError_t e = cudaFuncSetAttribute(se::router_logits_small_kernel<T>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            cudaError_t e = SE_LAUNCH_DEPENDENT("logits", se::router_logits_small_kernel<T>, dim3(se::ceil_div(experts, 2)),
                                                 dim3(32 * se::kRouterWarps), smem, stream, (const T*)x, gate, logits,
                                                 tokens, hidden, experts);
            if (e != cudaSuccess) return (int)e;
        } else if ((hidden & 3) == 0) {
            dim3 grid(se::ceil_div(tokens, se::kBigTokens), se::ceil_div(experts, se::kBigExperts));
            const int tiled_smem = se::kBigStages * (se::kBigTokens * 128 * (int)sizeof(T) + se::kBigExperts * 128 * (int)sizeof(float)) +
                                   8 * 4 * 64 * (int)sizeof(float);
            cudaError_t e = cudaFuncSetAttribute(se::router_logits_tiled_kernel<T>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, tiled_smem);
            if (e != cudaSuccess) return (int)e;
            se::router_logits_tiled_kernel<T><<<grid, 256, tiled_smem, stream>>>((const T*)x, gate, logits, tokens, hidden,
                                                                                  experts);
        } else {
            if (smem > 40 * 1024) {      // static shared memory counts against the 48 KB a kernel has without asking
                cudaError_t e = cudaFuncSetAttribute(se::router_logits_kernel<T>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            dim3 grid(se::ceil_div(tokens, se::kRouterTokens),
                      se::ceil_div(experts, se::kRouterWarps * se::kRouterExperts));
            se::router_logits_kernel<T><<<grid, 32 * se::kRouterWarps, smem, stream>>>((const T*)x, gate, logits, tokens,
                                                                                        hidden, experts);
        }
    });
    return launch_select(logits, 1, 1, bias, ids, weights, tokens, experts, top_k, score_fn, renormalize, routed_scale, 0,
                         stream);
}
