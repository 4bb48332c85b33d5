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

namespace se {

constexpr int kRouterTokens = 8;   // tokens that share one read of the gate weight

template <typename T>
__global__ void router_kernel(const T* __restrict__ x, const float* __restrict__ gate, const float* __restrict__ bias,
                              int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ logits_out,
                              int tokens, int hidden, int experts, int top_k, int score_fn, int renormalize,
                              float routed_scale, int tokens_per_block) {
    extern __shared__ float smem[];
    float* xs = smem;                                        // [tokens_per_block][hidden]
    float* prob = xs + (size_t)tokens_per_block * hidden;    // [tokens_per_block][experts]
    float* score = prob + (size_t)tokens_per_block * experts;
    int* ranks = (int*)(score + (size_t)tokens_per_block * experts);   // [experts]
    float* thr_s = (float*)(ranks + experts);
    const int t0 = blockIdx.x * tokens_per_block;
    const int nt = min(tokens_per_block, tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

    for (int i = threadIdx.x; i < nt * hidden; i += blockDim.x)
        xs[i] = to_float(x[(size_t)t0 * hidden + i]);
    __syncthreads();

    for (int e = warp; e < experts; e += nwarps) {
        float acc[kRouterTokens];
#pragma unroll
        for (int j = 0; j < kRouterTokens; ++j) acc[j] = 0.f;
        const float* g = gate + (size_t)e * hidden;
        for (int i = lane; i < hidden; i += 32) {
            const float gv = g[i];
#pragma unroll
            for (int j = 0; j < kRouterTokens; ++j)
                if (j < nt) acc[j] = fmaf(xs[j * hidden + i], gv, acc[j]);
        }
#pragma unroll
        for (int j = 0; j < kRouterTokens; ++j) {
            if (j < nt) {
                const float v = warp_sum(acc[j]);
                if (lane == 0) prob[j * experts + e] = v;   // logits for now
            }
        }
    }
    __syncthreads();

    for (int j = 0; j < nt; ++j) {
        float* pj = prob + j * experts;
        float* sj = score + j * experts;
        if (score_fn == 1) {   // softmax over experts
            float mx = -INFINITY;
            for (int e = threadIdx.x; e < experts; e += blockDim.x) mx = fmaxf(mx, pj[e]);
            __shared__ float red[33];
            mx = warp_max(mx);
            __syncthreads();
            if (lane == 0) red[warp] = mx;
            __syncthreads();
            mx = -INFINITY;
            for (int w = 0; w < nwarps; ++w) mx = fmaxf(mx, red[w]);
            float sum = 0.f;
            for (int e = threadIdx.x; e < experts; e += blockDim.x) sum += expf(pj[e] - mx);
            sum = block_sum(sum, red);
            for (int e = threadIdx.x; e < experts; e += blockDim.x) {
                if (logits_out) logits_out[(size_t)(t0 + j) * experts + e] = pj[e];
                pj[e] = expf(pj[e] - mx) / sum;
            }
        } else {
            for (int e = threadIdx.x; e < experts; e += blockDim.x) {
                if (logits_out) logits_out[(size_t)(t0 + j) * experts + e] = pj[e];
                pj[e] = 1.f / (1.f + expf(-pj[e]));
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < experts; e += blockDim.x) {
            float s = pj[e] + (bias ? bias[e] : 0.f);
            sj[e] = (s == s) ? s : INFINITY;
        }
        __syncthreads();
        // rank of e = number of experts that precede it in (score descending, index
        // ascending); ranks are a permutation, the chosen are the ranks below top_k and
        // the threshold is the score of rank top_k-1.
        for (int e = threadIdx.x; e < experts; e += blockDim.x) {
            const float s = sj[e];
            int rank = 0;
            for (int o = 0; o < experts; ++o) {
                const float so = sj[o];
                rank += (so > s) || (so == s && o < e);
            }
            ranks[e] = rank;
            if (rank == top_k - 1) *thr_s = s;
        }
        __syncthreads();
        const float thr = *thr_s;
        for (int e = threadIdx.x; e < experts; e += blockDim.x) {
            if (ranks[e] >= top_k) continue;
            // slot order: strictly greater than the threshold by ascending index, then
            // ties with it by ascending index.
            const float s = sj[e];
            int n_greater = 0, before_greater = 0, before_equal = 0;
            for (int o = 0; o < experts; ++o) {
                const float so = sj[o];
                n_greater += so > thr;
                before_greater += (so > thr) && o < e;
                before_equal += (so == thr) && o < e && ranks[o] < top_k;
            }
            const int slot = s > thr ? before_greater : n_greater + before_equal;
            ids[(size_t)(t0 + j) * top_k + slot] = e;
            weights[(size_t)(t0 + j) * top_k + slot] = pj[e];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float* w = weights + (size_t)(t0 + j) * top_k;
            float sum = 0.f;
            for (int s = 0; s < top_k; ++s) sum += w[s];
            for (int s = 0; s < top_k; ++s) w[s] = (renormalize ? w[s] / sum : w[s]) * routed_scale;
        }
        __syncthreads();
    }
}

}  // namespace se

extern "C" int se_router(const void* x, const float* gate, const float* bias, int* ids, float* weights,
                         float* logits_out, int tokens, int hidden, int experts, int top_k, int score_fn,
                         int renormalize, float routed_scale, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (top_k <= 0 || top_k > experts) return SE_ERR_ARGUMENT;
    int tpb = se::kRouterTokens;
    while (tpb > 1 && ((size_t)tpb * (hidden + 2 * experts) + experts + 1) * sizeof(float) > 160 * 1024) tpb >>= 1;
    if (tokens < 4 * 148) tpb = 1;   // few tokens: spread them over the SMs
    const size_t smem = ((size_t)tpb * (hidden + 2 * experts) + experts + 1) * sizeof(float);
    if (smem > 200 * 1024) return SE_ERR_UNSUPPORTED;
    SE_DISPATCH_DTYPE(dtype, T, {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(se::router_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        se::router_kernel<T><<<se::ceil_div(tokens, tpb), 256, smem, stream>>>(
            (const T*)x, gate, bias, ids, weights, logits_out, tokens, hidden, experts, top_k, score_fn, renormalize,
            routed_scale, tpb);
    });
    SE_LAUNCH_CHECK();
}
