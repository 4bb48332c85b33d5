// Sampling over the vocabulary, one block per row: greedy argmax, temperature, top-k,
// top-p, and the presence / repetition penalties.
//
// Reference semantics (src/sparseengine/layers/sampler.py:66-135): rows with temperature
// <= 1e-10 take argmax of the unscaled logits; others take p = softmax(logits / T) in
// 32-bit, keep the top-k (0 = all), then keep the smallest prefix of the sorted
// probabilities whose mass before each kept entry does not exceed top-p (the first is
// always kept), and draw by the exponential race argmax(p_i / e_i), e_i ~ Exp(1) clamped
// at 1e-10.  Here the two cuts are found without sorting, by bisection on the value of
// the threshold (entries that tie with the k-th value are all kept), and the noise
// comes from a counter-based generator (Philox 4x32-10) keyed by the row's own seed, so
// a request's draw does not depend on what else is in the batch.
// Penalties (src/sparseengine/layers/sampler.py:10-64): repetition divides positive logits
// and multiplies negative ones; presence subtracts.
#include "common.cuh"

namespace se {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ uint32_t ordered_key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct ArgMax {
    float v;
    int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    // larger value wins; NaN counts as larger than anything; ties go to the lower index
    const bool a_nan = a.v != a.v, b_nan = b.v != b.v;
    if (a.i < 0) return b;
    if (b.i < 0) return a;
    if (a_nan || b_nan) {
        if (a_nan && b_nan) return a.i < b.i ? a : b;
        return a_nan ? a : b;
    }
    if (a.v > b.v) return a;
    if (b.v > a.v) return b;
    return a.i < b.i ? a : b;
}

__device__ ArgMax block_argmax(ArgMax x, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    if (warp == 0) {
        ArgMax t = lane < nwarps ? scratch[lane] : ArgMax{0.f, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax y;
            y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, y);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

template <typename T>
__global__ void sample_kernel(const T* __restrict__ logits, const float* __restrict__ temperature,
                              const int* __restrict__ top_k, const float* __restrict__ top_p,
                              const unsigned long long* __restrict__ seeds, int* __restrict__ out,
                              float* __restrict__ logprob, int vocab) {
    __shared__ ArgMax am[33];
    __shared__ float red[33];
    const int row = blockIdx.x;
    const T* x = logits + (size_t)row * vocab;
    const float temp = temperature ? temperature[row] : 0.f;
    const bool greedy = temp <= 1e-10f;

    // pass 1: argmax of the raw logits (also the maximum for the softmax)
    ArgMax best{0.f, -1};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{to_float(x[i]), i});
    best = block_argmax(best, am);
    const float inv_t = greedy ? 1.f : 1.f / temp;
    const float mx = best.v * inv_t;

    int k = top_k ? top_k[row] : 0;
    float p_cut = top_p ? top_p[row] : 1.f;
    uint32_t thr = 0;   // keep entries with ordered_key(scaled) >= thr
    if (!greedy && k > 0 && k < vocab) {
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            float cnt = 0.f;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x)
                cnt += ordered_key(to_float(x[i]) * inv_t) >= cand ? 1.f : 0.f;
            cnt = block_sum(cnt, red);
            if (cnt >= (float)k) prefix = cand;
        }
        thr = prefix;
    }
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float s = to_float(x[i]) * inv_t;
        if (ordered_key(s) >= thr) z += expf(s - mx);
    }
    z = block_sum(z, red);
    if (logprob != nullptr && greedy && threadIdx.x == 0) {
        // log-probability of the chosen token under the unscaled distribution
        logprob[row] = -logf(z);
    }
    if (greedy) {
        if (threadIdx.x == 0) out[row] = best.i;
        return;
    }
    if (p_cut < 1.f) {
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            float mass = 0.f;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const float s = to_float(x[i]) * inv_t;
                const uint32_t key = ordered_key(s);
                if (key >= cand && key >= thr) mass += expf(s - mx);
            }
            mass = block_sum(mass, red);
            if (mass / z > p_cut) prefix = cand;
        }
        thr = max(thr, prefix);
    }
    const unsigned long long seed = seeds[row];
    ArgMax pick{0.f, -1};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float s = to_float(x[i]) * inv_t;
        if (ordered_key(s) < thr) continue;
        uint32_t r[4];
        philox4x32_10((uint32_t)(i >> 2), 0u, 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
        const float u = ((float)r[i & 3] + 0.5f) * 2.3283064365386963e-10f;   // (0, 1)
        const float e = fmaxf(-logf(u), 1e-10f);
        pick = better(pick, ArgMax{expf(s - mx) / e, i});
    }
    pick = block_argmax(pick, am);
    if (threadIdx.x == 0) {
        out[row] = pick.i;
        if (logprob != nullptr) logprob[row] = to_float(x[pick.i]) * inv_t - mx - logf(z);
    }
}

// Greedy over a large vocabulary with few rows: stage 1 reduces `chunks` slices of each row
// in parallel, stage 2 reduces the partial results (ties still go to the lower index).
template <typename T>
__global__ void argmax_partial_kernel(const T* __restrict__ logits, float* __restrict__ pval, int* __restrict__ pidx,
                                      int vocab, int chunks) {
    __shared__ ArgMax am[33];
    const int row = blockIdx.x, chunk = blockIdx.y;
    const int per = (vocab + chunks - 1) / chunks;
    const int a = chunk * per, b = min(vocab, a + per);
    const T* x = logits + (size_t)row * vocab;
    ArgMax best{0.f, -1};
    for (int i = a + threadIdx.x; i < b; i += blockDim.x) best = better(best, ArgMax{to_float(x[i]), i});
    best = block_argmax(best, am);
    if (threadIdx.x == 0) {
        pval[row * chunks + chunk] = best.v;
        pidx[row * chunks + chunk] = best.i;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx, int* __restrict__ out,
                                    int chunks) {
    __shared__ ArgMax am[33];
    const int row = blockIdx.x;
    ArgMax best{0.f, -1};
    for (int i = threadIdx.x; i < chunks; i += blockDim.x)
        best = better(best, ArgMax{pval[row * chunks + i], pidx[row * chunks + i]});
    best = block_argmax(best, am);
    if (threadIdx.x == 0) out[row] = best.i;
}

// pairs: n entries (row, token, flags); flags bit 0 = in prompt or completion (repetition),
// bit 1 = in completion (presence).  logits is float32 [rows, vocab], changed in place.
__global__ void penalties_kernel(float* logits, const int* __restrict__ pairs, int n, int vocab,
                                 const float* __restrict__ repetition, const float* __restrict__ presence) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int row = pairs[3 * i], tok = pairs[3 * i + 1], flags = pairs[3 * i + 2];
    if (tok < 0 || tok >= vocab) return;
    float v = logits[(size_t)row * vocab + tok];
    const float r = repetition[row], p = presence[row];
    if ((flags & 1) && r != 1.f) v = v > 0.f ? v / r : v * r;
    if ((flags & 2) && p != 0.f) v -= p;
    logits[(size_t)row * vocab + tok] = v;
}

template <typename T>
__global__ void to_float_kernel(const T* __restrict__ src, float* __restrict__ dst, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = to_float(src[i]);
}

}  // namespace se

// temperature/top_k/top_p/seeds may be null (then every row is greedy).
extern "C" int se_sample(const void* logits, const float* temperature, const int* top_k, const float* top_p,
                         const unsigned long long* seeds, int* out, float* logprob, int rows, int vocab, int dtype,
                         cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (temperature != nullptr && seeds == nullptr) return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T,
        se::sample_kernel<T><<<rows, se::kSampleThreads, 0, stream>>>((const T*)logits, temperature, top_k, top_p,
                                                                      seeds, out, logprob, vocab));
    SE_LAUNCH_CHECK();
}

// Greedy tokens only (no log-probabilities).  pval/pidx: workspaces of rows * 64 entries.
extern "C" int se_argmax(const void* logits, int* out, float* pval, int* pidx, int rows, int vocab, int dtype,
                         cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int chunks = 64;
    dim3 grid(rows, chunks);
    SE_DISPATCH_DTYPE(dtype, T,
        se::argmax_partial_kernel<T><<<grid, 256, 0, stream>>>((const T*)logits, pval, pidx, vocab, chunks));
    se::argmax_final_kernel<<<rows, 64, 0, stream>>>(pval, pidx, out, chunks);
    SE_LAUNCH_CHECK();
}

extern "C" int se_apply_penalties(float* logits, const int* pairs, int n, int vocab, const float* repetition,
                                  const float* presence, cudaStream_t stream) {
    if (n <= 0) return 0;
    se::penalties_kernel<<<se::ceil_div(n, 256), 256, 0, stream>>>(logits, pairs, n, vocab, repetition, presence);
    SE_LAUNCH_CHECK();
}

namespace se {

// The n most likely tokens of a row with their log-probabilities (log-softmax in 32-bit of the
// logits as given), most likely first, equal logits by ascending token id
// (src/sparseengine/engine/model_runner.py:2528-2569: log_softmax, then topk).  One block per
// listed row: a pass for the log-sum-exp, then one pass per entry for the best logit after the
// previous one in that order.
template <typename T>
__global__ void __launch_bounds__(256)
top_logprobs_kernel(const T* __restrict__ logits, const int* __restrict__ rows, int* __restrict__ ids,
                    float* __restrict__ values, int vocab, int n) {
    __shared__ float red[33];
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    __shared__ float prev_v_s;
    __shared__ int prev_i_s;
    const T* lg = logits + (size_t)rows[blockIdx.x] * vocab;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, to_float(lg[i]));
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) sum += expf(to_float(lg[i]) - mx);
    sum = block_sum(sum, red);
    const float lse = mx + logf(sum);
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int r = 0; r < n; ++r) {
        // the best (value descending, id ascending) strictly after (prev_v, prev_i)
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = to_float(lg[i]);
            const bool after = v < prev_v || (v == prev_v && i > prev_i);
            if (after && (v > bv || (v == bv && i < bi))) {
                bv = v;
                bi = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (lane == 0) {
            best_v[warp] = bv;
            best_i[warp] = bi;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
                if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) {
                    bv = best_v[w];
                    bi = best_i[w];
                }
            prev_v_s = bv;
            prev_i_s = bi;
            ids[(size_t)blockIdx.x * n + r] = bi == 0x7fffffff ? -1 : bi;        // -1: fewer than n tokens (NaN logits)
            values[(size_t)blockIdx.x * n + r] = bv - lse;
        }
        __syncthreads();
        prev_v = prev_v_s;
        prev_i = prev_i_s;
    }
}

}  // namespace se

// rows: int32 [count] row indices into logits [*, vocab]; ids int32 [count, n], values float [count, n].
extern "C" int se_top_logprobs(const void* logits, const int* rows, int* ids, float* values, int count, int vocab, int n,
                               int dtype, cudaStream_t stream) {
    if (count <= 0 || n <= 0) return 0;
    if (n > vocab) return SE_ERR_ARGUMENT;
    SE_DISPATCH_DTYPE(dtype, T,
        se::top_logprobs_kernel<T><<<count, 256, 0, stream>>>((const T*)logits, rows, ids, values, vocab, n));
    SE_LAUNCH_CHECK();
}

extern "C" int se_to_float(const void* src, float* dst, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 1023) / 1024 < 4096 ? (n + 1023) / 1024 : 4096);
    SE_DISPATCH_DTYPE(dtype, T, se::to_float_kernel<T><<<blocks, 256, 0, stream>>>((const T*)src, dst, (size_t)n));
    SE_LAUNCH_CHECK();
}
