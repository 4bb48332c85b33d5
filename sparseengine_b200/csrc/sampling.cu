// Sampling over the vocabulary, one block per row: greedy argmax, temperature, top-k,
// top-p, and the presence / repetition penalties.
//
// Reference semantics (src/sparseengine/layers/sampler.py:66-135): rows with temperature
// <= 1e-10 take argmax of the unscaled logits; others take p = softmax(logits / T) in
// 32-bit, keep the top-k (0 = all), then keep the smallest prefix of the sorted
// probabilities whose mass before each kept entry does not exceed top-p (the first is
// always kept), and draw by the exponential race argmax(p_i / e_i), e_i ~ Exp(1) clamped
// at 1e-10.  Here the two cuts are found without sorting, as thresholds on the value
// (entries that tie with the k-th value are all kept): by bisection over the bits of the
// threshold in the defining form of the kernel, and in its fast form byte by byte for top-k
// and over a short list of the entries that can still be chosen for top-p; the noise
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

// ---- helpers of the fast path ------------------------------------------------------------
constexpr int kCand = 8192;          // candidates a row may keep in shared memory (value, index, weight: 96 KB)
constexpr int kTaus = 8;
__device__ __constant__ float kTau[kTaus] = {1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 16.f};   // distances below the maximum

// The k-th largest selection key of a row (k >= 1, at most the number of entries), byte by byte
// from the top: a 256-bin count of the current byte among the entries that share the bytes found
// so far (lanes with the same byte add once per warp), then the byte in which the count from the
// top reaches what is still needed.  It equals what a bisection over the bits finds: the largest
// threshold that at least k keys reach.  The selection key of a bfloat16 row is the 16-bit
// ordered key of the logit itself (two bytes; scaling by 1/T keeps the order of distinct
// bfloat16 values), of a float row the 32-bit ordered key of the scaled logit (four bytes).
template <typename T> struct SelKey;
template <> struct SelKey<float> {
    static constexpr int kBytes = 4;
    static __device__ __forceinline__ uint32_t of(float v, float inv_t) { return ordered_key(v * inv_t); }
    static __device__ __forceinline__ uint32_t threshold(uint32_t key, float) { return key; }
};
template <> struct SelKey<__nv_bfloat16> {
    static constexpr int kBytes = 2;
    static __device__ __forceinline__ uint32_t of(__nv_bfloat16 v, float) {
        const uint32_t u = (uint32_t)__bfloat16_as_ushort(v);
        return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
    }
    // the threshold on scaled logits that the entries at or above this key reach
    static __device__ __forceinline__ uint32_t threshold(uint32_t key, float inv_t) {
        const uint32_t u = (key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu);
        return ordered_key(__bfloat162float(__ushort_as_bfloat16((unsigned short)u)) * inv_t);
    }
};

__device__ __forceinline__ void count_byte(int digit, int* hist) {      // digit 256: none; all lanes of the warp call
    const unsigned same = __match_any_sync(0xffffffffu, digit);
    if (digit < 256 && (int)(threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&hist[digit], __popc(same));
}

// From a filled count: the byte where the count from the top reaches `need`, and what is still
// needed inside that byte.  Every thread gets both.
__device__ void resolve_byte(const int* hist, int need, int* found, int* digit, int* rest) {
    __syncthreads();
    if (threadIdx.x == 0) {
        int above = 0, d = 255;
        for (; d > 0; --d) {
            if (above + hist[d] >= need) break;
            above += hist[d];
        }
        found[0] = d;
        found[1] = need - above;
    }
    __syncthreads();
    *digit = found[0];
    *rest = found[1];
    __syncthreads();
}

// Sums of N values over the block, in a fixed order; every thread gets them in v.
template <int N>
__device__ void block_sum_n(float (&v)[N], float (*part)[N]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = warp_sum(v[j]);
    __syncthreads();
    if (lane == 0)
#pragma unroll
        for (int j = 0; j < N; ++j) part[warp][j] = v[j];
    __syncthreads();
    if (threadIdx.x < N) {
        float t = 0.f;
        for (int w = 0; w < nwarps; ++w) t += part[w][threadIdx.x];
        part[32][threadIdx.x] = t;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = part[32][j];
}

// Exclusive prefix sum of one int per thread over the block (thread order); *total gets the sum.
__device__ int block_exclusive_scan(int mine, int* warp_tot, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += u;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int before = 0, all = 0;
    for (int w = 0; w < nwarps; ++w) {
        if (w < warp) before += warp_tot[w];
        all += warp_tot[w];
    }
    *total = all;
    return before + inc - mine;
}

// FAST: the top-k threshold by counting bytes of the key instead of bisecting over 32 bits, and, when
// the entries that can still be chosen are few (always with a usual top-k, and with top-p whenever
// the mass is concentrated), the top-p cut and the draw over a list of those entries in shared
// memory instead of over the whole row.  The chosen token is the same as without FAST: the
// kept set is defined by the same thresholds and the noise of an entry depends on its index only.
// (The mass above a candidate threshold is summed over the list instead of over the row, which
// can move the top-p cut only where two sums differ in their last bit.)
template <typename T, bool FAST>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const unsigned long long* __restrict__ seeds, int* __restrict__ out,
              float* __restrict__ logprob, float* __restrict__ spill, int vocab) {
    extern __shared__ __align__(16) uint8_t cand_raw[];         // FAST: float s[kCand], int index[kCand], float weight[kCand]
    __shared__ ArgMax am[33];
    __shared__ float red[33];
    __shared__ int hist[256];
    __shared__ int found[2];
    __shared__ int warp_tot[32];
    __shared__ float part[33][2 * kTaus + 1];
    const int row = blockIdx.x;
    const T* x = logits + (size_t)row * vocab;
    const float temp = temperature ? temperature[row] : 0.f;
    const bool greedy = temp <= 1e-10f;

    const float inv_t = greedy ? 1.f : 1.f / temp;
    int k = top_k ? top_k[row] : 0;
    float p_cut = top_p ? top_p[row] : 1.f;
    const bool cut_k = !greedy && k > 0 && k < vocab;
    constexpr int kTopShift = 8 * (SelKey<T>::kBytes - 1);

    // pass 1: argmax of the raw logits (also the maximum for the softmax); with FAST and a top-k
    // cut, the count of the selection keys' top byte in the same pass
    ArgMax best{0.f, -1};
    if (FAST && cut_k) {
        for (int t = threadIdx.x; t < 256; t += blockDim.x) hist[t] = 0;
        __syncthreads();
        for (int base = 0; base < vocab; base += blockDim.x) {
            const int i = base + threadIdx.x;
            int digit = 256;
            if (i < vocab) {
                best = better(best, ArgMax{to_float(x[i]), i});
                digit = (int)(SelKey<T>::of(x[i], inv_t) >> kTopShift);
            }
            count_byte(digit, hist);
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{to_float(x[i]), i});
    }
    best = block_argmax(best, am);
    const float mx = best.v * inv_t;

    uint32_t thr = 0;   // keep entries with ordered_key(scaled) >= thr
    if (cut_k) {
        if (FAST) {
            int digit, need;
            resolve_byte(hist, k, found, &digit, &need);
            uint32_t prefix = (uint32_t)digit << kTopShift;
            for (int shift = kTopShift - 8; shift >= 0; shift -= 8) {
                for (int t = threadIdx.x; t < 256; t += blockDim.x) hist[t] = 0;
                __syncthreads();
                for (int base = 0; base < vocab; base += blockDim.x) {
                    const int i = base + threadIdx.x;
                    int d = 256;
                    if (i < vocab) {
                        const uint32_t key = SelKey<T>::of(x[i], inv_t);
                        if ((key >> (shift + 8)) == (prefix >> (shift + 8))) d = (int)((key >> shift) & 255u);
                    }
                    count_byte(d, hist);
                }
                resolve_byte(hist, need, found, &digit, &need);
                prefix |= (uint32_t)digit << shift;
            }
            thr = SelKey<T>::threshold(prefix, inv_t);
        } else {
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
    }
    // the normaliser over the kept entries; with FAST also, in the same pass, how many of them and
    // how much of their mass lie within kTau[j] of the maximum
    float z = 0.f;
    float near[2 * kTaus + 1];                   // mass [0..7], count [8..15], count of all kept [16]
#pragma unroll
    for (int j = 0; j < 2 * kTaus + 1; ++j) near[j] = 0.f;
    const bool survey = FAST && !greedy && (p_cut < 1.f || thr != 0u);
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float s = to_float(x[i]) * inv_t;
        if (ordered_key(s) >= thr) {
            const float e = expf(s - mx);
            z += e;
            if (survey) {
                const float dist = mx - s;
                near[2 * kTaus] += 1.f;
#pragma unroll
                for (int j = 0; j < kTaus; ++j)
                    if (dist <= kTau[j]) {
                        near[j] += e;
                        near[kTaus + j] += 1.f;
                    }
            }
        }
    }
    float my_count[kTaus + 1];                  // this thread's own counts, before they become block sums
#pragma unroll
    for (int j = 0; j <= kTaus; ++j) my_count[j] = near[kTaus + j];
    z = block_sum(z, red);
    if (logprob != nullptr && greedy && threadIdx.x == 0) {
        // log-probability of the chosen token under the unscaled distribution
        logprob[row] = -logf(z);
    }
    if (greedy) {
        if (threadIdx.x == 0) out[row] = best.i;
        return;
    }
    // Which entries go on the list: all kept ones if they fit into shared memory; else, with a top-p
    // cut, those within the smallest distance whose mass is safely beyond the cut (what lies further
    // cannot be chosen); a list too long for shared memory goes to the row's workspace in global memory.
    bool listed = false, all_kept = false;
    float reach = INFINITY;
    int mine = 0;                                // entries of this thread that go on the list
    float listed_count = 0.f;
    if (survey) {
        block_sum_n<2 * kTaus + 1>(near, part);
        const float all = near[2 * kTaus];
        if (all >= 1.f) {
            all_kept = true;
            listed_count = all;
            mine = (int)my_count[kTaus];
            if (all > (float)kCand && p_cut < 1.f) {
#pragma unroll
                for (int j = 0; j < kTaus; ++j)
                    if (all_kept && near[j] > p_cut * z * 1.0001f && near[kTaus + j] >= 1.f) {
                        all_kept = false;
                        reach = kTau[j];
                        listed_count = near[kTaus + j];
                        mine = (int)my_count[j];
                    }
            }
            // a long list in global memory pays only while it is much shorter than the row
            listed = listed_count <= (float)kCand || (spill != nullptr && listed_count * 4.f <= (float)vocab);
        }
    }
    const unsigned long long seed = seeds[row];
    ArgMax pick{0.f, -1};
    if (listed) {
        const bool in_shared = listed_count <= (float)kCand;
        // a list in global memory is at most a quarter of the row long (see `listed` above)
        const size_t spill_stride = ((size_t)vocab + 3) / 4;
        float* spill_row = in_shared ? nullptr : spill + (size_t)row * 3 * spill_stride;
        float* cs = in_shared ? reinterpret_cast<float*>(cand_raw) : spill_row;
        int* ci = in_shared ? reinterpret_cast<int*>(cand_raw) + kCand : reinterpret_cast<int*>(spill_row + spill_stride);
        float* ce = in_shared ? reinterpret_cast<float*>(cand_raw) + 2 * kCand : spill_row + 2 * spill_stride;
        int n = 0;
        int at = block_exclusive_scan(mine, warp_tot, &n);
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float s = to_float(x[i]) * inv_t;
            if (ordered_key(s) >= thr && (all_kept || mx - s <= reach)) {      // as counted above
                cs[at] = s;
                ci[at] = i;
                ce[at] = expf(s - mx);
                ++at;
            }
        }
        __syncthreads();
        if (p_cut < 1.f) {
            uint32_t prefix = 0;
            for (int bit = 31; bit >= 0; --bit) {
                const uint32_t cand = prefix | (1u << bit);
                float mass = 0.f;
                for (int j = threadIdx.x; j < n; j += blockDim.x)
                    if (ordered_key(cs[j]) >= cand) mass += ce[j];
                mass = block_sum(mass, red);
                if (mass / z > p_cut) prefix = cand;
            }
            thr = max(thr, prefix);
        }
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            if (ordered_key(cs[j]) < thr) continue;
            const int i = ci[j];
            uint32_t r[4];
            philox4x32_10((uint32_t)(i >> 2), 0u, 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
            const float u = ((float)r[i & 3] + 0.5f) * 2.3283064365386963e-10f;   // (0, 1)
            const float e = fmaxf(-logf(u), 1e-10f);
            pick = better(pick, ArgMax{ce[j] / e, i});
        }
    } else {
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
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float s = to_float(x[i]) * inv_t;
            if (ordered_key(s) < thr) continue;
            uint32_t r[4];
            philox4x32_10((uint32_t)(i >> 2), 0u, 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
            const float u = ((float)r[i & 3] + 0.5f) * 2.3283064365386963e-10f;   // (0, 1)
            const float e = fmaxf(-logf(u), 1e-10f);
            pick = better(pick, ArgMax{expf(s - mx) / e, i});
        }
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

// Rows without a top-k or top-p cut, over a large vocabulary with few rows: like the two-stage
// argmax, every row is cut into `chunks` slices that blocks take in parallel.  After the partial
// maxima (argmax_partial_kernel) each block knows the row's maximum and takes, over its slice,
// the partial normaliser and the partial winner of the race; the last kernel merges them.  The
// winner is the one the one-block kernel finds (same value per entry, same rule for ties); the
// normaliser is summed slice by slice.
template <typename T>
__global__ void sample_plain_partial_kernel(const T* __restrict__ logits, const float* __restrict__ temperature,
                                            const unsigned long long* __restrict__ seeds,
                                            const float* __restrict__ pval, const int* __restrict__ pidx,
                                            float* __restrict__ zpart, float* __restrict__ rval, int* __restrict__ ridx,
                                            int vocab, int chunks) {
    __shared__ ArgMax am[33];
    __shared__ float red[33];
    const int row = blockIdx.x, chunk = blockIdx.y;
    const float temp = temperature[row];
    const bool greedy = temp <= 1e-10f;
    const float inv_t = greedy ? 1.f : 1.f / temp;
    ArgMax best{0.f, -1};
    for (int c = 0; c < chunks; ++c) best = better(best, ArgMax{pval[row * chunks + c], pidx[row * chunks + c]});
    const float mx = best.v * inv_t;
    const int per = (vocab + chunks - 1) / chunks;
    const int a = chunk * per, b = min(vocab, a + per);
    const T* x = logits + (size_t)row * vocab;
    const unsigned long long seed = seeds[row];
    float z = 0.f;
    ArgMax pick{0.f, -1};
    for (int i = a + threadIdx.x; i < b; i += blockDim.x) {
        const float s = to_float(x[i]) * inv_t;
        const float w = expf(s - mx);
        z += w;
        if (!greedy) {
            uint32_t r[4];
            philox4x32_10((uint32_t)(i >> 2), 0u, 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
            const float u = ((float)r[i & 3] + 0.5f) * 2.3283064365386963e-10f;   // (0, 1)
            const float e = fmaxf(-logf(u), 1e-10f);
            pick = better(pick, ArgMax{w / e, i});
        }
    }
    z = block_sum(z, red);
    pick = block_argmax(pick, am);
    if (threadIdx.x == 0) {
        zpart[row * chunks + chunk] = z;
        rval[row * chunks + chunk] = pick.v;
        ridx[row * chunks + chunk] = pick.i;
    }
}

__global__ void sample_plain_final_kernel(const void* __restrict__ logits, int dtype, const float* __restrict__ temperature,
                                          const float* __restrict__ pval, const int* __restrict__ pidx,
                                          const float* __restrict__ zpart, const float* __restrict__ rval,
                                          const int* __restrict__ ridx, int* __restrict__ out,
                                          float* __restrict__ logprob, int vocab, int chunks) {
    const int row = blockIdx.x;
    if (threadIdx.x != 0) return;
    const float temp = temperature[row];
    const bool greedy = temp <= 1e-10f;
    const float inv_t = greedy ? 1.f : 1.f / temp;
    ArgMax best{0.f, -1}, pick{0.f, -1};
    float z = 0.f;
    for (int c = 0; c < chunks; ++c) {
        best = better(best, ArgMax{pval[row * chunks + c], pidx[row * chunks + c]});
        pick = better(pick, ArgMax{rval[row * chunks + c], ridx[row * chunks + c]});
        z += zpart[row * chunks + c];
    }
    const int tok = greedy ? best.i : pick.i;
    out[row] = tok;
    if (logprob != nullptr) {
        if (greedy) {
            logprob[row] = -logf(z);
        } else {
            const float v = dtype == SE_DTYPE_BF16 ? to_float(((const __nv_bfloat16*)logits)[(size_t)row * vocab + tok])
                                                   : ((const float*)logits)[(size_t)row * vocab + tok];
            logprob[row] = v * inv_t - best.v * inv_t - logf(z);
        }
    }
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

// temperature/top_k/top_p/seeds may be null (then every row is greedy).  spill: optional workspace of
// rows * 3 * ceil(vocab / 4) floats for lists that do not fit into shared memory (without it such rows take the
// whole-row form).  impl: 0 = the fast
// path where it applies, 1 = every cut and the draw over the whole row (the definition; tests
// compare the two).
extern "C" int se_sample(const void* logits, const float* temperature, const int* top_k, const float* top_p,
                         const unsigned long long* seeds, int* out, float* logprob, float* spill, int rows, int vocab,
                         int dtype, int impl, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (temperature != nullptr && seeds == nullptr) return SE_ERR_ARGUMENT;
    if (impl != 0 && impl != 1) return SE_ERR_ARGUMENT;
    if (temperature != nullptr && impl == 0) {
        const int smem = 3 * se::kCand * (int)sizeof(float);
        SE_DISPATCH_DTYPE(dtype, T, {
            static bool configured = false;
            if (!configured) {
                cudaError_t e = cudaFuncSetAttribute(se::sample_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
                if (e != cudaSuccess) return (int)e;
                configured = true;
            }
            se::sample_kernel<T, true><<<rows, se::kSampleThreads, smem, stream>>>((const T*)logits, temperature, top_k,
                                                                                   top_p, seeds, out, logprob, spill, vocab);
        });
        SE_LAUNCH_CHECK();
    }
    SE_DISPATCH_DTYPE(dtype, T,
        (se::sample_kernel<T, false><<<rows, se::kSampleThreads, 0, stream>>>((const T*)logits, temperature, top_k, top_p,
                                                                              seeds, out, logprob, nullptr, vocab)));
    SE_LAUNCH_CHECK();
}

// Rows without top-k or top-p cuts (temperature rows and greedy rows), many blocks per row.
// Workspaces of rows * 64 entries each: pval, zpart, rval (float), pidx, ridx (int).
extern "C" int se_sample_plain(const void* logits, const float* temperature, const unsigned long long* seeds, int* out,
                               float* logprob, float* pval, int* pidx, float* zpart, float* rval, int* ridx, int rows,
                               int vocab, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (temperature == nullptr || seeds == nullptr) return SE_ERR_ARGUMENT;
    const int chunks = 64;
    dim3 grid(rows, chunks);
    SE_DISPATCH_DTYPE(dtype, T, {
        se::argmax_partial_kernel<T><<<grid, 256, 0, stream>>>((const T*)logits, pval, pidx, vocab, chunks);
        se::sample_plain_partial_kernel<T><<<grid, 256, 0, stream>>>((const T*)logits, temperature, seeds, pval, pidx,
                                                                     zpart, rval, ridx, vocab, chunks);
    });
    se::sample_plain_final_kernel<<<rows, 32, 0, stream>>>(logits, dtype, temperature, pval, pidx, zpart, rval, ridx, out,
                                                           logprob, vocab, chunks);
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
__global__ void __launch_bounds__(1024)
top_logprobs_kernel(const T* __restrict__ logits, const int* __restrict__ rows, int* __restrict__ ids,
                    float* __restrict__ values, int vocab, int n) {
    __shared__ float red[33];
    __shared__ float best_v[32];
    __shared__ int best_i[32];
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
        se::top_logprobs_kernel<T><<<count, vocab >= 8192 ? 1024 : 256, 0, stream>>>((const T*)logits, rows, ids, values, vocab, n));
    SE_LAUNCH_CHECK();
}

extern "C" int se_to_float(const void* src, float* dst, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 1023) / 1024 < 4096 ? (n + 1023) / 1024 : 4096);
    SE_DISPATCH_DTYPE(dtype, T, se::to_float_kernel<T><<<blocks, 256, 0, stream>>>((const T*)src, dst, (size_t)n));
    SE_LAUNCH_CHECK();
}
