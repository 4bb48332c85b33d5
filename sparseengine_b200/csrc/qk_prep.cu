// One pass over the packed qkv projection: whole-projection QK RMSNorm (32-bit
// statistics), rotary position encoding on the leading `rot` dims of each head, the
// query written out contiguously and K/V written into their cache page.
//
// Reference formulas: QK norm src/sparseengine/layers/layernorm.py:204-210 (the
// normalised value is rounded to the activation type before the weight multiply, which
// is itself done in the activation type); rotary src/sparseengine/layers/rotary_embedding.py:104-112
// (split-half pairing, 32-bit arithmetic), angle = position * inv_freq in 32-bit
// (:190-222); KV write src/sparseengine/kernels/triton/store_kvcache.py:10-30.
//
// Cache layout of one cache layer: [page][K|V][kv head][slot in page][head_dim].
#include "common.cuh"

namespace se {

template <typename T>
__global__ void qk_prep_kernel(const T* __restrict__ qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
                               const float* __restrict__ inv_freq, const int* __restrict__ positions,
                               const int* __restrict__ token_seq, const int* __restrict__ seq_rows,
                               const int* __restrict__ table, int table_stride, T* __restrict__ cache,
                               T* __restrict__ q_out, int hq, int hkv, int d, int rot, float eps,
                               float rope_scale, int page_size, int write_cache) {
    extern __shared__ float cs[];          // cos[rot/2], sin[rot/2]
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int qn = hq * d, kn = hkv * d;
    const T* row = qkv + (size_t)t * (qn + 2 * kn);
    const int pos = positions[t];
    const int half = rot / 2;

    float inv_q = 1.f, inv_k = 1.f;
    if (q_w != nullptr) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < qn; i += blockDim.x) { float v = to_float(row[i]); sq += v * v; }
        for (int i = threadIdx.x; i < kn; i += blockDim.x) { float v = to_float(row[qn + i]); sk += v * v; }
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        inv_q = 1.0f / sqrtf(sq / (float)qn + eps);
        inv_k = 1.0f / sqrtf(sk / (float)kn + eps);
    }
    if (inv_freq != nullptr) {
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float s, c;
            sincosf((float)pos * inv_freq[j], &s, &c);
            cs[j] = c * rope_scale;
            cs[half + j] = s * rope_scale;
        }
    }
    __syncthreads();

    T* k_dst = nullptr;
    T* v_dst = nullptr;
    if (write_cache) {
        const int page = table[(size_t)seq_rows[token_seq[t]] * table_stride + pos / page_size];
        const size_t page_elems = (size_t)2 * hkv * page_size * d;
        k_dst = cache + (size_t)page * page_elems + (size_t)(pos % page_size) * d;
        v_dst = k_dst + (size_t)hkv * page_size * d;
    }
    const size_t head_stride = (size_t)page_size * d;

    // Work items: (head, i) with i over [0, d - half): i < half is a rotated pair
    // (dims i and i+half), i >= half is the pass-through dim i + half.
    const int per_head = d - half;
    const int items_q = hq * per_head, items_k = write_cache ? hkv * per_head : 0;
    for (int it = threadIdx.x; it < items_q + items_k; it += blockDim.x) {
        const bool is_q = it < items_q;
        const int local = is_q ? it : it - items_q;
        const int h = local / per_head, i = local % per_head;
        const T* src = row + (is_q ? 0 : qn) + h * d;
        const T* w = is_q ? q_w : k_w;
        const float inv = is_q ? inv_q : inv_k;
        T* dst = is_q ? q_out + (size_t)t * qn + h * d : k_dst + h * head_stride;
        auto normed = [&](int dim) -> float {
            float v = to_float(src[dim]);
            if (w == nullptr) return v;
            // cast(x32 * inv) * cast(w), the product rounded once more
            return round_act<T>(round_act<T>(v * inv) * to_float(w[h * d + dim]));
        };
        if (inv_freq != nullptr && i < half) {
            const float x1 = normed(i), x2 = normed(i + half);
            const float c = cs[i], s = cs[half + i];
            dst[i] = from_float<T>(x1 * c - x2 * s);
            dst[i + half] = from_float<T>(x2 * c + x1 * s);
        } else if (inv_freq != nullptr) {
            dst[i + half] = from_float<T>(normed(i + half));
        } else {
            // no rotation: items cover dims [0, d - half) plus the tail below
            dst[i] = from_float<T>(normed(i));
            if (i < half) dst[per_head + i] = from_float<T>(normed(per_head + i));
        }
    }
    if (write_cache) {
        const T* vsrc = row + qn + kn;
        for (int i = threadIdx.x; i < kn; i += blockDim.x) {
            const int h = i / d, dim = i % d;
            v_dst[h * head_stride + dim] = vsrc[i];
        }
    }
}

}  // namespace se

extern "C" int se_qk_prep(const void* qkv, const void* q_w, const void* k_w, const float* inv_freq,
                          const int* positions, const int* token_seq, const int* seq_rows, const int* table,
                          int table_stride, void* cache, void* q_out, int tokens, int hq, int hkv, int d,
                          int rot, float eps, float rope_scale, int page_size, int write_cache, int dtype,
                          cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1)) return SE_ERR_ARGUMENT;
    if (inv_freq == nullptr) rot = 0;
    const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
    SE_DISPATCH_DTYPE(dtype, T,
        se::qk_prep_kernel<T><<<tokens, 256, smem, stream>>>(
            (const T*)qkv, (const T*)q_w, (const T*)k_w, rot > 0 ? inv_freq : nullptr, positions, token_seq,
            seq_rows, table, table_stride, (T*)cache, (T*)q_out, hq, hkv, d, rot, eps, rope_scale, page_size,
            write_cache));
    SE_LAUNCH_CHECK();
}
