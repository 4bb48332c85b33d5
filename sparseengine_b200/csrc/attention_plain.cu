// Plain paged attention: one block per (token, query head), any head size, any page
// size, float32 or bfloat16.  It is the 32-bit path's attention and the fallback for
// sizes the tensor-core kernels refuse.
//
// score = q·k * scale; query at position p sees keys max(0, p-window+1)..p of its own
// request (window 0 = all keys); softmax state and accumulators in 32-bit; the
// probability is rounded to the activation type before it multiplies V; the output is
// rounded once.  Reference: src/sparseengine/kernels/triton/context_flashattention_nopad.py:92-127,
// src/sparseengine/kernels/triton/gqa_flash_decoding_stage1.py:69-120.
//
// A block-table entry outside [0, num_pages) is not followed: the key is left out and a code
// goes to the error word (the reference checks such indices on the host behind a debug
// switch, src/sparseengine/layers/attention_backend.py:155-215).
#include "common.cuh"

namespace se {

constexpr int kAttnWarps = 4;
constexpr int kMaxDimPerLane = 8;   // head_dim <= 256

template <typename T>
__global__ void paged_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                                             const int* __restrict__ table, int table_stride,
                                             const int* __restrict__ seq_rows, const int* __restrict__ token_seq,
                                             const int* __restrict__ positions, T* __restrict__ out, int hq, int hkv,
                                             int d, int page_size, float scale, int window, int num_pages,
                                             int* __restrict__ error) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = h / (hq / hkv);
    const int pos = positions[t];
    const int* row_table = table + (size_t)seq_rows[token_seq[t]] * table_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const size_t page_elems = (size_t)2 * hkv * page_size * d;
    const size_t v_off = (size_t)hkv * page_size * d;
    const size_t head_off = (size_t)kvh * page_size * d;

    float qr[kMaxDimPerLane], acc[kMaxDimPerLane];
    const T* qp = q + ((size_t)t * hq + h) * d;
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) {
        const int dim = lane + 32 * i;
        qr[i] = dim < d ? to_float(qp[dim]) * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = lo + warp; j <= pos; j += kAttnWarps) {
        const int page = row_table[j / page_size];
        if (!page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_ATTN_PLAIN)) continue;     // warp-uniform: the key is left out
        const T* kp = cache + (size_t)page * page_elems + head_off + (size_t)(j % page_size) * d;
        const T* vp = kp + v_off;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxDimPerLane; ++i) {
            const int dim = lane + 32 * i;
            if (dim < d) s += qr[i] * to_float(kp[dim]);
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);   // m = -inf on the first key: exp(-inf) = 0
        const float p = expf(s - m_new);
        const float pr = round_act<T>(p);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < kMaxDimPerLane; ++i) {
            const int dim = lane + 32 * i;
            if (dim < d) acc[i] = acc[i] * corr + pr * to_float(vp[dim]);
        }
        m = m_new;
    }

    __shared__ float sm[kAttnWarps], sl[kAttnWarps];
    __shared__ float sacc[kAttnWarps][32 * kMaxDimPerLane];
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) sacc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mt = fmaxf(mt, sm[w]);
    float lt = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) lt += sm[w] == -INFINITY ? 0.f : sl[w] * expf(sm[w] - mt);
    T* op = out + ((size_t)t * hq + h) * d;
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) o += sm[w] == -INFINITY ? 0.f : sacc[w][dim] * expf(sm[w] - mt);
        op[dim] = from_float<T>(o / lt);
    }
}

}  // namespace se

extern "C" int se_paged_attention_plain(const void* q, const void* cache, const int* table, int table_stride,
                                        const int* seq_rows, const int* token_seq, const int* positions, void* out,
                                        int tokens, int hq, int hkv, int d, int page_size, float scale, int window,
                                        int num_pages, int* error, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d > 32 * se::kMaxDimPerLane || d <= 0 || hkv <= 0 || hq % hkv) return SE_ERR_UNSUPPORTED;
    dim3 grid(tokens, hq);
    SE_DISPATCH_DTYPE(dtype, T,
        se::paged_attention_plain_kernel<T><<<grid, 32 * se::kAttnWarps, 0, stream>>>(
            (const T*)q, (const T*)cache, table, table_stride, seq_rows, token_seq, positions, (T*)out, hq, hkv, d,
            page_size, scale, window, num_pages, error));
    SE_LAUNCH_CHECK();
}
