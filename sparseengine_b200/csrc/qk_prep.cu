// One kernel over the packed qkv projection: whole-projection QK RMSNorm (32-bit
// statistics), rotary position encoding on the leading `rot` dims of each head, the
// query written out contiguously and K/V written into their cache page.
//
// Reference formulas: QK norm src/sparseengine/layers/layernorm.py:204-210 (the
// normalised value is rounded to the activation type before the weight multiply, which
// is itself done in the activation type); rotary src/sparseengine/layers/rotary_embedding.py:104-112
// (split-half pairing, 32-bit arithmetic), angle = position * inv_freq in 32-bit
// (:190-222); KV write src/sparseengine/kernels/triton/store_kvcache.py:10-30.
//
// The position encoding is data: `inv_freq[rot/2]` is a table of one frequency per rotated
// pair (any scaling of the frequencies is done by whoever builds the table), `rope_scale`
// multiplies cos and sin, and `pairing` says which dims form pair i and where its results go:
// bit 0 set = the inputs are the adjacent dims (2i, 2i+1), clear = the split halves
// (i, i + rot/2); bit 1 says the same of the outputs.  0 is the split-half form, 3 the
// adjacent-pairs form, 1 reads adjacent pairs and writes split halves
// (src/sparseengine/layers/rotary_embedding.py:115-127).
//
// A block-table entry outside [0, num_pages) is not followed: the K/V write is skipped and a
// code goes to the error word.
//
// Cache layout of one cache layer: [page][K|V][kv head][slot in page][head_dim].
#include "common.cuh"

namespace se {

// grid (tokens, blocks of heads): a block handles `heads_per_block` of the hq query heads
// and hkv KV heads (a KV head means its key and its value) of one token.  With few tokens
// every head gets a block of its own, which recomputes the sum of squares of its whole
// projection (the rows are a few KB and sit in L2); with many tokens one block takes all
// heads of a token and the statistics come from a first kernel.
template <typename T>
__global__ void qk_prep_kernel(const T* qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
                               const float* __restrict__ inv_freq, const int* __restrict__ positions,
                               const int* __restrict__ token_seq, const int* __restrict__ seq_rows,
                               const int* __restrict__ table, int table_stride, T* __restrict__ cache,
                               T* __restrict__ q_out, int hq, int hkv, int d, int rot, float eps,
                               float rope_scale, int page_size, int write_cache, const float* __restrict__ inv_rms,
                               int heads_per_block, int pairing, int num_pages, int* __restrict__ error) {
    extern __shared__ float cs[];          // cos[rot/2], sin[rot/2]
    __shared__ float scratch[33];
    grid_dependency_trigger();             // the attention kernel that follows may find its keys' pages meanwhile
    // Where the positions are older than the projection that writes qkv, this kernel is launched
    // as its dependent, and the angles are ready when the projection ends.
    const int t = blockIdx.x;
    const int qn = hq * d, kn = hkv * d;
    const T* row = qkv + (size_t)t * (qn + 2 * kn);
    const int pos = positions[t];
    const int half = rot / 2;
    if (inv_freq != nullptr) {
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float s, c;
            sincosf((float)pos * inv_freq[j], &s, &c);
            cs[j] = c * rope_scale;
            cs[half + j] = s * rope_scale;
        }
    }
    grid_dependency_wait();      // qkv is not __restrict__: its loads must stay below this line
    const int total_heads = hq + (write_cache ? hkv : 0);
    const int h_begin = blockIdx.y * heads_per_block, h_end = min(total_heads, h_begin + heads_per_block);
    float inv_cached[2] = {-1.f, -1.f};       // statistics of the q and of the k projection, once per block
    for (int hh = h_begin; hh < h_end; ++hh) {
        const bool is_q = hh < hq;
        const int h = is_q ? hh : hh - hq;
        const T* w = is_q ? q_w : k_w;
        float inv = 1.f;
        if (w != nullptr && inv_rms != nullptr) {
            inv = inv_rms[2 * t + (is_q ? 0 : 1)];
        } else if (w != nullptr) {
            if (inv_cached[is_q ? 0 : 1] < 0.f) {
                const T* part = row + (is_q ? 0 : qn);
                const int n = is_q ? qn : kn;
                float ss = 0.f;
                if ((n & 7) == 0 && aligned8(part)) {
                    for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
                        float v[8];
                        load8(part + i, v);
#pragma unroll
                        for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
                    }
                } else {
                    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_float(part[i]); ss += v * v; }
                }
                ss = block_sum(ss, scratch);
                inv_cached[is_q ? 0 : 1] = 1.0f / sqrtf(ss / (float)n + eps);
            }
            inv = inv_cached[is_q ? 0 : 1];
        }
        __syncthreads();      // cos/sin are in shared memory (first pass) 

        T* k_dst = nullptr;
        if (!is_q) {
            const int page = table[(size_t)seq_rows[token_seq[t]] * table_stride + pos / page_size];
            if (!page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_QK_PREP)) continue;     // block-uniform
            const size_t page_elems = (size_t)2 * hkv * page_size * d;
            k_dst = cache + (size_t)page * page_elems + (size_t)h * page_size * d + (size_t)(pos % page_size) * d;
        }
        const T* src = row + (is_q ? 0 : qn) + h * d;
        T* dst = is_q ? q_out + (size_t)t * qn + h * d : k_dst;
        auto normed = [&](int dim) -> float {
            const float v = to_float(src[dim]);
            if (w == nullptr) return v;
            // cast(x32 * inv) * cast(w), the product rounded once more
            return round_act<T>(round_act<T>(v * inv) * to_float(w[h * d + dim]));
        };
        // items i over [0, d - half): i < half is rotated pair i (its dims by `pairing`), the
        // rest are the pass-through dims i + half
        for (int i = threadIdx.x; i < d - half; i += blockDim.x) {
            if (i < half) {
                const int in1 = (pairing & 1) ? 2 * i : i, in2 = (pairing & 1) ? 2 * i + 1 : i + half;
                const int out1 = (pairing & 2) ? 2 * i : i, out2 = (pairing & 2) ? 2 * i + 1 : i + half;
                const float x1 = normed(in1), x2 = normed(in2);
                const float c = cs[i], s = cs[half + i];
                dst[out1] = from_float<T>(x1 * c - x2 * s);
                dst[out2] = from_float<T>(x2 * c + x1 * s);
            } else {
                dst[i + half] = from_float<T>(normed(i + half));
            }
        }
        if (!is_q) {
            const T* vsrc = row + qn + kn + h * d;
            T* v_dst = k_dst + (size_t)hkv * page_size * d;
            for (int i = threadIdx.x; i < d; i += blockDim.x) v_dst[i] = vsrc[i];
        }
    }
}

// Many tokens: one block per token, every thread moves groups of 8 consecutive dims with
// 16-byte accesses.  A work item is (head, group): a group below rot/2 is rotated together
// with its partner group rot/2 dims further on, groups from rot on pass through, and the
// value heads are copied.  Same arithmetic per element as qk_prep_kernel; the block first takes
// the statistics of the token's whole q and k projections.  Needs d, rot/2 and the row pitch to
// be multiples of 8 elements.
template <typename T>
__global__ void __launch_bounds__(256)
qk_prep_vec_kernel(const T* __restrict__ qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
                   const float* __restrict__ inv_freq, const int* __restrict__ positions,
                   const int* __restrict__ token_seq, const int* __restrict__ seq_rows,
                   const int* __restrict__ table, int table_stride, T* __restrict__ cache, T* __restrict__ q_out,
                   int hq, int hkv, int d, int rot, float eps, float rope_scale, int page_size, int write_cache,
                   int num_pages, int* __restrict__ error) {
    extern __shared__ float cs[];          // cos[rot/2], sin[rot/2]
    __shared__ float scratch[33];
    grid_dependency_trigger();             // the attention kernel that follows may find its keys' pages meanwhile
    const int t = blockIdx.x;
    const int qn = hq * d, kn = hkv * d;
    const T* row = qkv + (size_t)t * (qn + 2 * kn);
    // The trips to memory that depend on one another (position and request -> table row -> page)
    // are started first and used last, so that they overlap the loads of the statistics.
    const int pos = positions[t];
    const int ts = write_cache ? token_seq[t] : 0;
    const int half = rot / 2;
    // statistics of the whole q and k projections of this token (the row is re-read from L1/L2 below)
    float ss_q = 0.f, ss_k = 0.f;
    if (q_w != nullptr) {
        for (int i = threadIdx.x * 8; i < qn; i += blockDim.x * 8) {
            float v[8];
            load8(row + i, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss_q += v[j] * v[j];
        }
        for (int i = threadIdx.x * 8; i < kn; i += blockDim.x * 8) {
            float v[8];
            load8(row + qn + i, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss_k += v[j] * v[j];
        }
    }
    const int table_row = write_cache ? seq_rows[ts] : 0;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        cs[j] = c * rope_scale;
        cs[half + j] = s * rope_scale;
    }
    const int page = write_cache ? table[(size_t)table_row * table_stride + pos / page_size] : 0;
    if (write_cache && !page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_QK_PREP)) write_cache = 0;   // q only
    float inv_q = 1.f, inv_k = 1.f;
    if (q_w != nullptr) {
        inv_q = 1.0f / sqrtf(block_sum(ss_q, scratch) / (float)qn + eps);
        inv_k = 1.0f / sqrtf(block_sum(ss_k, scratch) / (float)kn + eps);
    }
    __syncthreads();                       // cos/sin are in shared memory
    T* kv_base = nullptr;
    if (write_cache)
        kv_base = cache + (size_t)page * 2 * hkv * page_size * d + (size_t)(pos % page_size) * d;
    const int groups = d / 8, rot_groups = half / 8;
    const int live = groups - rot_groups;                  // items per head: rotated pairs, then pass-through groups
    const int qk_heads = hq + (write_cache ? hkv : 0);
    const int qk_items = qk_heads * live;
    const int v_items = write_cache ? hkv * groups : 0;
    for (int item = threadIdx.x; item < qk_items + v_items; item += blockDim.x) {
        if (item >= qk_items) {                            // value head: copy
            const int h = (item - qk_items) / groups, g = (item - qk_items) % groups;
            const T* src = row + qn + kn + h * d + 8 * g;
            T* dst = kv_base + (size_t)(hkv + h) * page_size * d + 8 * g;
            float v[8];
            load8(src, v);
            store8(dst, v);
            continue;
        }
        const int hh = item / live, i = item % live;
        const bool is_q = hh < hq;
        const int h = is_q ? hh : hh - hq;
        const T* w = is_q ? q_w : k_w;
        const float inv = is_q ? inv_q : inv_k;
        const T* src = row + (is_q ? 0 : qn) + h * d;
        T* dst = is_q ? q_out + (size_t)t * qn + h * d : kv_base + (size_t)h * page_size * d;
        auto normed8 = [&](int dim0, float* out) {
            load8(src + dim0, out);
            if (w != nullptr) {
                float wv[8];
                load8(w + h * d + dim0, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) out[j] = round_act<T>(round_act<T>(out[j] * inv) * wv[j]);
            }
        };
        if (i < rot_groups) {
            float x1[8], x2[8], o1[8], o2[8];
            normed8(8 * i, x1);
            normed8(8 * i + half, x2);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float c = cs[8 * i + j], sn = cs[half + 8 * i + j];
                o1[j] = x1[j] * c - x2[j] * sn;
                o2[j] = x2[j] * c + x1[j] * sn;
            }
            store8(dst + 8 * i, o1);
            store8(dst + 8 * i + half, o2);
        } else {
            float x[8];
            normed8(8 * (i + rot_groups), x);
            store8(dst + 8 * (i + rot_groups), x);
        }
    }
}

// The same for bfloat16 with fewer instructions (the kernel above spends its time issuing them,
// not waiting for memory): values stay packed in pairs, the product with the norm weight is a
// packed bfloat16 multiply (the exact product rounded once, which is what rounding the 32-bit
// product gives), and a thread steps through its work items without a division.  Bit for bit
// the results of the kernel above.
__global__ void __launch_bounds__(256)
qk_prep_vec_bf16_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_w,
                        const __nv_bfloat16* __restrict__ k_w, const float* __restrict__ inv_freq,
                        const int* __restrict__ positions, const int* __restrict__ token_seq,
                        const int* __restrict__ seq_rows, const int* __restrict__ table, int table_stride,
                        __nv_bfloat16* __restrict__ cache, __nv_bfloat16* __restrict__ q_out, int hq, int hkv, int d,
                        int rot, float eps, float rope_scale, int page_size, int write_cache, int num_pages,
                        int* __restrict__ error) {
    extern __shared__ float cs[];          // cos[rot/2], sin[rot/2]
    __shared__ float scratch[2][33];
    grid_dependency_trigger();             // the attention kernel that follows may find its keys' pages meanwhile
    const int t = blockIdx.x;
    const int qn = hq * d, kn = hkv * d;
    const __nv_bfloat16* row = qkv + (size_t)t * (qn + 2 * kn);
    const int pos = positions[t];
    const int ts = write_cache ? token_seq[t] : 0;
    const int half = rot / 2;
    auto sum_squares = [&](const __nv_bfloat16* part, int n) {
        float ss = 0.f;
        for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(part + i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {      // in the order of the elements, as the kernel above adds them
                const float2 f = __bfloat1622float2(h[j]);
                ss += f.x * f.x;
                ss += f.y * f.y;
            }
        }
        return ss;
    };
    float ss_q = 0.f, ss_k = 0.f;
    if (q_w != nullptr) {
        ss_q = sum_squares(row, qn);
        ss_k = sum_squares(row + qn, kn);
    }
    const int table_row = write_cache ? seq_rows[ts] : 0;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float sn, c;
        sincosf((float)pos * inv_freq[j], &sn, &c);
        cs[j] = c * rope_scale;
        cs[half + j] = sn * rope_scale;
    }
    const int page = write_cache ? table[(size_t)table_row * table_stride + pos / page_size] : 0;
    if (write_cache && !page_in_pool(page, num_pages, error, SE_CODE_BAD_PAGE_QK_PREP)) write_cache = 0;   // q only
    float inv_q = 1.f, inv_k = 1.f;
    if (q_w != nullptr) {
        inv_q = 1.0f / sqrtf(block_sum(ss_q, scratch[0]) / (float)qn + eps);
        inv_k = 1.0f / sqrtf(block_sum(ss_k, scratch[1]) / (float)kn + eps);
    }
    __syncthreads();                       // cos/sin are in shared memory
    __nv_bfloat16* kv_base = nullptr;
    if (write_cache)
        kv_base = cache + (size_t)page * 2 * hkv * page_size * d + (size_t)(pos % page_size) * d;
    const int groups = d / 8, rot_groups = half / 8;
    const int live = groups - rot_groups;                  // items per head: rotated pairs, then pass-through groups
    const int qk_heads = hq + (write_cache ? hkv : 0);
    // eight values of a head, normalised: cast(x * inv) * w, the product rounded once
    auto normed8 = [&](const __nv_bfloat16* src, const __nv_bfloat16* w, float inv, __nv_bfloat162 (&out)[4]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        if (w == nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) out[j] = x2[j];
            return;
        }
        const uint4 wraw = *reinterpret_cast<const uint4*>(w);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(x2[j]);
            out[j] = __hmul2(__floats2bfloat162_rn(f.x * inv, f.y * inv), w2[j]);
        }
    };
    // a thread's items are threadIdx.x, + 256, ...: (head, item of the head) without dividing each time
    const int step_h = (int)blockDim.x / live, step_i = (int)blockDim.x % live;
    int hh = (int)threadIdx.x / live, i = (int)threadIdx.x % live;
    for (; hh < qk_heads; hh += step_h, i += step_i) {
        if (i >= live) { i -= live; ++hh; if (hh >= qk_heads) break; }
        const bool is_q = hh < hq;
        const int h = is_q ? hh : hh - hq;
        const __nv_bfloat16* w = is_q ? q_w : k_w;
        const float inv = is_q ? inv_q : inv_k;
        const __nv_bfloat16* src = row + (is_q ? 0 : qn) + h * d;
        __nv_bfloat16* dst = is_q ? q_out + (size_t)t * qn + h * d : kv_base + (size_t)h * page_size * d;
        if (i < rot_groups) {
            __nv_bfloat162 x1[4], x2[4];
            normed8(src + 8 * i, w ? w + h * d + 8 * i : nullptr, inv, x1);
            normed8(src + 8 * i + half, w ? w + h * d + 8 * i + half : nullptr, inv, x2);
            uint4 o1, o2;
            __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(&o1);
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&o2);
            const float4* c4 = reinterpret_cast<const float4*>(cs + 8 * i);
            const float4* s4 = reinterpret_cast<const float4*>(cs + half + 8 * i);
            const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
            const float c[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
            const float sn[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = __bfloat1622float2(x1[j]), b = __bfloat1622float2(x2[j]);
                p1[j] = __floats2bfloat162_rn(a.x * c[2 * j] - b.x * sn[2 * j], a.y * c[2 * j + 1] - b.y * sn[2 * j + 1]);
                p2[j] = __floats2bfloat162_rn(b.x * c[2 * j] + a.x * sn[2 * j], b.y * c[2 * j + 1] + a.y * sn[2 * j + 1]);
            }
            *reinterpret_cast<uint4*>(dst + 8 * i) = o1;
            *reinterpret_cast<uint4*>(dst + 8 * i + half) = o2;
        } else {
            __nv_bfloat162 x[4];
            const int dim0 = 8 * (i + rot_groups);
            normed8(src + dim0, w ? w + h * d + dim0 : nullptr, inv, x);
            *reinterpret_cast<uint4*>(dst + dim0) = *reinterpret_cast<const uint4*>(x);
        }
    }
    if (write_cache) {                     // value heads: copies
        for (int item = threadIdx.x; item < hkv * groups; item += blockDim.x) {
            const int h = item / groups, g = item - h * groups;
            *reinterpret_cast<uint4*>(kv_base + (size_t)(hkv + h) * page_size * d + 8 * g) =
                *reinterpret_cast<const uint4*>(row + qn + kn + h * d + 8 * g);
        }
    }
}

// inv_rms[t] = (1/sqrt(mean(q^2)+eps), 1/sqrt(mean(k^2)+eps)) of token t's whole projections:
// for many tokens the statistics are taken once here instead of once per head.
template <typename T>
__global__ void qk_inv_rms_kernel(const T* __restrict__ qkv, float* __restrict__ inv_rms, int qn, int kn, float eps) {
    __shared__ float scratch[33];
    const T* row = qkv + (size_t)blockIdx.x * (qn + 2 * kn);
    for (int which = 0; which < 2; ++which) {
        const T* part = row + (which ? qn : 0);
        const int n = which ? kn : qn;
        float ss = 0.f;
        if ((n & 7) == 0 && aligned8(part)) {
            for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
                float v[8];
                load8(part + i, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
            }
        } else {
            for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_float(part[i]); ss += v * v; }
        }
        ss = block_sum(ss, scratch);
        if (threadIdx.x == 0) inv_rms[2 * blockIdx.x + which] = 1.0f / sqrtf(ss / (float)n + eps);
    }
}

}  // namespace se

// SE_QK_PREP_GENERIC=1: bfloat16 steps of many tokens take the kernel that also serves 32-bit (a
// testing aid: the two give the same bits).
static bool se_qk_prep_generic_vec() {
    static const bool v = [] { const char* e = ::getenv("SE_QK_PREP_GENERIC"); return e != nullptr && e[0] == '1'; }();
    return v;
}

extern "C" int se_qk_prep(const void* qkv, const void* q_w, const void* k_w, const float* inv_freq,
                          const int* positions, const int* token_seq, const int* seq_rows, const int* table,
                          int table_stride, void* cache, void* q_out, int tokens, int hq, int hkv, int d,
                          int rot, float eps, float rope_scale, int page_size, int write_cache, float* inv_rms,
                          int pairing, int num_pages, int* error, int settled, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || pairing < 0 || pairing > 3) return SE_ERR_ARGUMENT;
    if (inv_freq == nullptr) rot = 0;
    const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
    // many tokens and sizes that allow 16-byte groups: one block per token does everything
    const int elem = dtype == SE_DTYPE_BF16 ? 2 : 4;
    const bool vec = tokens > 64 && pairing == 0 && (q_w == nullptr) == (k_w == nullptr) && d % 8 == 0 && (rot / 2) % 8 == 0 &&
                     (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)cache | (uintptr_t)q_w | (uintptr_t)k_w) & 15) == 0 &&
                     ((size_t)page_size * d * elem) % 16 == 0;
    if (vec && dtype == SE_DTYPE_BF16 && !se_qk_prep_generic_vec()) {
        se::qk_prep_vec_bf16_kernel<<<tokens, 256, smem, stream>>>(
            (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, inv_freq, positions, token_seq,
            seq_rows, table, table_stride, (__nv_bfloat16*)cache, (__nv_bfloat16*)q_out, hq, hkv, d, rot, eps, rope_scale,
            page_size, write_cache, num_pages, error);
        SE_LAUNCH_CHECK();
    }
    if (vec) {
        SE_DISPATCH_DTYPE(dtype, T,
            se::qk_prep_vec_kernel<T><<<tokens, 256, smem, stream>>>(
                (const T*)qkv, (const T*)q_w, (const T*)k_w, inv_freq, positions, token_seq, seq_rows, table,
                table_stride, (T*)cache, (T*)q_out, hq, hkv, d, rot, eps, rope_scale, page_size, write_cache,
                num_pages, error));
        SE_LAUNCH_CHECK();
    }
    // inv_rms: optional float [tokens, 2] workspace; when given (many tokens) the statistics
    // are computed once per token by a first kernel
    const bool two_pass = inv_rms != nullptr && q_w != nullptr;
    if (two_pass) {
        SE_DISPATCH_DTYPE(dtype, T,
            se::qk_inv_rms_kernel<T><<<tokens, 256, 0, stream>>>((const T*)qkv, inv_rms, hq * d, hkv * d, eps));
    }
    const int heads_per_block = tokens > 64 ? 8 : 1;
    // as a dependent of the kernel before it, unless a kernel of this call came first
    SE_DISPATCH_DTYPE(dtype, T, {
        const dim3 grid(tokens, se::ceil_div(hq + hkv, heads_per_block));
        if (two_pass) {
            se::qk_prep_kernel<T><<<grid, 128, smem, stream>>>(
                (const T*)qkv, (const T*)q_w, (const T*)k_w, rot > 0 ? inv_freq : nullptr, positions, token_seq,
                seq_rows, table, table_stride, (T*)cache, (T*)q_out, hq, hkv, d, rot, eps, rope_scale, page_size,
                write_cache, inv_rms, heads_per_block, pairing, num_pages, error);
        } else {
            cudaError_t e = SE_LAUNCH_DEPENDENT_IF(
                settled != 0, "qk", se::qk_prep_kernel<T>, grid, dim3(128), smem, stream, (const T*)qkv, (const T*)q_w, (const T*)k_w,
                rot > 0 ? inv_freq : nullptr, positions, token_seq, seq_rows, table, table_stride, (T*)cache,
                (T*)q_out, hq, hkv, d, rot, eps, rope_scale, page_size, write_cache, (const float*)nullptr,
                heads_per_block, pairing, num_pages, error);
            if (e != cudaSuccess) return (int)e;
        }
    });
    SE_LAUNCH_CHECK();
}
