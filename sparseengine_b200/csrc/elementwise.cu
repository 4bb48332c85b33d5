// Embedding gather, RMSNorm (with and without the fused residual add), row gather and
// the block-table update kernel.
//
// RMSNorm follows src/sparseengine/kernels/triton/rmsnorm.py:17-66 of the reference:
// with a residual the 32-bit sum x+res is what gets normalised, and the residual is
// overwritten with the sum rounded to the activation type.
#include "common.cuh"

namespace se {

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    T* __restrict__ out, int hidden, int vocab) {
    const int t = blockIdx.x;
    int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * hidden;
    T* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? src[i] : from_float<T>(0.f);
}

// One block per row. x_sum (dynamic shared memory, `hidden` floats) keeps the 32-bit row.
template <typename T>
__global__ void rmsnorm_kernel(const T* x, const T* residual, const T* __restrict__ w,
                               T* y, T* residual_out, int hidden, float eps) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    grid_dependency_trigger();       // a projection that follows may start streaming its weights
    const size_t base = (size_t)blockIdx.x * hidden;
    const bool vec = (hidden & 7) == 0 && aligned8(x) && aligned8(y) && aligned8(w) &&
                     (residual == nullptr || (aligned8(residual) && aligned8(residual_out)));
    // Launched as a dependent of the kernel that writes x: a thread's first weights are asked for
    // before that kernel has ended (no kernel writes them).
    constexpr int kKeep = 2;
    float w_keep[kKeep][8];
    if (vec) {
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int i = (threadIdx.x + k * blockDim.x) * 8;
            if (i < hidden) load8(w + i, w_keep[k]);
        }
    }
    grid_dependency_wait();
    float ss = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float v[8];
            load8(x + base + i, v);
            if (residual != nullptr) {
                float r[8];
                load8(residual + base + i, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += r[j];
                store8(residual_out + base + i, v);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) { row[i + j] = v[j]; ss += v[j] * v[j]; }
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = to_float(x[base + i]);
            if (residual != nullptr) {
                v += to_float(residual[base + i]);
                residual_out[base + i] = from_float<T>(v);
            }
            row[i] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    if (vec) {
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int i = (threadIdx.x + k * blockDim.x) * 8;
            if (i < hidden) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = row[i + j] * inv * w_keep[k][j];
                store8(y + base + i, o);
            }
        }
        for (int i = (threadIdx.x + kKeep * blockDim.x) * 8; i < hidden; i += blockDim.x * 8) {
            float wv[8], o[8];
            load8(w + i, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = row[i + j] * inv * wv[j];
            store8(y + base + i, o);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x)
            y[base + i] = from_float<T>(row[i] * inv * to_float(w[i]));
    }
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ idx,
                                   T* __restrict__ dst, int width) {
    const size_t s = (size_t)idx[blockIdx.x] * width, d = (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[d + i] = src[s + i];
}

// updates: n triples (row, index, page); table[row * stride + index] = page.  A triple whose
// row, index or page lies outside the table or the pool is not applied, and a code goes to
// the error word.
__device__ __forceinline__ void apply_table_update(int* table, int rows, int stride, const int* __restrict__ updates,
                                                   int i, int num_pages, int* error) {
    const int row = updates[3 * i], index = updates[3 * i + 1], page = updates[3 * i + 2];
    if ((unsigned)row >= (unsigned)rows || (unsigned)index >= (unsigned)stride ||
        !page_in_pool(page, num_pages, nullptr, 0)) {
        if (error != nullptr) atomicCAS(error, 0, SE_CODE_BAD_TABLE_UPDATE);
        return;
    }
    table[(size_t)row * stride + index] = page;
}

__global__ void table_update_kernel(int* table, int rows, int stride, const int* __restrict__ updates, int n,
                                    int num_pages, int* error) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) apply_table_update(table, rows, stride, updates, i, num_pages, error);
}

// The same with the number of triples read from device memory (for replayed CUDA graphs,
// where the launch is fixed and the count changes from step to step).
__global__ void table_update_dyn_kernel(int* table, int rows, int stride, const int* __restrict__ updates,
                                        const int* __restrict__ count, int max_n, int num_pages, int* error) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < min(count[0], max_n)) apply_table_update(table, rows, stride, updates, i, num_pages, error);
}

}  // namespace se

extern "C" int se_embed_gather(const void* table, const int* ids, void* out, int tokens, int hidden,
                               int vocab, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    SE_DISPATCH_DTYPE(dtype, T,
        se::embed_gather_kernel<T><<<tokens, 256, 0, stream>>>((const T*)table, ids, (T*)out, hidden, vocab));
    SE_LAUNCH_CHECK();
}

// The widest row the norm takes: it is kept in shared memory in 32-bit (200 KB).
extern "C" int se_rmsnorm_max_width() { return 200 * 1024 / (int)sizeof(float); }

extern "C" int se_rmsnorm(const void* x, const void* residual, const void* w, void* y, void* residual_out,
                          int rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden > se_rmsnorm_max_width()) return SE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)hidden * sizeof(float);
    const int threads = hidden >= 8192 ? 512 : hidden >= 2048 ? 256 : 128;
    SE_DISPATCH_DTYPE(dtype, T, {
        if (smem > 40 * 1024) {      // static shared memory counts against the 48 KB a kernel has without asking
            cudaError_t e = cudaFuncSetAttribute(se::rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        cudaError_t e = SE_LAUNCH_DEPENDENT("norm", se::rmsnorm_kernel<T>, dim3(rows), dim3(threads), smem, stream, (const T*)x,
                                             (const T*)residual, (const T*)w, (T*)y, (T*)residual_out, hidden, eps);
        if (e != cudaSuccess) return (int)e;
    });
    SE_LAUNCH_CHECK();
}

extern "C" int se_gather_rows(const void* src, const int* idx, void* dst, int rows, int width, int dtype,
                              cudaStream_t stream) {
    if (rows <= 0) return 0;
    SE_DISPATCH_DTYPE(dtype, T,
        se::gather_rows_kernel<T><<<rows, 256, 0, stream>>>((const T*)src, idx, (T*)dst, width));
    SE_LAUNCH_CHECK();
}

extern "C" int se_table_update(int* table, int rows, int stride, const int* updates, int n, int num_pages, int* error,
                               cudaStream_t stream) {
    if (n <= 0) return 0;
    se::table_update_kernel<<<se::ceil_div(n, 256), 256, 0, stream>>>(table, rows, stride, updates, n, num_pages, error);
    SE_LAUNCH_CHECK();
}

extern "C" int se_table_update_dyn(int* table, int rows, int stride, const int* updates, const int* count, int max_n,
                                   int num_pages, int* error, cudaStream_t stream) {
    if (max_n <= 0) return 0;
    se::table_update_dyn_kernel<<<se::ceil_div(max_n, 256), 256, 0, stream>>>(table, rows, stride, updates, count, max_n,
                                                                              num_pages, error);
    SE_LAUNCH_CHECK();
}
