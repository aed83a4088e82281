// Residual add fused with layer norm, for one or two norms of the same row.
//   residual[r, :] += delta_a[r, :] + delta_b[r, :]      (float32 residual stream; either delta may be null)
//   out1[r, :] = (x - mean(x)) / sqrt(var(x) + eps) * gain1 + bias1,   var = mean((x - mean)^2)
//   out2[r, :] = the same with gain2, bias2               (skipped when out2 is null)
// A layer whose mixer and feed-forward read the same stream through two norms needs the mean and the variance of a row
// once: both outputs leave one kernel, and the adds of the layer in front ride along.  Mean, deviations, variance, square
// root and division are float32 (two passes over the row, which is kept in shared memory; no fast-math).  With `rows`
// given, output row r is computed from residual row rows[r] and the residual is left untouched.
#include "common.cuh"

namespace {
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
    return dtype == EG_BF16 ? __bfloat162float(((const bf16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void store_any(void* p, int dtype, size_t i, float v) {
    if (dtype == EG_BF16) ((bf16*)p)[i] = __float2bfloat16_rn(v);
    else ((float*)p)[i] = v;
}

__global__ void add_layernorm_kernel(float* __restrict__ residual, const void* __restrict__ delta_a, int dtype_a, const void* __restrict__ delta_b,
                                     int dtype_b, const int* __restrict__ rows, const float* __restrict__ gain1, const float* __restrict__ bias1,
                                     void* __restrict__ out1, const float* __restrict__ gain2, const float* __restrict__ bias2, void* __restrict__ out2,
                                     int out_dtype, int hidden, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float* x = residual + src;
    const bool write_back = rows == nullptr && (delta_a || delta_b);
    float sum = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = x[j];
        if (delta_a) v += load_any(delta_a, dtype_a, src + j);
        if (delta_b) v += load_any(delta_b, dtype_b, src + j);
        if (write_back) x[j] = v;
        row[j] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)hidden;
    float sq = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float d = row[j] - mean;
        sq += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + eps);
    const size_t dst = (size_t)r * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float n = (row[j] - mean) * inv;
        store_any(out1, out_dtype, dst + j, n * gain1[j] + bias1[j]);
        if (out2) store_any(out2, out_dtype, dst + j, n * gain2[j] + bias2[j]);
    }
}
}  // namespace

// dtypes: EG_F32 or EG_BF16.  rows, delta_a, delta_b and out2 (with gain2, bias2) may be null.
EG_API int eg_add_layernorm(cudaStream_t stream, float* residual, const void* delta_a, int dtype_a, const void* delta_b, int dtype_b, const int* rows,
                            const float* gain1, const float* bias1, void* out1, const float* gain2, const float* bias2, void* out2, int out_dtype,
                            int num_rows, int hidden, float eps) {
    if (num_rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(add_layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    int threads = 64;
    while (threads < 512 && threads * 4 < hidden) threads <<= 1;
    add_layernorm_kernel<<<num_rows, threads, smem, stream>>>(residual, delta_a, dtype_a, delta_b, dtype_b, rows, gain1, bias1, out1, gain2, bias2, out2,
                                                            out_dtype, hidden, eps);
    return eg_launch_status();
}
