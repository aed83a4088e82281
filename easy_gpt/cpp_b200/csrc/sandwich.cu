// Pieces of a layer whose branches are normed on both sides, x <- x + norm_b(f(shift(norm_a(x)))):
//
//   token shift      out[t] = h[t] + (h[t-1] - h[t]) * mu            h[t-1]: the row before t in its request; the request's
//                                                                    slot holds the last row of earlier steps (zeros at the start)
//   norm + shift     the same with h = gain * x / sqrt(mean(x^2) + eps) computed here from the float32 stream
//   norm and add     x[t] += gain * y[t] / sqrt(mean(y[t]^2) + eps)  a branch's output joins the stream through its norm
//   xIELU            a(z) = ap z^2 + z / 2 (z > 0),  an (e^z - 1 - z) + z / 2 (z <= 0)
//   scaled gather    x[t] = scale * table[id[t]]
//
// Sums, roots and divisions are float32.  The slot is read by the block of an entry's first token alone, which then
// stores the entry's last row in it: read and write of a slot sit in one thread each, so no block waits for another.
#include "common.cuh"

namespace {

// inverse root mean square of `row` (+ nothing): every thread gets it
__device__ __forceinline__ float inv_rms(const float* __restrict__ row, int hidden, float eps, float* scratch) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) ss = fmaf(row[j], row[j], ss);
    ss = block_sum(ss, scratch);
    return 1.0f / sqrtf(ss / (float)hidden + eps);
}

template <typename TO>
__global__ void token_shift_kernel(const float* __restrict__ rows, const float* __restrict__ mu, float* __restrict__ state, long long slot_floats,
                                   const int* __restrict__ token_seq, const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                                   TO* __restrict__ out, int hidden) {
    const int t = blockIdx.x, seq = token_seq[t], start = seq_starts[seq];
    const bool first = t == start;
    float* slot = state + (size_t)seq_slots[seq] * slot_floats;
    const float* prev = first ? slot : rows + (size_t)(t - 1) * hidden;
    const float* x = rows + (size_t)t * hidden;
    const float* last = rows + (size_t)(seq_starts[seq + 1] - 1) * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float v = x[j], p = prev[j];
        out[(size_t)t * hidden + j] = from_f32<TO>(fmaf(p - v, mu[j], v));
        if (first) slot[j] = last[j];
    }
}

template <typename TO>
__global__ void rmsnorm_shift_kernel(const float* __restrict__ stream, const float* __restrict__ gain, float eps, const float* __restrict__ mu,
                                     float* __restrict__ state, long long slot_floats, const int* __restrict__ token_seq,
                                     const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, TO* __restrict__ out, int hidden) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, seq = token_seq[t], start = seq_starts[seq];
    const bool first = t == start;
    float* slot = state + (size_t)seq_slots[seq] * slot_floats;
    const float* x = stream + (size_t)t * hidden;
    const float inv = inv_rms(x, hidden, eps, scratch);
    // the row in front: the stream's row t-1 normed again here, or the slot's row; the first token's block also norms the
    // entry's last row for the slot
    const float* other = stream + (size_t)(first ? seq_starts[seq + 1] - 1 : t - 1) * hidden;
    const float inv_other = (first && other == x) ? inv : inv_rms(other, hidden, eps, scratch);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float g = gain[j];
        const float v = g * (x[j] * inv);
        const float o = g * (other[j] * inv_other);
        const float p = first ? slot[j] : o;
        out[(size_t)t * hidden + j] = from_f32<TO>(fmaf(p - v, mu[j], v));
        if (first) slot[j] = o;
    }
}

template <typename TD>
__global__ void rmsnorm_add_kernel(float* __restrict__ stream, const TD* __restrict__ y, long long ldy, const float* __restrict__ gain, float eps,
                                   int hidden) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const TD* row = y + (size_t)t * ldy;
    float ss = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float v = to_f32<TD>(row[j]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    float* x = stream + (size_t)t * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) x[j] += gain[j] * (to_f32<TD>(row[j]) * inv);
}

__device__ __forceinline__ float xielu_f(float z, float ap, float an) {
    if (z > 0.f) return fmaf(ap * z, z, 0.5f * z);
    return fmaf(an, expm1f(z) - z, 0.5f * z);
}

template <typename TI, typename TO>
__global__ void xielu_kernel(const TI* __restrict__ x, long long ldx, TO* __restrict__ out, long long ldo, int tokens, int n, float ap, float an) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * n) return;
    const int t = (int)(i / n), c = (int)(i % n);
    out[(size_t)t * ldo + c] = from_f32<TO>(xielu_f(to_f32<TI>(x[(size_t)t * ldx + c]), ap, an));
}

template <typename T>
__global__ void embedding_scaled_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ stream, int hidden, int vocab,
                                        float scale, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* out = stream + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, EG_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = to_f32<T>(row[j]) * scale;
}

__global__ void scale_kernel(float* __restrict__ x, long long n, float s) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= s;
}

inline int row_threads(int hidden) {
    int threads = 64;
    while (threads < 512 && threads * 4 < hidden) threads <<= 1;
    return threads;
}

}  // namespace

// rows float32 [tokens, hidden], already normalised; out in out_dtype
EG_API int eg_token_shift(cudaStream_t stream, const float* rows, const float* mu, float* state, long long slot_floats, const int* token_seq,
                          const int* seq_starts, const int* seq_slots, void* out, int out_dtype, int tokens, int hidden) {
    if (tokens <= 0) return 0;
    const int threads = row_threads(hidden);
    if (out_dtype == EG_BF16)
        token_shift_kernel<bf16><<<tokens, threads, 0, stream>>>(rows, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (bf16*)out, hidden);
    else
        token_shift_kernel<float><<<tokens, threads, 0, stream>>>(rows, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (float*)out, hidden);
    return eg_launch_status();
}

// the norm of the float32 stream and the shift in one kernel
EG_API int eg_rmsnorm_shift(cudaStream_t stream, const float* residual, const float* gain, float eps, const float* mu, float* state,
                            long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, int out_dtype,
                            int tokens, int hidden) {
    if (tokens <= 0) return 0;
    const int threads = row_threads(hidden);
    if (out_dtype == EG_BF16)
        rmsnorm_shift_kernel<bf16><<<tokens, threads, 0, stream>>>(residual, gain, eps, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (bf16*)out,
                                                                   hidden);
    else
        rmsnorm_shift_kernel<float><<<tokens, threads, 0, stream>>>(residual, gain, eps, mu, state, slot_floats, token_seq, seq_starts, seq_slots, (float*)out,
                                                                    hidden);
    return eg_launch_status();
}

// residual[t] += gain * y[t] / rms(y[t])
EG_API int eg_rmsnorm_add(cudaStream_t stream, float* residual, const void* y, int y_dtype, long long ldy, const float* gain, float eps, int tokens,
                          int hidden) {
    if (tokens <= 0) return 0;
    const int threads = row_threads(hidden);
    if (y_dtype == EG_BF16) rmsnorm_add_kernel<bf16><<<tokens, threads, 0, stream>>>(residual, (const bf16*)y, ldy, gain, eps, hidden);
    else rmsnorm_add_kernel<float><<<tokens, threads, 0, stream>>>(residual, (const float*)y, ldy, gain, eps, hidden);
    return eg_launch_status();
}

// out[t, c] = xielu(x[t, c]); ap and an are the finished coefficients (softplus applied by the caller)
EG_API int eg_xielu(cudaStream_t stream, const void* x, int x_dtype, long long ldx, void* out, int out_dtype, long long ldo, int tokens, int n, float ap,
                    float an) {
    const long long total = (long long)tokens * n;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (x_dtype == EG_F32 && out_dtype == EG_F32) xielu_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)x, ldx, (float*)out, ldo, tokens, n, ap, an);
    else if (x_dtype == EG_F32) xielu_kernel<float, bf16><<<blocks, 256, 0, stream>>>((const float*)x, ldx, (bf16*)out, ldo, tokens, n, ap, an);
    else if (out_dtype == EG_F32) xielu_kernel<bf16, float><<<blocks, 256, 0, stream>>>((const bf16*)x, ldx, (float*)out, ldo, tokens, n, ap, an);
    else xielu_kernel<bf16, bf16><<<blocks, 256, 0, stream>>>((const bf16*)x, ldx, (bf16*)out, ldo, tokens, n, ap, an);
    return eg_launch_status();
}

EG_API int eg_embedding_gather_scaled(cudaStream_t stream, int dtype, const int* ids, const void* table, float* residual, int tokens, int hidden,
                                      int vocab, float scale, int* status) {
    if (tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == EG_BF16) embedding_scaled_kernel<bf16><<<tokens, threads, 0, stream>>>(ids, (const bf16*)table, residual, hidden, vocab, scale, status);
    else embedding_scaled_kernel<float><<<tokens, threads, 0, stream>>>(ids, (const float*)table, residual, hidden, vocab, scale, status);
    return eg_launch_status();
}

EG_API int eg_scale_f32(cudaStream_t stream, float* x, long long n, float s) {
    if (n <= 0) return 0;
    scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, n, s);
    return eg_launch_status();
}
