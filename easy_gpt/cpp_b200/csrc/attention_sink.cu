// Grouped-query attention whose keys and values have sizes of their own, over a paged cache that keeps either one row
// (key | value) per token and KV head or, where the two sizes are equal, keys and values in planes of their own (the
// layout the tensor-core kernels read): preparation of queries, keys and values, and the attention itself for the 32-bit
// path and for sizes the tensor-core kernels do not take.  A key lies at k[page * page_stride + head * head_stride +
// offset * row_stride], its value at the same place from v.
//
// Preparation, per token at position p (float32 throughout, from the float32 output of the projections):
//   the first rot_dims values of every query and key head are turned in pairs (i, i + rot_dims/2) by the angle
//   p * f_i: (u, v) -> (u c - v s, v c + u s) with (c, s) = magnitude * (cos, sin) from the step's table;
//   then, if unit_eps >= 0, every query and key head is divided by its root mean square (eps under the root);
//   queries go to q_out, keys and values to the token's row of the cache.
//
// Attention: token at position p of its request sees the keys first..p, first = 0 or p - window + 1;
//   score = (q . k) * scale;  weight_j = exp(s_j) / (sink ? exp(sink_logit) : 0 + sum_i exp(s_i))
// A sink is one more term of the denominator that has no value.  One warp per (token, query head), a running softmax
// over chunks of 32 keys that start at `first`: the order of the sums depends on the token's position and the window
// alone, never on how the request was cut into steps, on the batch or on the page ids.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 8;      // value size <= 256

// one warp per (token, head): heads 0..H-1 are queries, H..H+G-1 keys (each with its value row)
template <typename T>
__global__ void __launch_bounds__(128) sink_prepare_kernel(const float* __restrict__ proj, long long ld, const float2* __restrict__ table, int half,
                                                           float magnitude, const int* __restrict__ slot_map, T* __restrict__ k_cache,
                                                           T* __restrict__ v_cache, int row_stride, long long head_stride, int page_size,
                                                           long long page_stride, long long pool_slots, T* __restrict__ q_out, int tokens, int heads,
                                                           int kv_heads, int dk, int dv, float unit_eps, int* status) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)tokens * (heads + kv_heads)) return;
    const int t = (int)(w / (heads + kv_heads)), h = (int)(w % (heads + kv_heads));
    const bool is_q = h < heads;
    const float* src = proj + (size_t)t * ld + (size_t)h * dk;         // queries then keys, head after head
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * heads + h) * dk;
    } else {
        if (!k_cache) return;
        const long long slot = slot_map[t];
        if (slot < 0 || slot >= pool_slots) {
            if (lane == 0) atomicOr(status, EG_STATUS_BAD_SLOT);
            return;
        }
        const int g = h - heads;
        const long long at = (slot / page_size) * page_stride + g * head_stride + (slot % page_size) * (long long)row_stride;
        dst = k_cache + at;
        const float* v = proj + (size_t)t * ld + (size_t)(heads + kv_heads) * dk + (size_t)g * dv;
        for (int d = lane; d < dv; d += 32) v_cache[at + d] = from_f32<T>(v[d]);
    }
    const int rot = 2 * half;
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) {
        float x = src[d];
        if (d < rot) {
            const int i = d < half ? d : d - half;
            const float2 cs = table[(size_t)t * half + i];
            const float c = cs.x * magnitude, s = cs.y * magnitude;
            x = d < half ? x * c - src[d + half] * s : x * c + src[d - half] * s;
        }
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float inv = unit_eps >= 0.f ? 1.0f / sqrtf(ss / (float)dk + unit_eps) : 1.0f;
    for (int d = lane; d < dk; d += 32) {
        float x = src[d];
        if (d < rot) {
            const int i = d < half ? d : d - half;
            const float2 cs = table[(size_t)t * half + i];
            const float c = cs.x * magnitude, s = cs.y * magnitude;
            x = d < half ? x * c - src[d + half] * s : x * c + src[d - half] * s;
        }
        dst[d] = from_f32<T>(x * inv);
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
sink_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, int row_stride, long long head_stride,
                      const int* __restrict__ block_table, int table_stride,
                      const int* __restrict__ token_seq, const int* __restrict__ positions, const int* __restrict__ token_list, T* __restrict__ out,
                      long long ldo, int heads, int kv_heads, int dk, int dv, int page_size, long long page_stride, int num_pages, int window,
                      float scale, int has_sink, float sink_logit, int* status) {
    extern __shared__ float q_shared[];              // WARPS * dk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = token_list ? token_list[blockIdx.x] : blockIdx.x;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= heads) return;                           // no block-wide barrier below
    const int g = h / (heads / kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_seq[t] * table_stride;
    float* qs = q_shared + warp * dk;
    const T* qrow = q + ((size_t)t * heads + h) * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = to_f32<T>(qrow[d]);
    __syncwarp();

    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.0f;
    float acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.0f;
    for (int base = first; base <= pos; base += 32) {
        const int kpos = base + lane;
        long long row_off = -1;
        if (kpos <= pos) {
            const int page = table[kpos / page_size];
            if (page < 0 || page >= num_pages) atomicOr(status, EG_STATUS_BAD_PAGE);
            else row_off = (long long)page * page_stride + g * head_stride + (long long)(kpos % page_size) * row_stride;
        }
        float s = -INFINITY;
        if (row_off >= 0) {
            const T* krow = k_cache + row_off;
            float dot = 0.0f;
            for (int d = 0; d < dk; ++d) dot = fmaf(qs[d], to_f32<T>(krow[d]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float corr = expf(m - m_new);
        const float p = (row_off >= 0) ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] *= corr;
        const int nkeys = min(32, pos - base + 1);
        for (int j = 0; j < nkeys; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long off_j = __shfl_sync(0xffffffffu, row_off, j);
            if (off_j < 0) continue;
            const T* vrow = v_cache + off_j;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_f32<T>(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    if (has_sink) {
        const float m_new = fmaxf(m, sink_logit);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sink_logit - m_new);
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] *= corr;
    }
    T* orow = out + (size_t)t * ldo + (size_t)h * dv;
    const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<T>(acc[i] * inv_l);
    }
}
}  // namespace

// proj float32 [tokens, ld]: query heads, key heads, value heads side by side.  table: cos/sin [tokens, rot_dims/2, 2] or
// null with rot_dims 0.  k_cache null: nothing is stored (the entry reads another entry's cache).  q_out [tokens, heads, dk].
EG_API int eg_sink_attention_prepare(cudaStream_t stream, int dtype, const float* proj, long long ld, const float* table, int rot_dims, float magnitude,
                                     const int* slot_map, void* k_cache, void* v_cache, int row_stride, long long head_stride, int page_size,
                                     long long page_stride, long long pool_slots, void* q_out, int tokens, int heads, int kv_heads, int dk, int dv,
                                     float unit_eps, int* status) {
    if (tokens <= 0) return 0;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > dk || (rot_dims > 0 && !table)) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)tokens * (heads + kv_heads);
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (dtype == EG_BF16)
        sink_prepare_kernel<bf16><<<blocks, 128, 0, stream>>>(proj, ld, (const float2*)table, rot_dims / 2, magnitude, slot_map, (bf16*)k_cache, (bf16*)v_cache,
                                                              row_stride, head_stride, page_size, page_stride, pool_slots, (bf16*)q_out, tokens, heads, kv_heads, dk, dv, unit_eps, status);
    else
        sink_prepare_kernel<float><<<blocks, 128, 0, stream>>>(proj, ld, (const float2*)table, rot_dims / 2, magnitude, slot_map, (float*)k_cache, (float*)v_cache,
                                                               row_stride, head_stride, page_size, page_stride, pool_slots, (float*)q_out, tokens, heads, kv_heads, dk, dv, unit_eps, status);
    return eg_launch_status();
}

// q [tokens, heads, dk]; out [tokens, ldo] with head h at column h * dv.
// token_list: the tokens to work on (num_tokens of them), or null for all.  Returns cudaErrorInvalidValue for sizes it does not take.
EG_API int eg_sink_attention(cudaStream_t stream, int dtype, const void* q, const void* k_cache, const void* v_cache, int row_stride, long long head_stride,
                             const int* block_table, int table_stride,
                             const int* token_seq, const int* positions, const int* token_list, void* out, long long ldo, int num_tokens, int heads,
                             int kv_heads, int dk, int dv, int page_size, long long page_stride, int num_pages, int window, float scale, int has_sink,
                             float sink_logit, int* status) {
    if (num_tokens <= 0) return 0;
    if (dv > 32 * MAX_PER_LANE || dv <= 0 || dk <= 0 || dk > 4096 || kv_heads <= 0 || heads % kv_heads) return (int)cudaErrorInvalidValue;
    dim3 grid(num_tokens, (heads + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * dk * sizeof(float);
    if (dtype == EG_BF16)
        sink_attention_kernel<bf16><<<grid, WARPS * 32, smem, stream>>>((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, row_stride, head_stride, block_table,
                                                                        table_stride, token_seq, positions,
                                                                        token_list, (bf16*)out, ldo, heads, kv_heads, dk, dv, page_size, page_stride,
                                                                        num_pages, window, scale, has_sink, sink_logit, status);
    else
        sink_attention_kernel<float><<<grid, WARPS * 32, smem, stream>>>((const float*)q, (const float*)k_cache, (const float*)v_cache, row_stride, head_stride, block_table,
                                                                         table_stride, token_seq, positions, token_list, (float*)out, ldo, heads, kv_heads, dk, dv, page_size,
                                                                         page_stride, num_pages, window, scale, has_sink, sink_logit, status);
    return eg_launch_status();
}
