// Attention whose keys and values are expanded from one cached latent vector per token.
//
// Per token the cache holds ONE row of `rank + rot` values for all heads: the normalised latent c [rank] and a rotated
// key part k_r [rot].  With per-head maps Uk [dim, rank] and Uv [vdim, rank], the key of head h is (Uk_h c, k_r) and its
// value Uv_h c.  Because q . (Uk_h c) = (Uk_h^T q) . c, the kernels never expand keys or values: the query is carried
// into the latent space once per token (eg_latent_absorb), the attention runs over the cached rows themselves, each of
// which serves as key (all rank + rot values) and as value (its first rank values), and the result is expanded by Uv_h
// once per token (eg_latent_expand).
//
//   eg_latent_prepare   down-projected rows -> unit-RMS query latent, unit-RMS c and rotated k_r into the paged cache
//   eg_latent_absorb    q [T, H, dim + rot] -> qa [T, H, rank + rot] = scale * (Uk_h^T q_plain, rotate(q_rot))
//   eg_attention_latent softmax over the request's cached rows up to the token's position, with an optional sink
//                       (a learned logit per head that joins the denominator and has no value), float32
//   eg_latent_expand    o [T, H, rank] -> [T, H * vdim] = Uv_h o
//
// The rotation turns neighbouring pairs (2i, 2i+1) of the first `rot_dims` values of the rotated part by the angle
// position * inv_freq[i]; angles, sines and cosines are float32 (accurate sincosf).  Scores, weights, maxima and sums
// are float32; every sum's order depends on the token's own position only, never on the batch.
#include "common.cuh"

namespace {

__device__ __forceinline__ void store_any(void* p, int dtype, size_t i, float v) {
    if (dtype == EG_BF16) ((bf16*)p)[i] = __float2bfloat16_rn(v);
    else ((float*)p)[i] = v;
}

// one block per token
__global__ void latent_prepare_kernel(const float* __restrict__ down, long long ld, int q_rank, int rank, int rot, int rot_dims,
                                      const float* __restrict__ gain_q, const float* __restrict__ gain_c, float eps, const float* __restrict__ inv_freq,
                                      const int* __restrict__ positions, const int* __restrict__ slot_map, void* __restrict__ cache, int cache_dtype,
                                      int page_size, long long page_stride, long long pool_slots, void* __restrict__ cq, int cq_dtype,
                                      int* __restrict__ status) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* row = down + (size_t)t * ld;
    float ss = 0.f;
    for (int j = threadIdx.x; j < q_rank; j += blockDim.x) ss += row[j] * row[j];
    const float inv_q = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int j = threadIdx.x; j < q_rank; j += blockDim.x) store_any(cq, cq_dtype, (size_t)t * q_rank + j, row[j] * inv_q * gain_q[j]);
    if (!cache) return;
    const long long slot = slot_map[t];
    if (slot < 0 || slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(status, EG_STATUS_BAD_SLOT);
        return;
    }
    const float* c = row + q_rank;
    ss = 0.f;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) ss += c[j] * c[j];
    const float inv_c = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    const size_t at = (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * (rank + rot);
    for (int j = threadIdx.x; j < rank; j += blockDim.x) store_any(cache, cache_dtype, at + j, c[j] * inv_c * gain_c[j]);
    const float* kr = c + rank;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const float a = kr[2 * i], b = kr[2 * i + 1];
        store_any(cache, cache_dtype, at + rank + 2 * i, a * cs - b * sn);
        store_any(cache, cache_dtype, at + rank + 2 * i + 1, b * cs + a * sn);
    }
    for (int j = rot_dims + threadIdx.x; j < rot; j += blockDim.x) store_any(cache, cache_dtype, at + rank + j, kr[j]);
}

// one block per (token, head); Uk [heads * dim, rank] in TW
template <typename TW>
__global__ void latent_absorb_kernel(const float* __restrict__ q, long long ldq, const TW* __restrict__ Uk, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, int rot_dims, float scale, float* __restrict__ qa, int heads, int dim, int rot,
                                     int rank) {
    extern __shared__ float qs[];
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = q + (size_t)t * ldq + (size_t)h * (dim + rot);
    for (int d = threadIdx.x; d < dim + rot; d += blockDim.x) qs[d] = src[d];
    __syncthreads();
    float* out = qa + ((size_t)t * heads + h) * (rank + rot);
    const TW* W = Uk + (size_t)h * dim * rank;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        float acc = 0.f;
        for (int d = 0; d < dim; ++d) acc = fmaf(qs[d], to_f32<TW>(W[(size_t)d * rank + r]), acc);
        out[r] = acc * scale;
    }
    const float pos = (float)positions[t];
    const float* qr = qs + dim;
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const float a = qr[2 * i], b = qr[2 * i + 1];
        out[rank + 2 * i] = (a * cs - b * sn) * scale;
        out[rank + 2 * i + 1] = (b * cs + a * sn) * scale;
    }
    for (int j = rot_dims + threadIdx.x; j < rot; j += blockDim.x) out[rank + j] = qr[j] * scale;
}

// One block of WARPS warps per (token, head).  Warp w takes the keys j = w, w + WARPS, ...; a lane holds the values
// d = lane + 32 i of the query and of the key at hand, so that the cached row is read once for the score and for the
// weighted sum.  Each warp keeps a running maximum, sum and weighted sum; the block merges them, adds the sink to the
// denominator and writes o [rank].
template <typename TC, int VPL, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attention_latent_kernel(const float* __restrict__ qa, const TC* __restrict__ cache,
                                                                      const int* __restrict__ block_table, int table_stride,
                                                                      const int* __restrict__ token_seq, const int* __restrict__ positions,
                                                                      const float* __restrict__ sink, float* __restrict__ out, int heads, int rank, int rot,
                                                                      int page_size, long long page_stride, int num_pages, int* __restrict__ status) {
    extern __shared__ float merge[];            // [WARPS, rank] weighted sums, then [WARPS] maxima and [WARPS] sums
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int width = rank + rot;
    const float* qrow = qa + ((size_t)t * heads + h) * width;
    float qv[VPL], acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < width ? qrow[d] : 0.f;
        acc[i] = 0.f;
    }
    const int* table = block_table + (size_t)token_seq[t] * table_stride;
    const int last = positions[t];
    float m = -INFINITY, l = 0.f;
    for (int j = warp; j <= last; j += WARPS) {
        const int page = table[j / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(status, EG_STATUS_BAD_PAGE);
            continue;
        }
        const TC* krow = cache + (size_t)page * page_stride + (size_t)(j % page_size) * width;
        float kv[VPL], s = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int d = lane + 32 * i;
            kv[i] = d < width ? to_f32<TC>(krow[d]) : 0.f;
            s = fmaf(qv[i], kv[i], s);
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float keep = expf(m - m_new), p = expf(s - m_new);        // exp(-inf) = 0 at the first key
        l = l * keep + p;
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[i] = fmaf(p, kv[i], acc[i] * keep);
        m = m_new;
    }
    float* sums = merge;
    float* maxima = merge + (size_t)WARPS * rank;
    float* weights = maxima + WARPS;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) sums[(size_t)warp * rank + d] = acc[i];
    }
    if (lane == 0) {
        maxima[warp] = m;
        weights[warp] = l;
    }
    __syncthreads();
    float top = sink ? sink[h] : -INFINITY;
    for (int w = 0; w < WARPS; ++w) top = fmaxf(top, maxima[w]);
    float denom = sink ? expf(sink[h] - top) : 0.f;
    float f[WARPS];
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        f[w] = maxima[w] == -INFINITY ? 0.f : expf(maxima[w] - top);
        denom += weights[w] * f[w];
    }
    float* o = out + ((size_t)t * heads + h) * rank;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v = fmaf(sums[(size_t)w * rank + d], f[w], v);
        o[d] = v / denom;
    }
}

// one block per (token, head), a warp per output value; Uv [heads * vdim, rank] in TW
template <typename TW>
__global__ void latent_expand_kernel(const float* __restrict__ o, const TW* __restrict__ Uv, void* __restrict__ out, int out_dtype, long long ldo,
                                     int heads, int vdim, int rank) {
    extern __shared__ float os[];
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = o + ((size_t)t * heads + h) * rank;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) os[r] = src[r];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int e = warp; e < vdim; e += warps) {
        const TW* w = Uv + ((size_t)h * vdim + e) * rank;
        float acc = 0.f;
        for (int r = lane; r < rank; r += 32) acc = fmaf(os[r], to_f32<TW>(w[r]), acc);
        acc = warp_sum(acc);
        if (lane == 0) store_any(out, out_dtype, (size_t)t * ldo + (size_t)h * vdim + e, acc);
    }
}

}  // namespace

// down [T, ld] float32 holds per token (query latent [q_rank] | latent [rank] | rotated key part [rot]).  Writes the
// unit-RMS query latent times gain_q to cq [T, q_rank] (cq_dtype), and unit-RMS latent times gain_c followed by the
// rotated key part to the cache row of slot_map[t] (cache null: nothing is stored).  page_stride in elements.
EG_API int eg_latent_prepare(cudaStream_t stream, const float* down, long long ld, int q_rank, int rank, int rot, int rot_dims, const float* gain_q,
                             const float* gain_c, float eps, const float* inv_freq, const int* positions, const int* slot_map, void* cache, int cache_dtype,
                             int page_size, long long page_stride, long long pool_slots, void* cq, int cq_dtype, int tokens, int* status) {
    if (tokens <= 0) return 0;
    if (rot_dims % 2 || rot_dims > rot || q_rank <= 0 || rank <= 0) return (int)cudaErrorInvalidValue;
    latent_prepare_kernel<<<tokens, 128, 0, stream>>>(down, ld, q_rank, rank, rot, rot_dims, gain_q, gain_c, eps, inv_freq, positions, slot_map, cache,
                                                     cache_dtype, page_size, page_stride, pool_slots, cq, cq_dtype, status);
    return eg_launch_status();
}

// qa [T, heads, rank + rot] float32 from q [T, ldq] float32 (head by head: dim plain values, rot rotated ones)
EG_API int eg_latent_absorb(cudaStream_t stream, int w_dtype, const float* q, long long ldq, const void* Uk, const int* positions, const float* inv_freq,
                            int rot_dims, float scale, float* qa, int tokens, int heads, int dim, int rot, int rank) {
    if (tokens <= 0) return 0;
    const size_t smem = (size_t)(dim + rot) * sizeof(float);
    if (smem > 48 * 1024 || rot_dims % 2 || rot_dims > rot) return (int)cudaErrorInvalidValue;
    dim3 grid(tokens, heads);
    const int threads = rank >= 256 ? 256 : 128;
    if (w_dtype == EG_BF16)
        latent_absorb_kernel<bf16><<<grid, threads, smem, stream>>>(q, ldq, (const bf16*)Uk, positions, inv_freq, rot_dims, scale, qa, heads, dim, rot, rank);
    else
        latent_absorb_kernel<float><<<grid, threads, smem, stream>>>(q, ldq, (const float*)Uk, positions, inv_freq, rot_dims, scale, qa, heads, dim, rot, rank);
    return eg_launch_status();
}

// out [T, heads, rank] float32; sink [heads] float32 or null; page_stride in elements
EG_API int eg_attention_latent(cudaStream_t stream, int cache_dtype, const float* qa, const void* cache, const int* block_table, int table_stride,
                               const int* token_seq, const int* positions, const float* sink, float* out, int tokens, int heads, int rank, int rot,
                               int page_size, long long page_stride, int num_pages, int* status) {
    if (tokens <= 0) return 0;
    constexpr int WARPS = 4;
    const int vpl = (rank + rot + 31) / 32;
    const size_t smem = ((size_t)WARPS * rank + 2 * WARPS) * sizeof(float);
    if (vpl > 32 || smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid(tokens, heads);
#define EG_LATENT(TC, V) \
    attention_latent_kernel<TC, V, WARPS><<<grid, WARPS * 32, smem, stream>>>(qa, (const TC*)cache, block_table, table_stride, token_seq, positions, sink, out, \
                                                                              heads, rank, rot, page_size, page_stride, num_pages, status)
#define EG_LATENT_T(TC)                  \
    if (vpl <= 2) EG_LATENT(TC, 2);      \
    else if (vpl <= 4) EG_LATENT(TC, 4); \
    else if (vpl <= 8) EG_LATENT(TC, 8); \
    else if (vpl <= 18) EG_LATENT(TC, 18); \
    else EG_LATENT(TC, 32)
    if (cache_dtype == EG_BF16) { EG_LATENT_T(bf16); } else { EG_LATENT_T(float); }
#undef EG_LATENT_T
#undef EG_LATENT
    return eg_launch_status();
}

// out [T, ldo] (out_dtype), head by head vdim values, from o [T, heads, rank] float32
EG_API int eg_latent_expand(cudaStream_t stream, int w_dtype, const float* o, const void* Uv, void* out, int out_dtype, long long ldo, int tokens,
                            int heads, int vdim, int rank) {
    if (tokens <= 0) return 0;
    const size_t smem = (size_t)rank * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid(tokens, heads);
    if (w_dtype == EG_BF16) latent_expand_kernel<bf16><<<grid, 128, smem, stream>>>(o, (const bf16*)Uv, out, out_dtype, ldo, heads, vdim, rank);
    else latent_expand_kernel<float><<<grid, 128, smem, stream>>>(o, (const float*)Uv, out, out_dtype, ldo, heads, vdim, rank);
    return eg_launch_status();
}
