// Attention over cached latent rows on the warp-level tensor cores (bfloat16): the heads of a token are the rows of the
// product.
//
// All heads of a token attend the same cached rows (rank + rot values each, see attention_latent.cu), so 16 heads of one
// token against a tile of 64 keys is a 16 x 64 x (rank + rot) product, and the weighted sum a 16 x rank x 64 one: shapes
// that mma.sync m16n8k16 takes as they are, for a prompt's tokens and for single decoded tokens alike.  A CTA of four
// warps takes (token, group of 16 heads, part of the keys):
//   the queries qa [16, D] and, tile by tile, 64 cached rows [64, D] go to shared memory: one bulk copy (cp.async.bulk,
//     counted on an mbarrier) per cached row, issued by the lanes of the first warp, rows beyond the token's position
//     zeroed; the cached rows are read once for scores and values; the wait on the mbarrier is bounded;
//   scores: warp w computes the tile's keys 16 w .. 16 w + 15 for all 16 heads; row maxima and sums meet in shared memory;
//   the weights go to shared memory as bfloat16 and every warp adds its share of the value columns (columns 16 (w + 4 i)..)
//     from the same key tile, read transposed by ldmatrix;
//   at the end the sink joins the denominator (one part) or the part's (o, m, l) goes to scratch and a second kernel
//     merges the parts and the sink.
// Scores, maxima, sums and the accumulators are float32.  Takes D = rank + rot a multiple of 8, rank a multiple of 8 up
// to 512; anything else: cudaErrorInvalidValue, and the caller uses the generic kernel.
#include "mbarrier.cuh"
#include "mma_utils.cuh"

namespace {
constexpr int KT = 64, WARPS = 4, PAIRS = 8;        // keys per tile; warps; pairs of 8-column value tiles per warp

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

__global__ void __launch_bounds__(WARPS * 32) attention_latent_mma_kernel(const bf16* __restrict__ qa, const bf16* __restrict__ cache,
                                                                          const int* __restrict__ block_table, int table_stride,
                                                                          const int* __restrict__ token_seq, const int* __restrict__ positions,
                                                                          const float* __restrict__ sink, bf16* __restrict__ out, float* __restrict__ part_o,
                                                                          float* __restrict__ part_ml, int heads, int rank, int rot, int page_size,
                                                                          long long page_stride, int num_pages, int splits, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    const int D = rank + rot, D16 = (D + 15) / 16 * 16, DS = D16 + 8;           // row stride in elements: 16 bytes past a multiple of 32
    bf16* Qs = reinterpret_cast<bf16*>(smem);
    bf16* Ks = Qs + 16 * DS;
    bf16* Ps = Ks + KT * DS;
    float* red_max = reinterpret_cast<float*>(Ps + 16 * (KT + 8));
    float* red_sum = red_max + WARPS * 16;
    const int t = blockIdx.x, head0 = blockIdx.y * 16, part = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int last = positions[t];
    const int tiles = last / KT + 1, per = (tiles + splits - 1) / splits;
    const int tile0 = part * per, tile1 = min(tiles, tile0 + per);
    const int* table = block_table + (size_t)token_seq[t] * table_stride;

    // queries (zero rows for heads past the last one, zero columns past D), and the key tile's padding columns
    for (int i = threadIdx.x; i < 16 * (D / 8); i += blockDim.x) {          // 16 bytes a load
        const int h = i / (D / 8), c = i % (D / 8);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (head0 + h < heads) v = *reinterpret_cast<const uint4*>(qa + ((size_t)t * heads + head0 + h) * D + c * 8);
        *reinterpret_cast<uint4*>(Qs + h * DS + c * 8) = v;
    }
    for (int i = threadIdx.x; i < 16 * (DS - D); i += blockDim.x) Qs[(i / (DS - D)) * DS + D + i % (DS - D)] = __float2bfloat16(0.f);
    for (int i = threadIdx.x; i < KT * (DS - D); i += blockDim.x) Ks[(i / (DS - D)) * DS + D + i % (DS - D)] = __float2bfloat16(0.f);

    float o[PAIRS][2][4];
#pragma unroll
    for (int i = 0; i < PAIRS; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) o[i][j][k] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};      // rows lane / 4 and lane / 4 + 8
    const int chunks = D / 8;                                               // 16-byte pieces of a cached row
    const uint32_t row_bytes = (uint32_t)D * 2;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    for (int tile = tile0; tile < tile1; ++tile) {
        const int j0 = tile * KT;
        const int valid_rows = min(KT, last - j0 + 1);
        if (warp == 0) {
            // the buffer was last touched by ldmatrix and plain stores: order them before the copies that overwrite it
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            if (lane == 0) mbar_expect_tx(&bar, (uint32_t)valid_rows * row_bytes);
            __syncwarp();
            for (int r = lane; r < valid_rows; r += 32) {
                const int j = j0 + r, page = table[j / page_size];
                if (page < 0 || page >= num_pages) {             // a complaint, and the row's bytes from a page that exists
                    atomicOr(status, EG_STATUS_BAD_PAGE);
                }
                const int safe = (page < 0 || page >= num_pages) ? 0 : page;
                const bf16* src = cache + (size_t)safe * page_stride + (size_t)(j % page_size) * D;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_addr(Ks + r * DS)),
                             "l"(src), "r"(row_bytes), "r"(smem_addr(&bar))
                             : "memory");
            }
        } else {
            for (int i = threadIdx.x - 32; i < (KT - valid_rows) * chunks; i += blockDim.x - 32)      // rows past the token's position: zeros
                *reinterpret_cast<uint4*>(Ks + (valid_rows + i / chunks) * DS + (i % chunks) * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        if (!mbar_wait_bounded(&bar, (uint32_t)((tile - tile0) & 1), &abort_flag, status, 1u << 24)) break;
        __syncthreads();

        // scores of this warp's 16 keys for the 16 heads
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const bf16* a_at = Qs + (lane % 16) * DS + (lane / 16) * 8;
        const bf16* b_at = Ks + (warp * 16 + (lane % 8) + (lane / 16) * 8) * DS + ((lane / 8) % 2) * 8;
        for (int k0 = 0; k0 < D16; k0 += 16) {
            uint32_t a[4], b[4];
            ldmatrix_x4(a, a_at + k0);
            ldmatrix_x4(b, b_at + k0);
            mma_bf16_16816(s[0], a, b[0], b[1]);
            mma_bf16_16816(s[1], a, b[2], b[3]);
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + warp * 16 + i * 8 + 2 * (lane % 4) + (e & 1);
                if (j > last) s[i][e] = -INFINITY;
                tile_max[e >> 1] = fmaxf(tile_max[e >> 1], s[i][e]);
            }
        tile_max[0] = quad_max(tile_max[0]);
        tile_max[1] = quad_max(tile_max[1]);
        if (lane % 4 == 0) {
            red_max[warp * 16 + lane / 4] = tile_max[0];
            red_max[warp * 16 + lane / 4 + 8] = tile_max[1];
        }
        __syncthreads();
        float m_new[2], alpha[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float m = m_run[r];
#pragma unroll
            for (int w = 0; w < WARPS; ++w) m = fmaxf(m, red_max[w * 16 + lane / 4 + 8 * r]);
            m_new[r] = m;
            alpha[r] = m == -INFINITY ? 1.f : expf(m_run[r] - m);          // exp(-inf) = 0 at the first keys
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const float p = m_new[r] == -INFINITY ? 0.f : expf(s[i][e] - m_new[r]);
                s[i][e] = p;
                row_sum[r] += p;
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int col = warp * 16 + i * 8 + 2 * (lane % 4);
            *reinterpret_cast<uint32_t*>(Ps + (lane / 4) * (KT + 8) + col) = pack_bf16(s[i][0], s[i][1]);
            *reinterpret_cast<uint32_t*>(Ps + (lane / 4 + 8) * (KT + 8) + col) = pack_bf16(s[i][2], s[i][3]);
        }
        row_sum[0] = quad_sum(row_sum[0]);
        row_sum[1] = quad_sum(row_sum[1]);
        if (lane % 4 == 0) {
            red_sum[warp * 16 + lane / 4] = row_sum[0];
            red_sum[warp * 16 + lane / 4 + 8] = row_sum[1];
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) sum += red_sum[w * 16 + lane / 4 + 8 * r];
            l_run[r] = l_run[r] * alpha[r] + sum;
            m_run[r] = m_new[r];
        }
        // weighted sums: this warp's value columns 16 (warp + 4 i) .. + 15 over the tile's 64 keys
#pragma unroll
        for (int i = 0; i < PAIRS; ++i)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                o[i][j][0] *= alpha[0];
                o[i][j][1] *= alpha[0];
                o[i][j][2] *= alpha[1];
                o[i][j][3] *= alpha[1];
            }
        const bf16* p_at = Ps + (lane % 16) * (KT + 8) + (lane / 16) * 8;
        const bf16* v_at = Ks + ((lane % 8) + ((lane / 8) % 2) * 8) * DS + (lane / 16) * 8;
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(a, p_at + kk * 16);
#pragma unroll
            for (int i = 0; i < PAIRS; ++i) {
                const int col = 16 * (warp + WARPS * i);
                if (col < rank) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, v_at + (size_t)kk * 16 * DS + col);
                    mma_bf16_16816(o[i][0], a, b[0], b[1]);
                    mma_bf16_16816(o[i][1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                                    // the next tile overwrites the keys and the weights
    }

    if (abort_flag) return;                                                 // a wait gave up: the status word says so, nothing is written
    // a thread holds, per pair of column tiles, rows lane / 4 (values 0, 1) and lane / 4 + 8 (values 2, 3), columns 2 (lane % 4) + {0, 1}
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int head = head0 + lane / 4 + 8 * r;
        if (head >= heads) continue;
        const size_t row = (size_t)t * heads + head;
        float scale;
        if (splits == 1) {
            const float sk = sink ? sink[head] : -INFINITY;
            const float top = fmaxf(m_run[r], sk);
            const float f = m_run[r] == -INFINITY ? 0.f : expf(m_run[r] - top);
            const float denom = l_run[r] * f + (sink ? expf(sk - top) : 0.f);
            scale = f / denom;
        } else {
            scale = 1.f;
            if (lane % 4 == 0) {
                part_ml[(row * splits + part) * 2] = m_run[r];
                part_ml[(row * splits + part) * 2 + 1] = l_run[r];
            }
        }
#pragma unroll
        for (int i = 0; i < PAIRS; ++i)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int col = 16 * (warp + WARPS * i) + 8 * j + 2 * (lane % 4);
                if (col >= rank) continue;
                const float v0 = o[i][j][2 * r] * scale, v1 = o[i][j][2 * r + 1] * scale;
                if (splits == 1) *reinterpret_cast<uint32_t*>(out + row * rank + col) = pack_bf16(v0, v1);
                else *reinterpret_cast<float2*>(part_o + (row * splits + part) * rank + col) = make_float2(v0, v1);
            }
    }
}

// one block per (token, head): the parts' maxima, sums and weighted sums and the sink become the output row.  The parts'
// factors are worked out once, side by side (a thread per part), before the row is summed.
__global__ void attention_latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sink,
                                              bf16* __restrict__ out, int heads, int rank, int splits) {
    __shared__ float factor[64];
    __shared__ float inv_denom;
    const size_t row = blockIdx.x;
    const int head = (int)(row % heads);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m[2], l[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int s = lane + 32 * q;
            m[q] = s < splits ? part_ml[(row * splits + s) * 2] : -INFINITY;
            l[q] = s < splits ? part_ml[(row * splits + s) * 2 + 1] : 0.f;
        }
        const float sk = sink ? sink[head] : -INFINITY;
        const float top = fmaxf(sk, warp_max(fmaxf(m[0], m[1])));
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const float f = m[q] == -INFINITY ? 0.f : expf(m[q] - top);
            factor[lane + 32 * q] = f;
            sum += l[q] * f;
        }
        sum = warp_sum(sum) + (sink ? expf(sk - top) : 0.f);
        if (lane == 0) inv_denom = 1.0f / sum;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v = fmaf(part_o[(row * splits + s) * rank + d], factor[s], v);
        out[row * rank + d] = __float2bfloat16_rn(v * inv_denom);
    }
}

// one thread per (token, head, pair): the rotated part of the query, scaled, into qa [T, heads, rank + rot]
__global__ void latent_rotate_query_kernel(const bf16* __restrict__ q, long long ldq, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                           int rot_dims, float scale, bf16* __restrict__ qa, int tokens, int heads, int dim, int rot, int rank) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int half = (rot + 1) / 2;
    if (i >= (long long)tokens * heads * half) return;
    const int pair = (int)(i % half), h = (int)((i / half) % heads), t = (int)(i / ((long long)half * heads));
    const bf16* src = q + (size_t)t * ldq + (size_t)h * (dim + rot) + dim;
    bf16* dst = qa + ((size_t)t * heads + h) * (rank + rot) + rank;
    const int d = 2 * pair;
    if (d + 1 < rot_dims + 1 && d < rot_dims) {
        float sn, cs;
        sincosf((float)positions[t] * inv_freq[pair], &sn, &cs);
        const float a = __bfloat162float(src[d]), b = __bfloat162float(src[d + 1]);
        dst[d] = __float2bfloat16_rn((a * cs - b * sn) * scale);
        dst[d + 1] = __float2bfloat16_rn((b * cs + a * sn) * scale);
    } else {
        dst[d] = __float2bfloat16_rn(__bfloat162float(src[d]) * scale);
        if (d + 1 < rot) dst[d + 1] = __float2bfloat16_rn(__bfloat162float(src[d + 1]) * scale);
    }
}
}  // namespace

// whether eg_attention_latent_mma takes these sizes
EG_API int eg_attention_latent_mma_takes(int rank, int rot) {
    const int D = rank + rot, DS = (D + 15) / 16 * 16 + 8;
    const size_t smem = (size_t)(16 + KT) * DS * 2 + 16 * (KT + 8) * 2 + 2 * WARPS * 16 * 4;
    return D % 8 == 0 && rank % 8 == 0 && rank > 0 && rank <= 16 * WARPS * PAIRS && smem <= 200 * 1024;
}

// qa [T, heads, rank + rot] bfloat16 (scaled, rotated); cache rows bfloat16; out [T, heads, rank] bfloat16.  splits > 1:
// part_o [T, heads, splits, rank] and part_ml [T, heads, splits, 2] float32 scratch.  sink [heads] float32 or null.
EG_API int eg_attention_latent_mma(cudaStream_t stream, const void* qa, const void* cache, const int* block_table, int table_stride, const int* token_seq,
                                   const int* positions, const float* sink, void* out, float* part_o, float* part_ml, int tokens, int heads, int rank, int rot,
                                   int page_size, long long page_stride, int num_pages, int splits, int* status) {
    if (tokens <= 0) return 0;
    if (!eg_attention_latent_mma_takes(rank, rot) || splits < 1 || splits > 64 || (splits > 1 && (!part_o || !part_ml)) || page_stride % 8 || (uintptr_t)cache % 16 || (uintptr_t)qa % 16)
        return (int)cudaErrorInvalidValue;
    const int D = rank + rot, DS = (D + 15) / 16 * 16 + 8;
    const size_t smem = (size_t)(16 + KT) * DS * 2 + 16 * (KT + 8) * 2 + 2 * WARPS * 16 * 4;
    static size_t configured = 0;
    if (smem > configured) {
        const cudaError_t e = cudaFuncSetAttribute(attention_latent_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    dim3 grid(tokens, (heads + 15) / 16, splits);
    attention_latent_mma_kernel<<<grid, WARPS * 32, smem, stream>>>((const bf16*)qa, (const bf16*)cache, block_table, table_stride, token_seq, positions, sink,
                                                                     (bf16*)out, part_o, part_ml, heads, rank, rot, page_size, page_stride, num_pages, splits, status);
    if (splits > 1)
        attention_latent_merge_kernel<<<tokens * heads, 128, 0, stream>>>(part_o, part_ml, sink, (bf16*)out, heads, rank, splits);
    return eg_launch_status();
}

// the rotated, scaled part of the queries: qa[t, h, rank:] from q [T, ldq] (head by head: dim plain values, rot rotated ones)
EG_API int eg_latent_rotate_query(cudaStream_t stream, const void* q, long long ldq, const int* positions, const float* inv_freq, int rot_dims, float scale,
                                  void* qa, int tokens, int heads, int dim, int rot, int rank) {
    const long long n = (long long)tokens * heads * ((rot + 1) / 2);
    if (n <= 0) return 0;
    if (rot_dims % 2 || rot_dims > rot) return (int)cudaErrorInvalidValue;
    latent_rotate_query_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const bf16*)q, ldq, positions, inv_freq, rot_dims, scale, (bf16*)qa, tokens, heads,
                                                                               dim, rot, rank);
    return eg_launch_status();
}
