// The kernels of a selective state-space mixer (a causal convolution per channel, input-dependent step sizes, and a
// diagonal linear recurrence per channel and state) over a mixed batch: every entry of the batch is a run of tokens of
// one request that continues from the request's state slot.
//
// Per request the slot holds, in float32: the last taps-1 inputs of the convolution [taps-1, channels], then the
// recurrent state S [channels, states].  A slot is zero when a request first takes it, which is the convolution's
// zeros before the sequence and S = 0.
//
//   u[t, c]  = silu(cb[c] + sum_j cw[c, j] * x[t - (taps-1) + j, c])            (the last tap weighs the current token)
//   dt[t, c] = softplus(db[c] + sum_r dw[c, r] * low[t, r])                     (float32)
//   S[c, n] <- exp(dt[t, c] * A[c, n]) * S[c, n] + dt[t, c] * u[t, c] * B[t, n] (float32)
//   y[t, c]  = (sum_n S[c, n] * C[t, n] + D[c] * u[t, c]) * silu(z[t, c])
//
// Decays, step sizes, exponentials and the state are float32 in both precisions; the convolution's inputs and outputs
// are in the compute dtype with float32 sums.
#include <algorithm>

#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// exp(a * b) for a * b <= 0, rounded to nearest in all but rare cases.  A state that decays slowly is multiplied by
// thousands of such factors in a row, so an error with a sign of its own (the hardware's 2^x approximation behind expf
// has one) adds up over a long sequence where errors of either sign would not: measured on a sequence of 1,100 tokens,
// the logits were 4e-5 of their spread away from a float64 computation with expf and 1e-5 with this.  The product's rounding error is carried into
// the reduced argument; e^r on |r| <= ln2 / 2 is 1 + r + r^2 P(r) with the last addition the only rounding that counts.
__device__ __forceinline__ float decay_factor(float a, float b) {
    const float x = a * b;
    const float x_lo = fmaf(a, b, -x);
    if (x < -104.0f) return 0.0f;
    const float k = rintf(x * 1.442695041f);
    float r = fmaf(k, -0.693145751953125f, x);          // ln 2 in two pieces: the first has few enough bits for k * it to be exact
    r = fmaf(k, -1.428606765330187e-06f, r);
    r += x_lo;
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float e = 1.0f + fmaf(r * r, p, r);
    const int ki = (int)k;                              // 2^k by exponent arithmetic; results below the normal range go through two steps
    if (ki >= -125) return __int_as_float(__float_as_int(e) + (ki << 23));
    return __int_as_float(__float_as_int(e) + ((ki + 100) << 23)) * 7.888609052210118e-31f;      // 2^-100
}

// one thread per (token, channel)
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ cw, const float* __restrict__ cb,
                                 const float* __restrict__ state, long long slot_floats, const int* __restrict__ token_seq,
                                 const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, T* __restrict__ u, long long ldu, int tokens,
                                 int channels, int taps) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * channels) return;
    const int t = (int)(i / channels), c = (int)(i % channels);
    const int seq = token_seq[t], start = seq_starts[seq];
    const float* past = state + (size_t)seq_slots[seq] * slot_floats;
    float acc = cb ? cb[c] : 0.0f;                          // a convolution without bias hands none
    for (int j = 0; j < taps; ++j) {
        const int src = t - (taps - 1) + j;
        // before the entry's first token: the request's earlier inputs, the newest of which is row taps-2 of the slot
        const float v = src >= start ? to_f32<T>(x[(size_t)src * ldx + c]) : past[(size_t)(taps - 1 + src - start) * channels + c];
        acc = fmaf(cw[(size_t)c * taps + j], v, acc);
    }
    u[(size_t)t * ldu + c] = from_f32<T>(silu_f(acc));
}

// float32 rows whose channels come in fours on 16-byte boundaries: a thread takes four channels of a token, every tap one
// 16-byte load; the sums run over the taps in the same order as above
__global__ void conv_silu_vec4_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ cw, const float* __restrict__ cb,
                                      const float* __restrict__ state, long long slot_floats, const int* __restrict__ token_seq,
                                      const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, float* __restrict__ u, long long ldu,
                                      int tokens, int channels, int taps) {
    const int quads = channels / 4;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * quads) return;
    const int t = (int)(i / quads), c = (int)(i % quads) * 4;
    const int seq = token_seq[t], start = seq_starts[seq];
    const float* past = state + (size_t)seq_slots[seq] * slot_floats;
    float acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] = cb ? cb[c + e] : 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int src = t - (taps - 1) + j;
        const float4 v = src >= start ? *reinterpret_cast<const float4*>(x + (size_t)src * ldx + c)
                                      : *reinterpret_cast<const float4*>(past + (size_t)(taps - 1 + src - start) * channels + c);
        acc[0] = fmaf(cw[(size_t)c * taps + j], v.x, acc[0]);
        acc[1] = fmaf(cw[(size_t)(c + 1) * taps + j], v.y, acc[1]);
        acc[2] = fmaf(cw[(size_t)(c + 2) * taps + j], v.z, acc[2]);
        acc[3] = fmaf(cw[(size_t)(c + 3) * taps + j], v.w, acc[3]);
    }
    *reinterpret_cast<float4*>(u + (size_t)t * ldu + c) = make_float4(silu_f(acc[0]), silu_f(acc[1]), silu_f(acc[2]), silu_f(acc[3]));
}

// one thread per (entry, channel): the slot's rows become the last taps-1 inputs of the request after this step
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, long long ldx, float* __restrict__ state, long long slot_floats,
                                  const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, int num_seqs, int channels, int taps) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)num_seqs * channels) return;
    const int seq = (int)(i / channels), c = (int)(i % channels);
    const int start = seq_starts[seq], n = seq_starts[seq + 1] - start;
    float* past = state + (size_t)seq_slots[seq] * slot_floats;
    for (int r = 0; r < taps - 1; ++r) {                    // ascending: row r + n is read before any row >= r + 1 is written
        const int src = n - (taps - 1) + r;
        past[(size_t)r * channels + c] = src >= 0 ? to_f32<T>(x[(size_t)(start + src) * ldx + c]) : past[(size_t)(r + n) * channels + c];
    }
}

// one thread per (token, channel); low [tokens, ldl] float32, dw [channels, rank] float32
__global__ void step_size_kernel(const float* __restrict__ low, long long ldl, const float* __restrict__ dw, const float* __restrict__ db,
                                 float* __restrict__ dt, int tokens, int channels, int rank) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * channels) return;
    const int t = (int)(i / channels), c = (int)(i % channels);
    float acc = db[c];
    for (int r = 0; r < rank; ++r) acc = fmaf(dw[(size_t)c * rank + r], low[(size_t)t * ldl + r], acc);
    dt[i] = softplus_f(acc);
}

// The recurrence.  `lanes` threads share a channel; a thread keeps SPL states (n = lane + lanes * k) in registers for the
// whole run of tokens, so that a step costs its exponentials and two fused multiply-adds per state, and the sum over the
// states is a few shuffle steps.  A block covers blockDim.x / lanes channels of one entry and walks the entry's tokens in
// tiles: the block first brings a tile's step sizes (bias and softplus applied here, once per token and channel), inputs,
// gates and the tokens' B and C rows to shared memory with coalesced loads that are all in flight together, then runs the
// tile's steps out of shared memory, and writes the tile's outputs back in rows.  (Read straight from global memory, a
// step waited for its loads: 2,048 tokens of 4,096 channels with 16 states took 4.3 ms.)
template <typename T, int SPL>
__global__ void __launch_bounds__(128) selective_scan_kernel(const T* __restrict__ u, long long ldu, const float* __restrict__ dt,
                                                             const float* __restrict__ dt_bias, const float* __restrict__ low, long long ldl, int b_col,
                                                             int c_col, const float* __restrict__ A, const float* __restrict__ D, const T* __restrict__ z,
                                                             long long ldz, float* __restrict__ state, long long slot_floats, long long state_offset,
                                                             const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, T* __restrict__ y,
                                                             long long ldy, int channels, int states, int lanes, int tile_tokens) {
    extern __shared__ float tile[];
    const int per_block = blockDim.x / lanes;                   // channels of this block
    float* s_dt = tile;                                         // [tile_tokens, per_block] each
    float* s_u = s_dt + tile_tokens * per_block;
    float* s_z = s_u + tile_tokens * per_block;
    float* s_y = s_z + tile_tokens * per_block;
    float* s_b = s_y + tile_tokens * per_block;                 // [tile_tokens, states] each
    float* s_c = s_b + tile_tokens * states;
    const int seq = blockIdx.y;
    const int lane = threadIdx.x % lanes, local = threadIdx.x / lanes;
    const int c0 = blockIdx.x * per_block, c = c0 + local;
    const bool live = c < channels;
    const int cc = live ? c : channels - 1;
    float* S = state + (size_t)seq_slots[seq] * slot_floats + state_offset + (size_t)cc * states;
    float s[SPL], a[SPL];
#pragma unroll
    for (int k = 0; k < SPL; ++k) {
        const int n = lane + lanes * k;
        s[k] = n < states ? S[n] : 0.f;
        a[k] = n < states ? A[(size_t)cc * states + n] : 0.f;
    }
    const int t0 = seq_starts[seq], t1 = seq_starts[seq + 1];
    // A tile's values travel global memory -> registers -> shared memory; the loads of the next tile are issued before
    // the steps of this one, so their latency passes behind the recurrence.  (A tile has at most FETCH * 128 values of a
    // kind: the launcher sizes it so.)
    constexpr int FETCH = 4;
    float r_dt[FETCH], r_u[FETCH], r_z[FETCH], r_b[FETCH], r_c[FETCH];
    auto fetch = [&](int base) {
        const int count = min(tile_tokens, t1 - base);
#pragma unroll
        for (int q = 0; q < FETCH; ++q) {
            const int i = threadIdx.x + q * 128;
            if (i < count * per_block) {
                const int tt = i / per_block, ch = min(c0 + i % per_block, channels - 1);
                const size_t t = (size_t)(base + tt);
                r_dt[q] = dt[t * channels + ch];
                r_u[q] = to_f32<T>(u[t * ldu + ch]);
                r_z[q] = to_f32<T>(z[t * ldz + ch]);
            }
            if (i < count * states) {
                const size_t t = (size_t)(base + i / states);
                r_b[q] = low[t * ldl + b_col + i % states];
                r_c[q] = low[t * ldl + c_col + i % states];
            }
        }
    };
    if (t0 < t1) fetch(t0);
    for (int base = t0; base < t1; base += tile_tokens) {
        const int count = min(tile_tokens, t1 - base);
#pragma unroll
        for (int q = 0; q < FETCH; ++q) {
            const int i = threadIdx.x + q * 128;
            if (i < count * per_block) {
                float step = r_dt[q];
                if (dt_bias) step = softplus_f(step + dt_bias[min(c0 + i % per_block, channels - 1)]);   // dt held the projection alone
                s_dt[i] = step;
                s_u[i] = r_u[q];
                s_z[i] = r_z[q];
            }
            if (i < count * states) {
                s_b[i] = r_b[q];
                s_c[i] = r_c[q];
            }
        }
        __syncthreads();
        if (base + tile_tokens < t1) fetch(base + tile_tokens);
        // U steps at a time: their decay factors, drives and C values do not depend on the state, so they are computed
        // side by side; what remains in sequence per step is one fused multiply-add per state.  The sums over the states
        // of the U steps are reduced together, and the skip term and the gate wait for the tile's write-back.
        constexpr int U = SPL <= 2 ? 4 : SPL <= 4 ? 2 : 1;
        for (int tt0 = 0; tt0 < count; tt0 += U) {
            float dec[U][SPL], drv[U][SPL], cv[U][SPL], part[U];
#pragma unroll
            for (int q = 0; q < U; ++q) {
                const int tt = min(tt0 + q, count - 1);
                const float step = s_dt[tt * per_block + local], drive = step * s_u[tt * per_block + local];
#pragma unroll
                for (int k = 0; k < SPL; ++k) {
                    const int n = min(lane + lanes * k, states - 1);
                    dec[q][k] = decay_factor(step, a[k]);
                    drv[q][k] = drive * s_b[tt * states + n];
                    cv[q][k] = lane + lanes * k < states ? s_c[tt * states + n] : 0.f;
                }
            }
#pragma unroll
            for (int q = 0; q < U; ++q) {
                part[q] = 0.f;
                if (tt0 + q < count) {
#pragma unroll
                    for (int k = 0; k < SPL; ++k) {
                        s[k] = fmaf(dec[q][k], s[k], drv[q][k]);
                        part[q] = fmaf(s[k], cv[q][k], part[q]);
                    }
                }
            }
            for (int o = lanes >> 1; o > 0; o >>= 1)
#pragma unroll
                for (int q = 0; q < U; ++q) part[q] += __shfl_xor_sync(0xffffffffu, part[q], o);
            if (lane == 0)
#pragma unroll
                for (int q = 0; q < U; ++q)
                    if (tt0 + q < count) s_y[(tt0 + q) * per_block + local] = part[q];
        }
        __syncthreads();
        for (int i = threadIdx.x; i < count * per_block; i += blockDim.x) {
            const int ch = c0 + i % per_block;
            if (ch < channels) y[(size_t)(base + i / per_block) * ldy + ch] = from_f32<T>((s_y[i] + D[ch] * s_u[i]) * silu_f(s_z[i]));
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int k = 0; k < SPL; ++k) {
            const int n = lane + lanes * k;
            if (n < states) S[n] = s[k];
        }
    }
}

template <typename T, int SPL>
void launch_scan(cudaStream_t stream, const void* u, long long ldu, const float* dt, const float* dt_bias, const float* low, long long ldl, int b_col, int c_col,
                 const float* A, const float* D, const void* z, long long ldz, float* state, long long slot_floats, long long state_offset,
                 const int* seq_starts, const int* seq_slots, void* y, long long ldy, int num_seqs, int channels, int states, int lanes) {
    const int per_block = 128 / lanes;
    // a tile: up to 32 tokens, and no more than 512 values of a kind (a thread fetches four of each ahead)
    const size_t per_token = (size_t)(4 * per_block + 2 * states) * sizeof(float);
    const int tile_tokens = std::max(1, std::min({32, 512 / per_block, 512 / states}));
    dim3 grid((channels + per_block - 1) / per_block, num_seqs);
    selective_scan_kernel<T, SPL><<<grid, 128, tile_tokens * per_token, stream>>>((const T*)u, ldu, dt, dt_bias, low, ldl, b_col, c_col, A, D, (const T*)z, ldz, state,
                                                                                 slot_floats, state_offset, seq_starts, seq_slots, (T*)y, ldy, channels, states,
                                                                                 lanes, tile_tokens);
}

}  // namespace

// u[t, c] = silu(conv(x)) for every token of the batch, reading what lies before an entry from the request's slot.
// The slots are not changed: eg_conv_state does that afterwards.
EG_API int eg_conv_silu(cudaStream_t stream, int dtype, const void* x, long long ldx, const float* conv_w, const float* conv_b, const float* state,
                        long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* u, long long ldu, int tokens,
                        int channels, int taps) {
    const long long n = (long long)tokens * channels;
    if (n <= 0) return 0;
    if (taps < 1) return (int)cudaErrorInvalidValue;
    if (dtype == EG_F32 && channels % 4 == 0 && ldx % 4 == 0 && ldu % 4 == 0 && slot_floats % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)u % 16 == 0 &&
        (uintptr_t)state % 16 == 0) {
        conv_silu_vec4_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, stream>>>((const float*)x, ldx, conv_w, conv_b, state, slot_floats, token_seq,
                                                                                 seq_starts, seq_slots, (float*)u, ldu, tokens, channels, taps);
        return eg_launch_status();
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == EG_BF16)
        conv_silu_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)x, ldx, conv_w, conv_b, state, slot_floats, token_seq, seq_starts, seq_slots, (bf16*)u,
                                                          ldu, tokens, channels, taps);
    else
        conv_silu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, ldx, conv_w, conv_b, state, slot_floats, token_seq, seq_starts, seq_slots,
                                                           (float*)u, ldu, tokens, channels, taps);
    return eg_launch_status();
}

// the slots' convolution rows after this step's tokens
EG_API int eg_conv_state(cudaStream_t stream, int dtype, const void* x, long long ldx, float* state, long long slot_floats, const int* seq_starts,
                         const int* seq_slots, int num_seqs, int channels, int taps) {
    const long long n = (long long)num_seqs * channels;
    if (n <= 0 || taps <= 1) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == EG_BF16) conv_state_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)x, ldx, state, slot_floats, seq_starts, seq_slots, num_seqs, channels, taps);
    else conv_state_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, ldx, state, slot_floats, seq_starts, seq_slots, num_seqs, channels, taps);
    return eg_launch_status();
}

// dt [tokens, channels] float32 = softplus(low[:, :rank] dw^T + db)
EG_API int eg_step_sizes(cudaStream_t stream, const float* low, long long ldl, const float* dw, const float* db, float* dt, int tokens, int channels,
                         int rank) {
    const long long n = (long long)tokens * channels;
    if (n <= 0) return 0;
    step_size_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(low, ldl, dw, db, dt, tokens, channels, rank);
    return eg_launch_status();
}

// The recurrence over every entry's tokens, from and back into the slots' states, and the gated output y.
// dt_bias null: dt holds the step sizes.  Otherwise dt holds their projection alone and the step size is
// softplus(dt + dt_bias[c]) (the projection then came from a matrix product, and this kernel finishes it).
// states_per_lane: 1, 2, 4, 8, 16 or 32 (how many states a thread keeps; fewer means more threads per channel).
EG_API int eg_selective_scan(cudaStream_t stream, int dtype, const void* u, long long ldu, const float* dt, const float* dt_bias, const float* low,
                             long long ldl, int b_col, int c_col, const float* A, const float* D, const void* z, long long ldz, float* state, long long slot_floats,
                             long long state_offset, const int* seq_starts, const int* seq_slots, void* y, long long ldy, int num_seqs, int channels,
                             int states, int states_per_lane) {
    if (num_seqs <= 0 || channels <= 0) return 0;
    if (states <= 0 || states > 512) return (int)cudaErrorInvalidValue;
    int spl = states_per_lane;
    while ((states + spl - 1) / spl > 32) spl *= 2;
    if (spl > 32) return (int)cudaErrorInvalidValue;
    int lanes = 1;
    while (lanes * spl < states) lanes <<= 1;
#define EG_SCAN(T, S) \
    launch_scan<T, S>(stream, u, ldu, dt, dt_bias, low, ldl, b_col, c_col, A, D, z, ldz, state, slot_floats, state_offset, seq_starts, seq_slots, y, ldy, num_seqs, \
                      channels, states, lanes)
#define EG_SCAN_T(T)                      \
    switch (spl) {                        \
        case 1: EG_SCAN(T, 1); break;     \
        case 2: EG_SCAN(T, 2); break;     \
        case 4: EG_SCAN(T, 4); break;     \
        case 8: EG_SCAN(T, 8); break;     \
        case 16: EG_SCAN(T, 16); break;   \
        case 32: EG_SCAN(T, 32); break;   \
        default: return (int)cudaErrorInvalidValue; \
    }
    if (dtype == EG_BF16) { EG_SCAN_T(bf16) } else { EG_SCAN_T(float) }
#undef EG_SCAN_T
#undef EG_SCAN
    return eg_launch_status();
}
