// A gated diagonal linear recurrence with a short causal convolution in front of it (the recurrent block of
// Griffin: "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models",
// De, Smith et al., 2024). Per request the state is, per channel, the recurrence's S (float32) and the last
// taps - 1 inputs of the convolution; a request's slot holds [S | inputs] as float32 [taps][width] (row 0: S,
// rows 1..taps-1: the inputs, oldest first), zero when the request starts.
//
//   causal_conv : u[t][c] = bias[c] + sum_k w[c][k] * in[t - (taps-1-k)][c]; inputs before the step's first token
//                 come from the slot, inputs before the request's start are zero (the slot was zeroed)
//   gated_scan  : a = exp(-decay * r * softplus(lam)), S <- a S + sqrt(1 - a^2) * (i * u), out = S * gelu_tanh(y);
//                 one thread per (request, channel) walks the request's tokens of this step in order, then stores S
//                 and the convolution's newest inputs back into the slot
// r, i: float32 gates [T][2 * width] laid out per block as [r of the block | i of the block]. Decays, their
// logarithms, softplus, exponentials and the state are float32; u, y and the output are in the compute dtype.
#include "common.cuh"

constexpr int RC_MAX_TAPS = 16;

template <typename T>
__global__ void causal_conv_kernel(T* __restrict__ u, const T* __restrict__ in, int ld_in, int in_off,
                                   const float* __restrict__ state, const float* __restrict__ w, const float* __restrict__ bias,
                                   const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ state_slots, int width, int taps) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int seq = token_seq[t];
    const int local = t - cu_seqlens[seq];              // tokens of this request before t in this step
    const float* hist = state + (size_t)state_slots[seq] * taps * width + width;     // [taps-1][width], oldest first
    float acc = bias ? bias[c] : 0.f;
    for (int k = 0; k < taps; ++k) {                    // column taps-1 is the current token's
        const int back = taps - 1 - k;
        float v;
        if (local - back >= 0) v = to_f32(in[(size_t)(t - back) * ld_in + in_off + c]);
        else v = hist[(size_t)(taps - 1 + local - back) * width + c];
        acc = fmaf(w[(size_t)c * taps + k], v, acc);
    }
    u[(size_t)t * width + c] = from_f32<T>(acc);
}

TI_API int ti_causal_conv(void* u, const void* in, int ld_in, int in_off, const float* state, const float* w, const float* bias,
                          const int* token_seq, const int* cu_seqlens, const int* state_slots, int num_tokens, int width,
                          int taps, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && width > 0 && taps >= 1 && taps <= RC_MAX_TAPS, "causal_conv: bad sizes (taps 1..%d)", RC_MAX_TAPS);
    TI_REQUIRE(num_tokens <= 65535, "causal_conv: more than 65535 tokens in one step");
    if (num_tokens == 0) return 0;
    dim3 grid((width + 127) / 128, num_tokens);
    if (dtype == TI_F32)
        ti_launch(causal_conv_kernel<float>, grid, 128, 0, stream, (float*)u, (const float*)in, ld_in, in_off, state, w, bias,
                  token_seq, cu_seqlens, state_slots, width, taps);
    else if (dtype == TI_BF16)
        ti_launch(causal_conv_kernel<__nv_bfloat16>, grid, 128, 0, stream, (__nv_bfloat16*)u, (const __nv_bfloat16*)in, ld_in,
                  in_off, state, w, bias, token_seq, cu_seqlens, state_slots, width, taps);
    else TI_REQUIRE(false, "causal_conv: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("causal_conv");
    return 0;
}

__device__ __forceinline__ float rc_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float rc_gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void gated_scan_kernel(T* __restrict__ out, float* __restrict__ state, const T* __restrict__ u,
                                  const float* __restrict__ gates, const T* __restrict__ yx, int ld_yx, int y_off, int x_off,
                                  const float* __restrict__ lam, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ state_slots, int width, int block_width, int taps, float decay) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];
    float* slot = state + (size_t)state_slots[seq] * taps * width;
    const int blk = c / block_width, o = c % block_width;
    const size_t g_off = (size_t)blk * 2 * block_width + o;      // r; i lies block_width further on
    const float rate = decay * rc_softplus(lam[c]);
    float S = slot[c];
    for (int t = row0; t < row1; ++t) {
        const float r = gates[(size_t)t * 2 * width + g_off];
        const float g = gates[(size_t)t * 2 * width + g_off + block_width];
        const float log_a = -rate * r;
        const float a = expf(log_a);
        const float mult = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f));       // sqrt(1 - a^2) without the cancellation
        S = fmaf(a, S, mult * (g * to_f32(u[(size_t)t * width + c])));
        const float y = rc_gelu_tanh(to_f32(yx[(size_t)t * ld_yx + y_off + c]));
        out[(size_t)t * width + c] = from_f32<T>(S * y);
    }
    slot[c] = S;
    // the convolution's last taps - 1 inputs: from this step's rows, or, where the step was shorter, moved up
    const int n = row1 - row0, keep = taps - 1;
    float fresh[RC_MAX_TAPS];
    for (int j = 0; j < keep; ++j) {
        const int idx = n - keep + j;                  // local index of the input that becomes entry j
        fresh[j] = idx >= 0 ? to_f32(yx[(size_t)(row0 + idx) * ld_yx + x_off + c])
                            : slot[(size_t)(1 + keep + idx) * width + c];
    }
    for (int j = 0; j < keep; ++j) slot[(size_t)(1 + j) * width + c] = fresh[j];
}

TI_API int ti_gated_scan(void* out, float* state, const void* u, const float* gates, const void* yx, int ld_yx, int y_off,
                         int x_off, const float* lam, const int* cu_seqlens, const int* state_slots, int num_seqs, int width,
                         int block_width, int taps, float decay, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_seqs >= 0 && width > 0 && block_width > 0 && width % block_width == 0, "gated_scan: bad sizes");
    TI_REQUIRE(taps >= 1 && taps <= RC_MAX_TAPS, "gated_scan: taps must be 1..%d", RC_MAX_TAPS);
    TI_REQUIRE(num_seqs <= 65535, "gated_scan: too many requests");
    if (num_seqs == 0) return 0;
    dim3 grid((width + 63) / 64, num_seqs);
    if (dtype == TI_F32)
        ti_launch(gated_scan_kernel<float>, grid, 64, 0, stream, (float*)out, state, (const float*)u, gates, (const float*)yx,
                  ld_yx, y_off, x_off, lam, cu_seqlens, state_slots, width, block_width, taps, decay);
    else if (dtype == TI_BF16)
        ti_launch(gated_scan_kernel<__nv_bfloat16>, grid, 64, 0, stream, (__nv_bfloat16*)out, state, (const __nv_bfloat16*)u, gates,
                  (const __nv_bfloat16*)yx, ld_yx, y_off, x_off, lam, cu_seqlens, state_slots, width, block_width, taps, decay);
    else TI_REQUIRE(false, "gated_scan: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("gated_scan");
    return 0;
}
