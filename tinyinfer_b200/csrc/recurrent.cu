// A gated diagonal linear recurrence with a short causal convolution in front of it (the recurrent block of
// Griffin: "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models",
// De, Smith et al., 2024). Per request the state is, per channel, the recurrence's S (float32) and the last
// taps - 1 inputs of the convolution; a request's slot holds [S | inputs] as float32 [taps][width] (row 0: S,
// rows 1..taps-1: the inputs, oldest first), zero when the request starts.
//
//   causal_conv : u[t][c] = bias[c] + sum_k w[c][k] * in[t - (taps-1-k)][c]; inputs before the step's first token
//                 come from the slot, inputs before the request's start are zero (the slot was zeroed)
//   gated_scan  : a = exp(-decay * r * softplus(lam)), S <- a S + sqrt(1 - a^2) * (i * u), out = S * gelu_tanh(y)
//                 over a request's tokens of this step in order (in stretches that are scanned side by side and
//                 joined), then S and the convolution's newest inputs go back into the slot
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

// A block is 32 channels x 32 stretches of a request's tokens of this step. A recurrence S <- a S + b composes:
// a stretch is (A, B) = (product of its a, its own scan from zero), so the stretches are scanned side by side, their
// (A, B) folded in order by the first row of threads, and each stretch scanned again from its true start to write the
// outputs. A step of single decoded tokens is launched with one stretch (blockDim.y = 1).
constexpr int GS_CH = 32, GS_PARTS = 32;

template <typename T>
__global__ void __launch_bounds__(GS_CH * GS_PARTS) gated_scan_kernel(
    T* __restrict__ out, float* __restrict__ state, const T* __restrict__ u, const float* __restrict__ gates,
    const T* __restrict__ yx, int ld_yx, int y_off, int x_off, const float* __restrict__ lam,
    const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int width, int block_width, int taps, float decay) {
    __shared__ float prod[GS_PARTS][GS_CH + 1], own[GS_PARTS][GS_CH + 1], start[GS_PARTS][GS_CH + 1];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int seq = blockIdx.y;
    const int cx = threadIdx.x, part = threadIdx.y;
    const int c = blockIdx.x * GS_CH + cx;
    const bool live = c < width;
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];
    const int n = row1 - row0;
    const int parts = blockDim.y;
    const int len = (n + parts - 1) / parts;
    const int t0 = min(row1, row0 + part * len), t1 = min(row1, t0 + len);
    float* slot = state + (size_t)state_slots[seq] * taps * width;
    size_t g_off = 0;
    float rate = 0.f;
    if (live) {
        const int blk = c / block_width, o = c % block_width;
        g_off = (size_t)blk * 2 * block_width + o;              // r; i lies block_width further on
        rate = decay * rc_softplus(lam[c]);
    }
    auto terms = [&](int t, float& a, float& b) {
        const float r = gates[(size_t)t * 2 * width + g_off];
        const float g = gates[(size_t)t * 2 * width + g_off + block_width];
        const float log_a = -rate * r;
        a = expf(log_a);
        const float mult = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f));       // sqrt(1 - a^2) without the cancellation
        b = mult * (g * to_f32(u[(size_t)t * width + c]));
    };
    float A = 1.f, B = 0.f;
    if (live) {
#pragma unroll 4
        for (int t = t0; t < t1; ++t) {
            float a, b;
            terms(t, a, b);
            B = fmaf(a, B, b);
            A *= a;
        }
    }
    prod[part][cx] = A;
    own[part][cx] = B;
    __syncthreads();
    if (part == 0 && live) {
        float S = slot[c];
        for (int k = 0; k < parts; ++k) {
            start[k][cx] = S;
            S = fmaf(prod[k][cx], S, own[k][cx]);
        }
        slot[c] = S;
    }
    __syncthreads();
    if (!live) return;
    float S = start[part][cx];
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        float a, b;
        terms(t, a, b);
        S = fmaf(a, S, b);
        const float y = rc_gelu_tanh(to_f32(yx[(size_t)t * ld_yx + y_off + c]));
        out[(size_t)t * width + c] = from_f32<T>(S * y);
    }
    if (part != 0) return;
    // the convolution's last taps - 1 inputs: from this step's rows, or, where the step was shorter, moved up
    const int keep = taps - 1;
    float fresh[RC_MAX_TAPS];
    for (int j = 0; j < keep; ++j) {
        const int idx = n - keep + j;                  // local index of the input that becomes entry j
        fresh[j] = idx >= 0 ? to_f32(yx[(size_t)(row0 + idx) * ld_yx + x_off + c])
                            : slot[(size_t)(1 + keep + idx) * width + c];
    }
    for (int j = 0; j < keep; ++j) slot[(size_t)(1 + j) * width + c] = fresh[j];
}

TI_API int ti_gated_scan(void* out, float* state, const void* u, const float* gates, const void* yx, int ld_yx, int y_off,
                         int x_off, const float* lam, const int* cu_seqlens, const int* state_slots, int num_seqs, int num_tokens,
                         int width, int block_width, int taps, float decay, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_seqs >= 0 && width > 0 && block_width > 0 && width % block_width == 0, "gated_scan: bad sizes");
    TI_REQUIRE(taps >= 1 && taps <= RC_MAX_TAPS, "gated_scan: taps must be 1..%d", RC_MAX_TAPS);
    TI_REQUIRE(num_seqs <= 65535, "gated_scan: too many requests");
    if (num_seqs == 0) return 0;
    dim3 grid((width + GS_CH - 1) / GS_CH, num_seqs), block(GS_CH, num_tokens == num_seqs ? 1 : GS_PARTS);
    if (dtype == TI_F32)
        ti_launch(gated_scan_kernel<float>, grid, block, 0, stream, (float*)out, state, (const float*)u, gates, (const float*)yx,
                  ld_yx, y_off, x_off, lam, cu_seqlens, state_slots, width, block_width, taps, decay);
    else if (dtype == TI_BF16)
        ti_launch(gated_scan_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)out, state, (const __nv_bfloat16*)u, gates,
                  (const __nv_bfloat16*)yx, ld_yx, y_off, x_off, lam, cu_seqlens, state_slots, width, block_width, taps, decay);
    else TI_REQUIRE(false, "gated_scan: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("gated_scan");
    return 0;
}
