// A residual stream kept in float32 beside a copy in the compute dtype, for designs whose residual sum is
// 32-bit whatever the matrix products run in: the products read the copy, the sums go to the float32 rows.
//   embedding_scaled : x32 = table[id] * scale, copy = round(x32)
//   norm_add         : x32 += w * y * rsqrt(mean(y^2) + eps) (the norm sits on a sublayer's OUTPUT), copy = round(x32)
//   rmsnorm_rows32   : w * x32[rows] * rsqrt(mean(x32[rows]^2) + eps) in the compute dtype (the norm before the head)
// All arithmetic in float32; the copy is the only rounding. In a float32 model the copy is left out.
#include "common.cuh"

template <typename T>
__global__ void embedding_scaled_kernel(float* __restrict__ x32, T* __restrict__ copy, const T* __restrict__ table,
                                        const int* __restrict__ ids, int hidden, int vocab, float scale) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = ok ? to_f32(src[i]) * scale : 0.f;
        x32[(size_t)t * hidden + i] = v;
        if (copy) copy[(size_t)t * hidden + i] = from_f32<T>(v);
    }
}

TI_API int ti_embedding_scaled(float* x32, void* copy, const void* table, const int* ids, int num_tokens, int hidden,
                               int vocab, float scale, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && hidden > 0 && vocab > 0, "embedding_scaled: bad sizes");
    if (num_tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == TI_F32)
        ti_launch(embedding_scaled_kernel<float>, num_tokens, threads, 0, stream, x32, (float*)copy, (const float*)table, ids, hidden, vocab, scale);
    else if (dtype == TI_BF16)
        ti_launch(embedding_scaled_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, x32, (__nv_bfloat16*)copy, (const __nv_bfloat16*)table, ids, hidden, vocab, scale);
    else TI_REQUIRE(false, "embedding_scaled: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("embedding_scaled");
    return 0;
}

// One block per row. y is read once into shared memory (size floats), so the row may be any length that fits.
template <typename TY, typename TC>
__global__ void norm_add_kernel(float* __restrict__ x32, TC* __restrict__ copy, const TY* __restrict__ y,
                                const float* __restrict__ w, int size, float eps) {
    extern __shared__ float row[];
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t base = (size_t)blockIdx.x * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = to_f32(y[base + i]);
        row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = x32[base + i] + w[i] * row[i] * inv;
        x32[base + i] = v;
        if (copy) copy[base + i] = from_f32<TC>(v);
    }
}

// y_dtype: what the sublayer's output is stored in; copy_dtype: the compute dtype (copy may be null).
TI_API int ti_norm_add(float* x32, void* copy, const void* y, const float* weight, int num_rows, int size, float eps,
                       int y_dtype, int copy_dtype, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && size > 0 && size <= 48 * 1024 / 4, "norm_add: bad sizes");
    if (num_rows == 0) return 0;
    int threads = 32;
    while (threads < 512 && threads * 4 < size) threads <<= 1;
    const size_t smem = (size_t)size * sizeof(float);
    typedef __nv_bfloat16 B;
    if (y_dtype == TI_F32 && copy_dtype == TI_F32)
        ti_launch(norm_add_kernel<float, float>, num_rows, threads, smem, stream, x32, (float*)copy, (const float*)y, weight, size, eps);
    else if (y_dtype == TI_F32 && copy_dtype == TI_BF16)
        ti_launch(norm_add_kernel<float, B>, num_rows, threads, smem, stream, x32, (B*)copy, (const float*)y, weight, size, eps);
    else if (y_dtype == TI_BF16 && copy_dtype == TI_BF16)
        ti_launch(norm_add_kernel<B, B>, num_rows, threads, smem, stream, x32, (B*)copy, (const B*)y, weight, size, eps);
    else TI_REQUIRE(false, "norm_add: unsupported dtypes %d -> %d", y_dtype, copy_dtype);
    TI_CHECK_LAUNCH("norm_add");
    return 0;
}

template <typename T>
__global__ void rmsnorm_rows32_kernel(T* __restrict__ out, const float* __restrict__ x32, const float* __restrict__ w,
                                      const int* __restrict__ rows, int size, float eps) {
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int r = blockIdx.x;
    const float* src = x32 + (size_t)(rows ? rows[r] : r) * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) ss += src[i] * src[i];
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        out[(size_t)r * size + i] = from_f32<T>(w[i] * src[i] * inv);
}

TI_API int ti_rmsnorm_rows32(void* out, const float* x32, const float* weight, const int* rows, int num_rows, int size,
                             float eps, int out_dtype, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && size > 0, "rmsnorm_rows32: bad sizes");
    if (num_rows == 0) return 0;
    int threads = 32;
    while (threads < 512 && threads * 4 < size) threads <<= 1;
    if (out_dtype == TI_F32)
        ti_launch(rmsnorm_rows32_kernel<float>, num_rows, threads, 0, stream, (float*)out, x32, weight, rows, size, eps);
    else if (out_dtype == TI_BF16)
        ti_launch(rmsnorm_rows32_kernel<__nv_bfloat16>, num_rows, threads, 0, stream, (__nv_bfloat16*)out, x32, weight, rows, size, eps);
    else TI_REQUIRE(false, "rmsnorm_rows32: unknown dtype %d", out_dtype);
    TI_CHECK_LAUNCH("rmsnorm_rows32");
    return 0;
}

// max(v, 0)^2, the activation of a feed-forward whose up projection has no gate; float32 arithmetic, one rounding.
template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ out, const T* __restrict__ x, size_t n) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = fmaxf(to_f32(x[i]), 0.f);
        out[i] = from_f32<T>(v * v);
    }
}

TI_API int ti_relu_squared(void* out, const void* x, long long n, int dtype, cudaStream_t stream) {
    TI_REQUIRE(n >= 0, "relu_squared: bad size");
    if (n == 0) return 0;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == TI_F32)
        ti_launch(relu_squared_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)x, (size_t)n);
    else if (dtype == TI_BF16)
        ti_launch(relu_squared_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, (size_t)n);
    else TI_REQUIRE(false, "relu_squared: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("relu_squared");
    return 0;
}
