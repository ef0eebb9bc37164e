// Residual-stream kernels of decoders whose blocks scale what they add:
//
//   embed_gather_scaled   out[t,:] = table[id[t],:] * scale               (bad id -> NaN)
//   add_table_rows        x[t,:] += table[index[t],:]                     learned additive positions
//   add_scaled_rmsnorm    x[t,:] += s[:] * sum_k delta_k[t,:];  out[t,:] = x[t,:] / sqrt(mean(x^2) + eps) * w[:]
//   add_scaled_inplace    x[t,:] += s[:] * sum_k delta_k[t,:]
//   stream_entry          x[t,:] += (x0 ? x0[t,:] : 0) + v[:]             what a pass of looped layers adds first
//
// `s` is a per-column factor (a layer scale times the block's residual multiplier), null for none.  All sums are
// fp32; one block per row with a fixed number of threads, so that a row's result never depends on the batch.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int ROW_THREADS = 256;

template <typename TableT>
__global__ void embed_scaled_kernel(const TableT* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                    int tokens, int width, int vocab, float scale) {
    pdl_prologue();
    const int t = blockIdx.x;
    if (t >= tokens) return;
    const int id = ids[t];
    float* dst = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = nanf("");
        return;
    }
    const TableT* src = table + (size_t)id * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = to_f32(src[c]) * scale;
}

template <typename TableT>
__global__ void add_table_rows_kernel(float* __restrict__ x, const TableT* __restrict__ table, const int* __restrict__ index,
                                      int tokens, int width, int rows) {
    pdl_prologue();
    const int t = blockIdx.x;
    if (t >= tokens) return;
    const int r = index[t];
    float* dst = x + (size_t)t * width;
    if (r < 0 || r >= rows) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = nanf("");
        return;
    }
    const TableT* src = table + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] += to_f32(src[c]);
}

__device__ __forceinline__ float delta_sum(const float* delta, int n_delta, long long stride, size_t at) {
    float d = delta[at];
    for (int k = 1; k < n_delta; ++k) d += delta[(size_t)k * stride + at];
    return d;
}

template <typename OutT>
__global__ void __launch_bounds__(ROW_THREADS)
add_scaled_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta, long long delta_stride,
                          const float* __restrict__ col_scale, const float* __restrict__ weight, OutT* __restrict__ out,
                          int width, float eps) {
    pdl_prologue();
    __shared__ float scratch[32];
    const size_t row = (size_t)blockIdx.x * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
        float d = delta_sum(delta, n_delta, delta_stride, row + c);
        if (col_scale) d *= col_scale[c];
        const float v = x[row + c] + d;
        x[row + c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) out[row + c] = from_f32<OutT>(x[row + c] * inv * weight[c]);
}

__global__ void add_scaled_inplace_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta,
                                          long long delta_stride, const float* __restrict__ col_scale, int width, size_t n) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float d = delta_sum(delta, n_delta, delta_stride, i);
    if (col_scale) d *= col_scale[i % width];
    x[i] += d;
}

__global__ void stream_entry_kernel(float* __restrict__ x, const float* __restrict__ x0, const float* __restrict__ v,
                                    int width, size_t n) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a = x[i];
    if (x0) a += x0[i];
    x[i] = a + v[i % width];
}

}  // namespace

MLB_EXPORT int mlb_embed_gather_scaled(const void* table, int table_dtype, const int* ids, float* out, int tokens, int width,
                                       int vocab, float scale, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || vocab <= 0) return fail(MLB_INVALID_ARGUMENT, "embed_gather_scaled: bad sizes");
    if (tokens == 0) return MLB_OK;
    if (table_dtype == MLB_F32)
        launch_kernel(embed_scaled_kernel<float>, tokens, ROW_THREADS, 0, stream, (const float*)table, ids, out, tokens, width, vocab, scale);
    else if (table_dtype == MLB_BF16)
        launch_kernel(embed_scaled_kernel<__nv_bfloat16>, tokens, ROW_THREADS, 0, stream, (const __nv_bfloat16*)table, ids, out, tokens, width, vocab, scale);
    else
        return fail(MLB_INVALID_ARGUMENT, "embed_gather_scaled: unknown table dtype %d", table_dtype);
    return check_launch("embed_gather_scaled");
}

MLB_EXPORT int mlb_add_table_rows(float* x, const void* table, int table_dtype, const int* index, int tokens, int width,
                                  int rows, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || rows <= 0) return fail(MLB_INVALID_ARGUMENT, "add_table_rows: bad sizes");
    if (tokens == 0) return MLB_OK;
    if (table_dtype == MLB_F32)
        launch_kernel(add_table_rows_kernel<float>, tokens, ROW_THREADS, 0, stream, x, (const float*)table, index, tokens, width, rows);
    else if (table_dtype == MLB_BF16)
        launch_kernel(add_table_rows_kernel<__nv_bfloat16>, tokens, ROW_THREADS, 0, stream, x, (const __nv_bfloat16*)table, index, tokens, width, rows);
    else
        return fail(MLB_INVALID_ARGUMENT, "add_table_rows: unknown table dtype %d", table_dtype);
    return check_launch("add_table_rows");
}

MLB_EXPORT int mlb_add_scaled_rmsnorm(float* residual, const float* delta, int n_delta, long long delta_stride,
                                      const float* col_scale, const float* weight, void* out, int out_dtype, int n_rows,
                                      int width, float eps, cudaStream_t stream) {
    if (n_rows < 0 || width <= 0 || !(eps > 0.0f) || !delta || n_delta < 1)
        return fail(MLB_INVALID_ARGUMENT, "add_scaled_rmsnorm: bad sizes, eps or delta");
    if (n_rows == 0) return MLB_OK;
    if (out_dtype == MLB_F32)
        launch_kernel(add_scaled_rmsnorm_kernel<float>, n_rows, ROW_THREADS, 0, stream, residual, delta, n_delta, delta_stride, col_scale, weight, (float*)out, width, eps);
    else if (out_dtype == MLB_BF16)
        launch_kernel(add_scaled_rmsnorm_kernel<__nv_bfloat16>, n_rows, ROW_THREADS, 0, stream, residual, delta, n_delta, delta_stride, col_scale, weight, (__nv_bfloat16*)out, width, eps);
    else
        return fail(MLB_INVALID_ARGUMENT, "add_scaled_rmsnorm: unknown output dtype %d", out_dtype);
    return check_launch("add_scaled_rmsnorm");
}

MLB_EXPORT int mlb_add_scaled_inplace(float* x, const float* delta, int n_delta, long long delta_stride, const float* col_scale,
                                      int width, long long n, cudaStream_t stream) {
    if (n < 0 || n_delta < 1 || width <= 0) return fail(MLB_INVALID_ARGUMENT, "add_scaled_inplace: bad sizes");
    if (n == 0) return MLB_OK;
    launch_kernel(add_scaled_inplace_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, delta, n_delta, delta_stride, col_scale, width, (size_t)n);
    return check_launch("add_scaled_inplace");
}

MLB_EXPORT int mlb_stream_entry(float* x, const float* x0, const float* v, int width, long long n, cudaStream_t stream) {
    if (n < 0 || width <= 0 || !v) return fail(MLB_INVALID_ARGUMENT, "stream_entry: bad sizes");
    if (n == 0) return MLB_OK;
    launch_kernel(stream_entry_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, x0, v, width, (size_t)n);
    return check_launch("stream_entry");
}
