// Layer norm with weight and bias, fp32:  y = (v - mean(v)) / sqrt(mean((v - mean)^2) + eps) * w + b.
//
//   mlb_layernorm             y[r] = LN(x[rows[r]] or x[r]), stored in the compute dtype (the final norm on selected rows)
//   mlb_scale_add_layernorm   x[r] <- LN(alpha * x[r] + s1 * sum_k d1[k][r] + s2 * sum_k d2[k][r]) in place (the stream of a
//                             block that normalises AFTER its sums), and a copy of the new x[r] in the compute dtype
//                             for the products that read it next.  d1/d2 may be K-split partial results, added in
//                             split order; d2 is optional (two mixers side by side whose results are weighted).
//
// One block of a fixed size per row, the row kept in shared memory between the passes (mean, then the squared
// deviations: the two-pass form), reductions in a fixed tree: a row's result depends on the row alone.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int LN_THREADS = 256;

struct LnParams {
    float* x;                 // [*, width] fp32 (written by scale_add)
    const float* d1; int n1; long long stride1; float s1;
    const float* d2; int n2; long long stride2; float s2;
    float alpha;
    const float* weight; const float* bias;
    void* out;                // compute-dtype copy, may be null
    const int* rows;          // plain norm: source row of each output row, may be null
    int width; float eps;
};

// sum over the partial results at one float4, eight loads in flight, added in split order
__device__ __forceinline__ float4 partial_sum4(const float* at, int n, long long stride) {
    float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < n; k0 += 8) {
        float4 part[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            part[k] = k0 + k < n ? *reinterpret_cast<const float4*>(at + (size_t)(k0 + k) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 8; ++k) { total.x += part[k].x; total.y += part[k].y; total.z += part[k].z; total.w += part[k].w; }
    }
    return total;
}

constexpr int LN_VECS = 4;          // float4 a thread keeps in registers: rows of up to 4 * LN_VECS * LN_THREADS columns

// FEW: a step of few rows (decoding), where what counts is the time from the predecessor's end to this kernel's:
// weight and bias wait in registers.  Many rows: fewer registers a thread, more rows in flight on an SM.
template <typename OutT, bool ADD, bool FEW>
__global__ void __launch_bounds__(LN_THREADS) layernorm_kernel(LnParams p) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float row_s[];
    __shared__ float scratch[32];
    const int r = blockIdx.x, W = p.width;
    if (ADD && (W & 3) == 0 && W <= 4 * LN_VECS * LN_THREADS) {
        // The row stays in registers between the passes.  Weight and bias are never written by a kernel: they are
        // fetched before the wait for the predecessor.
        float4 wv[FEW ? LN_VECS : 1], bv[FEW ? LN_VECS : 1], v[LN_VECS];
        if (FEW) {
#pragma unroll
            for (int i = 0; i < LN_VECS; ++i) {
                const int c = (threadIdx.x + i * LN_THREADS) * 4;
                if (c < W) { wv[i] = *reinterpret_cast<const float4*>(p.weight + c); bv[i] = *reinterpret_cast<const float4*>(p.bias + c); }
            }
        }
        pdl_wait();
        float* xr = p.x + (size_t)r * W;
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < LN_VECS; ++i) {
            const int c = (threadIdx.x + i * LN_THREADS) * 4;
            if (c >= W) break;
            float4 x = *reinterpret_cast<const float4*>(xr + c);
            x.x *= p.alpha; x.y *= p.alpha; x.z *= p.alpha; x.w *= p.alpha;
            const float4 a = partial_sum4(p.d1 + (size_t)r * W + c, p.n1, p.stride1);
            x.x = fmaf(p.s1, a.x, x.x); x.y = fmaf(p.s1, a.y, x.y); x.z = fmaf(p.s1, a.z, x.z); x.w = fmaf(p.s1, a.w, x.w);
            if (p.d2) {
                const float4 b = partial_sum4(p.d2 + (size_t)r * W + c, p.n2, p.stride2);
                x.x = fmaf(p.s2, b.x, x.x); x.y = fmaf(p.s2, b.y, x.y); x.z = fmaf(p.s2, b.z, x.z); x.w = fmaf(p.s2, b.w, x.w);
            }
            v[i] = x;
            sum += (x.x + x.y) + (x.z + x.w);
        }
        const float mean = block_sum(sum, scratch) / (float)W;
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < LN_VECS; ++i) {
            const int c = (threadIdx.x + i * LN_THREADS) * 4;
            if (c >= W) break;
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
        }
        const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)W + p.eps);
        OutT* yr = p.out ? (OutT*)p.out + (size_t)r * W : nullptr;
#pragma unroll
        for (int i = 0; i < LN_VECS; ++i) {
            const int c = (threadIdx.x + i * LN_THREADS) * 4;
            if (c >= W) break;
            const float4 w4 = FEW ? wv[FEW ? i : 0] : *reinterpret_cast<const float4*>(p.weight + c);
            const float4 b4 = FEW ? bv[FEW ? i : 0] : *reinterpret_cast<const float4*>(p.bias + c);
            float4 y;
            y.x = v[i].x * inv * w4.x + b4.x; y.y = v[i].y * inv * w4.y + b4.y;
            y.z = v[i].z * inv * w4.z + b4.z; y.w = v[i].w * inv * w4.w + b4.w;
            *reinterpret_cast<float4*>(xr + c) = y;
            if (yr) { yr[c] = from_f32<OutT>(y.x); yr[c + 1] = from_f32<OutT>(y.y); yr[c + 2] = from_f32<OutT>(y.z); yr[c + 3] = from_f32<OutT>(y.w); }
        }
        return;
    }
    pdl_wait();
    const size_t src = (!ADD && p.rows) ? (size_t)p.rows[r] : (size_t)r;
    float* xr = p.x + src * W;
    float sum = 0.0f;
    if (ADD && (W & 3) == 0) {
        // four columns a thread, the partial results' loads issued eight at a time (they are independent; only their sum
        // is taken in split order)
        for (int c = threadIdx.x * 4; c < W; c += LN_THREADS * 4) {
            float4 v = *reinterpret_cast<const float4*>(xr + c);
            v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha;
            const float4 a = partial_sum4(p.d1 + src * W + c, p.n1, p.stride1);
            v.x = fmaf(p.s1, a.x, v.x); v.y = fmaf(p.s1, a.y, v.y); v.z = fmaf(p.s1, a.z, v.z); v.w = fmaf(p.s1, a.w, v.w);
            if (p.d2) {
                const float4 b = partial_sum4(p.d2 + src * W + c, p.n2, p.stride2);
                v.x = fmaf(p.s2, b.x, v.x); v.y = fmaf(p.s2, b.y, v.y); v.z = fmaf(p.s2, b.z, v.z); v.w = fmaf(p.s2, b.w, v.w);
            }
            *reinterpret_cast<float4*>(row_s + c) = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
    } else
    for (int c = threadIdx.x; c < W; c += LN_THREADS) {
        float v = xr[c];
        if (ADD) {
            v *= p.alpha;
            float a = 0.0f;
            for (int k = 0; k < p.n1; ++k) a += p.d1[(size_t)k * p.stride1 + src * W + c];
            v = fmaf(p.s1, a, v);
            if (p.d2) {
                float b = 0.0f;
                for (int k = 0; k < p.n2; ++k) b += p.d2[(size_t)k * p.stride2 + src * W + c];
                v = fmaf(p.s2, b, v);
            }
        }
        row_s[c] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)W;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < W; c += LN_THREADS) { const float d = row_s[c] - mean; sq = fmaf(d, d, sq); }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)W + p.eps);
    OutT* yr = p.out ? (OutT*)p.out + (size_t)r * W : nullptr;
    for (int c = threadIdx.x; c < W; c += LN_THREADS) {
        const float y = (row_s[c] - mean) * inv * p.weight[c] + p.bias[c];
        if (ADD) xr[c] = y;
        if (yr) yr[c] = from_f32<OutT>(y);
    }
}

int launch(const LnParams& p, int n, int out_dtype, bool add, cudaStream_t stream, const char* what) {
    if (n < 0 || p.width <= 0) return fail(MLB_INVALID_ARGUMENT, "%s: bad sizes", what);
    if ((size_t)p.width * sizeof(float) > 200 * 1024) return fail(MLB_UNSUPPORTED_SIZE, "%s: a row of %d floats does not fit shared memory", what, p.width);
    if (n == 0) return MLB_OK;
    const size_t smem = (size_t)p.width * sizeof(float);
    const bool few = add && n <= 2 * sm_count();
    auto go = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            static bool raised[MAX_DEVICES][8] = {};
            const int slot = (few ? 4 : 0) + (add ? 2 : 0) + (out_dtype == MLB_BF16 ? 1 : 0);
            if (!raised[device_index()][slot]) {
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
                    return fail(MLB_CUDA_ERROR, "%s: cannot raise the shared-memory limit", what);
                raised[device_index()][slot] = true;
            }
        }
        launch_kernel(kernel, (unsigned)n, LN_THREADS, smem, stream, p);
        return check_launch(what);
    };
    if (add && few) return out_dtype == MLB_BF16 ? go(layernorm_kernel<__nv_bfloat16, true, true>) : go(layernorm_kernel<float, true, true>);
    if (add) return out_dtype == MLB_BF16 ? go(layernorm_kernel<__nv_bfloat16, true, false>) : go(layernorm_kernel<float, true, false>);
    return out_dtype == MLB_BF16 ? go(layernorm_kernel<__nv_bfloat16, false, false>) : go(layernorm_kernel<float, false, false>);
}

}  // namespace

MLB_EXPORT int mlb_layernorm(const float* x, const float* weight, const float* bias, void* out, int out_dtype, const int* rows,
                             int n, int width, float eps, cudaStream_t stream) {
    if (!x || !weight || !bias || !out) return fail(MLB_INVALID_ARGUMENT, "layernorm: null operand");
    LnParams p{};
    p.x = const_cast<float*>(x); p.weight = weight; p.bias = bias; p.out = out; p.rows = rows; p.width = width; p.eps = eps;
    return launch(p, n, out_dtype, false, stream, "layernorm");
}

MLB_EXPORT int mlb_scale_add_layernorm(float* x, float alpha, const float* d1, int n1, long long stride1, float s1, const float* d2,
                                       int n2, long long stride2, float s2, const float* weight, const float* bias, void* out,
                                       int out_dtype, int n, int width, float eps, cudaStream_t stream) {
    if (!x || !d1 || !weight || !bias || n1 < 1 || (d2 && n2 < 1)) return fail(MLB_INVALID_ARGUMENT, "scale_add_layernorm: bad operands");
    LnParams p{};
    p.x = x; p.d1 = d1; p.n1 = n1; p.stride1 = stride1; p.s1 = s1; p.d2 = d2; p.n2 = n2; p.stride2 = stride2; p.s2 = s2;
    p.alpha = alpha; p.weight = weight; p.bias = bias; p.out = out; p.width = width; p.eps = eps;
    return launch(p, n, out_dtype, true, stream, "scale_add_layernorm");
}
