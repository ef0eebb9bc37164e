// Routing of tokens to experts, on the device from start to end (nothing here needs the host to know a count):
//
//   moe_route     per token: z[e] = x . Wr[e] + b[e] in fp32; the `top` largest (ties: the smaller index) in order of
//                 size; weights = softmax over those chosen logits only.  Optionally one more dot product with a
//                 single row (the gate of a shared expert) whose sigmoid is stored per token.
//   moe_align     from ids[T*top] to a list of the pairs (token, choice) sorted by expert: offsets[E+1] and
//                 sorted[T*top] (pair indices); the order inside an expert is arbitrary, every pair's result is
//                 computed on its own.
//   moe_combine   out[t,:] = (sum_j w[t,j] * y[t*top + j,:] + g[t] * sum_k shared_k[t,:]) * s[:]
//                 j in order of choice; shared (may be split partial sums), g and s are optional.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int ROUTE_WARPS = 4;
constexpr int MAX_EXPERTS = 1024;
constexpr int MAX_TOP = 32;

template <typename XT, typename WT>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const XT* __restrict__ x, const WT* __restrict__ wr, const float* __restrict__ bias,
                 const WT* __restrict__ shared_gate, int tokens, int width, int experts, int top,
                 int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ gate_out) {
    pdl_prologue();
    extern __shared__ float logits_s[];                 // [ROUTE_WARPS][experts]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= tokens) return;
    float* z = logits_s + (size_t)warp * experts;
    const XT* xr = x + (size_t)t * width;
    for (int e = 0; e < experts; ++e) {
        const WT* w = wr + (size_t)e * width;
        float part = 0.0f;
        for (int c = lane; c < width; c += 32) part = fmaf(to_f32(xr[c]), to_f32(w[c]), part);
        part = warp_sum(part);
        if (lane == 0) z[e] = part + (bias ? bias[e] : 0.0f);
    }
    if (shared_gate && gate_out) {
        float part = 0.0f;
        for (int c = lane; c < width; c += 32) part = fmaf(to_f32(xr[c]), to_f32(shared_gate[c]), part);
        part = warp_sum(part);
        if (lane == 0) gate_out[t] = 1.0f / (1.0f + expf(-part));
    }
    __syncwarp();
    if (lane == 0) {
        float chosen[MAX_TOP];
        unsigned taken[MAX_EXPERTS / 32];
        for (int e = 0; e < (experts + 31) / 32; ++e) taken[e] = 0u;
        for (int j = 0; j < top; ++j) {
            int best = -1;
            float best_v = -INFINITY;
            for (int e = 0; e < experts; ++e) {
                if ((taken[e >> 5] >> (e & 31)) & 1u) continue;
                const float v = z[e];
                if (best < 0 || v > best_v) { best = e; best_v = v; }
            }
            chosen[j] = best_v;
            ids[(size_t)t * top + j] = best;
            taken[best >> 5] |= 1u << (best & 31);
        }
        const float m = chosen[0];                      // the first choice is the largest
        float sum = 0.0f;
        for (int j = 0; j < top; ++j) { chosen[j] = expf(chosen[j] - m); sum += chosen[j]; }
        for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] = chosen[j] / sum;
    }
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ offsets, int* __restrict__ sorted,
                 int* __restrict__ error_flag) {
    pdl_prologue();
    __shared__ int count[MAX_EXPERTS];
    __shared__ int cursor[MAX_EXPERTS];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
        else if (error_flag) atomicExch(error_flag, 3);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) { offsets[e] = at; cursor[e] = at; at += count[e]; }
        offsets[experts] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < experts) sorted[atomicAdd(&cursor[e], 1)] = i;
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, const float* __restrict__ shared,
                                   int n_shared, long long shared_stride, const float* __restrict__ gate,
                                   const float* __restrict__ col_scale, float* __restrict__ out, int tokens, int width, int top) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    float acc = 0.0f;
    for (int j = 0; j < top; ++j) acc = fmaf(weights[(size_t)t * top + j], y[((size_t)t * top + j) * width + c], acc);
    if (shared) {
        float s = shared[i];
        for (int k = 1; k < n_shared; ++k) s += shared[(size_t)k * shared_stride + i];
        acc += gate ? gate[t] * s : s;
    }
    out[i] = col_scale ? acc * col_scale[c] : acc;
}

}  // namespace

MLB_EXPORT int mlb_moe_route(const void* x, const void* router, const float* bias, const void* shared_gate, int dtype, int tokens,
                             int width, int experts, int top, int* ids, float* weights, float* gate_out, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || experts <= 0 || experts > MAX_EXPERTS || top <= 0 || top > experts || top > MAX_TOP)
        return fail(MLB_INVALID_ARGUMENT, "moe_route: bad sizes (experts %d, top %d; at most %d and %d)", experts, top, MAX_EXPERTS, MAX_TOP);
    if (tokens == 0) return MLB_OK;
    const unsigned blocks = (tokens + ROUTE_WARPS - 1) / ROUTE_WARPS;
    const size_t smem = (size_t)ROUTE_WARPS * experts * sizeof(float);
    if (dtype == MLB_F32)
        launch_kernel(moe_route_kernel<float, float>, blocks, ROUTE_WARPS * 32, smem, stream, (const float*)x, (const float*)router, bias,
                      (const float*)shared_gate, tokens, width, experts, top, ids, weights, gate_out);
    else if (dtype == MLB_BF16)
        launch_kernel(moe_route_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, ROUTE_WARPS * 32, smem, stream, (const __nv_bfloat16*)x,
                      (const __nv_bfloat16*)router, bias, (const __nv_bfloat16*)shared_gate, tokens, width, experts, top, ids, weights, gate_out);
    else
        return fail(MLB_INVALID_ARGUMENT, "moe_route: unknown dtype %d", dtype);
    return check_launch("moe_route");
}

MLB_EXPORT int mlb_moe_align(const int* ids, int pairs, int experts, int* offsets, int* sorted, int* error_flag, cudaStream_t stream) {
    if (pairs < 0 || experts <= 0 || experts > MAX_EXPERTS) return fail(MLB_INVALID_ARGUMENT, "moe_align: bad sizes");
    launch_kernel(moe_align_kernel, 1, 1024, 0, stream, ids, pairs, experts, offsets, sorted, error_flag);
    return check_launch("moe_align");
}

MLB_EXPORT int mlb_moe_combine(const float* y, const float* weights, const float* shared, int n_shared, long long shared_stride,
                               const float* gate, const float* col_scale, float* out, int tokens, int width, int top,
                               cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || top <= 0 || (shared && n_shared < 1)) return fail(MLB_INVALID_ARGUMENT, "moe_combine: bad sizes");
    if (tokens == 0) return MLB_OK;
    const long long n = (long long)tokens * width;
    launch_kernel(moe_combine_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, y, weights, shared, n_shared, shared_stride,
                  gate, col_scale, out, tokens, width, top);
    return check_launch("moe_combine");
}
