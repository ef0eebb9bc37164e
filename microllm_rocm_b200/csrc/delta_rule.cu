// Gated delta rule with one decay per head and key channel, fp32 throughout.  Per head, with S [DK, DV]:
//
//   S <- diag(g_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t
//
//   mlb_delta_prepare   what enters the recurrence besides v: q and k as unit vectors per head (x / sqrt(sum x^2 + 1e-6),
//                       q also times DK^-1/2), beta = sigmoid(b), g = exp(-exp(A_log[h]) * softplus(W2 a + dt_bias)) with a
//                       the (narrow) output of the first of the decay's two projections; W2 is applied here.
//   mlb_delta_scan      the recurrence over the new tokens of every sequence of the step, from the state in the
//                       sequence's slot ([slots, H, DK, DV] fp32; taken as zero when the sequence starts at position 0)
//                       and back into it.  The columns of S never meet: a CTA owns 16 of them for one (sequence,
//                       head), eight lanes share a column's DK rows in registers and meet by shuffles twice a token.
//   mlb_delta_output    o / rms(o) per head * weight * sigmoid(W2g a_g), stored in the compute dtype.
//
// The order of every addition depends on the token's place in its sequence only, never on how the sequence was cut
// into steps: a token's result is the same bits however it is scheduled.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;
constexpr int PER_LANE = MAX_D / 32;

struct Columns {
    const float* base; long long ld; int n_partials; long long partial_stride;
    __device__ __forceinline__ float at(long long row, int col) const {
        const float* p = base + row * ld + col;
        float v = p[0];
        for (int k = 1; k < n_partials; ++k) v += p[(size_t)k * partial_stride];
        return v;
    }
};

__device__ __forceinline__ float sigmoid(float v) {
    if (v >= 0.0f) return 1.0f / (1.0f + expf(-v));
    const float e = expf(v);
    return e / (1.0f + e);
}

__device__ __forceinline__ float softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// ------------------------------------------------------------------------------ prepare
struct PrepareParams {
    const float* qkv; long long ld_qkv;      // convolved and activated [T, G*DK | G*DK | H*DV]
    Columns proj; int beta_col, a_col;       // the input projection's fp32 output: beta pre-activations [H], a [a_rank]
    const float* w2;                         // [H * DK, a_rank]; unused when `pre` is given
    Columns pre;                             // W2 a already made by a product [T, H * DK] (base null: made here)
    const float* dt_bias;                    // [H * DK]
    const float* a_log;                      // [H]
    float* qn; float* kn;                    // [T, G * DK]
    float* g;                                // [T, H * DK]
    float* beta;                             // [T, H]
    int T, H, G, DK, a_rank;
};

__global__ void __launch_bounds__(WARPS * 32) delta_prepare_kernel(PrepareParams p) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items = 2 * p.G + p.H;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.T * items) return;
    const int t = (int)(item / items), which = (int)(item % items);
    if (which < 2 * p.G) {                   // a head of q or of k: unit vector
        const bool is_q = which < p.G;
        const int head = is_q ? which : which - p.G;
        const float* src = p.qkv + (size_t)t * p.ld_qkv + (is_q ? 0 : p.G * p.DK) + head * p.DK;
        float x[PER_LANE];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int c = lane + 32 * i;
            x[i] = c < p.DK ? src[c] : 0.0f;
            ss = fmaf(x[i], x[i], ss);
        }
        float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
        if (is_q) inv *= 1.0f / sqrtf((float)p.DK);
        float* dst = (is_q ? p.qn : p.kn) + ((size_t)t * p.G + head) * p.DK;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) { const int c = lane + 32 * i; if (c < p.DK) dst[c] = x[i] * inv; }
        return;
    }
    const int h = which - 2 * p.G;
    const float rate = expf(p.a_log[h]);
    for (int c = lane; c < p.DK; c += 32) {
        float pre = 0.0f;
        if (p.pre.base) {
            pre = p.pre.at(t, h * p.DK + c);
        } else {
            const float* w = p.w2 + ((size_t)h * p.DK + c) * p.a_rank;
            for (int r = 0; r < p.a_rank; ++r) pre = fmaf(w[r], p.proj.at(t, p.a_col + r), pre);
        }
        pre += p.dt_bias[h * p.DK + c];
        p.g[((size_t)t * p.H + h) * p.DK + c] = expf(-rate * softplus(pre));
    }
    if (lane == 0) p.beta[(size_t)t * p.H + h] = sigmoid(p.proj.at(t, p.beta_col + h));
}

// ------------------------------------------------------------------------------ the recurrence
struct ScanParams {
    const float* qn; const float* kn;        // [T, G * DK]
    const float* g;                          // [T, H * DK]
    const float* beta;                       // [T, H]
    const float* v; long long ld_v;          // [T, H * DV] (a column block of the convolved rows)
    float* o;                                // [T, H * DV]
    float* state;                            // [slots + 1, H, DK, DV]
    const int* slots; int num_slots;
    const int* seq_starts; const int* seq_pos0;
    int A, H, G, DK, DV;
    int* error_flag;
};

constexpr int SCAN_LANES = 8, SCAN_THREADS = 128, SCAN_COLS = SCAN_THREADS / SCAN_LANES;

// ROWS: rows of a column that one lane keeps (DK <= 8 * ROWS).  CHUNK: tokens whose q, k, g, v and beta are staged in
// shared memory at a time; the next chunk's values are fetched into registers before the present chunk is computed
// and stored behind it, so the recurrence never waits for global memory inside a chunk.
template <int ROWS, int CHUNK>
__global__ void __launch_bounds__(SCAN_THREADS) delta_scan_kernel(ScanParams p) {
    pdl_prologue();
    constexpr int DKP = SCAN_LANES * ROWS;                    // padded key width
    constexpr int PER_TOKEN = 3 * DKP + SCAN_COLS + 1;        // q | k | g | v of this CTA's columns | beta
    constexpr int STAGED = CHUNK * PER_TOKEN;
    constexpr int FETCH = (STAGED + SCAN_THREADS - 1) / SCAN_THREADS;
    __shared__ float stage_s[2][STAGED];
    const int col_blocks = (p.DV + SCAN_COLS - 1) / SCAN_COLS;
    const int cb = blockIdx.x % col_blocks, h = (blockIdx.x / col_blocks) % p.H, a = blockIdx.x / (col_blocks * p.H);
    const int part = threadIdx.x & (SCAN_LANES - 1);
    const int local_col = threadIdx.x / SCAN_LANES;
    const int col = cb * SCAN_COLS + local_col;
    const bool col_ok = col < p.DV;
    const int start = p.seq_starts[a], n = p.seq_starts[a + 1] - start;
    const int slot = p.slots[a];
    if (slot < 0 || slot >= p.num_slots) {
        if (threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 3);
        return;
    }
    const int kvh = h / (p.H / p.G);
    const int row0 = part * ROWS;
    float S[ROWS];
    float* st = p.state + (((size_t)slot * p.H + h) * p.DK) * p.DV;
    const bool fresh = p.seq_pos0[a] == 0;
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
        S[i] = (!fresh && col_ok && row0 + i < p.DK) ? st[(size_t)(row0 + i) * p.DV + col] : 0.0f;

    // element e of a chunk's staging area, for the chunk that begins at token `first`
    auto fetch = [&](int first, int e) -> float {
        const int tok = e / PER_TOKEN, w = e % PER_TOKEN;
        if (e >= STAGED || first + tok >= n) return 0.0f;
        const size_t t = (size_t)start + first + tok;
        if (w < 3 * DKP) {
            const int which = w / DKP, c = w % DKP;
            if (c >= p.DK) return which == 2 ? 1.0f : 0.0f;
            return which == 0 ? p.qn[(t * p.G + kvh) * p.DK + c] : (which == 1 ? p.kn[(t * p.G + kvh) * p.DK + c] : p.g[(t * p.H + h) * p.DK + c]);
        }
        if (w < 3 * DKP + SCAN_COLS) {
            const int c = cb * SCAN_COLS + (w - 3 * DKP);
            return c < p.DV ? p.v[t * p.ld_v + (size_t)h * p.DV + c] : 0.0f;
        }
        return p.beta[t * p.H + h];
    };
    float next[FETCH];
#pragma unroll
    for (int f = 0; f < FETCH; ++f) {
        const int e = threadIdx.x + f * SCAN_THREADS;
        if (e < STAGED) stage_s[0][e] = fetch(0, e);
    }
    __syncthreads();
    for (int first = 0, buf = 0; first < n; first += CHUNK, buf ^= 1) {
        const bool more = first + CHUNK < n;
        if (more) {
#pragma unroll
            for (int f = 0; f < FETCH; ++f) next[f] = fetch(first + CHUNK, threadIdx.x + f * SCAN_THREADS);
        }
        const int count = min(CHUNK, n - first);
        for (int tok = 0; tok < count; ++tok) {
            const float* row = stage_s[buf] + tok * PER_TOKEN;
            const float* qs = row + row0; const float* ks = row + DKP + row0; const float* gs = row + 2 * DKP + row0;
            const float v = row[3 * DKP + local_col], beta = row[3 * DKP + SCAN_COLS];
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) { S[i] *= gs[i]; dot = fmaf(S[i], ks[i], dot); }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            const float u = beta * (v - dot);
            float out = 0.0f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) { S[i] = fmaf(ks[i], u, S[i]); out = fmaf(S[i], qs[i], out); }
            out += __shfl_xor_sync(0xffffffffu, out, 1);
            out += __shfl_xor_sync(0xffffffffu, out, 2);
            out += __shfl_xor_sync(0xffffffffu, out, 4);
            if (part == 0 && col_ok) p.o[((size_t)start + first + tok) * ((size_t)p.H * p.DV) + (size_t)h * p.DV + col] = out;
        }
        if (more) {
#pragma unroll
            for (int f = 0; f < FETCH; ++f) {
                const int e = threadIdx.x + f * SCAN_THREADS;
                if (e < STAGED) stage_s[buf ^ 1][e] = next[f];
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
        if (col_ok && row0 + i < p.DK) st[(size_t)(row0 + i) * p.DV + col] = S[i];
}

// ------------------------------------------------------------------------------ output norm and gate
struct OutputParams {
    const float* o;                          // [T, H * DV]
    const float* weight;                     // [DV]
    Columns proj; int g_col;                 // the narrow output of the gate's first projection [g_rank]
    const float* w2;                         // [H * DV, g_rank]; unused when `pre` is given
    Columns pre;                             // W2g a_g already made by a product [T, H * DV] (base null: made here)
    void* out;                               // [T, H * DV]
    int T, H, DV, g_rank; float eps;
};

template <typename OutT>
__global__ void __launch_bounds__(WARPS * 32) delta_output_kernel(OutputParams p) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.T * p.H) return;
    const int t = (int)(item / p.H), h = (int)(item % p.H);
    const float* src = p.o + ((size_t)t * p.H + h) * p.DV;
    float x[PER_LANE];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        x[i] = c < p.DV ? src[c] : 0.0f;
        ss = fmaf(x[i], x[i], ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)p.DV + p.eps);
    OutT* dst = (OutT*)p.out + ((size_t)t * p.H + h) * p.DV;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c >= p.DV) continue;
        float pre = 0.0f;
        if (p.pre.base) {
            pre = p.pre.at(t, h * p.DV + c);
        } else {
            const float* w = p.w2 + ((size_t)h * p.DV + c) * p.g_rank;
            for (int r = 0; r < p.g_rank; ++r) pre = fmaf(w[r], p.proj.at(t, p.g_col + r), pre);
        }
        dst[c] = from_f32<OutT>(x[i] * inv * p.weight[c] * sigmoid(pre));
    }
}

// out[t, c] = src[t, col0 + c] (partial results summed in split order), stored in the compute dtype: the narrow output of
// a first projection made ready for the second one.
template <typename OutT>
__global__ void take_columns_kernel(Columns src, int col0, int n, int T, OutT* out) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)T * n) return;
    out[i] = from_f32<OutT>(src.at(i / n, col0 + (int)(i % n)));
}

}  // namespace

MLB_EXPORT int mlb_take_columns(const float* src, long long ld, int n_partials, long long partial_stride, int col0, int n, int T,
                                void* out, int out_dtype, cudaStream_t stream) {
    if (!src || !out || n <= 0 || T < 0) return fail(MLB_INVALID_ARGUMENT, "take_columns: bad operands");
    if (T == 0) return MLB_OK;
    Columns c{src, ld, n_partials < 1 ? 1 : n_partials, partial_stride};
    const unsigned blocks = (unsigned)(((long long)T * n + 255) / 256);
    if (out_dtype == MLB_BF16) launch_kernel(take_columns_kernel<__nv_bfloat16>, blocks, 256, 0, stream, c, col0, n, T, (__nv_bfloat16*)out);
    else launch_kernel(take_columns_kernel<float>, blocks, 256, 0, stream, c, col0, n, T, (float*)out);
    return check_launch("take_columns");
}

MLB_EXPORT int mlb_delta_prepare(const float* qkv, long long ld_qkv, const float* proj, long long ld_proj, int n_partials,
                                 long long partial_stride, int beta_col, int a_col, const float* w2, const float* pre, long long ld_pre,
                                 int pre_partials, long long pre_partial_stride, const float* dt_bias,
                                 const float* a_log, float* qn, float* kn, float* g, float* beta, int T, int H, int G, int DK,
                                 int a_rank, cudaStream_t stream) {
    if (T < 0 || H <= 0 || G <= 0 || H % G || DK <= 0 || DK > MAX_D || a_rank <= 0)
        return fail(MLB_UNSUPPORTED_SIZE, "delta_prepare: heads %d/%d, key width %d (at most %d), rank %d", H, G, DK, MAX_D, a_rank);
    if (!qkv || !proj || (!w2 && !pre) || !dt_bias || !a_log || !qn || !kn || !g || !beta) return fail(MLB_INVALID_ARGUMENT, "delta_prepare: null operand");
    if (T == 0) return MLB_OK;
    PrepareParams p{qkv, ld_qkv, Columns{proj, ld_proj, n_partials < 1 ? 1 : n_partials, partial_stride}, beta_col, a_col, w2,
                    Columns{pre, ld_pre, pre_partials < 1 ? 1 : pre_partials, pre_partial_stride}, dt_bias, a_log, qn, kn, g, beta, T, H, G, DK, a_rank};
    const long long items = (long long)T * (2 * G + H);
    launch_kernel(delta_prepare_kernel, (unsigned)((items + WARPS - 1) / WARPS), WARPS * 32, 0, stream, p);
    return check_launch("delta_prepare");
}

MLB_EXPORT int mlb_delta_scan(const float* qn, const float* kn, const float* g, const float* beta, const float* v, long long ld_v,
                              float* o, float* state, const int* slots, int num_slots, const int* seq_starts, const int* seq_pos0,
                              int A, int H, int G, int DK, int DV, int* error_flag, cudaStream_t stream) {
    if (A < 0 || H <= 0 || G <= 0 || H % G || DK <= 0 || DK > MAX_D || DV <= 0)
        return fail(MLB_UNSUPPORTED_SIZE, "delta_scan: heads %d/%d, widths %d (at most %d) / %d", H, G, DK, MAX_D, DV);
    if (!qn || !kn || !g || !beta || !v || !o || !state || !slots || !seq_starts || !seq_pos0)
        return fail(MLB_INVALID_ARGUMENT, "delta_scan: null operand");
    if (A == 0) return MLB_OK;
    ScanParams p{qn, kn, g, beta, v, ld_v, o, state, slots, num_slots, seq_starts, seq_pos0, A, H, G, DK, DV, error_flag};
    const unsigned blocks = (unsigned)((long long)A * H * ((DV + SCAN_COLS - 1) / SCAN_COLS));
    if (DK <= 32) launch_kernel(delta_scan_kernel<4, 16>, blocks, SCAN_THREADS, 0, stream, p);
    else if (DK <= 64) launch_kernel(delta_scan_kernel<8, 16>, blocks, SCAN_THREADS, 0, stream, p);
    else if (DK <= 128) launch_kernel(delta_scan_kernel<16, 8>, blocks, SCAN_THREADS, 0, stream, p);
    else launch_kernel(delta_scan_kernel<32, 4>, blocks, SCAN_THREADS, 0, stream, p);
    return check_launch("delta_scan");
}

MLB_EXPORT int mlb_delta_output(const float* o, const float* weight, const float* proj, long long ld_proj, int n_partials,
                                long long partial_stride, int g_col, const float* w2, const float* pre, long long ld_pre,
                                int pre_partials, long long pre_partial_stride, void* out, int out_dtype, int T, int H,
                                int DV, int g_rank, float eps, cudaStream_t stream) {
    if (T < 0 || H <= 0 || DV <= 0 || DV > MAX_D || g_rank <= 0)
        return fail(MLB_UNSUPPORTED_SIZE, "delta_output: value width %d (at most %d), rank %d", DV, MAX_D, g_rank);
    if (!o || !weight || !proj || (!w2 && !pre) || !out) return fail(MLB_INVALID_ARGUMENT, "delta_output: null operand");
    if (T == 0) return MLB_OK;
    OutputParams p{o, weight, Columns{proj, ld_proj, n_partials < 1 ? 1 : n_partials, partial_stride}, g_col, w2,
                   Columns{pre, ld_pre, pre_partials < 1 ? 1 : pre_partials, pre_partial_stride}, out, T, H, DV, g_rank, eps};
    const long long items = (long long)T * H;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (out_dtype == MLB_BF16) launch_kernel(delta_output_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, p);
    else launch_kernel(delta_output_kernel<float>, blocks, WARPS * 32, 0, stream, p);
    return check_launch("delta_output");
}
