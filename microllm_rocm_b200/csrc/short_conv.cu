// Short causal convolution over time, per channel, with the last taps - 1 inputs of every sequence kept as state:
//
//   y[t, c] = act( sum_j w[c, j] * u[t - taps + 1 + j, c] ),   u = 0 before the sequence's start, act = identity | silu
//
// u is a block of columns of a projection's fp32 output (or of its K-split partial results, added in split
// order).  Tokens of a step are the flat batch of the engine: a sequence's tokens are consecutive, it held `pos0`
// tokens before the step; inputs of positions before the step come from the state of the sequence's slot
// ([slots, taps - 1, C] fp32, oldest first), inputs of positions before 0 are zero whatever the slot holds (a slot
// is never cleared when a new request takes it).  `mlb_short_conv_state` then moves the state on; it runs after the
// convolution has read the old one.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int MAX_TAPS = 16;

struct ConvParams {
    const float* u; long long ld; int n_partials; long long partial_stride; int col0;
    const float* w;            // [C, taps]
    float* state;              // [slots + 1, taps - 1, C]
    const int* slots;          // [A]
    int num_slots;
    const int* seq_starts;     // [A + 1]
    const int* seq_pos0;       // [A]
    const int* token_seq;      // [T]
    float* y; long long ldy;
    int T, A, C, taps, act;
    int* error_flag;
    int run = 1;               // tokens a thread of the four-channel kernel walks
};

__device__ __forceinline__ float input_at(const ConvParams& p, long long row, int c) {
    const float* at = p.u + row * p.ld + p.col0 + c;
    float v = at[0];
    for (int k = 1; k < p.n_partials; ++k) v += at[(size_t)k * p.partial_stride];
    return v;
}

__global__ void short_conv_kernel(ConvParams p) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.T * p.C) return;
    const int t = (int)(i / p.C), c = (int)(i % p.C);
    const int a = p.token_seq[t];
    const int start = p.seq_starts[a], pos0 = p.seq_pos0[a];
    const int local = t - start;
    const int slot = p.slots[a];
    const int hist = p.taps - 1;
    const bool slot_ok = hist == 0 || (slot >= 0 && slot < p.num_slots);      // one tap keeps no state: any slot will do
    if (!slot_ok && p.error_flag) atomicExch(p.error_flag, 3);
    float acc = 0.0f;
    for (int j = 0; j < p.taps; ++j) {
        const int src = local - hist + j;              // index among this step's tokens of the sequence
        float u = 0.0f;
        if (src >= 0) u = input_at(p, (long long)start + src, c);
        else if (pos0 + src >= 0 && slot_ok) u = p.state[((size_t)slot * hist + (hist + src)) * p.C + c];
        acc = fmaf(p.w[(size_t)c * p.taps + j], u, acc);
    }
    if (p.act == 1) acc = acc / (1.0f + expf(-acc));
    p.y[(size_t)t * p.ldy + c] = acc;
}

// Four channels and RUN consecutive tokens of the flat batch a thread: every row a multiple of four floats and 16-byte
// aligned, the number of taps known when compiling.  A sequence's tokens are consecutive rows, so a token's earlier
// inputs are the rows right above it and stay in registers from one token to the next (every row is fetched once, plus
// TAPS - 1 rows per run); only the first tokens of a sequence's portion take theirs from the state, or zero.
constexpr int CONV_RUN = 8;            // for steps of many tokens; a thread of a small step takes one token

__device__ __forceinline__ float4 conv_row(const ConvParams& p, long long row, int c) {
    const float* at = p.u + row * p.ld + p.col0 + c;
    float4 u = *reinterpret_cast<const float4*>(at);
    for (int k = 1; k < p.n_partials; ++k) {
        const float4 more = *reinterpret_cast<const float4*>(at + (size_t)k * p.partial_stride);
        u.x += more.x; u.y += more.y; u.z += more.z; u.w += more.w;
    }
    return u;
}

template <int TAPS>
__global__ void short_conv_x4_kernel(ConvParams p) {
    pdl_launch_dependents();
    constexpr int HIST = TAPS - 1;
    const int C4 = p.C / 4;
    const int runs = (p.T + p.run - 1) / p.run;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool active = i < (long long)runs * C4;
    const int c = active ? (int)(i % C4) * 4 : 0;
    float wreg[4 * TAPS];               // the weights are never written by a kernel: fetched before the wait for the predecessor
#pragma unroll
    for (int k = 0; k < 4 * TAPS; ++k) wreg[k] = p.w[(size_t)c * TAPS + k];
    pdl_wait();
    if (!active) return;
    const int t0 = (int)(i / C4) * p.run;
    float4 win[HIST > 0 ? HIST : 1];    // rows t - HIST .. t - 1 of the flat batch, as they are
#pragma unroll
    for (int m = 0; m < HIST; ++m) win[m] = t0 - HIST + m >= 0 ? conv_row(p, t0 - HIST + m, c) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = t0; t < min(t0 + p.run, p.T); ++t) {
        const float4 now = conv_row(p, t, c);
        const int a = p.token_seq[t];
        const int local = t - p.seq_starts[a];
        float4 acc = make_float4(wreg[HIST] * now.x, wreg[TAPS + HIST] * now.y, wreg[2 * TAPS + HIST] * now.z, wreg[3 * TAPS + HIST] * now.w);
        if (local >= HIST) {
#pragma unroll
            for (int j = 0; j < HIST; ++j) {
                acc.x = fmaf(wreg[j], win[j].x, acc.x); acc.y = fmaf(wreg[TAPS + j], win[j].y, acc.y);
                acc.z = fmaf(wreg[2 * TAPS + j], win[j].z, acc.z); acc.w = fmaf(wreg[3 * TAPS + j], win[j].w, acc.w);
            }
        } else {                        // one of the first tokens of a portion: some inputs lie before it
            const int pos0 = p.seq_pos0[a], slot = p.slots[a];
            const bool slot_ok = slot >= 0 && slot < p.num_slots;
            if (!slot_ok && p.error_flag) atomicExch(p.error_flag, 3);
#pragma unroll
            for (int j = 0; j < HIST; ++j) {
                const int src = local - HIST + j;
                float4 u = win[j];
                if (src < 0) {
                    u = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (pos0 + src >= 0 && slot_ok) u = *reinterpret_cast<const float4*>(p.state + ((size_t)slot * HIST + (HIST + src)) * p.C + c);
                }
                acc.x = fmaf(wreg[j], u.x, acc.x); acc.y = fmaf(wreg[TAPS + j], u.y, acc.y);
                acc.z = fmaf(wreg[2 * TAPS + j], u.z, acc.z); acc.w = fmaf(wreg[3 * TAPS + j], u.w, acc.w);
            }
        }
        if (p.act == 1) {
            acc.x = acc.x / (1.0f + expf(-acc.x)); acc.y = acc.y / (1.0f + expf(-acc.y));
            acc.z = acc.z / (1.0f + expf(-acc.z)); acc.w = acc.w / (1.0f + expf(-acc.w));
        }
        *reinterpret_cast<float4*>(p.y + (size_t)t * p.ldy + c) = acc;
#pragma unroll
        for (int m = 0; m + 1 < HIST; ++m) win[m] = win[m + 1];
        if (HIST > 0) win[HIST - 1] = now;
    }
}

__global__ void short_conv_state_kernel(ConvParams p) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.A * p.C) return;
    const int a = (int)(i / p.C), c = (int)(i % p.C);
    const int start = p.seq_starts[a], n = p.seq_starts[a + 1] - start;
    const int slot = p.slots[a];
    if (slot < 0 || slot >= p.num_slots) return;
    const int hist = p.taps - 1;
    float keep[MAX_TAPS];
    float* st = p.state + (size_t)slot * hist * p.C + c;
#pragma unroll
    for (int m = 0; m < MAX_TAPS; ++m) {
        if (m >= hist) break;
        const int src = n - hist + m;
        keep[m] = src >= 0 ? input_at(p, (long long)start + src, c) : st[(size_t)(m + n) * p.C];
    }
#pragma unroll
    for (int m = 0; m < MAX_TAPS; ++m) {
        if (m >= hist) break;
        st[(size_t)m * p.C] = keep[m];
    }
}

int check(const ConvParams& p, const char* what) {
    if (p.T < 0 || p.A < 0 || p.C <= 0 || p.taps < 1 || p.taps > MAX_TAPS + 1 || p.n_partials < 1 || p.num_slots <= 0)
        return fail(MLB_INVALID_ARGUMENT, "%s: bad sizes (taps 1..%d)", what, MAX_TAPS + 1);
    if (!p.u || !p.w || !p.slots || !p.seq_starts || !p.seq_pos0 || !p.token_seq || (p.taps > 1 && !p.state))
        return fail(MLB_INVALID_ARGUMENT, "%s: null operand", what);
    return MLB_OK;
}

}  // namespace

MLB_EXPORT int mlb_short_conv(const float* u, long long ld, int n_partials, long long partial_stride, int col0, const float* w,
                              float* state, const int* slots, int num_slots, const int* seq_starts, const int* seq_pos0,
                              const int* token_seq, float* y, long long ldy, int T, int A, int C, int taps, int act,
                              int* error_flag, cudaStream_t stream) {
    ConvParams p{u, ld, n_partials, partial_stride, col0, w, state, slots, num_slots, seq_starts, seq_pos0, token_seq, y, ldy,
                 T, A, C, taps, act, error_flag};
    if (int s = check(p, "short_conv")) return s;
    if (!y) return fail(MLB_INVALID_ARGUMENT, "short_conv: null output");
    if (T == 0) return MLB_OK;
    const long long n = (long long)T * C;
    const bool x4 = C % 4 == 0 && ld % 4 == 0 && ldy % 4 == 0 && col0 % 4 == 0 && partial_stride % 4 == 0 &&
                    ((uintptr_t)u | (uintptr_t)y | (uintptr_t)state) % 16 == 0;
    p.run = T >= 64 * CONV_RUN ? CONV_RUN : 1;
    const long long x4_threads = ((long long)T + p.run - 1) / p.run * (C / 4);
    const unsigned x4_blocks = (unsigned)((x4_threads + 127) / 128);
    if (x4 && taps == 2) launch_kernel(short_conv_x4_kernel<2>, x4_blocks, 128, 0, stream, p);
    else if (x4 && taps == 3) launch_kernel(short_conv_x4_kernel<3>, x4_blocks, 128, 0, stream, p);
    else if (x4 && taps == 4) launch_kernel(short_conv_x4_kernel<4>, x4_blocks, 128, 0, stream, p);
    else if (x4 && taps == 5) launch_kernel(short_conv_x4_kernel<5>, x4_blocks, 128, 0, stream, p);
    else launch_kernel(short_conv_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, p);
    return check_launch("short_conv");
}

MLB_EXPORT int mlb_short_conv_state(const float* u, long long ld, int n_partials, long long partial_stride, int col0, float* state,
                                    const int* slots, int num_slots, const int* seq_starts, int A, int C, int taps,
                                    cudaStream_t stream) {
    ConvParams p{u, ld, n_partials, partial_stride, col0, u, state, slots, num_slots, seq_starts, seq_starts, seq_starts, nullptr, 0,
                 0, A, C, taps, 0, nullptr};
    if (int s = check(p, "short_conv_state")) return s;
    if (A == 0 || taps == 1) return MLB_OK;
    const long long n = (long long)A * C;
    launch_kernel(short_conv_state_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, p);
    return check_launch("short_conv_state");
}
