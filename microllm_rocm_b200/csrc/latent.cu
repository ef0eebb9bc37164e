// Attention over a compressed key/value cache ("latent attention").
//
// Per token the cache holds ONE row for all heads: c[R] (the normalised latent from which every head's key and
// value would be expanded, k_h = Wuk_h c, v_h = Wuv_h c) followed by kr[Dr] (a rotated key part that all heads
// share).  The expansion is never materialised: with a[h] = Wuk_h^T q_h (computed by a product per head before this
// kernel) the score of head h against key j is
//
//     s = (a[h] . c_j + qr[h] . kr_j) * scale
//
// and the head's output in latent space is sum_j p_j c_j, which a second product per head turns into Wuv_h (sum_j p_j c_j).
// So every head attends to the same rows: Dk = R + Dr wide for the score, the first R of them again as the value.
//
//   latent_prepare   from the fused projection output [T, ld] fp32 (or its split partial sums):
//                      columns q_col..   : H heads of (dim plain, Dr rotated) query elements
//                      columns kv_col..  : R latent elements, then Dr shared rotated-key elements
//                      columns gate_col..: gate_width pre-activations of an output gate (optional)
//                    -> q_plain[T, H*dim]           the plain query parts, input of the product with Wuk
//                       q_full[T, H*(R+Dr)]         only its last Dr columns per head: the rotated query parts
//                       pages[page, slot, 0:R]      c = rms(latent) * norm_weight;  [R:R+Dr] = rotated kr
//                       gate_out[T, gate_width]     sigmoid of the pre-activations, fp32
//                    rotation: element i of the first rot_dims is paired with i + rot_dims/2, angle = pos * inv_freq[i]
//   latent_attention_plain   one warp per (token, head); keys in tiles of 32 at absolute multiples of 32, running
//                    maximum and sum in fp32; a learned per-head sink enters the denominator once, unscaled, with
//                    no value.  Bit-stable under any cutting of the tokens into steps.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

struct PrepareParams {
    const float* proj; long long ld; int n_partials; long long partial_stride;
    long long q_col, kv_col, gate_col;
    const float* norm_weight; float eps;
    const int* positions; const int* token_seq; const int* block_table; int max_blocks;
    const float* inv_freq; int rot_dims;
    void* q_plain; void* q_full; void* pages; float* gate_out;
    int num_pages, page_size, tokens, heads, dim, rot_dim, rank, gate_width;
    int* error_flag;
};

__device__ __forceinline__ float proj_at(const PrepareParams& p, size_t row_base, long long col) {
    float v = p.proj[row_base + col];
    for (int k = 1; k < p.n_partials; ++k) v += p.proj[(size_t)k * p.partial_stride + row_base + col];
    return v;
}

constexpr int SLICE = 1024;        // query and gate columns per block

template <typename QT, typename KVT>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(PrepareParams p) {
    pdl_prologue();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const size_t row = (size_t)t * p.ld;
    const int pos = p.positions[t];
    const int half = p.rot_dims / 2;
    const int Dk = p.rank + p.rot_dim;

    // blockIdx.y == 0: the token's cache row; blockIdx.y >= 1: a slice of SLICE query and gate columns
    if (blockIdx.y > 0) {
        const int per_head = p.dim + p.rot_dim;
        const int q_cols = p.heads * per_head;
        const int lo = (blockIdx.y - 1) * SLICE, hi = min(lo + SLICE, q_cols + (p.gate_out ? p.gate_width : 0));
        for (int e = lo + threadIdx.x; e < hi; e += blockDim.x) {
            if (e >= q_cols) {                                   // the gate's sigmoid
                const int c = e - q_cols;
                const float z = proj_at(p, row, p.gate_col + c);
                p.gate_out[(size_t)t * p.gate_width + c] = 1.0f / (1.0f + expf(-z));
                continue;
            }
            // queries: plain parts to q_plain, rotated parts into the tail of each head's row of q_full
            const int h = e / per_head, i = e % per_head;
            const float v = proj_at(p, row, p.q_col + e);
            if (i < p.dim) {
                ((QT*)p.q_plain)[((size_t)t * p.heads + h) * p.dim + i] = from_f32<QT>(v);
                continue;
            }
            const int r = i - p.dim;
            float out = v;
            if (r < p.rot_dims) {
                const int pair = r < half ? r : r - half;
                const float angle = (float)pos * p.inv_freq[pair];
                const float cs = cosf(angle), sn = sinf(angle);
                const float other = proj_at(p, row, p.q_col + (long long)h * per_head + p.dim + (r < half ? r + half : r - half));
                out = r < half ? v * cs - other * sn : v * cs + other * sn;
            }
            ((QT*)p.q_full)[((size_t)t * p.heads + h) * Dk + p.rank + r] = from_f32<QT>(out);
        }
        return;
    }
    // where this token's cache row lives
    KVT* cache_row = nullptr;
    if (p.pages) {
        const int block = pos / p.page_size;
        const int page = block < p.max_blocks ? p.block_table[(size_t)p.token_seq[t] * p.max_blocks + block] : -1;
        if (page < 0 || page >= p.num_pages) {
            if (threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 1);
        } else {
            cache_row = (KVT*)p.pages + ((size_t)page * p.page_size + pos % p.page_size) * Dk;
        }
        // the latent, divided by its root mean square, times the norm's weight
        float ss = 0.0f;
        for (int c = threadIdx.x; c < p.rank; c += blockDim.x) {
            const float v = proj_at(p, row, p.kv_col + c);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)p.rank + p.eps);
        if (cache_row) {
            for (int c = threadIdx.x; c < p.rank; c += blockDim.x)
                cache_row[c] = from_f32<KVT>(proj_at(p, row, p.kv_col + c) * inv * p.norm_weight[c]);
            // the shared key part: pairs (i, i + half) of its first rot_dims turned, the rest passed on
            for (int i = threadIdx.x; i < p.rot_dim; i += blockDim.x) {
                float out;
                const float v = proj_at(p, row, p.kv_col + p.rank + i);
                if (i < p.rot_dims) {
                    const int pair = i < half ? i : i - half;
                    const float angle = (float)pos * p.inv_freq[pair];
                    const float cs = cosf(angle), sn = sinf(angle);
                    const float other = proj_at(p, row, p.kv_col + p.rank + (i < half ? i + half : i - half));
                    out = i < half ? v * cs - other * sn : v * cs + other * sn;
                } else {
                    out = v;
                }
                cache_row[p.rank + i] = from_f32<KVT>(out);
            }
        }
    }
}

constexpr int WARPS = 4;
constexpr int MAX_DK = 640;
constexpr int MAX_R = 512;

struct AttnParams {
    const void* q;           // [T, H*(R+Dr)]
    const void* pages;       // [num_pages, page_size, R+Dr]
    void* out;               // [T, H*R]
    const float* sink;       // [H] or null
    const int* positions; const int* token_seq; const int* block_table;
    int max_blocks, num_pages, page_size, tokens, heads, rank, rot_dim, window;
    float scale;
    int* error_flag;
};

template <typename QT, typename KVT, typename OutT>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_plain_kernel(AttnParams p) {
    pdl_prologue();
    __shared__ float q_s[WARPS][MAX_DK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.tokens * p.heads) return;
    const int t = (int)(item / p.heads), h = (int)(item % p.heads);
    const int R = p.rank, Dk = p.rank + p.rot_dim;
    const int pos = p.positions[t];
    const int seq = p.token_seq[t];
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const QT* qrow = (const QT*)p.q + ((size_t)t * p.heads + h) * Dk;
    for (int c = lane; c < Dk; c += 32) q_s[warp][c] = to_f32(qrow[c]);
    __syncwarp();

    constexpr int PER_LANE = MAX_R / 32;
    float acc[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) acc[i] = 0.0f;
    // the sink is one more term of the denominator: exp(sink) with no key and no value
    float m = p.sink ? p.sink[h] : -INFINITY;
    float l = p.sink ? 1.0f : 0.0f;
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    for (int base = (lo / 32) * 32; base <= pos; base += 32) {
        const int kp = base + lane;
        bool valid = kp >= lo && kp <= pos;
        long long k_off = -1;
        if (valid) {
            const int block = kp / p.page_size;
            const int page = block < p.max_blocks ? table[block] : -1;
            if (page < 0 || page >= p.num_pages) {
                if (p.error_flag) atomicExch(p.error_flag, 2);
                valid = false;
            } else {
                k_off = (long long)(((size_t)page * p.page_size + kp % p.page_size) * Dk);
            }
        }
        float s = -INFINITY;
        if (valid) {
            const KVT* krow = (const KVT*)p.pages + k_off;
            float dot = 0.0f;
            for (int c = 0; c < Dk; ++c) dot = fmaf(q_s[warp][c], to_f32(krow[c]), dot);
            s = dot * p.scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float prob = valid ? expf(s - m_new) : 0.0f;
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + warp_sum(prob);
        m = m_new;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) acc[i] *= corr;
        const unsigned valid_mask = __ballot_sync(0xffffffffu, valid);
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, prob, j);
            const long long off_j = __shfl_sync(0xffffffffu, k_off, j);
            if (!((valid_mask >> j) & 1u)) continue;
            const KVT* vrow = (const KVT*)p.pages + off_j;
#pragma unroll
            for (int i = 0; i < PER_LANE; ++i) {
                const int c = lane + 32 * i;
                if (c < R) acc[i] = fmaf(pj, to_f32(vrow[c]), acc[i]);
            }
        }
    }
    OutT* orow = (OutT*)p.out + ((size_t)t * p.heads + h) * R;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < R) orow[c] = from_f32<OutT>(acc[i] * inv);
    }
}

}  // namespace

MLB_EXPORT int mlb_latent_prepare(const float* proj, long long ld, int n_partials, long long partial_stride, long long q_col,
                                  long long kv_col, long long gate_col, const float* norm_weight, float eps,
                                  const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                                  const float* inv_freq, int rot_dims, void* q_plain, void* q_full, int q_dtype, void* pages,
                                  int kv_dtype, float* gate_out, int num_pages, int page_size, int tokens, int heads, int dim,
                                  int rot_dim, int rank, int gate_width, int* error_flag, cudaStream_t stream) {
    if (tokens < 0 || heads <= 0 || dim <= 0 || rot_dim < 0 || rank <= 0 || n_partials < 1 || !(eps > 0.0f))
        return fail(MLB_INVALID_ARGUMENT, "latent_prepare: bad sizes");
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > rot_dim) return fail(MLB_INVALID_ARGUMENT, "latent_prepare: rot_dims %d must be even and at most %d", rot_dims, rot_dim);
    if (pages && (page_size <= 0 || num_pages <= 0 || max_blocks <= 0)) return fail(MLB_INVALID_ARGUMENT, "latent_prepare: bad cache geometry");
    if (tokens == 0) return MLB_OK;
    PrepareParams p{proj, ld, n_partials, partial_stride, q_col, kv_col, gate_col, norm_weight, eps, positions, token_seq,
                    block_table, max_blocks, inv_freq, rot_dims, q_plain, q_full, pages, gate_out, num_pages, page_size,
                    tokens, heads, dim, rot_dim, rank, gate_width, error_flag};
    const int columns = heads * (dim + rot_dim) + (gate_out ? gate_width : 0);
    const dim3 grid(tokens, 1 + (columns + SLICE - 1) / SLICE);
    if (q_dtype == MLB_F32 && (kv_dtype == MLB_F32 || !pages))
        launch_kernel(latent_prepare_kernel<float, float>, grid, 256, 0, stream, p);
    else if (q_dtype == MLB_BF16 && (kv_dtype == MLB_BF16 || !pages))
        launch_kernel(latent_prepare_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, p);
    else
        return fail(MLB_INVALID_ARGUMENT, "latent_prepare: unsupported dtypes %d / %d", q_dtype, kv_dtype);
    return check_launch("latent_prepare");
}

MLB_EXPORT int mlb_latent_attention_plain(const void* q, int q_dtype, const void* pages, int kv_dtype, void* out, int out_dtype,
                                          const float* sink, const int* positions, const int* token_seq,
                                          const int* block_table, int max_blocks, int num_pages, int page_size, int tokens,
                                          int heads, int rank, int rot_dim, int window, float scale, int* error_flag,
                                          cudaStream_t stream) {
    if (tokens < 0 || heads <= 0 || rank <= 0 || rot_dim < 0) return fail(MLB_INVALID_ARGUMENT, "latent_attention_plain: bad sizes");
    if (rank > MAX_R || rank + rot_dim > MAX_DK)
        return fail(MLB_UNSUPPORTED_SIZE, "latent_attention_plain: latent %d + rotated %d exceed %d / %d", rank, rot_dim, MAX_R, MAX_DK);
    if (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0) return fail(MLB_INVALID_ARGUMENT, "latent_attention_plain: bad cache geometry");
    if (tokens == 0) return MLB_OK;
    AttnParams p{q, pages, out, sink, positions, token_seq, block_table, max_blocks, num_pages, page_size, tokens, heads, rank,
                 rot_dim, window, scale, error_flag};
    const long long items = (long long)tokens * heads;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (q_dtype == MLB_F32 && kv_dtype == MLB_F32 && out_dtype == MLB_F32)
        launch_kernel(latent_attention_plain_kernel<float, float, float>, blocks, WARPS * 32, 0, stream, p);
    else if (q_dtype == MLB_BF16 && kv_dtype == MLB_BF16 && out_dtype == MLB_BF16)
        launch_kernel(latent_attention_plain_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, blocks, WARPS * 32, 0, stream, p);
    else
        return fail(MLB_INVALID_ARGUMENT, "latent_attention_plain: unsupported dtypes %d/%d/%d", q_dtype, kv_dtype, out_dtype);
    return check_launch("latent_attention_plain");
}
