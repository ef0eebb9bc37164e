// Grouped matrix product on CUDA cores:  for every group g and every row r of the group
//
//     C[c_row(r), g * c_group_cols + n] = epilogue( sum_k A[a_row(r), g * a_group_cols + k] * W[g][n, k] )
//
// with W[g] = W + g * w_group_stride, stored [N, K] (K contiguous) like every weight of the library.
// Two ways of saying which rows a group has:
//   * `group_offsets` [G + 1]: the rows are the places offsets[g] .. offsets[g+1]-1 of a sorted list (tokens routed
//     to experts); `a_rows` / `c_rows` (either may be null) map a place to the row read and the row written, and
//     the row read is a_rows[place] / a_row_div (a list of (token, choice) pairs reads the token's row);
//   * null: every group takes all M rows (one product per head over the same tokens).
// Each output element is accumulated by ONE thread over k = 0..K-1 in increasing order with fp32 FMA, so its value
// depends neither on the tile it falls in nor on which other rows its group holds: the fp32 path stays
// bit-stable, and the bf16 path (bf16 operands, fp32 accumulation) differs from it only by the operands' rounding.
// The optional epilogue multiplies by a factor read from an fp32 matrix at the output's own (row, column).
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int BN = 64, BK = 16, TN = 4;
constexpr int MAX_GROUPS = 1024;       // with a list of offsets (the offsets travel through shared memory)

struct GroupedParams {
    const void* A; long long lda; long long a_group_cols;
    const void* W; long long ldw; long long w_group_stride;
    void* C; long long ldc; long long c_group_cols;
    const int* group_offsets;
    const int* a_rows;
    const int* c_rows;
    int a_row_div;
    const float* factor; long long ldf;      // null: no epilogue
    int M, N, K, G;
};

template <typename AT, typename WT, typename OutT, int TM>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(GroupedParams p) {
    constexpr int BM = 16 * TM;
    pdl_prologue();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int src_row[BM];
    __shared__ int dst_row[BM];
    __shared__ int tile_info[3];             // group, first place, places in this tile
    __shared__ int offsets_s[MAX_GROUPS + 1];
    const int tid = threadIdx.x;
    if (p.group_offsets) {
        for (int g = tid; g <= p.G; g += blockDim.x) offsets_s[g] = p.group_offsets[g];
        __syncthreads();
    }
    if (tid == 0) {
        int group = -1, first = 0, count = 0;
        if (p.group_offsets == nullptr) {
            const int tiles_per_group = (p.M + BM - 1) / BM;
            group = blockIdx.y / tiles_per_group;
            first = (blockIdx.y % tiles_per_group) * BM;
            count = min(BM, p.M - first);
            if (group >= p.G) group = -1;
        } else {
            int tile = blockIdx.y;
            for (int g = 0; g < p.G; ++g) {
                const int lo = offsets_s[g], n = offsets_s[g + 1] - lo;
                const int tiles = (n + BM - 1) / BM;
                if (tile < tiles) { group = g; first = lo + tile * BM; count = min(BM, n - tile * BM); break; }
                tile -= tiles;
            }
        }
        tile_info[0] = group; tile_info[1] = first; tile_info[2] = count;
    }
    __syncthreads();
    const int group = tile_info[0], first = tile_info[1], count = tile_info[2];
    if (group < 0 || count <= 0) return;
    if (tid < BM) {
        int a = -1, c = -1;
        if (tid < count) {
            const int place = first + tid;
            a = p.a_rows ? p.a_rows[place] / p.a_row_div : place;
            c = p.c_rows ? p.c_rows[place] : place;
        }
        src_row[tid] = a; dst_row[tid] = c;
    }
    __syncthreads();
    const AT* A = (const AT*)p.A + (size_t)group * p.a_group_cols;
    const WT* W = (const WT*)p.W + (size_t)group * p.w_group_stride;
    const int tx = tid % 16, ty = tid / 16;
    const int n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < (BM * BK + 255) / 256; ++i) {
            const int e = tid + i * 256;
            if (e < BM * BK) {
                const int row = e / BK, kk = e % BK, k = k0 + kk;
                const int a = src_row[row];
                As[kk][row] = (a >= 0 && k < p.K) ? to_f32(A[(size_t)a * p.lda + k]) : 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int row = e / BK, kk = e % BK, k = k0 + kk;
            const int n = n0 + row;
            Ws[kk][row] = (n < p.N && k < p.K) ? to_f32(W[(size_t)n * p.ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int c = dst_row[ty * TM + i];
        if (c < 0) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= p.N) continue;
            const size_t col = (size_t)group * p.c_group_cols + n;
            float v = acc[i][j];
            if (p.factor) v *= p.factor[(size_t)c * p.ldf + col];
            ((OutT*)p.C)[(size_t)c * p.ldc + col] = from_f32<OutT>(v);
        }
    }
}

template <typename AT, typename WT, typename OutT>
void launch(const GroupedParams& p, int row_tile, unsigned tiles_y, cudaStream_t stream) {
    dim3 grid((p.N + BN - 1) / BN, tiles_y);
    if (row_tile == 16) launch_kernel(grouped_gemm_kernel<AT, WT, OutT, 1>, grid, 256, 0, stream, p);
    else launch_kernel(grouped_gemm_kernel<AT, WT, OutT, 4>, grid, 256, 0, stream, p);
}

}  // namespace

// dtype: operands (A and W alike); out_dtype: C.  row_tile: 16 or 64 rows per CTA (few rows per group: 16).
MLB_EXPORT int mlb_grouped_gemm(const void* A, long long lda, long long a_group_cols, const void* W, long long ldw,
                                long long w_group_stride, void* C, long long ldc, long long c_group_cols,
                                const int* group_offsets, const int* a_rows, const int* c_rows, int a_row_div,
                                const float* factor, long long ldf, int M, int N, int K, int G, int dtype, int out_dtype,
                                int row_tile, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || G <= 0 || a_row_div <= 0 || (row_tile != 16 && row_tile != 64))
        return fail(MLB_INVALID_ARGUMENT, "grouped_gemm: bad sizes M=%d N=%d K=%d G=%d", M, N, K, G);
    if (group_offsets && G > MAX_GROUPS) return fail(MLB_UNSUPPORTED_SIZE, "grouped_gemm: more than %d groups", MAX_GROUPS);
    if (M == 0) return MLB_OK;
    GroupedParams p{A, lda, a_group_cols, W, ldw, w_group_stride, C, ldc, c_group_cols, group_offsets, a_rows, c_rows,
                    a_row_div, factor, ldf, M, N, K, G};
    const long long per = (M + row_tile - 1) / row_tile;
    const long long tiles = group_offsets ? per + G : per * G;
    if (tiles > 65535) return fail(MLB_UNSUPPORTED_SIZE, "grouped_gemm: %lld row tiles exceed one launch", tiles);
    if (dtype == MLB_F32 && out_dtype == MLB_F32) launch<float, float, float>(p, row_tile, (unsigned)tiles, stream);
    else if (dtype == MLB_BF16 && out_dtype == MLB_F32) launch<__nv_bfloat16, __nv_bfloat16, float>(p, row_tile, (unsigned)tiles, stream);
    else if (dtype == MLB_BF16 && out_dtype == MLB_BF16) launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(p, row_tile, (unsigned)tiles, stream);
    else return fail(MLB_INVALID_ARGUMENT, "grouped_gemm: unsupported dtypes %d -> %d", dtype, out_dtype);
    return check_launch("grouped_gemm");
}
