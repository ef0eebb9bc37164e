// Grouped matrix product on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulation): the bf16 path's
// form of grouped_gemm.cu, with the same meaning of groups, row lists and column blocks:
//
//     C[c_row(r), g * c_group_cols + n] = epilogue( sum_k A[a_row(r), g * a_group_cols + k] * W[g][n, k] )
//
// A CTA owns a tile of BM rows (128 or 64, or 16 when groups hold few rows) of ONE group by 64 output columns, and walks K in
// steps of 64 through a three-stage ring filled with cp.async (16-byte pieces: rows of A are gathered through the
// row list on the way in).  Fragments come out of shared memory with ldmatrix; rows of the ring are padded to 144
// bytes, which keeps the eight rows of an ldmatrix phase in different banks.
// Epilogues: none; times a factor read at the output's own place (fp32); or DUAL: the weight holds two row blocks
// (gate rows, then `dual_rows` further down the up rows), both are multiplied in the same pass and the result is
// silu(gate) * up.
// Sizes must suit 16-byte pieces (K, the row pitches and the column blocks multiples of 8 elements); the caller
// sends everything else to the CUDA-core kernel.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int BN = 64, STAGES = 3;
// K elements per step: 64, but 32 for the 128-row tile with two weight blocks (its accumulators leave no registers for
// the fragments of four 16-wide steps; measured 609 against 736 us for gate/up of 12,288 rows)
__host__ __device__ constexpr int bk_of(int bm, bool dual) { return (bm == 128 && dual) ? 32 : 64; }
constexpr int MAX_GROUPS = 1024;       // with a list of offsets (the offsets travel through shared memory)

struct MmaParams {
    const __nv_bfloat16* A; long long lda; long long a_group_cols;
    const __nv_bfloat16* W; long long ldw; long long w_group_stride;
    void* C; long long ldc; long long c_group_cols;
    const int* group_offsets; const int* a_rows; const int* c_rows; int a_row_div;
    const float* factor; long long ldf;
    long long dual_rows;                       // DUAL: the second row block starts this many rows further down
    int M, N, K, G;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                           // 0: the piece is filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float silu(float g) { return g / (1.0f + expf(-g)); }

__host__ __device__ constexpr int threads_of(int bm) { return bm == 128 ? 256 : 128; }
constexpr size_t smem_of(int bm, bool dual) {
    return (size_t)STAGES * (bm + (dual ? 2 : 1) * BN) * (bk_of(bm, dual) + 8) * sizeof(__nv_bfloat16) + (2 * bm + 4 + MAX_GROUPS + 1) * sizeof(int);
}

template <typename OutT, int BM, bool DUAL>
__global__ void __launch_bounds__(threads_of(BM), BM == 128 ? 2 : 1)
grouped_mma_kernel(MmaParams p) {
    constexpr int THREADS = threads_of(BM);
    constexpr int BK = bk_of(BM, DUAL), PITCH = BK + 8, PIECES = BK / 8;    // padded row of the ring; 16-byte pieces per row
    constexpr int WARPS_M = BM >= 64 ? 4 : 1;        // BM 128 and 64: four warps under one another; BM 16: side by side
    constexpr int MT = BM / (16 * WARPS_M);          // 16-row tiles per warp: 2 (BM 128: a weight fragment serves both) or 1
    constexpr int WARPS_N = (THREADS / 32) / WARPS_M;   // 2 (BM 128: eight warps), 1 or 4
    constexpr int WN = BN / WARPS_N;                 // columns per warp: 32, 64 or 16
    constexpr int NT = WN / 8;                       // n-tiles per warp: 4, 8 or 2
    constexpr int NB = DUAL ? 2 : 1;
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    typedef __nv_bfloat16 (*ATile)[BM][PITCH];
    typedef __nv_bfloat16 (*WTile)[NB][BN][PITCH];
    ATile As = reinterpret_cast<ATile>(smem_raw);                                                   // [STAGES][BM][PITCH]
    WTile Ws = reinterpret_cast<WTile>(smem_raw + (size_t)STAGES * BM * PITCH * sizeof(__nv_bfloat16));   // [STAGES][NB][BN][PITCH]
    int* src_row = reinterpret_cast<int*>(smem_raw + (size_t)STAGES * (BM + NB * BN) * PITCH * sizeof(__nv_bfloat16));
    int* dst_row = src_row + BM;
    int* tile_info = dst_row + BM;
    int* offsets_s = tile_info + 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (p.group_offsets) {                           // fetched by all threads at once, walked by one
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
    const __nv_bfloat16* A = p.A + (size_t)group * p.a_group_cols;
    const __nv_bfloat16* W = p.W + (size_t)group * p.w_group_stride;
    const int n0 = blockIdx.x * BN;
    const int k_tiles = (p.K + BK - 1) / BK;

    // Which pieces this thread copies never changes from one K tile to the next: their global addresses (null: zeros)
    // and their places in a stage are worked out once, a K tile only adds its offset.
    constexpr int A_PER = (BM * PIECES + THREADS - 1) / THREADS, W_PER = (BN * PIECES + THREADS - 1) / THREADS;
    const __nv_bfloat16* a_src[A_PER];
    const __nv_bfloat16* w_src[NB][W_PER];
    int a_dst[A_PER], w_dst[W_PER], a_k[A_PER], w_k[W_PER];
#pragma unroll
    for (int i = 0; i < A_PER; ++i) {
        const int e = tid + i * THREADS;
        const int row = (e / PIECES) % BM, piece = e % PIECES;
        const int a = e < BM * PIECES ? src_row[row] : -1;
        a_src[i] = a >= 0 ? A + (size_t)a * p.lda + piece * 8 : nullptr;
        a_dst[i] = e < BM * PIECES ? row * PITCH + piece * 8 : -1;
        a_k[i] = piece * 8;
    }
#pragma unroll
    for (int i = 0; i < W_PER; ++i) {
        const int e = tid + i * THREADS;
        const int row = (e / PIECES) % BN, piece = e % PIECES;
        const int n = n0 + row;
#pragma unroll
        for (int b = 0; b < NB; ++b)
            w_src[b][i] = (e < BN * PIECES && n < p.N) ? W + ((size_t)n + (size_t)b * p.dual_rows) * p.ldw + piece * 8 : nullptr;
        w_dst[i] = e < BN * PIECES ? row * PITCH + piece * 8 : -1;
        w_k[i] = piece * 8;
    }
    auto load_stage = [&](int stage, int kt) {
        const int k0 = kt * BK;
        __nv_bfloat16* a_stage = &As[stage][0][0];
#pragma unroll
        for (int i = 0; i < A_PER; ++i) {
            if (a_dst[i] < 0) continue;
            const bool ok = a_src[i] != nullptr && k0 + a_k[i] < p.K;
            cp_async16(a_stage + a_dst[i], ok ? (const void*)(a_src[i] + k0) : (const void*)p.A, ok);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            __nv_bfloat16* w_stage = &Ws[stage][b][0][0];
#pragma unroll
            for (int i = 0; i < W_PER; ++i) {
                if (w_dst[i] < 0) continue;
                const bool ok = w_src[b][i] != nullptr && k0 + w_k[i] < p.K;
                cp_async16(w_stage + w_dst[i], ok ? (const void*)(w_src[b][i] + k0) : (const void*)p.W, ok);
            }
        }
    };

    float acc[MT][NB][NT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[m][b][j][i] = 0.0f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < k_tiles) load_stage(s, s);
        cp_async_commit();
    }
    const int warp_m = warp % WARPS_M, warp_n = warp / WARPS_M;
    const int a_row = warp_m * 16 * MT + (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
    const int b_row = (lane & 7) + 8 * (lane >> 4), b_col = 8 * ((lane >> 3) & 1);
    for (int kt = 0; kt < k_tiles; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                              // stage kt has landed for everyone; stage kt-1 is free to refill
        if (kt + STAGES - 1 < k_tiles) load_stage((kt + STAGES - 1) % STAGES, kt + STAGES - 1);
        cp_async_commit();
        const int stage = kt % STAGES;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            unsigned a[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m) ldmatrix_x4(a[m], &As[stage][a_row + 16 * m][ks * 16 + a_col]);
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    unsigned w[4];
                    ldmatrix_x4(w, &Ws[stage][b][warp_n * WN + j * 8 + b_row][ks * 16 + b_col]);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        mma_bf16(acc[m][b][j], a[m], w[0], w[1]);
                        mma_bf16(acc[m][b][j + 1], a[m], w[2], w[3]);
                    }
                }
        }
    }
    cp_async_wait<0>();
    // accumulator element i of n-tile j: row (lane / 4) + 8 * (i / 2), column 2 * (lane % 4) + (i % 2)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int c = dst_row[warp_m * 16 * MT + 16 * m + (lane >> 2) + 8 * half];
        if (c < 0) continue;
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int n = n0 + warp_n * WN + j * 8 + 2 * (lane & 3) + i;
                if (n >= p.N) continue;
                const size_t col = (size_t)group * p.c_group_cols + n;
                float v = acc[m][0][j][half * 2 + i];
                if (DUAL) v = silu(v) * acc[m][NB - 1][j][half * 2 + i];
                if (p.factor) v *= p.factor[(size_t)c * p.ldf + col];
                ((OutT*)p.C)[(size_t)c * p.ldc + col] = from_f32<OutT>(v);
            }
    }
}

template <typename OutT, int BM, bool DUAL>
void launch_tile(const MmaParams& p, dim3 grid, cudaStream_t stream) {
    static bool configured[MAX_DEVICES] = {false};               // the larger tiles need more shared memory than the default limit
    constexpr size_t smem = smem_of(BM, DUAL);
    if (smem > 48 * 1024 && !configured[device_index()]) {
        cudaFuncSetAttribute(grouped_mma_kernel<OutT, BM, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured[device_index()] = true;
    }
    launch_kernel(grouped_mma_kernel<OutT, BM, DUAL>, grid, threads_of(BM), smem, stream, p);
}

template <typename OutT, bool DUAL>
void launch(const MmaParams& p, int row_tile, unsigned tiles_y, cudaStream_t stream) {
    dim3 grid((p.N + BN - 1) / BN, tiles_y);
    if (row_tile == 16) launch_tile<OutT, 16, DUAL>(p, grid, stream);
    else if (row_tile == 64) launch_tile<OutT, 64, DUAL>(p, grid, stream);
    else launch_tile<OutT, 128, DUAL>(p, grid, stream);
}

}  // namespace

// dual_rows > 0: W holds gate rows [0, N) and up rows [dual_rows, dual_rows + N) per group; C = silu(A gate^T) * (A up^T).
MLB_EXPORT int mlb_grouped_mma(const void* A, long long lda, long long a_group_cols, const void* W, long long ldw,
                               long long w_group_stride, void* C, long long ldc, long long c_group_cols,
                               const int* group_offsets, const int* a_rows, const int* c_rows, int a_row_div,
                               const float* factor, long long ldf, long long dual_rows, int M, int N, int K, int G,
                               int out_dtype, int row_tile, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || G <= 0 || a_row_div <= 0 || dual_rows < 0 || (row_tile != 16 && row_tile != 64 && row_tile != 128))
        return fail(MLB_INVALID_ARGUMENT, "grouped_mma: bad sizes M=%d N=%d K=%d G=%d", M, N, K, G);
    if (K % 8 || lda % 8 || ldw % 8 || a_group_cols % 8 || w_group_stride % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16)
        return fail(MLB_UNSUPPORTED_SIZE, "grouped_mma: K, the row pitches and the column blocks must be multiples of 8 elements");
    if (group_offsets && G > MAX_GROUPS) return fail(MLB_UNSUPPORTED_SIZE, "grouped_mma: more than %d groups", MAX_GROUPS);
    if (M == 0) return MLB_OK;
    MmaParams p{(const __nv_bfloat16*)A, lda, a_group_cols, (const __nv_bfloat16*)W, ldw, w_group_stride, C, ldc, c_group_cols,
                group_offsets, a_rows, c_rows, a_row_div, factor, ldf, dual_rows, M, N, K, G};
    const long long per = (M + row_tile - 1) / row_tile;
    const long long tiles = group_offsets ? per + G : per * G;
    if (tiles > 65535) return fail(MLB_UNSUPPORTED_SIZE, "grouped_mma: %lld row tiles exceed one launch", tiles);
    const bool dual = dual_rows > 0;
    if (out_dtype == MLB_F32) { if (dual) launch<float, true>(p, row_tile, (unsigned)tiles, stream); else launch<float, false>(p, row_tile, (unsigned)tiles, stream); }
    else if (out_dtype == MLB_BF16) { if (dual) launch<__nv_bfloat16, true>(p, row_tile, (unsigned)tiles, stream); else launch<__nv_bfloat16, false>(p, row_tile, (unsigned)tiles, stream); }
    else return fail(MLB_INVALID_ARGUMENT, "grouped_mma: unsupported output dtype %d", out_dtype);
    return check_launch("grouped_mma");
}
