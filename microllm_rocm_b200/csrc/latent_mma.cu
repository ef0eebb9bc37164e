// Latent attention on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 scores, weights and accumulation),
// for prompt portions and decoded tokens alike.  Compiled per model: -DLAT_R (latent width) -DLAT_DR (rotated width).
//
// All heads read the same cache rows (see latent.cu): a query row is one (token, head) pair, and q [T*H, Dk] /
// out [T*H, R] are plain row-major matrices with Dk = R + DR.  A CTA of four warps owns 16 consecutive query rows
// of ONE sequence (a work item: sequence, first row among the sequence's new rows) and walks the keys those rows may
// see in tiles of 32 at absolute multiples of 32, through a two-stage ring filled by cp.async straight from the pages.
//   scores   warp w multiplies every fourth 16-wide step of the contraction (w, w + 4, ...) for all 32 keys, with its
//            columns of Q held in registers as A fragments for the whole kernel; the four partial S[16 x 32] meet in
//            shared memory, and from there on warp w owns keys 8 w .. 8 w + 7
//   softmax  running maximum and sum per row in fp32; the warps meet in shared memory for the row's maximum and sum
//   values   P[16 x 32] goes to shared memory as bf16; each warp owns a quarter of the R output columns and adds
//            P V for them (V = the first R columns of the same cache rows, fetched with ldmatrix.trans)
// A sink (one learned number per head) enters the denominator once, with no value.
// With `splits` > 1 a work item's key tiles are divided among that many CTAs, which leave unnormalised partial
// outputs with their maximum and sum in a workspace; latent_merge_kernel puts them together (and adds the sink).
#include "common.cuh"

#ifndef LAT_R
#error "compile with -DLAT_R=<latent width> -DLAT_DR=<rotated width>"
#endif

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int R = LAT_R, DR = LAT_DR, DK = R + DR;
constexpr int BM = 16, BN = 32, KP = DK + 8, PP = BN + 8;      // padded pitches in elements
constexpr int WR = R / 4, NT = WR / 8;                          // output columns and n-tiles per warp
static_assert(BN * 4 == 128, "four threads per cache row of a key tile");
static_assert(R % 32 == 0 && DK % 16 == 0, "latent width must be a multiple of 32, latent + rotated a multiple of 16");

struct Params {
    const __nv_bfloat16* q; const __nv_bfloat16* pages; __nv_bfloat16* out;
    const float* sink;
    const int* seq_starts; const int* seq_pos0; const int* block_table; const int* work;   // work: (sequence, first row) pairs
    float* part_o; float* part_ml;         // [splits, rows, R] and [splits, rows, 2], rows = T * H
    int max_blocks, num_pages, page_size, heads, window, splits, total_rows;
    float scale;
    int* error_flag;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// STAGES key tiles are in shared memory or on their way: 2 for prompt portions (two CTAs share a multiprocessor), 4
// for decoding, where a CTA owns few tiles and has all of them in flight at once.
constexpr int KS = DK / 16;               // 16-wide steps along the score's contraction
constexpr int KW = (KS + 3) / 4;          // of which a warp takes every fourth: w, w + 4, ...
constexpr int SP = BN + 4;                // pitch of a row of partial scores, in floats

template <int STAGES>
struct Smem {
    __nv_bfloat16 k[STAGES][BN][KP];
    __nv_bfloat16 p[BM][PP];
    float part[4][BM][SP];                // each warp's partial scores of the tile
    float red_max[4][BM];
    float red_sum[4][BM];
};

template <int STAGES>
__global__ void __launch_bounds__(128)
latent_mma_kernel(Params p) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem<STAGES>& s = *reinterpret_cast<Smem<STAGES>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.work[2 * blockIdx.x], first_row = p.work[2 * blockIdx.x + 1];
    const int split = blockIdx.y;
    const int H = p.heads;
    const int seq_start = p.seq_starts[seq], n_new = p.seq_starts[seq + 1] - seq_start;
    const int pos0 = p.seq_pos0[seq];
    const int rows = min(BM, n_new * H - first_row);                       // rows of this tile that exist
    const size_t row_base = (size_t)seq_start * H + first_row;             // global (token, head) row of the tile's first row
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    // what the tile's rows may see: from the first row's lower edge to the last row's own position
    const int pos_first = pos0 + first_row / H, pos_last = pos0 + (first_row + rows - 1) / H;
    const int lo_tile = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int tile_first = lo_tile / BN, tile_count_all = pos_last / BN - tile_first + 1;
    const int t_begin = tile_first + (int)((long long)tile_count_all * split / p.splits);
    const int t_end = tile_first + (int)((long long)tile_count_all * (split + 1) / p.splits);

    // Q never touches shared memory: warp w multiplies the 16-wide steps w, w + 4, ... of the contraction for ALL 32 keys
    // of a tile, so it needs only those columns of Q, and keeps them as A fragments for the whole kernel
    // (fragment registers: (row g, k 2t..), (row g + 8, k 2t..), (row g, k 2t + 8..), (row g + 8, k 2t + 8..); g = lane / 4, t = lane % 4)
    unsigned qa[KW][4];
    {
        const int g = lane >> 2, t2 = 2 * (lane & 3);
        const __nv_bfloat16* q0 = p.q + (row_base + g) * DK;
        const __nv_bfloat16* q1 = p.q + (row_base + g + 8) * DK;
#pragma unroll
        for (int i = 0; i < KW; ++i) {
            const int col = (warp + 4 * i) * 16 + t2;
            const bool in = warp + 4 * i < KS;
            qa[i][0] = in && g < rows ? *reinterpret_cast<const unsigned*>(q0 + col) : 0u;
            qa[i][1] = in && g + 8 < rows ? *reinterpret_cast<const unsigned*>(q1 + col) : 0u;
            qa[i][2] = in && g < rows ? *reinterpret_cast<const unsigned*>(q0 + col + 8) : 0u;
            qa[i][3] = in && g + 8 < rows ? *reinterpret_cast<const unsigned*>(q1 + col + 8) : 0u;
        }
    }
    // Four threads share a cache row: each looks the row's page up ONCE per tile and copies every fourth 16-byte piece.
    auto load_keys = [&](int stage, int tile) {
        const int row = tid >> 2;
        const int kp = tile * BN + row;
        bool ok = kp >= lo_tile && kp <= pos_last;
        const __nv_bfloat16* src = p.pages;
        if (ok) {
            const int block = kp / p.page_size;
            const int page = block < p.max_blocks ? table[block] : -1;
            if (page < 0 || page >= p.num_pages) {
                if (p.error_flag) atomicExch(p.error_flag, 2);
                ok = false;
            } else {
                src = p.pages + ((size_t)page * p.page_size + kp % p.page_size) * DK;
            }
        }
#pragma unroll
        for (int piece = tid & 3; piece < DK / 8; piece += 4)
            cp_async16(&s.k[stage][row][piece * 8], ok ? src + piece * 8 : p.pages, ok);
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (t_begin + i < t_end) load_keys(i, t_begin + i);
        cp_async_commit();
    }

    // this thread's two rows (lane / 4 and lane / 4 + 8): position and lower edge of each
    int row_pos[2], row_lo[2];
    float m_run[2], l_run[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + 8 * h;
        const bool exists = r < rows;
        row_pos[h] = exists ? pos0 + (first_row + r) / H : -1;             // -1: sees nothing
        row_lo[h] = (p.window > 0 && row_pos[h] - p.window + 1 > 0) ? row_pos[h] - p.window + 1 : 0;
        const bool own_sink = p.sink != nullptr && p.splits == 1 && exists;
        m_run[h] = own_sink ? p.sink[(first_row + r) % H] : -INFINITY;
        l_run[h] = own_sink ? 1.0f : 0.0f;
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
    for (int tile = t_begin; tile < t_end; ++tile) {
        const int stage = (tile - t_begin) % STAGES;
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                    // this tile's keys have landed; the stage used last is free
        if (tile + STAGES - 1 < t_end) load_keys((tile - t_begin + STAGES - 1) % STAGES, tile + STAGES - 1);
        cp_async_commit();
        // ---- partial scores of all 32 keys over this warp's steps of the contraction (four independent accumulators)
        float sp[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) sp[j][i] = 0.0f;
#pragma unroll
        for (int i = 0; i < KW; ++i) {
            const int ks = warp + 4 * i;
            if (ks < KS) {                                  // the same for the whole warp
                unsigned b0[4], b1[4];
                ldmatrix_x4(b0, &s.k[stage][(lane & 7) + 8 * (lane >> 4)][ks * 16 + 8 * ((lane >> 3) & 1)]);
                ldmatrix_x4(b1, &s.k[stage][16 + (lane & 7) + 8 * (lane >> 4)][ks * 16 + 8 * ((lane >> 3) & 1)]);
                mma_bf16(sp[0], qa[i], b0[0], b0[1]);
                mma_bf16(sp[1], qa[i], b0[2], b0[3]);
                mma_bf16(sp[2], qa[i], b1[0], b1[1]);
                mma_bf16(sp[3], qa[i], b1[2], b1[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<float2*>(&s.part[warp][lane >> 2][j * 8 + 2 * (lane & 3)]) = make_float2(sp[j][0], sp[j][1]);
            *reinterpret_cast<float2*>(&s.part[warp][(lane >> 2) + 8][j * 8 + 2 * (lane & 3)]) = make_float2(sp[j][2], sp[j][3]);
        }
        __syncthreads();
        // ---- from here on warp w owns keys 8 w .. 8 w + 7 of the tile: their scores are the four warps' partial sums, in order
        float sc[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float2 v = *reinterpret_cast<const float2*>(&s.part[0][(lane >> 2) + 8 * h][warp * 8 + 2 * (lane & 3)]);
#pragma unroll
            for (int w2 = 1; w2 < 4; ++w2) {
                const float2 u = *reinterpret_cast<const float2*>(&s.part[w2][(lane >> 2) + 8 * h][warp * 8 + 2 * (lane & 3)]);
                v.x += u.x; v.y += u.y;
            }
            sc[2 * h] = v.x; sc[2 * h + 1] = v.y;
        }
        const int key0 = tile * BN + warp * 8 + 2 * (lane & 3);
        float part_max[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int kp = key0 + i;
                const bool seen = kp <= row_pos[h] && kp >= row_lo[h];
                sc[2 * h + i] = seen ? sc[2 * h + i] * p.scale : -INFINITY;
            }
            float v = fmaxf(sc[2 * h], sc[2 * h + 1]);
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
            part_max[h] = v;
        }
        if ((lane & 3) == 0) { s.red_max[warp][lane >> 2] = part_max[0]; s.red_max[warp][(lane >> 2) + 8] = part_max[1]; }
        __syncthreads();
        float corr[2], part_sum[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (lane >> 2) + 8 * h;
            const float m_new = fmaxf(fmaxf(fmaxf(s.red_max[0][r], s.red_max[1][r]), fmaxf(s.red_max[2][r], s.red_max[3][r])), m_run[h]);
            corr[h] = (m_run[h] == -INFINITY) ? 0.0f : expf(m_run[h] - m_new);      // m_new >= m_run; both -inf: nothing seen yet
            const float p0 = sc[2 * h] == -INFINITY ? 0.0f : expf(sc[2 * h] - m_new);
            const float p1 = sc[2 * h + 1] == -INFINITY ? 0.0f : expf(sc[2 * h + 1] - m_new);
            m_run[h] = m_new;
            *reinterpret_cast<__nv_bfloat162*>(&s.p[r][warp * 8 + 2 * (lane & 3)]) = __floats2bfloat162_rn(p0, p1);
            float v = p0 + p1;
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            part_sum[h] = v;
        }
        if ((lane & 3) == 0) { s.red_sum[warp][lane >> 2] = part_sum[0]; s.red_sum[warp][(lane >> 2) + 8] = part_sum[1]; }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (lane >> 2) + 8 * h;
            l_run[h] = l_run[h] * corr[h] + ((s.red_sum[0][r] + s.red_sum[1][r]) + (s.red_sum[2][r] + s.red_sum[3][r]));
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) { acc[j][0] *= corr[0]; acc[j][1] *= corr[0]; acc[j][2] *= corr[1]; acc[j][3] *= corr[1]; }
        // ---- this warp's quarter of the output columns: acc += P V
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            unsigned a[4];
            ldmatrix_x4(a, &s.p[a_row][ks * 16 + a_col]);
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                unsigned v[4];
                ldmatrix_x4_trans(v, &s.k[stage][ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][warp * WR + j * 8 + 8 * (lane >> 4)]);
                mma_bf16(acc[j], a, v[0], v[1]);
                if (j + 1 < NT) mma_bf16(acc[j + 1], a, v[2], v[3]);
            }
        }
    }
    cp_async_wait<0>();
    // ---- results
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + 8 * h;
        if (r >= rows) continue;
        const size_t g = row_base + r;
        if (p.splits == 1) {
            const float inv = l_run[h] > 0.0f ? 1.0f / l_run[h] : 0.0f;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int c = warp * WR + j * 8 + 2 * (lane & 3);
                *reinterpret_cast<__nv_bfloat162*>(p.out + g * R + c) = __floats2bfloat162_rn(acc[j][2 * h] * inv, acc[j][2 * h + 1] * inv);
            }
        } else {
            float* o = p.part_o + ((size_t)split * p.total_rows + g) * R;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int c = warp * WR + j * 8 + 2 * (lane & 3);
                *reinterpret_cast<float2*>(o + c) = make_float2(acc[j][2 * h], acc[j][2 * h + 1]);
            }
            if (warp == 0 && (lane & 3) == 0) {
                float* ml = p.part_ml + ((size_t)split * p.total_rows + g) * 2;
                ml[0] = m_run[h]; ml[1] = l_run[h];
            }
        }
    }
}

// out[g, :] = sum_s O_s e^(m_s - m) / (sum_s l_s e^(m_s - m) + e^(sink - m)),  m = max(m_s, sink); splits in order.
// One block per row; the splits' weights are worked out once, then every thread sums four columns.
constexpr int MAX_SPLITS = 64;
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sink,
                    __nv_bfloat16* __restrict__ out, int splits, int total_rows, int heads) {
    pdl_prologue();
    __shared__ float weight[MAX_SPLITS];
    const int g = blockIdx.x;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float ms[MAX_SPLITS / 32], ls[MAX_SPLITS / 32];
        float m = sink ? sink[g % heads] : -INFINITY;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS / 32; ++i) {
            const int sp = lane + 32 * i;
            ms[i] = -INFINITY; ls[i] = 0.0f;
            if (sp < splits) {
                const float2 v = *reinterpret_cast<const float2*>(part_ml + ((size_t)sp * total_rows + g) * 2);
                ms[i] = v.x; ls[i] = v.y;
            }
            m = fmaxf(m, ms[i]);
        }
        m = warp_max(m);
        float l = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS / 32; ++i) {
            ms[i] = ms[i] == -INFINITY ? 0.0f : expf(ms[i] - m);
            l += ls[i] * ms[i];
        }
        l = warp_sum(l) + (sink ? expf(sink[g % heads] - m) : 0.0f);
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS / 32; ++i)
            if (lane + 32 * i < splits) weight[lane + 32 * i] = ms[i] * inv;
    }
    __syncthreads();
    for (int c = threadIdx.x * 4; c < R; c += blockDim.x * 4) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < splits; ++sp) {
            const float4 v = *reinterpret_cast<const float4*>(part_o + ((size_t)sp * total_rows + g) * R + c);
            const float w = weight[sp];
            o.x = fmaf(v.x, w, o.x); o.y = fmaf(v.y, w, o.y); o.z = fmaf(v.z, w, o.z); o.w = fmaf(v.w, w, o.w);
        }
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)g * R + c) = __floats2bfloat162_rn(o.x, o.y);
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)g * R + c + 2) = __floats2bfloat162_rn(o.z, o.w);
    }
}

template <int STAGES>
int launch_attention(const Params& p, int num_work, cudaStream_t stream) {
    static bool configured[MAX_DEVICES] = {false};
    const size_t smem = sizeof(Smem<STAGES>);
    if (!configured[device_index()]) {
        if (cudaFuncSetAttribute(latent_mma_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return fail(MLB_UNSUPPORTED_SIZE, "latent_attention_mma: %zu bytes of shared memory per CTA are not available", smem);
        configured[device_index()] = true;
    }
    launch_kernel(latent_mma_kernel<STAGES>, dim3(num_work, p.splits), 128, smem, stream, p);
    return check_launch("latent_attention_mma");
}

}  // namespace

MLB_EXPORT int mlb_latent_mma_widths(int which) { return which == 0 ? R : DR; }

// q [T*H, R+DR] bf16, pages [num_pages, page_size, R+DR] bf16, out [T*H, R] bf16.  work: num_work (sequence, first row)
// pairs, each a tile of up to 16 (token, head) rows of one sequence.  splits > 1 needs part_o [splits, T*H, R] and
// part_ml [splits, T*H, 2] fp32.
MLB_EXPORT int mlb_latent_attention_mma(const void* q, const void* pages, void* out, const float* sink, const int* seq_starts,
                                        const int* seq_pos0, const int* block_table, const int* work, int num_work,
                                        float* part_o, float* part_ml, int max_blocks, int num_pages, int page_size,
                                        int heads, int window, int splits, int total_rows, float scale, int* error_flag,
                                        cudaStream_t stream) {
    if (num_work < 0 || heads <= 0 || splits < 1 || splits > MAX_SPLITS || total_rows < 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0)
        return fail(MLB_INVALID_ARGUMENT, "latent_attention_mma: bad sizes");
    if (splits > 1 && (!part_o || !part_ml)) return fail(MLB_INVALID_ARGUMENT, "latent_attention_mma: split keys need a workspace");
    if (num_work == 0) return MLB_OK;
    Params p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, (__nv_bfloat16*)out, sink, seq_starts, seq_pos0, block_table, work,
             part_o, part_ml, max_blocks, num_pages, page_size, heads, window, splits, total_rows, scale, error_flag};
    // shared keys: few tiles per CTA, all of them in flight at once (if four stages fit this device's shared memory)
    const bool deep = splits > 1 && sizeof(Smem<4>) <= 200 * 1024;
    int status = deep ? launch_attention<4>(p, num_work, stream) : launch_attention<2>(p, num_work, stream);
    if (status != MLB_OK || splits == 1) return status;
    launch_kernel(latent_merge_kernel, total_rows, 128, 0, stream, (const float*)part_o, (const float*)part_ml, sink,
                  (__nv_bfloat16*)out, splits, total_rows, heads);
    return check_launch("latent_merge");
}
