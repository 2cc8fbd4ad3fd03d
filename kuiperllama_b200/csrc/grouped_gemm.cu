// Many small matrix products in one launch: C_g = A_g W_g^T for groups g that each have weights of
// their own, [N, K] row-major as everywhere in this package.  Two ways to say which rows belong to
// which group:
//
//   * batched (tile_group == null): every group takes all M rows; group g reads the columns of A that
//     start at g * a_gs and writes the columns of C that start at g * c_gs.  This is a per-head
//     projection ([tokens, heads, k] x [heads, n, k]) or a block-diagonal matrix.
//   * routed (tile_group given): the rows are positions of a list that is sorted by group and padded
//     so that every tile of BM rows lies in one group; tile_group[tile] names it (-1: no rows) and
//     a_rows[position] the row of A to read (-1: padding; null: the position itself).  This is a
//     mixture of experts: the list holds (token, choice) pairs.
//
// Epilogues: plain (optionally times sigmoid of one number per row and group, `row_gate`: a head's output gate on a
// per-head projection, or with `gate_elems` of one number per row and output, at column group * N + n of the gate's row; optionally an activation of the result, `act` 1: the squared relu max(y, 0)^2), or a gated activation over weights that hold N gate rows followed by N up rows (or,
// `interleaved`, blocks of 64 gate rows each followed by the 64 up rows of the same outputs, N % 64 == 0):
//     g = min(gate, limit), u = clamp(up, -limit, limit) (no clamp when limit <= 0),
//     y = g * sigmoid(alpha * g) * (u + shift).
// Arithmetic is 32-bit FMA for both dtypes; every output is one thread's sum in ascending k, so a row's
// result does not depend on which other rows share its tile.  ExiledOfCode/KuiperLLama has single
// products alone (matmul_kernel.cu:6-54).
#include "common.cuh"

namespace kl {

constexpr int GG_BN = 64, GG_BK = 16, GG_THREADS = 256;
enum : int { GG_PLAIN = 0, GG_GATED = 1 };

template <typename TI, typename TO, int BM, int EPI>
__global__ void __launch_bounds__(GG_THREADS)
grouped_gemm_kernel(const TI* __restrict__ A, long long lda, long long a_gs, const int* __restrict__ a_rows,
                    const TI* __restrict__ W, long long w_gs, TO* __restrict__ C, long long ldc, long long c_gs,
                    const int* __restrict__ tile_group, int M, int N, int K, float limit, float alpha, float shift, int interleaved,
                    const TI* __restrict__ row_gate, long long gate_ld, int act, int gate_elems) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int RM = BM / 16;                                   // rows per thread
    __shared__ float As[GG_BK][BM + 4];
    __shared__ float Ws[EPI == GG_GATED ? 2 : 1][GG_BK][GG_BN + 4];
    __shared__ int src[BM];
    const int g = tile_group ? tile_group[blockIdx.y] : (int)blockIdx.z;
    if (g < 0) return;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * GG_BN;
    for (int i = threadIdx.x; i < BM; i += GG_THREADS) {
        const int m = m0 + i;
        src[i] = m < M ? (a_rows ? a_rows[m] : m) : -1;
    }
    __syncthreads();
    const TI* Ag = A + (size_t)g * a_gs;
    const TI* Wg = W + (size_t)g * w_gs;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[EPI == GG_GATED ? 2 : 1][RM][4];
#pragma unroll
    for (int z = 0; z < (EPI == GG_GATED ? 2 : 1); ++z)
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[z][i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        for (int e = threadIdx.x; e < BM * GG_BK; e += GG_THREADS) {
            const int row = e / GG_BK, kk = e % GG_BK, gk = k0 + kk;
            const int s = src[row];
            As[kk][row] = (s >= 0 && gk < K) ? to_f32(Ag[(size_t)s * lda + gk]) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = threadIdx.x + r * GG_THREADS;
            const int row = e / GG_BK, kk = e % GG_BK, gn = n0 + row, gk = k0 + kk;
            const bool ok = gn < N && gk < K;
            // gate rows then up rows, or (interleaved) 64 gate rows, the 64 up rows of the same outputs, and so on
            const size_t gate_row = (EPI == GG_GATED && interleaved) ? (size_t)(gn / 64) * 128 + gn % 64 : (size_t)gn;
            const size_t up_row = interleaved ? gate_row + 64 : (size_t)N + gn;
            Ws[0][kk][row] = ok ? to_f32(Wg[gate_row * K + gk]) : 0.f;
            if (EPI == GG_GATED) Ws[1][kk][row] = ok ? to_f32(Wg[up_row * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[RM];
#pragma unroll
            for (int i = 0; i < RM; ++i) a[i] = As[kk][ty * RM + i];
#pragma unroll
            for (int z = 0; z < (EPI == GG_GATED ? 2 : 1); ++z) {
                float b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Ws[z][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < RM; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[z][i][j] = fmaf(a[i], b[j], acc[z][i][j]);
            }
        }
        __syncthreads();
    }
    TO* Cg = C + (size_t)g * c_gs;
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        const int row = ty * RM + i;
        if (src[row] < 0) continue;
        TO* crow = Cg + (size_t)(m0 + row) * ldc;
        // one number per row and group on the result (a head's output gate), if given
        // (with gate_elems: one number per row and output instead, at column g * N + n of the gate's row)
        const float rg = (row_gate && !gate_elems) ? 1.0f / (1.0f + expf(-to_f32(row_gate[(size_t)(m0 + row) * gate_ld + g]))) : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float y = acc[0][i][j] * rg;
            if (row_gate && gate_elems) y *= 1.0f / (1.0f + expf(-to_f32(row_gate[(size_t)(m0 + row) * gate_ld + (size_t)g * N + gn])));
            if (EPI != GG_GATED && act == 1) y = y > 0.f ? y * y : 0.f;      // the plain epilogue's activation: squared relu
            if (EPI == GG_GATED) {
                float gt = y, up = acc[1][i][j];
                if (limit > 0.f) { gt = fminf(gt, limit); up = fminf(fmaxf(up, -limit), limit); }
                y = gt / (1.0f + expf(-alpha * gt)) * (up + shift);
            }
            crow[gn] = from_f32<TO>(y);
        }
    }
}

// The batched form on the tensor cores (bfloat16, mma.sync m16n8k16, 32-bit sums): per-head projections of a prompt's rows,
// whose k and n are a head's sizes (tens to hundreds) and whose groups are the heads.  A CTA of four warps makes a tile of
// 64 rows x 64 outputs of one group, 64 k at a time through shared memory (rows 72 elements apart: no bank conflicts for
// ldmatrix); each warp 16 rows x 64 outputs.  Operands' rows and group offsets must lie on 16-byte boundaries.
__device__ __forceinline__ void gg_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void gg_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int GM_TILE = 64, GM_LD = 72;

__global__ void __launch_bounds__(128)
grouped_gemm_mma_kernel(const bf16* __restrict__ A, long long lda, long long a_gs, const bf16* __restrict__ W, long long w_gs,
                        bf16* __restrict__ C, long long ldc, long long c_gs, int M, int N, int K,
                        const bf16* __restrict__ row_gate, long long gate_ld, int gate_elems) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) bf16 As[GM_TILE][GM_LD];
    __shared__ __align__(16) bf16 Ws[GM_TILE][GM_LD];
    const int g = blockIdx.z, m0 = blockIdx.y * GM_TILE, n0 = blockIdx.x * GM_TILE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* Ag = A + (size_t)g * a_gs;
    const bf16* Wg = W + (size_t)g * w_gs;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[n][c] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GM_TILE) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 128, r = e >> 3, c = (e & 7) * 8;      // 64 rows x 8 pieces of 16 bytes
            uint4 va = make_uint4(0u, 0u, 0u, 0u), vw = va;
            if (k0 + c < K) {
                if (m0 + r < M) va = *reinterpret_cast<const uint4*>(Ag + (size_t)(m0 + r) * lda + k0 + c);
                if (n0 + r < N) vw = *reinterpret_cast<const uint4*>(Wg + (size_t)(n0 + r) * K + k0 + c);
            }
            *reinterpret_cast<uint4*>(&As[r][c]) = va;
            *reinterpret_cast<uint4*>(&Ws[r][c]) = vw;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GM_TILE; kk += 16) {
            if (k0 + kk >= K) break;
            uint32_t a[4];
            gg_ldmatrix_x4(a, &As[warp * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
                uint32_t b[4];
                gg_ldmatrix_x4(b, &Ws[n2 * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
                gg_mma_bf16(acc[2 * n2], a, b[0], b[1]);
                gg_mma_bf16(acc[2 * n2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    bf16* Cg = C + (size_t)g * c_gs;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = m0 + warp * 16 + (lane >> 2) + 8 * i;
        if (row >= M) continue;
        const float rg = (row_gate && !gate_elems) ? 1.0f / (1.0f + expf(-to_f32(row_gate[(size_t)row * gate_ld + g]))) : 1.0f;
        const bf16* erow = (row_gate && gate_elems) ? row_gate + (size_t)row * gate_ld + (size_t)g * N : nullptr;     // a gate number per output
        auto eg = [&](int col) { return erow ? 1.0f / (1.0f + expf(-to_f32(erow[col]))) : 1.0f; };
        bf16* crow = Cg + (size_t)row * ldc;
        const bool pairs = (((uintptr_t)Cg | (uintptr_t)(ldc * 2)) & 3) == 0;      // two neighbours as one 4-byte store
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const int col = n0 + n * 8 + 2 * (lane & 3);
            if (pairs && col + 1 < N) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(acc[n][2 * i] * rg * eg(col), acc[n][2 * i + 1] * rg * eg(col + 1));
                *reinterpret_cast<__nv_bfloat162*>(crow + col) = v;
            } else {
                if (col < N) crow[col] = __float2bfloat16_rn(acc[n][2 * i] * rg * eg(col));
                if (col + 1 < N) crow[col + 1] = __float2bfloat16_rn(acc[n][2 * i + 1] * rg * eg(col + 1));
            }
        }
    }
}

// Few rows per group (a decode step's experts): the product is bound by reading each group's weights once.
// A warp takes four weight rows (four outputs, or two outputs' gate and up rows), every lane 16 bytes of each
// row per step, and multiplies them with up to GV_ROWS list places of the tile at once (their rows of A come
// from L1 after the first touch); shuffles add the lanes.  bfloat16 operands, 32-bit sums, K % 8 == 0.
constexpr int GV_ROWS = 8, GV_WARPS = 8;

__device__ __forceinline__ void bf16x8_to_float(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(p[j]);
        f[2 * j] = v.x;
        f[2 * j + 1] = v.y;
    }
}

template <typename TO, bool GATED>
__global__ void __launch_bounds__(GV_WARPS * 32)
grouped_gemv_kernel(const bf16* __restrict__ A, long long lda, const int* __restrict__ a_rows, const int* __restrict__ live_rows,
                    const bf16* __restrict__ W, long long w_gs,
                    TO* __restrict__ C, long long ldc, const int* __restrict__ tile_group, int tile_rows, int N, int K,
                    float limit, float alpha, float shift, int interleaved, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int g = tile_group[blockIdx.y];
    if (g < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int OUTS = GATED ? 2 : 4;                           // outputs per warp
    const int n0 = (blockIdx.x * GV_WARPS + warp) * OUTS;
    if (n0 >= N) return;
    const bf16* Wg = W + (size_t)g * w_gs;
    const bf16* wrow[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        int n = min(n0 + (GATED ? c / 2 : c), N - 1);
        size_t row = n;
        if (GATED) {
            const size_t gate_row = interleaved ? (size_t)(n / 64) * 128 + n % 64 : (size_t)n;
            row = (c & 1) ? (interleaved ? gate_row + 64 : (size_t)N + n) : gate_row;
        }
        wrow[c] = Wg + row * K;
    }
    const int m0 = blockIdx.y * tile_rows;
    for (int r0 = 0; r0 < tile_rows; r0 += GV_ROWS) {
        int src[GV_ROWS];
        bool any = false;
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
            const int place = m0 + r0 + r;
            src[r] = -1;
            if (r0 + r < tile_rows) src[r] = a_rows ? a_rows[place] : (live_rows == nullptr || live_rows[place] >= 0 ? place : -1);
            any = any || src[r] >= 0;
        }
        if (!any) continue;
        float acc[GV_ROWS][4];
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
        // two steps of 256 columns at a time: eight 16-byte loads of weights in flight per lane (four steps at a time
        // were measured slower: 119 against 76 us for 16 experts' gate and up rows of 2,048 x 2,048, the registers cost warps)
        for (int k = lane * 8; k < K; k += 512) {
            const bool second = k + 256 < K;
            uint4 raw[2][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                raw[0][c] = *reinterpret_cast<const uint4*>(wrow[c] + k);
                raw[1][c] = second ? *reinterpret_cast<const uint4*>(wrow[c] + k + 256) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (h == 1 && !second) break;
                float w[4][8];
#pragma unroll
                for (int c = 0; c < 4; ++c) bf16x8_to_float(raw[h][c], w[c]);
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r) {
                    if (src[r] < 0) continue;
                    float x[8];
                    bf16x8_to_float(*reinterpret_cast<const uint4*>(A + (size_t)src[r] * lda + k + 256 * h), x);
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[r][c] = fmaf(x[j], w[c][j], acc[r][c]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
            if (src[r] < 0) continue;
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][c] = warp_sum(acc[r][c]);
            if (lane != 0) continue;
            TO* crow = C + (size_t)(m0 + r0 + r) * ldc;
            if (GATED) {
#pragma unroll
                for (int o = 0; o < 2; ++o) {
                    if (n0 + o >= N) continue;
                    float gt = acc[r][2 * o], up = acc[r][2 * o + 1];
                    if (limit > 0.f) { gt = fminf(gt, limit); up = fminf(fmaxf(up, -limit), limit); }
                    crow[n0 + o] = from_f32<TO>(gt / (1.0f + expf(-alpha * gt)) * (up + shift));
                }
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (n0 + c < N) crow[n0 + c] = from_f32<TO>(act == 1 ? (acc[r][c] > 0.f ? acc[r][c] * acc[r][c] : 0.f) : acc[r][c]);
            }
        }
    }
}

}  // namespace kl

using namespace kl;

// The batched product on the tensor cores (see grouped_gemm_mma_kernel): bfloat16 in and out, K % 8 == 0, rows and group
// offsets of A on 16-byte boundaries.
KL_API int kl_grouped_gemm_mma(const void* A, long long lda, long long a_gs, const void* W, long long w_gs, void* C, long long ldc,
                               long long c_gs, int groups, int M, int N, int K, const void* row_gate, long long gate_ld,
                               int gate_elems, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || groups <= 0) return KL_OK;
    if (K <= 0 || K % 8 || lda % 8 || a_gs % 8 || w_gs % 8) return KL_ERR_BAD_ALIGN;
    if ((((uintptr_t)A | (uintptr_t)W) & 15) != 0) return KL_ERR_BAD_ALIGN;
    const dim3 grid((N + GM_TILE - 1) / GM_TILE, (M + GM_TILE - 1) / GM_TILE, groups);
    if (grid.y > 65535 || grid.z > 65535) return KL_ERR_BAD_SIZE;
    launch_kernel(grouped_gemm_mma_kernel, grid, 128, 0, stream, (const bf16*)A, lda, a_gs, (const bf16*)W, w_gs, (bf16*)C, ldc, c_gs,
                  M, N, K, (const bf16*)row_gate, gate_ld, gate_elems);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// The routed product for few rows per group (see grouped_gemv_kernel): bfloat16 operands with 16-byte aligned rows.
// a_rows: the row of A every list place reads (-1: padding); or null: the place itself, where live_rows (if given) is not negative.
KL_API int kl_grouped_gemv(const void* A, long long lda, const int* a_rows, const int* live_rows, const void* W, long long w_gs, void* C, long long ldc,
                           const int* tile_group, int tiles, int tile_rows, int N, int K, int gated, float limit, float alpha,
                           float shift, int interleaved, int out_dtype, int act, cudaStream_t stream) {
    if (tiles <= 0 || N <= 0) return KL_OK;
    if (act != 0 && (act != 1 || gated)) return KL_ERR_BAD_SIZE;
    if (K <= 0 || K % 8 || lda % 8 || tile_rows <= 0 || tile_group == nullptr || (interleaved && (!gated || N % 64))) return KL_ERR_BAD_SIZE;
    if ((((uintptr_t)A | (uintptr_t)W) & 15) != 0) return KL_ERR_BAD_ALIGN;
    if (tiles > 65535) return KL_ERR_BAD_SIZE;
    const int per_cta = GV_WARPS * (gated ? 2 : 4);
    const dim3 grid((N + per_cta - 1) / per_cta, tiles);
#define KL_GV(TO, G)                                                                                                      \
    launch_kernel(grouped_gemv_kernel<TO, G>, grid, GV_WARPS * 32, 0, stream, (const bf16*)A, lda, a_rows, live_rows, (const bf16*)W, w_gs, \
                  (TO*)C, ldc, tile_group, tile_rows, N, K, limit, alpha, shift, interleaved, act)
    if (out_dtype == KL_BF16) { if (gated) KL_GV(bf16, true); else KL_GV(bf16, false); }
    else if (out_dtype == KL_F32) { if (gated) KL_GV(float, true); else KL_GV(float, false); }
    else return KL_ERR_BAD_DTYPE;
#undef KL_GV
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// groups: the number of groups of a batched call (ignored for a routed one, whose tile_group has
// `tiles` entries).  gated: 0 plain (W_g is [N, K]), 1 gated activation (W_g is [2 N, K]).  act: the plain
// epilogue's activation (0 none, 1 squared relu).
KL_API int kl_grouped_gemm(const void* A, long long lda, long long a_gs, const int* a_rows, const void* W, long long w_gs,
                           void* C, long long ldc, long long c_gs, const int* tile_group, int tiles, int tile_rows, int groups,
                           int M, int N, int K, int gated, float limit, float alpha, float shift, int interleaved, const void* row_gate,
                           long long gate_ld, int in_dtype, int out_dtype, int act, int gate_elems, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KL_OK;
    if (act != 0 && (act != 1 || gated)) return KL_ERR_BAD_SIZE;
    if (K <= 0 || (tile_rows != 16 && tile_rows != 64) || (interleaved && (!gated || N % 64))) return KL_ERR_BAD_SIZE;
    const int my = tile_group ? tiles : (M + tile_rows - 1) / tile_rows;
    const int gz = tile_group ? 1 : groups;
    if (my <= 0 || gz <= 0) return KL_OK;
    if (my > 65535 || gz > 65535) return KL_ERR_BAD_SIZE;
    const dim3 grid((N + GG_BN - 1) / GG_BN, my, gz);
#define KL_GG(TI, TO, BM, EPI)                                                                                              \
    launch_kernel(grouped_gemm_kernel<TI, TO, BM, EPI>, grid, GG_THREADS, 0, stream, (const TI*)A, lda, a_gs, a_rows,         \
                  (const TI*)W, w_gs, (TO*)C, ldc, c_gs, tile_group, M, N, K, limit, alpha, shift, interleaved, (const TI*)row_gate, gate_ld, act, gate_elems)
#define KL_GG_BY(TI, TO)                                                                                                    \
    do {                                                                                                                    \
        if (tile_rows == 16) { if (gated) KL_GG(TI, TO, 16, GG_GATED); else KL_GG(TI, TO, 16, GG_PLAIN); }                  \
        else { if (gated) KL_GG(TI, TO, 64, GG_GATED); else KL_GG(TI, TO, 64, GG_PLAIN); }                                  \
    } while (0)
    if (in_dtype == KL_F32 && out_dtype == KL_F32) KL_GG_BY(float, float);
    else if (in_dtype == KL_BF16 && out_dtype == KL_BF16) KL_GG_BY(bf16, bf16);
    else if (in_dtype == KL_BF16 && out_dtype == KL_F32) KL_GG_BY(bf16, float);
    else return KL_ERR_BAD_DTYPE;
#undef KL_GG_BY
#undef KL_GG
    KL_LAUNCH_CHECK();
    return KL_OK;
}
