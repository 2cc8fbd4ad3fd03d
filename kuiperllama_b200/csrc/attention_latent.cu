// Causal attention of many query heads over ONE key head whose values are the leading columns of its keys:
// what attention over a shared latent comes to once the per-head key and value maps have been moved to
// the query's and the result's side.  bfloat16, tensor cores (mma.sync m16n8k16), flash-attention form.
//
// A CTA of four warps holds 64 query rows of one sequence: TT consecutive tokens times HB heads (all heads
// when there are at most 64), so the cache rows a CTA fetches serve every head at once; for a decode step
// that is one token's heads.  Keys arrive page by page (64 rows of Dk columns) by cp.async into two
// buffers; S = Q K^T per warp (16 rows x 64 keys), softmax on the fly in 32 bits (running maximum and sum,
// exp2), P as the A operand straight from the accumulators, O += P V with V = the same page's first Dv
// columns read through ldmatrix.trans.  O stays in registers (16 x Dv per warp), so Dv <= 256 here; wider
// latents and float32 take the plain kernel (attention_simt.cu).  A sink per head joins the denominator at
// the end.  With a window a row sees the keys of its last `window` positions only, and a CTA starts at the page of its
// first token's first key.  In a decode step a sequence's pages are cut over several CTAs (split-KV) whose pieces a small kernel
// merges, so that few sequences still fill the machine.  Rows of shared memory are Dk + 8 elements apart, which keeps the eight rows of an ldmatrix on
// different banks when Dk is a multiple of 16.
//
// Every row's sums run over the pages in ascending order whatever the step brings, so the result does not
// depend on how a prompt was cut; it does differ from the plain kernel's in the last bits (bfloat16 P).
// ExiledOfCode/KuiperLLama's attention is one head per CTA with scores through global memory
// (mha_kernel.cu:61,74-106).
#include "common.cuh"

namespace kl {

constexpr int LA_ROWS = 64, LA_THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// NVT: value tiles of 8 columns a warp keeps (Dv <= 8 NVT).
template <int NVT>
__global__ void __launch_bounds__(LA_THREADS)
latent_attention_mma_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ cache,
                            const int* __restrict__ block_table, int blocks_per_seq, const int* __restrict__ cu_tokens,
                            const int* __restrict__ seq_slots, const int* __restrict__ seq_starts, const int* __restrict__ seq_new,
                            const float* __restrict__ sink, int H, int HB, int TT, int Dk, int Dv, float scale_log2,
                            int splits, float* __restrict__ part, int stages, int window) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int ld = Dk + 8;                                          // elements between rows of shared memory
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                   // [64][ld]
    bf16* Ks = Qs + (size_t)LA_ROWS * ld;                           // [stages][64][ld]

    const int s = blockIdx.z, n_new = seq_new[s], t0 = blockIdx.x * TT, h0 = (blockIdx.y / splits) * HB, piece = blockIdx.y % splits;
    const int slot = seq_slots[s];
    if (t0 >= n_new || slot < 0) return;
    const int start = seq_starts[s], row0 = cu_tokens[s];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = Dk / 8;                                      // 16-byte pieces per row
    const int* table = block_table + (size_t)slot * blocks_per_seq;
    const int tokens_here = min(TT, n_new - t0);
    // this CTA's pages: all of them, or (splits > 1, a decode step) one of `splits` runs of pages
    // (with a window: from the page that holds the first key the tile's first token still sees)
    const int all_pages = (start + t0 + tokens_here - 1) / PAGE + 1;
    const int low_page = window > 0 ? max(0, start + t0 - window + 1) / PAGE : 0;
    const int per = (all_pages - low_page + splits - 1) / splits;
    const int first_page = low_page + piece * per, last_page = min(all_pages, first_page + per) - 1;

    auto load_page = [&](int j, int buf) {
        const bf16* src = cache + (size_t)table[j] * PAGE * Dk;
        bf16* dst = Ks + (size_t)buf * LA_ROWS * ld;
        for (int e = threadIdx.x; e < PAGE * chunks; e += LA_THREADS) {
            const int r = e / chunks, c = e - r * chunks;
            cp_async16(dst + (size_t)r * ld + c * 8, src + (size_t)r * Dk + c * 8);
        }
    };
    if (first_page <= last_page) load_page(first_page, 0);
    cp_async_commit();
    // the query rows: row r is token t0 + r / HB, head h0 + r % HB; rows beyond the tile's tokens or heads are zeros
    for (int e = threadIdx.x; e < LA_ROWS * chunks; e += LA_THREADS) {
        const int r = e / chunks, c = e - r * chunks;
        const int tt = r / HB, h = h0 + r % HB;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (tt < tokens_here && h < H) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + t0 + tt) * H + h) * Dk + c * 8);
        *reinterpret_cast<uint4*>(Qs + (size_t)r * ld + c * 8) = v;
    }

    // this thread's two rows of the warp's 16: g and g + 8
    const int g = lane >> 2, quad = lane & 3;
    int pos[2], lo[2];
    bool live[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + g + 8 * i, tt = r / HB;
        live[i] = tt < tokens_here && h0 + r % HB < H;
        pos[i] = live[i] ? start + t0 + tt : -1;
        lo[i] = window > 0 ? max(0, pos[i] - window + 1) : 0;          // the first key the row sees
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[NVT][4];
#pragma unroll
    for (int n = 0; n < NVT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
    const int nv = Dv / 8;                                          // value tiles in use (uniform)

    for (int j = first_page; j <= last_page; ++j) {
        // two buffers: the next page is on its way while this one is worked on.  One buffer (prompts: two CTAs then fit a
        // multiprocessor and overlap each other's loads, softmax and products): the page is fetched here.
        const int buf = stages == 2 ? (j - first_page) & 1 : 0;
        if (stages == 2) {
            if (j < last_page) load_page(j + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            if (j > first_page) load_page(j, 0);
            cp_async_commit();
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* K = Ks + (size_t)buf * LA_ROWS * ld;
        // S = Q K^T: 16 rows x 64 keys per warp
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) sc[n][c] = 0.f;
        for (int k0 = 0; k0 < Dk; k0 += 16) {
            uint32_t a[4];
            ldmatrix_x4(a, Qs + (size_t)(warp * 16 + (lane & 15)) * ld + k0 + (lane >> 4) * 8);
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
                uint32_t b[4];
                ldmatrix_x4(b, K + (size_t)(n2 * 16 + (lane & 7) + (lane >> 4) * 8) * ld + k0 + ((lane >> 3) & 1) * 8);
                mma_bf16(sc[2 * n2], a, b[0], b[1]);
                mma_bf16(sc[2 * n2 + 1], a, b[2], b[3]);
            }
        }
        // scale, mask, running maximum and sum
        const int key0 = j * PAGE + 2 * quad;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = key0 + n * 8 + (c & 1);
                const float v = (key <= pos[c >> 1] && key >= lo[c >> 1]) ? sc[n][c] * scale_log2 : -INFINITY;
                sc[n][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
            }
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m[i], mx[i]);
            corr[i] = m_new == -INFINITY ? 1.f : exp2f(m[i] - m_new);      // exp2(-inf) = 0 at a row's first keys
            m[i] = m_new;
            l[i] *= corr[i];
        }
        uint32_t p[8][2];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            float e[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                e[c] = m[c >> 1] == -INFINITY ? 0.f : exp2f(sc[n][c] - m[c >> 1]);
                l[c >> 1] += e[c];
            }
            p[n][0] = pack_bf16(e[0], e[1]);
            p[n][1] = pack_bf16(e[2], e[3]);
        }
#pragma unroll
        for (int n = 0; n < NVT; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
        // O += P V, V = the page's first Dv columns
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t a[4] = {p[2 * ks][0], p[2 * ks][1], p[2 * ks + 1][0], p[2 * ks + 1][1]};
#pragma unroll
            for (int n2 = 0; n2 < NVT / 2; ++n2) {
                if (2 * n2 < nv) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, K + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + n2 * 16 + (lane >> 4) * 8);
                    mma_bf16(o[2 * n2], a, b[0], b[1]);
                    mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                            // the buffer is free for the page after next
    }
    cp_async_wait<0>();
    // the rows' sums over the quad, the sink's share, and out
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        if (!live[i]) continue;
        const int r = warp * 16 + g + 8 * i, tt = r / HB, h = h0 + r % HB;
        if (splits > 1) {
            // a piece: the sums as they are (relative to this piece's maximum), the maximum and the sum of weights
            float* pr = part + (((size_t)(row0 + t0 + tt) * H + h) * splits + piece) * (Dv + 2);
#pragma unroll
            for (int n = 0; n < NVT; ++n)
                if (n < nv) *reinterpret_cast<float2*>(pr + n * 8 + 2 * quad) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
            if (quad == 0) { pr[Dv] = m[i]; pr[Dv + 1] = l[i]; }
            continue;
        }
        float w = 1.f, denom = l[i];
        if (sink != nullptr) {
            const float sk = sink[h] * 1.4426950408889634f;           // in the exp2 domain, as the scores are
            const float top = fmaxf(m[i], sk);
            w = exp2f(m[i] - top);
            denom = l[i] * w + exp2f(sk - top);
        }
        const float f = w / denom;
        bf16* orow = out + ((size_t)(row0 + t0 + tt) * H + h) * Dv;
#pragma unroll
        for (int n = 0; n < NVT; ++n)
            if (n < nv) *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * quad) = pack_bf16(o[n][2 * i] * f, o[n][2 * i + 1] * f);
    }
}

// The pieces of a decode step's rows put together: a warp per (token, head); out = sum_p O_p 2^(m_p - M) / (sum_p l_p 2^(m_p - M) +
// 2^(sink - M)), M the largest of the maxima and the sink, pieces in ascending order.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ part, int splits, const float* __restrict__ sink, int rows, int H, int Dv,
                              bf16* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* pr = part + (size_t)row * splits * (Dv + 2);
    const float sk = sink ? sink[row % H] * 1.4426950408889634f : -INFINITY;
    // lane p holds piece p's maximum and sum of weights (splits <= 32), then its factor 2^(m_p - M)
    const float mp = lane < splits ? pr[(size_t)lane * (Dv + 2) + Dv] : -INFINITY;
    const float lp = lane < splits ? pr[(size_t)lane * (Dv + 2) + Dv + 1] : 0.f;
    const float M = fmaxf(warp_max(mp), sk);
    const float f = mp == -INFINITY ? 0.f : exp2f(mp - M);
    const float denom = warp_sum(lp * f) + (sink ? exp2f(sk - M) : 0.f);
    for (int d0 = 0; d0 < Dv; d0 += 32) {
        const int d = d0 + lane;
        float acc = 0.f;
#pragma unroll 8
        for (int p = 0; p < splits; ++p) {
            const float fp = __shfl_sync(0xffffffffu, f, p);
            if (d < Dv) acc = fmaf(pr[(size_t)p * (Dv + 2) + d], fp, acc);
        }
        if (d < Dv) out[(size_t)row * Dv + d] = __float2bfloat16_rn(acc / denom);
    }
}

// KL_LATENT_BUFFERS=2 in the environment keeps two page buffers for prompts too (for comparisons).
static bool latent_two_buffers() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("KL_LATENT_BUFFERS");
        v = (e != nullptr && e[0] == '2') ? 1 : 0;
    }
    return v != 0;
}

}  // namespace kl

using namespace kl;

// q: [tokens, H, Dk], out: [tokens, H, Dv], cache: [pages, 1, 64, Dk], all bfloat16; Dk % 16 == 0, Dv % 16 == 0, Dv <= 256
// and <= Dk.  scale multiplies the dot products; sink: float32 [H] or null; window: keys a token sees (0: all).  max_new: the most tokens a sequence brings.
// splits > 1 (a decode step: one token per sequence): every sequence's pages are cut into that many runs, each a CTA that
// leaves its sums in part (float32 [n_tokens * H][splits][Dv + 2]), and a second kernel puts the pieces together.
KL_API int kl_latent_attention_mma(const void* q, void* out, const void* cache, const int* block_table, int blocks_per_seq,
                                   const int* cu_tokens, const int* seq_slots, const int* seq_starts, const int* seq_new, int n_seqs,
                                   int max_new, const float* sink, int H, int Dk, int Dv, float scale, int splits, float* part,
                                   int n_tokens, int window, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return KL_OK;
    if (splits < 1 || splits > 32 || (splits > 1 && (part == nullptr || max_new != 1 || Dv % 2))) return KL_ERR_BAD_SIZE;
    if (H <= 0 || Dk % 16 || Dv % 16 || Dv <= 0 || Dv > 256 || Dv > Dk) return KL_ERR_BAD_SIZE;
    if ((((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) & 15) != 0) return KL_ERR_BAD_ALIGN;
    const int HB = H < LA_ROWS ? H : LA_ROWS, TT = LA_ROWS / HB;
    const dim3 grid((max_new + TT - 1) / TT, ((H + HB - 1) / HB) * splits, n_seqs);
    if (grid.y > 65535 || grid.z > 65535) return KL_ERR_BAD_SIZE;
    // prompts: one page buffer where that lets two CTAs share a multiprocessor; decode steps (a chain of pages per CTA): two
    const size_t one = (size_t)LA_ROWS * (Dk + 8) * sizeof(bf16);
    const int stages = (max_new > 1 && 2 * (2 * one + 1024) <= 220 * 1024 && !latent_two_buffers()) ? 1 : 2;
    const size_t smem = (size_t)(1 + stages) * one;
    if (smem > 220 * 1024) return KL_ERR_BAD_SIZE;
    const float scale_log2 = scale * 1.4426950408889634f;
#define KL_LA(NVT)                                                                                                            \
    do {                                                                                                                      \
        static size_t allowed = 0;                                                                                            \
        if (smem > allowed) {                                                                                                 \
            KL_CUDA(cudaFuncSetAttribute(latent_attention_mma_kernel<NVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            allowed = smem;                                                                                                   \
        }                                                                                                                     \
        launch_kernel(latent_attention_mma_kernel<NVT>, grid, LA_THREADS, smem, stream, (const bf16*)q, (bf16*)out,           \
                      (const bf16*)cache, block_table, blocks_per_seq, cu_tokens, seq_slots, seq_starts, seq_new, sink, H, HB, TT, \
                      Dk, Dv, scale_log2, splits, part, stages, window);                                                      \
    } while (0)
    if (Dv <= 64) KL_LA(8);
    else if (Dv <= 128) KL_LA(16);
    else if (Dv <= 192) KL_LA(24);
    else KL_LA(32);
#undef KL_LA
    KL_LAUNCH_CHECK();
    if (splits > 1) {
        const int rows = n_tokens * H;
        launch_kernel(latent_attention_merge_kernel, (rows + 3) / 4, 128, 0, stream, (const float*)part, splits, sink, rows, H, Dv, (bf16*)out);
        KL_LAUNCH_CHECK();
    }
    return KL_OK;
}
