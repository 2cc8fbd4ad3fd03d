// Attention over a window of recent keys and, before the window, one pooled key and value per block of
// positions; plain SIMT arithmetic in 32 bits, for both dtypes.
//
// Query token t of slot s at position p sees
//   * the keys j with 0 <= p - j < window (all keys up to p without a window), and
//   * for every block b of `pool` positions that lies wholly before the window, (b + 1) pool - 1 <= p - window,
//     the block's mean key and mean value (rows in the cache's dtype that pool_blocks_kernel wrote, from 32-bit sums,
//     when the block's last position arrived; a position that has left the window while its block is still incomplete is not seen).
// Pooled rows and keys are treated alike: score = (q . k) * scale, and the weight of what is seen is either
//   softmax over everything seen, optionally with a sink exp(sink[h]) in the denominator, or
//   sigmoid(score + head_bias[h]), not normalised over the keys.
// Head h reads kv head h / (H / KV).  One CTA of four warps per (token, query head); the pooled rows and the
// keys are cut into chunks of 32 by their own index and dealt to the warps in turn, so the order of every sum
// depends on the token's position alone: not on the step's cut, the batch or the pages.
// ExiledOfCode/KuiperLLama's attention reads every earlier key with a softmax (mha_kernel.cu:61,74-106).
#include "common.cuh"

namespace kl {

constexpr int AP_WARPS = 4;
constexpr int AP_MAX_VALUE_DIM = 512;

template <typename TK>
__device__ __forceinline__ float ap_dot(const TK* __restrict__ k, const float* __restrict__ q, int hd) {
    float s = 0.f;
    if constexpr (sizeof(TK) == 4) {
        if ((hd & 3) == 0) {
            for (int i = 0; i < hd; i += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(k + i);
                s += kv.x * q[i] + kv.y * q[i + 1] + kv.z * q[i + 2] + kv.w * q[i + 3];
            }
            return s;
        }
    } else {
        if ((hd & 7) == 0) {
            for (int i = 0; i < hd; i += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(p[j]);
                    s += f.x * q[i + 2 * j] + f.y * q[i + 2 * j + 1];
                }
            }
            return s;
        }
    }
    for (int i = 0; i < hd; ++i) s += to_f32(k[i]) * q[i];
    return s;
}

// One chunk of up to 32 rows (lane j holds row j's weight or score): folds it into the warp's running state.
template <typename TV, int PL, bool SIGMOID>
__device__ __forceinline__ void ap_fold(float s, bool valid, int j_lo, int j_hi, const TV* __restrict__ vbase, int v_ld, int vd,
                                        float bias, float& m, float& l, float (&acc)[PL]) {
    const int lane = threadIdx.x & 31;
    float p;
    if (SIGMOID) {
        p = valid ? 1.0f / (1.0f + expf(-(s + bias))) : 0.f;
    } else {
        const float m_new = fmaxf(m, warp_max(valid ? s : -INFINITY));
        const float corr = expf(m - m_new);                          // exp(-inf) = 0 at the first chunk
        p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < PL; ++i) acc[i] *= corr;
    }
    for (int j = j_lo; j <= j_hi; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const TV* vrow = vbase + (size_t)j * v_ld;
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int d = lane + 32 * i;
            if (d < vd) acc[i] += pj * to_f32(vrow[d]);
        }
    }
}

template <typename T, int PL, bool SIGMOID>
__global__ void __launch_bounds__(AP_WARPS * 32)
attention_pooled_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out,
                        const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        const int* __restrict__ block_table, int blocks_per_seq,
                        const T* __restrict__ pool_k, const T* __restrict__ pool_v,
                        const int* __restrict__ pool_table, int pool_blocks_per_seq, int pool,
                        const int* __restrict__ positions, const int* __restrict__ token_slot,
                        int H, int KV, int hd, float scale, int window, int vd,
                        const float* __restrict__ sink, const float* __restrict__ head_bias) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* q_s = smem;                               // [hd]
    float* m_s = q_s + hd;                           // [AP_WARPS]
    float* l_s = m_s + AP_WARPS;                     // [AP_WARPS]
    float* acc_s = l_s + AP_WARPS;                   // [AP_WARPS][vd]

    const int t = blockIdx.x, h = blockIdx.y;
    const int slot = token_slot[t];
    if (slot < 0) return;                            // a padding row: nothing is written
    const int pos = positions[t];
    const int g = h / (H / KV);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) q_s[i] = to_f32(qrow[i]);
    __syncthreads();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_blocks = (window > 0 && pool > 0) ? max(0, pos - window + 1) / pool : 0;     // blocks wholly before the window
    const int pool_chunks = (n_blocks + 31) / 32;
    const int first_chunk = lo / 32, key_chunks = pos / 32 - first_chunk + 1;
    const float bias = head_bias ? head_bias[h] : 0.f;
    float m = -INFINITY, l = 0.f;
    float acc[PL];
#pragma unroll
    for (int i = 0; i < PL; ++i) acc[i] = 0.f;

    const int* table = block_table + (size_t)slot * blocks_per_seq;
    const int* ptable = pool_table ? pool_table + (size_t)slot * pool_blocks_per_seq : nullptr;
    for (int u = warp; u < pool_chunks + key_chunks; u += AP_WARPS) {
        if (u < pool_chunks) {
            const int base = u * 32;                                     // 32 pooled rows inside one page
            const size_t row0 = ((size_t)ptable[base / PAGE] * KV + g) * PAGE + (base % PAGE);
            const bool valid = base + lane < n_blocks;
            float s = 0.f;
            if (valid) s = ap_dot<T>(pool_k + (row0 + lane) * (size_t)hd, q_s, hd) * scale;
            ap_fold<T, PL, SIGMOID>(s, valid, 0, min(n_blocks - base, 32) - 1, pool_v + row0 * (size_t)vd, vd, vd, bias, m, l, acc);
        } else {
            const int base = (first_chunk + u - pool_chunks) * 32;      // 32 keys inside one page
            const size_t row0 = ((size_t)table[base / PAGE] * KV + g) * PAGE + (base % PAGE);
            const int key = base + lane;
            const bool valid = key >= lo && key <= pos;
            float s = 0.f;
            if (valid) s = ap_dot<T>(k_cache + (row0 + lane) * (size_t)hd, q_s, hd) * scale;
            ap_fold<T, PL, SIGMOID>(s, valid, max(lo - base, 0), min(pos - base, 31), v_cache + row0 * (size_t)vd, vd, vd, bias, m, l, acc);
        }
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) acc_s[warp * vd + d] = acc[i];
    }
    __syncthreads();
    T* orow = out + ((size_t)t * H + h) * vd;
    if (SIGMOID) {
        for (int d = threadIdx.x; d < vd; d += blockDim.x) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < AP_WARPS; ++w) o += acc_s[w * vd + d];
            orow[d] = from_f32<T>(o);
        }
        return;
    }
    float M = m_s[0];
#pragma unroll
    for (int w = 1; w < AP_WARPS; ++w) M = fmaxf(M, m_s[w]);
    const float snk = sink ? sink[h] : -INFINITY;
    M = fmaxf(M, snk);
    float L = sink ? expf(snk - M) : 0.f;
    float wgt[AP_WARPS];
#pragma unroll
    for (int w = 0; w < AP_WARPS; ++w) {
        wgt[w] = m_s[w] == -INFINITY ? 0.f : expf(m_s[w] - M);
        L += l_s[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < vd; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < AP_WARPS; ++w) o += acc_s[w * vd + d] * wgt[w];
        orow[d] = from_f32<T>(o / L);
    }
}

// The means of the blocks that became complete in this step: grid (sequence, block of the step, kv head).
template <typename T>
__global__ void __launch_bounds__(128)
pool_blocks_kernel(const T* __restrict__ k_cache, const T* __restrict__ v_cache, const int* __restrict__ block_table, int blocks_per_seq,
                   T* __restrict__ pool_k, T* __restrict__ pool_v, const int* __restrict__ pool_table, int pool_blocks_per_seq,
                   int pool, const int* __restrict__ seq_slots, const int* __restrict__ seq_starts, const int* __restrict__ seq_new,
                   int KV, int hd, int vd) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, g = blockIdx.z;
    const int slot = seq_slots[s];
    if (slot < 0) return;
    const int start = seq_starts[s], end = start + seq_new[s];
    const int b = start / pool + blockIdx.y;                  // complete now: its last position is one of the step's
    if (b >= end / pool) return;
    const size_t prow = ((size_t)pool_table[(size_t)slot * pool_blocks_per_seq + b / PAGE] * KV + g) * PAGE + (b % PAGE);
    for (int d = threadIdx.x; d < hd + vd; d += blockDim.x) {
        const bool key = d < hd;
        const int width = key ? hd : vd, e = key ? d : d - hd;
        const T* src = key ? k_cache : v_cache;
        float sum = 0.f;
        for (int j = 0; j < pool; ++j)
            sum += to_f32(src[cache_row_offset(block_table, blocks_per_seq, slot, b * pool + j, g, KV, width) + e]);
        (key ? pool_k : pool_v)[prow * (size_t)width + e] = from_f32<T>(sum / (float)pool);
    }
}

}  // namespace kl

using namespace kl;

// q: rows of q_stride elements, head h at column h * hd.  out: [tokens, H * vd].  Caches [pages, KV, PAGE, hd] and
// [pages, KV, PAGE, vd]; pooled rows in the same dtype in pages of their own (pool <= 0: none).  weights: 0 softmax (sink float32 [H] or
// null), 1 sigmoid (head_bias float32 [H] or null).
KL_API int kl_attention_pooled(const void* q, long long q_stride, void* out, const void* k_cache, const void* v_cache,
                               const int* block_table, int blocks_per_seq, const void* pool_k, const void* pool_v,
                               const int* pool_table, int pool_blocks_per_seq, int pool, const int* positions,
                               const int* token_slot, int n_tokens, int H, int KV, int hd, float scale, int window, int vd,
                               const float* sink, const float* head_bias, int weights, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return KL_OK;
    if (vd <= 0 || vd > AP_MAX_VALUE_DIM || hd <= 0 || KV <= 0 || H % KV || H > 65535) return KL_ERR_BAD_SIZE;
    if (pool > 0 && (window <= 0 || pool_k == nullptr || pool_v == nullptr || pool_table == nullptr)) return KL_ERR_BAD_SIZE;
    if (weights != 0 && weights != 1) return KL_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, H);
    const size_t smem = (size_t)(hd + 2 * AP_WARPS + AP_WARPS * vd) * sizeof(float);
    if (smem > 48 * 1024) return KL_ERR_BAD_SIZE;
#define KL_AP(T, PL, SG)                                                                                                        \
    launch_kernel(attention_pooled_kernel<T, PL, SG>, grid, AP_WARPS * 32, smem, stream, (const T*)q, q_stride, (T*)out,        \
                  (const T*)k_cache, (const T*)v_cache, block_table, blocks_per_seq, (const T*)pool_k, (const T*)pool_v, pool_table, \
                  pool_blocks_per_seq, pool, positions, token_slot, H, KV, hd, scale, window, vd, sink, head_bias)
#define KL_AP_T(T)                                                                    \
    do {                                                                              \
        if (weights == 1) { if (vd <= 256) KL_AP(T, 8, true); else KL_AP(T, 16, true); } \
        else { if (vd <= 256) KL_AP(T, 8, false); else KL_AP(T, 16, false); }         \
    } while (0)
    if (dtype == KL_F32) KL_AP_T(float);
    else if (dtype == KL_BF16) KL_AP_T(bf16);
    else return KL_ERR_BAD_DTYPE;
#undef KL_AP_T
#undef KL_AP
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_pool_blocks(const void* k_cache, const void* v_cache, const int* block_table, int blocks_per_seq, void* pool_k,
                          void* pool_v, const int* pool_table, int pool_blocks_per_seq, int pool, const int* seq_slots,
                          const int* seq_starts, const int* seq_new, int n_seqs, int max_new, int KV, int hd, int vd, int dtype,
                          cudaStream_t stream) {
    if (n_seqs <= 0) return KL_OK;
    if (pool <= 0 || KV <= 0 || hd <= 0 || vd <= 0 || max_new <= 0) return KL_ERR_BAD_SIZE;
    const int per_seq = max_new / pool + 1;               // the most blocks a sequence can complete with max_new tokens
    if (per_seq > 65535 || KV > 65535) return KL_ERR_BAD_SIZE;
    const dim3 grid(n_seqs, per_seq, KV);
    if (dtype == KL_F32)
        launch_kernel(pool_blocks_kernel<float>, grid, 128, 0, stream, (const float*)k_cache, (const float*)v_cache, block_table,
                      blocks_per_seq, (float*)pool_k, (float*)pool_v, pool_table, pool_blocks_per_seq, pool, seq_slots, seq_starts, seq_new, KV, hd, vd);
    else if (dtype == KL_BF16)
        launch_kernel(pool_blocks_kernel<bf16>, grid, 128, 0, stream, (const bf16*)k_cache, (const bf16*)v_cache, block_table,
                      blocks_per_seq, (bf16*)pool_k, (bf16*)pool_v, pool_table, pool_blocks_per_seq, pool, seq_slots, seq_starts, seq_new, KV, hd, vd);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
