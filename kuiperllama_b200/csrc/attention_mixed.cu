// Softmax attention whose heads exchange their weights after the softmax, over the paged cache:
//
//   s_h(i, j) = scale * q_h(i) . k_kv(h)(j);   s <- cap * tanh(s / cap)  (cap > 0);   s <- s - r1_h * ln(1 + r2_h * (i - j))
//   visible:    j <= i and (i - j < window or j < keep_first)            (window 0: every earlier key)
//   p_h(i, .) = softmax of s_h(i, .) over the visible keys
//   w_h(i, j) = sum_g talk[h, g] * p_g(i, j)                             (talk null: w = p)
//   out_h(i)  = out_scale * sigmoid(gate[i, h]) * sum_j w_h(i, j) v_kv(h)(j)      (gate null: no gate)
//
// No rotation: positions enter through the distance bias alone; kept first tokens keep their true distances.  Keys
// have `dim` and values `vdim` elements per head (two cache tensors of their own shapes).  Everything is computed
// in 32 bits from the stored keys and values; the compute dtype is only what q, the cache and the output hold.
//
//   attention_mixed_kernel<T>   the plain form (attention_mixed_tiled.cu runs wherever its shared memory holds the sizes):
//       a CTA per token with all its heads.  Because w mixes normalised weights of all heads
//       at the same key, the keys are walked twice, in chunks of 32 by absolute position: once for every head's
//       maximum and sum, once more for p, the mix and the product with the values.  The chunks and the order of the
//       sums depend on positions only, so a row's result does not depend on the step it arrived in.  Pages wholly
//       outside the window and the kept first tokens are never touched.
//   kv_append_kernel<T>         keys and values of the step's tokens into their pages.
//
// ExiledOfCode/KuiperLLama's attention is mha_kernel.cu:61,74-106 (one sequence, no window, no bias).
#include "common.cuh"

namespace kl {

constexpr int AM_THREADS = 256;
constexpr int AM_CHUNK = 32;
constexpr int AM_ACC = 16;          // outputs per thread: heads * vdim <= AM_THREADS * AM_ACC

struct MixedArgs {
    const void* q; long long q_stride;               // [rows, >= heads * dim]
    const void* gate; long long gate_stride;         // [rows, >= heads] or null
    void* out; long long out_stride;                 // [rows, >= heads * vdim]
    const void* k_cache; const void* v_cache;        // [pages, kv_heads, PAGE, dim] and [pages, kv_heads, PAGE, vdim]
    const int* block_table; int blocks_per_seq;
    const int* positions; const int* token_slot;
    const float* r1; const float* r2; const float* talk;
    int heads, kv_heads, dim, vdim, window, keep_first;
    float scale, softcap, out_scale;
};

template <typename T>
__global__ void __launch_bounds__(AM_THREADS)
attention_mixed_kernel(const MixedArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int t = blockIdx.x;
    const int slot = A.token_slot[t];
    if (slot < 0) return;
    const int i = A.positions[t];
    const int H = A.heads, G = A.kv_heads, d = A.dim, dv = A.vdim, per = H / G;
    const int kd = d + 1;
    float* qs = sm;                            // [H][d]
    float* Ks = qs + H * d;                    // [G][CHUNK][d + 1]
    float* Vs = Ks + G * AM_CHUNK * kd;        // [G][CHUNK][dv]
    float* sc = Vs + G * AM_CHUNK * dv;        // [H][CHUNK]
    float* mx = sc + H * AM_CHUNK;             // [H][CHUNK]  (the mixed weights)
    float* mrow = mx + H * AM_CHUNK;           // [H] maxima
    float* lrow = mrow + H;                    // [H] sums
    const T* q = (const T*)A.q + (size_t)t * A.q_stride;
    for (int idx = threadIdx.x; idx < H * d; idx += AM_THREADS) qs[idx] = to_f32(q[idx]);
    for (int h = threadIdx.x; h < H; h += AM_THREADS) { mrow[h] = -INFINITY; lrow[h] = 0.f; }
    const int lo = A.window > 0 ? max(0, i - A.window + 1) : 0;
    const int keep = A.window > 0 ? A.keep_first : 0;
    const int n_chunks = i / AM_CHUNK + 1;
    const int* table = A.block_table + (size_t)slot * A.blocks_per_seq;
    const T* kc = (const T*)A.k_cache;
    const T* vc = (const T*)A.v_cache;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    float acc[AM_ACC];
#pragma unroll
    for (int a = 0; a < AM_ACC; ++a) acc[a] = 0.f;

    for (int pass = 0; pass < 2; ++pass) {
        for (int c = 0; c < n_chunks; ++c) {
            const int j0 = c * AM_CHUNK;
            if (!(j0 + AM_CHUNK - 1 >= lo || j0 < keep)) continue;          // no visible key in the chunk
            const int page = table[j0 / PAGE];
            const int in_page = j0 % PAGE;
            __syncthreads();                                                // the buffers of the chunk before are free
            for (int idx = threadIdx.x; idx < G * AM_CHUNK * d; idx += AM_THREADS) {
                const int g = idx / (AM_CHUNK * d), r = idx - g * (AM_CHUNK * d);
                const int j = r / d, e = r - j * d;
                Ks[(g * AM_CHUNK + j) * kd + e] = (j0 + j <= i) ? to_f32(kc[(((size_t)page * G + g) * PAGE + in_page + j) * d + e]) : 0.f;
            }
            if (pass == 1)
                for (int idx = threadIdx.x; idx < G * AM_CHUNK * dv; idx += AM_THREADS) {
                    const int g = idx / (AM_CHUNK * dv), r = idx - g * (AM_CHUNK * dv);
                    const int j = r / dv;
                    Vs[idx] = (j0 + j <= i) ? to_f32(vc[(((size_t)page * G + g) * PAGE + in_page) * dv + r]) : 0.f;
                }
            __syncthreads();
            for (int idx = threadIdx.x; idx < H * AM_CHUNK; idx += AM_THREADS) {
                const int h = idx / AM_CHUNK, j = idx - h * AM_CHUNK;
                const int pos = j0 + j;
                float s = -INFINITY;
                if (pos <= i && (pos >= lo || pos < keep)) {
                    const float* kr = Ks + ((h / per) * AM_CHUNK + j) * kd;
                    const float* qr = qs + h * d;
                    float dot = 0.f;
                    for (int e = 0; e < d; ++e) dot = fmaf(qr[e], kr[e], dot);
                    s = dot * A.scale;
                    if (A.softcap > 0.f) s = A.softcap * tanhf(s / A.softcap);
                    if (A.r1 != nullptr) s -= A.r1[h] * log1pf(A.r2[h] * (float)(i - pos));
                }
                sc[idx] = s;
            }
            __syncthreads();
            if (pass == 0) {
                for (int h = warp; h < H; h += AM_THREADS / 32) {
                    const float s = sc[h * AM_CHUNK + lane];
                    const float m_old = mrow[h];
                    const float m_new = fmaxf(m_old, warp_max(s));
                    const float add = warp_sum(s == -INFINITY ? 0.f : expf(s - m_new));
                    if (lane == 0) {
                        lrow[h] = lrow[h] * (m_old == -INFINITY ? 0.f : expf(m_old - m_new)) + add;
                        mrow[h] = m_new;
                    }
                }
            } else {
                for (int idx = threadIdx.x; idx < H * AM_CHUNK; idx += AM_THREADS) {
                    const int h = idx / AM_CHUNK;
                    const float s = sc[idx];
                    sc[idx] = s == -INFINITY ? 0.f : expf(s - mrow[h]) / lrow[h];
                }
                __syncthreads();
                const float* w = sc;
                if (A.talk != nullptr) {
                    for (int idx = threadIdx.x; idx < H * AM_CHUNK; idx += AM_THREADS) {
                        const int h = idx / AM_CHUNK, j = idx - h * AM_CHUNK;
                        float m = 0.f;
                        for (int g = 0; g < H; ++g) m = fmaf(A.talk[h * H + g], sc[g * AM_CHUNK + j], m);
                        mx[idx] = m;
                    }
                    __syncthreads();
                    w = mx;
                }
#pragma unroll
                for (int a = 0; a < AM_ACC; ++a) {
                    const int o = a * AM_THREADS + threadIdx.x;
                    if (o < H * dv) {
                        const int h = o / dv, cc = o - h * dv;
                        const float* wr = w + h * AM_CHUNK;
                        const float* vr = Vs + (h / per) * AM_CHUNK * dv + cc;
                        float x = acc[a];
                        for (int j = 0; j < AM_CHUNK; ++j) x = fmaf(wr[j], vr[j * dv], x);
                        acc[a] = x;
                    }
                }
            }
        }
        __syncthreads();
    }
    T* out = (T*)A.out + (size_t)t * A.out_stride;
    const T* gate = A.gate != nullptr ? (const T*)A.gate + (size_t)t * A.gate_stride : nullptr;
#pragma unroll
    for (int a = 0; a < AM_ACC; ++a) {
        const int o = a * AM_THREADS + threadIdx.x;
        if (o < H * dv) {
            float y = acc[a] * A.out_scale;
            if (gate != nullptr) y *= 1.0f / (1.0f + expf(-to_f32(gate[o / dv])));
            out[o] = from_f32<T>(y);
        }
    }
}

template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ src, long long ld, int k_col, int v_col, T* __restrict__ k_cache,
                                 T* __restrict__ v_cache, const int* __restrict__ block_table, int blocks_per_seq,
                                 const int* __restrict__ positions, const int* __restrict__ token_slot, int rows, int kv_heads, int dim,
                                 int vdim) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = kv_heads * (dim + vdim);
    const size_t total = (size_t)rows * per_row;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / per_row), r = (int)(idx - (size_t)t * per_row);
        const int slot = token_slot[t];
        if (slot < 0) continue;
        const int pos = positions[t];
        if (r < kv_heads * dim) {
            const int g = r / dim, e = r - g * dim;
            k_cache[cache_row_offset(block_table, blocks_per_seq, slot, pos, g, kv_heads, dim) + e] = src[(size_t)t * ld + k_col + r];
        } else {
            const int rr = r - kv_heads * dim;
            const int g = rr / vdim, e = rr - g * vdim;
            v_cache[cache_row_offset(block_table, blocks_per_seq, slot, pos, g, kv_heads, vdim) + e] = src[(size_t)t * ld + v_col + rr];
        }
    }
}

}  // namespace kl

using namespace kl;

KL_API int kl_attention_mixed(const void* q, long long q_stride, const void* gate, long long gate_stride, void* out, long long out_stride,
                              const void* k_cache, const void* v_cache, const int* block_table, int blocks_per_seq,
                              const int* positions, const int* token_slot, int rows, int heads, int kv_heads, int dim, int vdim,
                              float scale, float softcap, const float* r1, const float* r2, const float* talk, int window,
                              int keep_first, float out_scale, int dtype, cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || window < 0 || keep_first < 0) return KL_ERR_BAD_SIZE;
    if (heads * vdim > AM_THREADS * AM_ACC) return KL_ERR_BAD_SIZE;
    if ((r1 == nullptr) != (r2 == nullptr)) return KL_ERR_BAD_SIZE;
    const size_t smem = sizeof(float) * ((size_t)heads * dim + (size_t)kv_heads * AM_CHUNK * (dim + 1 + vdim) + 2 * (size_t)heads * AM_CHUNK + 2 * heads);
    if (smem > 220 * 1024) return KL_ERR_BAD_SIZE;
    MixedArgs A;
    A.q = q; A.q_stride = q_stride; A.gate = gate; A.gate_stride = gate_stride; A.out = out; A.out_stride = out_stride;
    A.k_cache = k_cache; A.v_cache = v_cache; A.block_table = block_table; A.blocks_per_seq = blocks_per_seq;
    A.positions = positions; A.token_slot = token_slot; A.r1 = r1; A.r2 = r2; A.talk = talk;
    A.heads = heads; A.kv_heads = kv_heads; A.dim = dim; A.vdim = vdim; A.window = window; A.keep_first = keep_first;
    A.scale = scale; A.softcap = softcap; A.out_scale = out_scale;
    if (dtype == KL_F32) {
        if (smem > 48 * 1024) KL_CUDA(cudaFuncSetAttribute(attention_mixed_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_kernel(attention_mixed_kernel<float>, rows, AM_THREADS, smem, stream, A);
    } else if (dtype == KL_BF16) {
        if (smem > 48 * 1024) KL_CUDA(cudaFuncSetAttribute(attention_mixed_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_kernel(attention_mixed_kernel<bf16>, rows, AM_THREADS, smem, stream, A);
    } else {
        return KL_ERR_BAD_DTYPE;
    }
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_kv_append(const void* src, long long ld, int k_col, int v_col, void* k_cache, void* v_cache, const int* block_table,
                        int blocks_per_seq, const int* positions, const int* token_slot, int rows, int kv_heads, int dim, int vdim,
                        int dtype, cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    const int blocks = kl::strided_grid((size_t)rows * kv_heads * (dim + vdim), 256, 8);
    if (dtype == KL_F32)
        launch_kernel(kv_append_kernel<float>, blocks, 256, 0, stream, (const float*)src, ld, k_col, v_col, (float*)k_cache, (float*)v_cache,
                      block_table, blocks_per_seq, positions, token_slot, rows, kv_heads, dim, vdim);
    else if (dtype == KL_BF16)
        launch_kernel(kv_append_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)src, ld, k_col, v_col, (bf16*)k_cache, (bf16*)v_cache,
                      block_table, blocks_per_seq, positions, token_slot, rows, kv_heads, dim, vdim);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
