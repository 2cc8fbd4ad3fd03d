// What grouped-query attention needs between its input product and the scores, as one kernel per step with
// every step optional: for every token
//
//   * a bias is added to the projected q, k and v (float32 vectors),
//   * the first `rot` elements of every q and k head turn by the token's position, in pairs (2i, 2i + 1)
//     (interleaved) or (i, i + rot / 2); angle = position * inv_freq[i] in 32 bits with sincosf,
//   * every q and k head is divided by its root mean square over the head (eps inside the root) and
//     multiplied by a weight per element (one vector for the q heads, one for the k heads) where one is given,
//   * q is written back where it came from, k into the token's row of the paged cache, and v (as projected,
//     with its bias) into the value cache, whose rows may have another size than the keys'; with v_col < 0
//     there is no value projection and the key heads as projected (with bias, before rotation and norm)
//     are stored as values.
//
// A token's heads are dealt to the CTAs of its grid row, a warp per head, and the head passes through a row of
// shared memory, so the order of a head's sum of squares depends on the head size only.  ExiledOfCode/KuiperLLama
// rotates whole heads from tables and has neither biases nor norms on q and k (rope_kernel.cu:5-49,
// kuiper/source/model/llama3.cpp:610-639).
#include "common.cuh"

namespace kl {

constexpr int QKP_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(QKP_WARPS * 32)
qk_prepare_kernel(T* __restrict__ proj, long long ld, int q_col, int k_col, int v_col,
                  const float* __restrict__ q_bias, const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                  const float* __restrict__ inv_freq, int rot, int interleaved,
                  int head_norm, float eps, const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                  const int* __restrict__ positions, const int* __restrict__ token_slot,
                  const int* __restrict__ block_table, int blocks_per_seq,
                  T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int KV, int hd, int vd) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* cs = smem;                                   // [rot]: cos, sin of every pair
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;                               // a padding row
    const int pos = positions[t];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* buf = smem + rot + (size_t)warp * hd;        // [hd] per warp
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[2 * i] = c;
        cs[2 * i + 1] = s;
    }
    __syncthreads();
    T* row = proj + (size_t)t * ld;
    const bool write = k_cache != nullptr;
    const int half = rot / 2;
    for (int head = blockIdx.y * QKP_WARPS + warp; head < H + KV; head += gridDim.y * QKP_WARPS) {
        const bool is_q = head < H;
        if (!is_q && !write) continue;
        const int g = is_q ? head : head - H;
        T* src = row + (is_q ? q_col + (size_t)g * hd : k_col + (size_t)g * hd);
        const float* bias = is_q ? q_bias : k_bias;
        T* vdst = (!is_q && v_col < 0) ? v_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, vd) : nullptr;
        for (int i = lane; i < hd; i += 32) {
            const float x = to_f32(src[i]) + (bias ? bias[(size_t)g * hd + i] : 0.f);
            buf[i] = x;
            if (vdst != nullptr) vdst[i] = from_f32<T>(x);          // the values are the keys as projected
        }
        __syncwarp();
        for (int i = lane; i < half; i += 32) {
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
            const float u = buf[a], v = buf[b], c = cs[2 * i], s = cs[2 * i + 1];
            buf[a] = u * c - v * s;
            buf[b] = v * c + u * s;
        }
        __syncwarp();
        float inv = 1.f;
        if (head_norm) {
            float ss = 0.f;
            for (int i = lane; i < hd; i += 32) ss += buf[i] * buf[i];
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)hd + eps);
        }
        const float* w = is_q ? q_norm_w : k_norm_w;
        T* dst = is_q ? src : k_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, hd);
        for (int i = lane; i < hd; i += 32) dst[i] = from_f32<T>(w ? buf[i] * inv * w[i] : buf[i] * inv);
        __syncwarp();
    }
    if (write && v_col >= 0) {
        for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < KV * vd; idx += gridDim.y * blockDim.x) {
            const int g = idx / vd, e = idx - g * vd;
            T* dst = v_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, vd);
            dst[e] = from_f32<T>(to_f32(row[(size_t)v_col + idx]) + (v_bias ? v_bias[idx] : 0.f));
        }
    }
}

}  // namespace kl

using namespace kl;

// proj: rows of `ld` elements; q heads from column q_col, k heads from k_col, v heads from v_col (< 0: none).
// Caches: [pages, KV, PAGE, hd] and [pages, KV, PAGE, vd]; both null: a layer that only reads a cache.
KL_API int kl_qk_prepare(void* proj, long long ld, int q_col, int k_col, int v_col, const float* q_bias, const float* k_bias,
                         const float* v_bias, const float* inv_freq, int rot, int interleaved, int head_norm, float eps,
                         const float* q_norm_w, const float* k_norm_w, const int* positions, const int* token_slot,
                         const int* block_table, int blocks_per_seq, void* k_cache, void* v_cache, int n_tokens, int H, int KV,
                         int hd, int vd, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return KL_OK;
    if (rot % 2 || rot < 0 || rot > hd || H <= 0 || KV <= 0 || hd <= 0 || vd <= 0) return KL_ERR_BAD_SIZE;
    if (rot > 0 && inv_freq == nullptr) return KL_ERR_BAD_SIZE;
    if ((k_cache == nullptr) != (v_cache == nullptr)) return KL_ERR_BAD_SIZE;
    if (v_col < 0 && vd != hd) return KL_ERR_BAD_SIZE;
    const size_t smem = (size_t)(rot + QKP_WARPS * hd) * sizeof(float);
    if (smem > 48 * 1024 || (H + KV + QKP_WARPS - 1) / QKP_WARPS > 65535) return KL_ERR_BAD_SIZE;
#define KL_QKP(T)                                                                                                                  \
    launch_kernel(qk_prepare_kernel<T>, dim3(n_tokens, (H + KV + QKP_WARPS - 1) / QKP_WARPS), QKP_WARPS * 32, smem, stream, (T*)proj, ld, q_col, k_col, v_col, q_bias, k_bias, \
                  v_bias, inv_freq, rot, interleaved, head_norm, eps, q_norm_w, k_norm_w, positions, token_slot, block_table,      \
                  blocks_per_seq, (T*)k_cache, (T*)v_cache, H, KV, hd, vd)
    if (dtype == KL_F32) KL_QKP(float);
    else if (dtype == KL_BF16) KL_QKP(bf16);
    else return KL_ERR_BAD_DTYPE;
#undef KL_QKP
    KL_LAUNCH_CHECK();
    return KL_OK;
}
