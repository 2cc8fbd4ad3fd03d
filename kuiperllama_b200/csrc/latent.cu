// What attention over a shared latent needs before the scores: one kernel per step that, for every token,
//
//   * norms the first kv_rank columns of the down-projection (RMS norm, 32-bit statistics, plain weight)
//     and writes them to the token's row of the paged cache: the latent c,
//   * rotates the rot_dim columns after them by the token's position and writes them behind c in the
//     same row: the key part that all heads share,
//   * rotates the rot_dim part of every head's query and puts it behind that head's kv_rank columns of
//     the query buffer [tokens, heads, kv_rank + rot_dim], whose first kv_rank columns a grouped product
//     fills with W_uk^T q (the unrotated part taken through the key up-projection, so that scores are
//     plain dot products with cache rows).
//
// A layer that reads another layer's latent runs the query part alone (kv_col < 0).  The queries may lie in a
// matrix of their own (`qsrc`, rows `q_ld` apart: queries that came through a latent and a second product).  Rotation: pair i of
// the first rot_dims elements is (2i, 2i+1) (interleaved) or (i, i + rot_dims/2); angle = position *
// inv_freq[i] in 32 bits, and cos and sin are multiplied by `mscale` (1 without frequency scaling).
// ExiledOfCode/KuiperLLama rotates whole heads of q and k from tables (rope_kernel.cu:38-49,124-135).
#include "common.cuh"

namespace kl {

template <typename T>
__device__ __forceinline__ void rotate_into(const T* __restrict__ src, T* __restrict__ dst, int rot_dim, int rot_dims,
                                            const float* __restrict__ cs, int interleaved, int i) {
    // i < rot_dim / 2 handles one pair (or, beyond the rotated pairs, two elements that pass unchanged)
    const int half = rot_dims / 2;
    if (i < half) {
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        const float u = to_f32(src[a]), v = to_f32(src[b]);
        const float c = cs[2 * i], s = cs[2 * i + 1];
        dst[a] = from_f32<T>(u * c - v * s);
        dst[b] = from_f32<T>(v * c + u * s);
    } else {
        const int a = rot_dims + 2 * (i - half);
        dst[a] = src[a];
        if (a + 1 < rot_dim) dst[a + 1] = src[a + 1];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, long long ld, const T* __restrict__ qsrc, long long q_ld, int q_col, int kv_col, const float* __restrict__ norm_w, float eps,
                      const float* __restrict__ inv_freq, int rot_dims, float mscale, int interleaved,
                      const int* __restrict__ positions, const int* __restrict__ token_slot,
                      const int* __restrict__ block_table, int blocks_per_seq, T* __restrict__ cache, T* __restrict__ qfull,
                      int H, int dim, int rot_dim, int kv_rank) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* cs = smem;                         // [rot_dims] cos, sin of every pair
    float* scratch = smem + rot_dims;         // [33]
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[2 * i] = c * mscale;
        cs[2 * i + 1] = s * mscale;
    }
    __syncthreads();
    const T* row = proj + (size_t)t * ld;
    const int Dk = kv_rank + rot_dim, pairs = (rot_dim + 1) / 2;
    for (int e = threadIdx.x; e < H * pairs; e += blockDim.x) {
        const int h = e / pairs, i = e % pairs;
        rotate_into(qsrc + (size_t)t * q_ld + q_col + (size_t)h * (dim + rot_dim) + dim, qfull + ((size_t)t * H + h) * Dk + kv_rank, rot_dim, rot_dims,
                    cs, interleaved, i);
    }
    if (kv_col < 0) return;
    T* crow = cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, 0, 1, Dk);
    const T* kv = row + kv_col;
    float ss = 0.f;
    for (int j = threadIdx.x; j < kv_rank; j += blockDim.x) { const float v = to_f32(kv[j]); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    for (int j = threadIdx.x; j < kv_rank; j += blockDim.x) crow[j] = from_f32<T>(to_f32(kv[j]) * inv * norm_w[j]);
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) rotate_into(kv + kv_rank, crow + kv_rank, rot_dim, rot_dims, cs, interleaved, i);
}

}  // namespace kl

using namespace kl;

KL_API int kl_latent_prepare(const void* proj, long long ld, const void* qsrc, long long q_ld, int q_col, int kv_col, const float* norm_w, float eps,
                             const float* inv_freq, int rot_dims, float mscale, int interleaved, const int* positions,
                             const int* token_slot, const int* block_table, int blocks_per_seq, void* cache, void* qfull,
                             int n_tokens, int H, int dim, int rot_dim, int kv_rank, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return KL_OK;
    if (rot_dims % 2 || rot_dims > rot_dim || rot_dims < 0 || H <= 0 || kv_rank <= 0 || dim < 0) return KL_ERR_BAD_SIZE;
    if (rot_dims > 0 && inv_freq == nullptr) return KL_ERR_BAD_SIZE;
    if (qsrc == nullptr) return KL_ERR_BAD_SIZE;
    if (kv_col >= 0 && (cache == nullptr || norm_w == nullptr || block_table == nullptr)) return KL_ERR_BAD_SIZE;
    const size_t smem = (size_t)(rot_dims + 33) * sizeof(float);
    if (dtype == KL_F32)
        launch_kernel(latent_prepare_kernel<float>, n_tokens, 128, smem, stream, (const float*)proj, ld, (const float*)qsrc, q_ld, q_col, kv_col, norm_w, eps,
                      inv_freq, rot_dims, mscale, interleaved, positions, token_slot, block_table, blocks_per_seq, (float*)cache,
                      (float*)qfull, H, dim, rot_dim, kv_rank);
    else if (dtype == KL_BF16)
        launch_kernel(latent_prepare_kernel<bf16>, n_tokens, 128, smem, stream, (const bf16*)proj, ld, (const bf16*)qsrc, q_ld, q_col, kv_col, norm_w, eps,
                      inv_freq, rot_dims, mscale, interleaved, positions, token_slot, block_table, blocks_per_seq, (bf16*)cache,
                      (bf16*)qfull, H, dim, rot_dim, kv_rank);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
