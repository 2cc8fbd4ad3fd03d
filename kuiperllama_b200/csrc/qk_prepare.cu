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

// The same for bfloat16 rows on 16-byte boundaries and head sizes of 8 L with L a power of two up to 32: a lane holds eight
// neighbouring elements of a head (one 16-byte access each way), L lanes a head, so a warp carries 512 bytes a load instead
// of 64 and a tenth as many warps move the same rows.  Interleaved pairs lie inside a lane's eight elements; a pair
// (i, i + rot / 2) has its partner rot / 16 lanes away (rot a multiple of 16) and comes by shuffle.  The head's sum of squares
// is added over the lane's elements in order, then over the L lanes by shuffles.
template <int L>
__global__ void __launch_bounds__(256)
qk_prepare_vec_kernel(bf16* __restrict__ proj, long long ld, int q_col, int k_col, int v_col,
                      const float* __restrict__ q_bias, const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                      const float* __restrict__ inv_freq, int rot, int interleaved,
                      int head_norm, float eps, const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                      const int* __restrict__ positions, const int* __restrict__ token_slot,
                      const int* __restrict__ block_table, int blocks_per_seq,
                      bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int H, int KV, int vd) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int hd = 8 * L;
    extern __shared__ float smem[];
    float* cs = smem;                                   // [rot]: cos, sin of every pair
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;                               // a padding row
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
        float sn, c;
        sincosf((float)pos * inv_freq[i], &sn, &c);
        cs[2 * i] = c;
        cs[2 * i + 1] = sn;
    }
    __syncthreads();
    bf16* row = proj + (size_t)t * ld;
    const bool write = k_cache != nullptr;
    const int half = rot / 2;
    const int part = threadIdx.x % L;                   // which eight elements of the head
    const int e0 = part * 8;
    // every thread of the warp walks the same number of turns, so the shuffles below are whole
    const int per_turn = gridDim.y * (blockDim.x / L);
    for (int base = blockIdx.y * (blockDim.x / L); base < H + KV; base += per_turn) {
        const int head = base + threadIdx.x / L;
        const bool live = head < H + KV && (head < H || write);
        const bool is_q = head < H;
        const int g = is_q ? head : head - H;
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = 0.f;
        bf16* src = row + (is_q ? q_col + (size_t)g * hd : k_col + (size_t)g * hd) + e0;
        if (live) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p[e]); x[2 * e] = f.x; x[2 * e + 1] = f.y; }
            const float* bias = is_q ? q_bias : k_bias;
            if (bias != nullptr) {
                const float4 b0 = *reinterpret_cast<const float4*>(bias + (size_t)g * hd + e0), b1 = *reinterpret_cast<const float4*>(bias + (size_t)g * hd + e0 + 4);
                x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w; x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
            }
            if (!is_q && v_col < 0) {                   // the values are the keys as projected
                uint4 out;
                __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
                *reinterpret_cast<uint4*>(v_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, vd) + e0) = out;
            }
        }
        if (rot > 0) {
            if (interleaved) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = (e0 >> 1) + e;        // the pair's index in the head
                    if (i < half) {
                        const float u = x[2 * e], v = x[2 * e + 1], c = cs[2 * i], sn = cs[2 * i + 1];
                        x[2 * e] = u * c - v * sn;
                        x[2 * e + 1] = v * c + u * sn;
                    }
                }
            } else {
                // the partner of element a < rot / 2 is a + rot / 2, rot / 16 lanes up; of a in [rot / 2, rot) it is rot / 16 lanes down
                const int away = half >> 3;
                const bool low = e0 < half, in = e0 < rot;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float up = __shfl_down_sync(0xffffffffu, x[e], away), down = __shfl_up_sync(0xffffffffu, x[e], away);
                    if (in) {
                        const int i = (low ? e0 : e0 - half) + e;
                        const float c = cs[2 * i], sn = cs[2 * i + 1];
                        x[e] = low ? x[e] * c - up * sn : x[e] * c + down * sn;
                    }
                }
            }
        }
        float inv = 1.f;
        if (head_norm) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            inv = 1.0f / sqrtf(ss / (float)hd + eps);
        }
        if (!live) continue;
        const float* w = is_q ? q_norm_w : k_norm_w;
        if (w != nullptr) {
            const float4 w0 = *reinterpret_cast<const float4*>(w + e0), w1 = *reinterpret_cast<const float4*>(w + e0 + 4);
            x[0] *= w0.x; x[1] *= w0.y; x[2] *= w0.z; x[3] *= w0.w; x[4] *= w1.x; x[5] *= w1.y; x[6] *= w1.z; x[7] *= w1.w;
        }
        uint4 out;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(x[2 * e] * inv, x[2 * e + 1] * inv);
        bf16* dst = is_q ? src : k_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, hd) + e0;
        *reinterpret_cast<uint4*>(dst) = out;
    }
    if (write && v_col >= 0) {
        for (int idx = (blockIdx.y * blockDim.x + threadIdx.x) * 8; idx < KV * vd; idx += gridDim.y * blockDim.x * 8) {
            const int g = idx / vd, e = idx - g * vd;
            const uint4 raw = *reinterpret_cast<const uint4*>(row + (size_t)v_col + idx);
            uint4 out = raw;
            if (v_bias != nullptr) {
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
                __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(p[j]);
                    o[j] = __floats2bfloat162_rn(f.x + v_bias[idx + 2 * j], f.y + v_bias[idx + 2 * j + 1]);
                }
            }
            *reinterpret_cast<uint4*>(v_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, vd) + e) = out;
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
    // bfloat16 rows on 16-byte boundaries, head sizes 8 L with L a power of two: the form with eight elements a lane
    const int L = hd / 8;
    const bool pairs_ok = rot == 0 || interleaved || rot % 16 == 0;
    if (dtype == KL_BF16 && hd % 8 == 0 && L <= 32 && (L & (L - 1)) == 0 && vd % 8 == 0 && ld % 8 == 0 && q_col % 8 == 0 && k_col % 8 == 0 &&
        (v_col < 0 || v_col % 8 == 0) && pairs_ok && (((uintptr_t)proj | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0 &&
        (((uintptr_t)q_bias | (uintptr_t)k_bias | (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) & 15) == 0) {
        const int heads_per_cta = 256 / L;
        const dim3 grid(n_tokens, (H + KV + heads_per_cta - 1) / heads_per_cta);
        const size_t table = (size_t)rot * sizeof(float);
#define KL_QKV(LL)                                                                                                                 \
    launch_kernel(qk_prepare_vec_kernel<LL>, grid, 256, table, stream, (bf16*)proj, ld, q_col, k_col, v_col, q_bias, k_bias, v_bias, \
                  inv_freq, rot, interleaved, head_norm, eps, q_norm_w, k_norm_w, positions, token_slot, block_table, blocks_per_seq, \
                  (bf16*)k_cache, (bf16*)v_cache, H, KV, vd)
        switch (L) {
            case 1: KL_QKV(1); break;
            case 2: KL_QKV(2); break;
            case 4: KL_QKV(4); break;
            case 8: KL_QKV(8); break;
            case 16: KL_QKV(16); break;
            default: KL_QKV(32); break;
        }
#undef KL_QKV
        KL_LAUNCH_CHECK();
        return KL_OK;
    }
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
