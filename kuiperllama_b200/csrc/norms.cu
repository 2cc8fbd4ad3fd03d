// Norms around a float32 residual stream, with what a sandwich of norms needs folded in.
//
// One kernel does, for a row s of the step,
//
//     d = delta[s]                                  (the sublayer's result, compute dtype)
//     d = d * sigmoid(gate[s] + gate_bias)          (a gated residual, if a gate is given)
//     d = norm_post(d)                              (a norm after the sublayer, if one is given)
//     x = residual[s] + d;  residual[s] = x         (32-bit sum, written back)
//     out[r] = norm(x)                              (the norm before the next sublayer, if out is given; it may be
//                                                    "none": the row itself in the compute dtype)
//
// so that a block whose sublayers are normed before and after costs one row-wise kernel per
// sublayer, as the pre-norm block's add_rmsnorm does.  Each norm is a layer norm
// ((x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b, the variance from the deviations, not
// from E[x^2] - mean^2) or an RMS norm (x / sqrt(mean(x^2) + eps) * w).  All statistics, the
// sigmoid and the sum are 32-bit.  ExiledOfCode/KuiperLLama has the RMS norm alone
// (rmsnorm_kernel.cu:70-106) and its add as a kernel of its own (add_kernel.cu:4-12).
//
// A second kernel is the per-head RMS norm with an output gate that linear-attention mixers
// end with: out[t, h, :] = x[t, h, :] / rms(x[t, h, :]) * w * silu(gate[t, h, :]).
#include "common.cuh"

namespace kl {

enum : int { NORM_LAYER = 0, NORM_RMS = 1, NORM_NONE = 2 };     // NORM_NONE: the rows as they are (no weight is read)

// Normalise buf[0..n) in place (shared memory, every thread strides over it).
__device__ __forceinline__ void norm_in_place(float* buf, int n, const float* __restrict__ w, const float* __restrict__ b,
                                              float eps, int kind, float* scratch) {
    if (kind == NORM_NONE) return;
    float mean = 0.f;
    if (kind == NORM_LAYER) {
        float s = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) s += buf[i];
        mean = block_sum(s, scratch) / (float)n;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float d = buf[i] - mean; ss += d * d; }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float y = (buf[i] - mean) * inv * w[i];
        if (b != nullptr) y += b[i];
        buf[i] = y;
    }
}

// Four neighbouring elements of a row in the compute dtype, as floats.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// Sum over the CTA with one barrier: every warp adds up all warps' partial sums itself.  `scratch` (32
// floats) must not be written again before every warp has read it, so each call of a kernel gets its own.
__device__ __forceinline__ float block_sum_once(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    return warp_sum(lane < nwarps ? scratch[lane] : 0.f);
}

// One norm over a row that lies in registers, VPT float4 per thread (lanes beyond the row hold zeros and
// stay out of the sums).
template <int THREADS, int VPT>
__device__ __forceinline__ void norm_in_registers(float4 (&v)[VPT], int n4, int n, const float* __restrict__ w,
                                                  const float* __restrict__ b, float eps, int kind, float* scratch) {
    if (kind == NORM_NONE) return;
    float mean = 0.f;
    if (kind == NORM_LAYER) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        mean = block_sum_once(s, scratch) / (float)n;
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        if ((int)threadIdx.x + j * THREADS < n4) {
            const float a = v[j].x - mean, c = v[j].y - mean, e = v[j].z - mean, f = v[j].w - mean;
            ss += (a * a + c * c) + (e * e + f * f);
        }
    }
    ss = block_sum_once(ss, scratch + 32);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i4 = threadIdx.x + j * THREADS;
        if (i4 < n4) {
            const float4 ww = *reinterpret_cast<const float4*>(w + 4 * i4);
            float4 y = make_float4((v[j].x - mean) * inv * ww.x, (v[j].y - mean) * inv * ww.y, (v[j].z - mean) * inv * ww.z,
                                   (v[j].w - mean) * inv * ww.w);
            if (b != nullptr) {
                const float4 bb = *reinterpret_cast<const float4*>(b + 4 * i4);
                y.x += bb.x; y.y += bb.y; y.z += bb.z; y.w += bb.w;
            }
            v[j] = y;
        }
    }
}

// The chain with the row in registers and 8- or 16-byte accesses: rows of hidden % 4 == 0 elements up to
// 4 THREADS VPT whose pointers and strides are aligned for it.  `partials`: the delta as float32 pieces
// [n_partials][rows][hidden] of a product whose K range was cut, added in ascending order.
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
norm_chain_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta, long long delta_ld,
                      const float* __restrict__ partials, int n_partials, long long partial_stride,
                      const T* __restrict__ gate, long long gate_ld, const float* __restrict__ gate_bias,
                      const float* __restrict__ post_w, const float* __restrict__ post_b, float post_eps, int post_kind,
                      const float* __restrict__ w, const float* __restrict__ b, float eps, int kind,
                      T* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[4 * 32];                   // a row of its own for each of the four sums
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    const int n4 = hidden >> 2;
    float* x = residual + (size_t)s * hidden;
    const bool adds = delta != nullptr || n_partials > 0;
    float4 v[VPT], xr[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i4 = threadIdx.x + j * THREADS;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        xr[j] = v[j];
        if (i4 < n4) {
            xr[j] = *reinterpret_cast<const float4*>(x + 4 * i4);
            if (delta != nullptr) v[j] = Vec4<T>::load(delta + (size_t)s * delta_ld + 4 * i4);
            for (int z0 = 0; z0 < n_partials; z0 += 8) {          // eight pieces on their way at a time, added in ascending order
                float4 p[8];
#pragma unroll
                for (int zz = 0; zz < 8; ++zz)
                    p[zz] = z0 + zz < n_partials
                                ? *reinterpret_cast<const float4*>(partials + (size_t)(z0 + zz) * partial_stride + (size_t)s * hidden + 4 * i4)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int zz = 0; zz < 8; ++zz)
                    if (z0 + zz < n_partials) { v[j].x += p[zz].x; v[j].y += p[zz].y; v[j].z += p[zz].z; v[j].w += p[zz].w; }
            }
            if (gate != nullptr) {
                float4 a = Vec4<T>::load(gate + (size_t)s * gate_ld + 4 * i4);
                if (gate_bias != nullptr) {
                    const float4 gb = *reinterpret_cast<const float4*>(gate_bias + 4 * i4);
                    a.x += gb.x; a.y += gb.y; a.z += gb.z; a.w += gb.w;
                }
                v[j].x *= 1.0f / (1.0f + expf(-a.x)); v[j].y *= 1.0f / (1.0f + expf(-a.y));
                v[j].z *= 1.0f / (1.0f + expf(-a.z)); v[j].w *= 1.0f / (1.0f + expf(-a.w));
            }
        }
    }
    if (adds) {
        if (post_w != nullptr) norm_in_registers<THREADS, VPT>(v, n4, hidden, post_w, post_b, post_eps, post_kind, scratch);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i4 = threadIdx.x + j * THREADS;
            v[j].x += xr[j].x; v[j].y += xr[j].y; v[j].z += xr[j].z; v[j].w += xr[j].w;
            if (i4 < n4 && rows == nullptr) *reinterpret_cast<float4*>(x + 4 * i4) = v[j];
        }
    } else {
#pragma unroll
        for (int j = 0; j < VPT; ++j) v[j] = xr[j];
    }
    if (out == nullptr) return;
    norm_in_registers<THREADS, VPT>(v, n4, hidden, w, b, eps, kind, scratch + 64);
    T* o = out + (size_t)r * hidden;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i4 = threadIdx.x + j * THREADS;
        if (i4 < n4) Vec4<T>::store(o + 4 * i4, v[j]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
norm_chain_kernel(float* __restrict__ residual, const T* __restrict__ delta, long long delta_ld,
                  const float* __restrict__ partials, int n_partials, long long partial_stride,
                  const T* __restrict__ gate, long long gate_ld, const float* __restrict__ gate_bias,
                  const float* __restrict__ post_w, const float* __restrict__ post_b, float post_eps, int post_kind,
                  const float* __restrict__ w, const float* __restrict__ b, float eps, int kind,
                  T* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* buf = smem;                 // [hidden]
    float* scratch = smem + hidden;    // [33]
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* x = residual + (size_t)s * hidden;
    if (delta != nullptr || n_partials > 0) {
        const T* d = delta ? delta + (size_t)s * delta_ld : nullptr;
        const T* g = gate ? gate + (size_t)s * gate_ld : nullptr;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = d ? to_f32(d[i]) : 0.f;
            for (int z = 0; z < n_partials; ++z) v += partials[(size_t)z * partial_stride + (size_t)s * hidden + i];
            if (g != nullptr) {
                const float a = to_f32(g[i]) + (gate_bias ? gate_bias[i] : 0.f);
                v *= 1.0f / (1.0f + expf(-a));
            }
            buf[i] = v;
        }
        if (post_w != nullptr) {
            __syncthreads();
            norm_in_place(buf, hidden, post_w, post_b, post_eps, post_kind, scratch);
        }
        // every thread touches the same indices in each pass, so its own elements need no barrier here
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = x[i] + buf[i];
            buf[i] = v;
            if (rows == nullptr) x[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) buf[i] = x[i];
    }
    if (out == nullptr) return;
    __syncthreads();
    norm_in_place(buf, hidden, w, b, eps, kind, scratch);
    T* o = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(buf[i]);
}

// x: float32 [tokens, heads * dim]; gate: compute dtype, row stride gate_ld, same columns;
// w: float32 [dim] shared by the heads (or null).  One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_rmsnorm_gate_kernel(const float* __restrict__ x, const T* __restrict__ gate, long long gate_ld, const float* __restrict__ w,
                         T* __restrict__ out, long long out_ld, float out_scale, int tokens, int heads, int dim, float eps, int gate_first,
                         int wide_weight) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
    const float* xr = x + ((size_t)t * heads + h) * dim;
    const T* g = gate ? gate + (size_t)t * gate_ld + (size_t)h * dim : nullptr;
    const float* wr = w != nullptr ? w + (wide_weight ? (size_t)h * dim : 0) : nullptr;
    T* o = out + (size_t)t * out_ld + (size_t)h * dim;
    if (gate_first && g != nullptr) {
        // the gate comes before the norm: y = x silu(g), then y / rms(y) * w
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) {
            const float a = to_f32(g[i]);
            const float y = xr[i] * (a / (1.0f + expf(-a)));
            ss += y * y;
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        for (int i = lane; i < dim; i += 32) {
            const float a = to_f32(g[i]);
            float y = xr[i] * (a / (1.0f + expf(-a))) * inv;
            if (wr != nullptr) y *= wr[i];
            o[i] = from_f32<T>(y * out_scale);
        }
        return;
    }
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) ss += xr[i] * xr[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = lane; i < dim; i += 32) {
        float y = xr[i] * inv;
        if (wr != nullptr) y *= wr[i];
        if (g != nullptr) { const float a = to_f32(g[i]); y *= a / (1.0f + expf(-a)); }
        o[i] = from_f32<T>(y * out_scale);
    }
}

// The same for long rows (a norm over hundreds of channels or more): one CTA per (token, head).
template <typename T>
__global__ void __launch_bounds__(1024)
head_rmsnorm_gate_block_kernel(const float* __restrict__ x, const T* __restrict__ gate, long long gate_ld, const float* __restrict__ w,
                               T* __restrict__ out, long long out_ld, float out_scale, int heads, int dim, float eps, int gate_first,
                               int wide_weight) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x / heads, h = blockIdx.x - t * heads;
    const float* xr = x + ((size_t)t * heads + h) * dim;
    const T* g = gate ? gate + (size_t)t * gate_ld + (size_t)h * dim : nullptr;
    const float* wr = w != nullptr ? w + (wide_weight ? (size_t)h * dim : 0) : nullptr;
    T* o = out + (size_t)t * out_ld + (size_t)h * dim;
    const bool first = gate_first && g != nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float y = xr[i];
        if (first) { const float a = to_f32(g[i]); y *= a / (1.0f + expf(-a)); }
        ss += y * y;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float y = xr[i];
        if (first) {
            const float a = to_f32(g[i]);
            y = y * (a / (1.0f + expf(-a))) * inv;
            if (wr != nullptr) y *= wr[i];
        } else {
            y *= inv;
            if (wr != nullptr) y *= wr[i];
            if (g != nullptr) { const float a = to_f32(g[i]); y *= a / (1.0f + expf(-a)); }
        }
        o[i] = from_f32<T>(y * out_scale);
    }
}

// The norms of a block whose two sublayers read the same stream: x = residual + (d1 + d2) (each delta rows in the
// compute dtype or float32 pieces, or absent), written back; one root mean square; out1 = x / rms * w1 and
// out2 = x / rms * w2 (out2 optional).  With `rows` only those rows are read, into out1[0..), and the stream stays.
struct PairDelta {
    const void* rows; long long ld;          // compute dtype [n, hidden], or null
    const float* pieces; int n_pieces; long long piece_stride;   // float32 [S, n, hidden], or null
};

template <typename T>
__global__ void __launch_bounds__(1024)
pair_rmsnorm_kernel(float* __restrict__ residual, const PairDelta d1, const PairDelta d2, const float* __restrict__ w1,
                    const float* __restrict__ w2, float eps, T* __restrict__ out1, T* __restrict__ out2, const int* __restrict__ rows,
                    int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xrow[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t row = rows != nullptr ? (size_t)rows[r] : (size_t)r;
    float* x = residual + row * hidden;
    const bool has = d1.rows != nullptr || d1.pieces != nullptr || d2.rows != nullptr || d2.pieces != nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = x[i];
        if (has) {
            float add = 0.f;
            if (d1.rows != nullptr) add += to_f32(((const T*)d1.rows)[row * d1.ld + i]);
#pragma unroll 4
            for (int p = 0; p < d1.n_pieces; ++p) add += d1.pieces[(size_t)p * d1.piece_stride + row * hidden + i];
            if (d2.rows != nullptr) add += to_f32(((const T*)d2.rows)[row * d2.ld + i]);
#pragma unroll 4
            for (int p = 0; p < d2.n_pieces; ++p) add += d2.pieces[(size_t)p * d2.piece_stride + row * hidden + i];
            v += add;
            if (rows == nullptr) x[i] = v;
        }
        xrow[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xrow[i] * inv;
        if (out1 != nullptr) out1[(size_t)r * hidden + i] = from_f32<T>(v * w1[i]);
        if (out2 != nullptr) out2[(size_t)r * hidden + i] = from_f32<T>(v * w2[i]);
    }
}

}  // namespace kl

using namespace kl;

// delta, gate, out: compute dtype (`dtype`); everything else float32.  Null pointers switch steps off:
// no delta (nothing is added), no gate, no post norm (post_w null), no output (out null: only the sum).
KL_API int kl_norm_chain(float* residual, const void* delta, long long delta_ld, const float* partials, int n_partials,
                         long long partial_stride, const void* gate, long long gate_ld,
                         const float* gate_bias, const float* post_w, const float* post_b, float post_eps, int post_kind,
                         const float* w, const float* b, float eps, int kind, void* out, const int* rows, int n_rows,
                         int hidden, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return KL_OK;
    if (hidden <= 0 || (out != nullptr && w == nullptr && kind != NORM_NONE)) return KL_ERR_BAD_SIZE;
    if (kind < NORM_LAYER || kind > NORM_NONE || post_kind < NORM_LAYER || post_kind > NORM_NONE) return KL_ERR_BAD_SIZE;
    if (n_partials < 0 || (n_partials > 0 && (partials == nullptr || delta != nullptr))) return KL_ERR_BAD_SIZE;
    const bool bf = dtype == KL_BF16;
    if (dtype != KL_F32 && !bf) return KL_ERR_BAD_DTYPE;
    {
        // the form with the row in registers, where everything is aligned for 8-byte (bfloat16) or 16-byte (float) accesses
        const uintptr_t m = bf ? 7 : 15;
        auto ok_t = [&](const void* p, long long ld) { return p == nullptr || ((((uintptr_t)p) & m) == 0 && ld % 4 == 0); };
        auto ok_f = [&](const void* p) { return (((uintptr_t)p) & 15) == 0; };
        const int n4 = hidden / 4;
        if (hidden % 4 == 0 && n4 <= 256 * 8 && ok_t(delta, delta_ld) && ok_t(gate, gate_ld) && ok_t(out, hidden) && ok_f(residual) &&
            ok_f(partials) && ok_f(gate_bias) && ok_f(post_w) && ok_f(post_b) && ok_f(w) && ok_f(b)) {
#define KL_VEC(T, THREADS, VPT)                                                                                              \
            launch_kernel(norm_chain_vec_kernel<T, THREADS, VPT>, n_rows, THREADS, 0, stream, residual, (const T*)delta, delta_ld, partials, \
                          n_partials, partial_stride, (const T*)gate, gate_ld, gate_bias, post_w, post_b, post_eps, post_kind, w, b, eps, kind, \
                          (T*)out, rows, hidden)
#define KL_VEC_BY_SIZE(T)                                                                                                    \
            do {                                                                                                             \
                /* few rows of a wide model (decode): a row over 1,024 threads, so that one round of loads fetches it */      \
                if (n_rows <= 256 && n4 > 256 && n4 <= 1024) KL_VEC(T, 1024, 1);                                             \
                else if (n_rows <= 256 && n4 > 1024) KL_VEC(T, 1024, 2);                                                      \
                else if (n4 <= 64) KL_VEC(T, 64, 1); else if (n4 <= 128) KL_VEC(T, 128, 1); else if (n4 <= 256) KL_VEC(T, 256, 1);        \
                else if (n4 <= 512) KL_VEC(T, 256, 2); else if (n4 <= 1024) KL_VEC(T, 512, 2); else KL_VEC(T, 512, 4);             \
            } while (0)
            if (bf) KL_VEC_BY_SIZE(bf16); else KL_VEC_BY_SIZE(float);
#undef KL_VEC_BY_SIZE
#undef KL_VEC
            KL_LAUNCH_CHECK();
            return KL_OK;
        }
    }
    const size_t smem = (size_t)(hidden + 33) * sizeof(float);
    if (smem > 200 * 1024) return KL_ERR_BAD_SIZE;
    const int threads = hidden >= 1024 ? 256 : 128;
#define KL_CHAIN(T)                                                                                                        \
    do {                                                                                                                   \
        if (smem > 48 * 1024) KL_CUDA(cudaFuncSetAttribute(norm_chain_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        launch_kernel(norm_chain_kernel<T>, n_rows, threads, smem, stream, residual, (const T*)delta, delta_ld, partials, n_partials, partial_stride, (const T*)gate, gate_ld, \
                      gate_bias, post_w, post_b, post_eps, post_kind, w, b, eps, kind, (T*)out, rows, hidden);                \
    } while (0)
    if (dtype == KL_F32) KL_CHAIN(float);
    else if (dtype == KL_BF16) KL_CHAIN(bf16);
    else return KL_ERR_BAD_DTYPE;
#undef KL_CHAIN
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_head_rmsnorm_gate(const float* x, const void* gate, long long gate_ld, const float* w, void* out, long long out_ld,
                                float out_scale, int tokens, int heads, int dim, float eps, int gate_first, int wide_weight, int dtype,
                                cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0) return KL_OK;
    if (dim <= 0) return KL_ERR_BAD_SIZE;
    const long long items = (long long)tokens * heads;
    if (dim >= 512) {
        if (dtype == KL_F32)
            launch_kernel(head_rmsnorm_gate_block_kernel<float>, (int)items, dim >= 2048 ? 1024 : 256, 0, stream, x, (const float*)gate, gate_ld, w, (float*)out, out_ld, out_scale, heads, dim, eps, gate_first, wide_weight);
        else if (dtype == KL_BF16)
            launch_kernel(head_rmsnorm_gate_block_kernel<bf16>, (int)items, dim >= 2048 ? 1024 : 256, 0, stream, x, (const bf16*)gate, gate_ld, w, (bf16*)out, out_ld, out_scale, heads, dim, eps, gate_first, wide_weight);
        else
            return KL_ERR_BAD_DTYPE;
        KL_LAUNCH_CHECK();
        return KL_OK;
    }
    const int blocks = (int)((items + 3) / 4);
    if (dtype == KL_F32)
        launch_kernel(head_rmsnorm_gate_kernel<float>, blocks, 128, 0, stream, x, (const float*)gate, gate_ld, w, (float*)out, out_ld, out_scale, tokens, heads, dim, eps, gate_first, wide_weight);
    else if (dtype == KL_BF16)
        launch_kernel(head_rmsnorm_gate_kernel<bf16>, blocks, 128, 0, stream, x, (const bf16*)gate, gate_ld, w, (bf16*)out, out_ld, out_scale, tokens, heads, dim, eps, gate_first, wide_weight);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// RMS norm of rows in the compute dtype that are no part of the residual stream (a latent between two products):
// out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w, statistics in 32 bits; rows of x may be `x_ld` elements apart.
namespace kl {
template <typename T>
__global__ void __launch_bounds__(256)
rows_rmsnorm_kernel(const T* __restrict__ x, long long x_ld, const float* __restrict__ w, T* __restrict__ out, long long out_ld,
                    int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const T* row = x + (size_t)blockIdx.x * x_ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = to_f32(row[i]); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    T* o = out + (size_t)blockIdx.x * out_ld;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<T>(to_f32(row[i]) * inv * (w ? w[i] : 1.f));
}
}  // namespace kl

KL_API int kl_rows_rmsnorm(const void* x, long long x_ld, const float* w, void* out, long long out_ld, int rows, int width, float eps,
                           int dtype, cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    if (width <= 0) return KL_ERR_BAD_SIZE;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == KL_F32)
        launch_kernel(rows_rmsnorm_kernel<float>, rows, threads, 0, stream, (const float*)x, x_ld, w, (float*)out, out_ld, width, eps);
    else if (dtype == KL_BF16)
        launch_kernel(rows_rmsnorm_kernel<bf16>, rows, threads, 0, stream, (const bf16*)x, x_ld, w, (bf16*)out, out_ld, width, eps);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// d*_rows: compute dtype; d*_pieces: float32 [S, n, hidden].  out2 may be null; with `rows` the stream is not written.
KL_API int kl_pair_rmsnorm(float* residual, const void* d1_rows, long long d1_ld, const float* d1_pieces, int d1_n, long long d1_stride,
                           const void* d2_rows, long long d2_ld, const float* d2_pieces, int d2_n, long long d2_stride,
                           const float* w1, const float* w2, float eps, void* out1, void* out2, const int* rows, int n_rows, int hidden,
                           int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return KL_OK;
    if (hidden <= 0 || hidden > 48 * 1024 || (out1 != nullptr && w1 == nullptr) || (out2 != nullptr && w2 == nullptr)) return KL_ERR_BAD_SIZE;
    PairDelta a{d1_rows, d1_ld, d1_pieces, d1_pieces ? d1_n : 0, d1_stride};
    PairDelta b{d2_rows, d2_ld, d2_pieces, d2_pieces ? d2_n : 0, d2_stride};
    const size_t smem = (size_t)hidden * sizeof(float);
    // few rows: a row's loads (the stream, the rows or pieces of two results) are a chain per thread, so many threads
    const int pair_threads = n_rows <= 64 && hidden >= 2048 ? 1024 : 256;
    if (dtype == KL_F32) {
        if (smem > 48 * 1024) KL_CUDA(cudaFuncSetAttribute(pair_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_kernel(pair_rmsnorm_kernel<float>, n_rows, pair_threads, smem, stream, residual, a, b, w1, w2, eps, (float*)out1, (float*)out2, rows, hidden);
    } else if (dtype == KL_BF16) {
        if (smem > 48 * 1024) KL_CUDA(cudaFuncSetAttribute(pair_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_kernel(pair_rmsnorm_kernel<bf16>, n_rows, pair_threads, smem, stream, residual, a, b, w1, w2, eps, (bf16*)out1, (bf16*)out2, rows, hidden);
    } else {
        return KL_ERR_BAD_DTYPE;
    }
    KL_LAUNCH_CHECK();
    return KL_OK;
}
