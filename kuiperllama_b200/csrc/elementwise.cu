// Element-wise kernels between matrix products: activations of a plain (ungated) feed-forward
// and a sigmoid gate on a mixer's output.  The arithmetic is 32-bit; inputs and outputs are in
// the compute dtype and may be column slices of a wider matrix (a row stride of their own).
// ExiledOfCode/KuiperLLama's only activation is SwiGLU (swiglu_kernel.cu:18-21).
#include "common.cuh"

namespace kl {

enum : int { ACT_XIELU = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_RELU2 = 3 };     // relu2: max(z, 0)^2

// xIELU with a_pos = softplus(p) and a_neg = 1/2 + softplus(q) (both made at load, params[0..1]):
//   z > 0:  a_pos z^2 + z / 2          z <= 0:  a_neg (exp(z) - 1 - z) + z / 2
// FAST (a result that is rounded to bfloat16): exp(z) - 1 from the fast exponential; its absolute error near
// zero, 1e-7, stands beside z / 2 and is far below that format's step.
template <bool FAST>
__device__ __forceinline__ float activate(float z, int kind, float a_pos, float a_neg) {
    if (kind == ACT_XIELU) return z > 0.f ? a_pos * z * z + 0.5f * z : a_neg * ((FAST ? __expf(z) - 1.0f : expm1f(z)) - z) + 0.5f * z;
    if (kind == ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
    if (kind == ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.0f + (FAST ? __expf(-z) : expf(-z)));
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, long long ld_x, T* __restrict__ out, long long ld_out, int tokens, int n,
                                  int kind, const float* __restrict__ params) {
    pdl_launch_dependents();
    pdl_wait();
    const float a_pos = params ? params[0] : 0.f, a_neg = params ? params[1] : 0.f;
    const size_t total = (size_t)tokens * n;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        const int i = (int)(idx - t * n);
        out[t * ld_out + i] = from_f32<T>(activate<sizeof(T) == 2>(to_f32(x[t * ld_x + i]), kind, a_pos, a_neg));
    }
}

// The same, 16 bytes per access (rows whose starts and widths are multiples of 16 bytes).
template <typename T>
__global__ void activation_vec_kernel(const T* __restrict__ x, long long ld_x, T* __restrict__ out, long long ld_out, int tokens, int n,
                                      int kind, const float* __restrict__ params) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int V = 16 / sizeof(T);
    const float a_pos = params ? params[0] : 0.f, a_neg = params ? params[1] : 0.f;
    const int nv = n / V;
    const size_t total = (size_t)tokens * nv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / nv;
        const int i = (int)(idx - t * nv) * V;
        uint4 raw = *reinterpret_cast<const uint4*>(x + t * ld_x + i);
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int k = 0; k < V; ++k) e[k] = from_f32<T>(activate<sizeof(T) == 2>(to_f32(e[k]), kind, a_pos, a_neg));
        *reinterpret_cast<uint4*>(out + t * ld_out + i) = raw;
    }
}

// x[t, i] *= sigmoid(gate[t, i / group]) in place: group = 1 gates element by element, group = a head's
// width gates every head by one number.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, long long ld_x, const T* __restrict__ gate, long long ld_gate, int tokens, int n,
                                    int group) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)tokens * n;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        const int i = (int)(idx - t * n);
        const float g = to_f32(gate[t * ld_gate + i / group]);
        x[t * ld_x + i] = from_f32<T>(to_f32(x[t * ld_x + i]) * (1.0f / (1.0f + expf(-g))));
    }
}

}  // namespace kl

using namespace kl;

KL_API int kl_activation(const void* x, long long ld_x, void* out, long long ld_out, int tokens, int n, int kind,
                         const float* params, int dtype, cudaStream_t stream) {
    if (tokens <= 0 || n <= 0) return KL_OK;
    if (kind < ACT_XIELU || kind > ACT_RELU2 || (kind == ACT_XIELU && params == nullptr)) return KL_ERR_BAD_SIZE;
    const int threads = 256;
    if (dtype != KL_F32 && dtype != KL_BF16) return KL_ERR_BAD_DTYPE;
    const int v = dtype == KL_F32 ? 4 : 8;
    if (n % v == 0 && ld_x % v == 0 && ld_out % v == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        const int blocks = kl::strided_grid((size_t)tokens * (n / v), threads, 16);
        if (dtype == KL_F32)
            launch_kernel(activation_vec_kernel<float>, blocks, threads, 0, stream, (const float*)x, ld_x, (float*)out, ld_out, tokens, n, kind, params);
        else
            launch_kernel(activation_vec_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)x, ld_x, (bf16*)out, ld_out, tokens, n, kind, params);
        KL_LAUNCH_CHECK();
        return KL_OK;
    }
    const int blocks = kl::strided_grid((size_t)tokens * n, threads, 16);
    if (dtype == KL_F32)
        launch_kernel(activation_kernel<float>, blocks, threads, 0, stream, (const float*)x, ld_x, (float*)out, ld_out, tokens, n, kind, params);
    else
        launch_kernel(activation_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)x, ld_x, (bf16*)out, ld_out, tokens, n, kind, params);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_sigmoid_gate(void* x, long long ld_x, const void* gate, long long ld_gate, int tokens, int n, int group, int dtype,
                           cudaStream_t stream) {
    if (tokens <= 0 || n <= 0) return KL_OK;
    if (group <= 0 || n % group) return KL_ERR_BAD_SIZE;
    const int threads = 256;
    const int blocks = kl::strided_grid((size_t)tokens * n, threads, 16);
    if (dtype == KL_F32)
        launch_kernel(sigmoid_gate_kernel<float>, blocks, threads, 0, stream, (float*)x, ld_x, (const float*)gate, ld_gate, tokens, n, group);
    else if (dtype == KL_BF16)
        launch_kernel(sigmoid_gate_kernel<bf16>, blocks, threads, 0, stream, (bf16*)x, ld_x, (const bf16*)gate, ld_gate, tokens, n, group);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
