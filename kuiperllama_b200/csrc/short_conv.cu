// A short causal convolution over time, one filter per channel, for a ragged step:
//
//   y[t, c] = act( (add_input ? x[t, c] : 0) + bias[c] + sum_j w[c, j] * x[t - (taps - 1) + j, c] )
//
// x before a sequence's first token is zero; x before the step's first token of a sequence that is already
// running comes from the slot's state, which holds the last taps - 1 inputs (oldest first) as [taps - 1, C]
// float32.  Two uses: the convolution in front of a mixer that is added to its own input (output in the
// compute dtype), and the convolution with bias and SiLU over the channels of a state-space mixer (output
// float32, since it enters a recurrence).  The sums run in 32 bits in the order j = 0 .. taps - 1, whatever
// the cut of the prompt, so a result does not depend on the cut.
//
//   short_conv_kernel         a CTA per (sequence, tile of tokens), threads over channels.
//   short_conv_state_kernel   a thread per (sequence, channel): the state after the step.  It runs after the
//                             convolution (stream order), because the convolution's CTAs read the old state.
//
// ExiledOfCode/KuiperLLama has no convolution (its layers are kuiper/source/model/llama3.cpp:146-166).
#include "common.cuh"

namespace kl {

constexpr int SC_MAX_TAPS = 16;
constexpr int SC_TILE = 8;         // tokens per CTA

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
short_conv_kernel(const T* __restrict__ x, long long ld_x, const float* __restrict__ w, const float* __restrict__ bias, int taps,
                  const float* __restrict__ state, long long ld_state, const int* __restrict__ cu_tokens,
                  const int* __restrict__ seq_slots, int channels, int add_input, int act_silu, TO* __restrict__ out, long long ld_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    const int row0 = cu_tokens[s], n_new = cu_tokens[s + 1] - row0;
    const int first = blockIdx.x * SC_TILE;
    if (first >= n_new) return;
    const int last = min(first + SC_TILE, n_new);
    const int slot = seq_slots[s];
    const float* st = state + (size_t)slot * ld_state;
    for (int c = blockIdx.z * blockDim.x + threadIdx.x; c < channels; c += gridDim.z * blockDim.x) {
        float wj[SC_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < SC_MAX_TAPS; ++j) wj[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
        const float b = bias != nullptr ? bias[c] : 0.f;
        for (int t = first; t < last; ++t) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < SC_MAX_TAPS; ++j) {
                if (j < taps) {
                    const int li = t - (taps - 1) + j;              // index among the step's tokens of this sequence
                    float v;
                    if (li >= 0) v = to_f32(x[(size_t)(row0 + li) * ld_x + c]);
                    else v = st[(size_t)(taps - 1 + li) * channels + c];   // zero in a fresh slot: nothing before the first token
                    acc = fmaf(wj[j], v, acc);
                }
            }
            float y = acc + b;
            if (add_input) y += to_f32(x[(size_t)(row0 + t) * ld_x + c]);
            if (act_silu) y = y / (1.0f + expf(-y));
            out[(size_t)(row0 + t) * ld_out + c] = from_f32<TO>(y);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const T* __restrict__ x, long long ld_x, int taps, float* __restrict__ state, long long ld_state,
                        const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots, int channels) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    const int row0 = cu_tokens[s], n_new = cu_tokens[s + 1] - row0;
    if (n_new <= 0) return;
    float* st = state + (size_t)seq_slots[s] * ld_state;
    const int keep = taps - 1;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
        float next[SC_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < SC_MAX_TAPS; ++k) {
            if (k < keep) {
                const int li = n_new - keep + k;
                next[k] = li >= 0 ? to_f32(x[(size_t)(row0 + li) * ld_x + c]) : st[(size_t)(keep + li) * channels + c];
            }
        }
#pragma unroll
        for (int k = 0; k < SC_MAX_TAPS; ++k)
            if (k < keep) st[(size_t)k * channels + c] = next[k];
    }
}

}  // namespace kl

using namespace kl;

// x: compute dtype `dtype`; out: float32 if out_f32 else the compute dtype.  state: float32, the slot's row starts at
// state + slot * ld_state and holds [taps - 1, channels].  With update_state the state moves on in a second launch.
KL_API int kl_short_conv(const void* x, long long ld_x, const float* w, const float* bias, int taps, float* state, long long ld_state,
                         const int* cu_tokens, const int* seq_slots, int n_seqs, int max_new, int channels, int add_input,
                         int act_silu, void* out, long long ld_out, int out_f32, int update_state, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0 || channels <= 0) return KL_OK;
    if (taps < 1 || taps > SC_MAX_TAPS) return KL_ERR_BAD_SIZE;
    if (dtype != KL_F32 && dtype != KL_BF16) return KL_ERR_BAD_DTYPE;
    const int threads = channels >= 256 ? 256 : ((channels + 31) / 32) * 32;
    const int tiles = (max_new + SC_TILE - 1) / SC_TILE;
    int zblocks = (channels + threads - 1) / threads;
    if (zblocks > 64) zblocks = 64;
    dim3 grid(tiles, n_seqs, zblocks);
#define KL_SC(T, TO)                                                                                                          \
    launch_kernel(short_conv_kernel<T, TO>, grid, threads, 0, stream, (const T*)x, ld_x, w, bias, taps, (const float*)state, ld_state, \
                  cu_tokens, seq_slots, channels, add_input, act_silu, (TO*)out, ld_out)
    if (dtype == KL_F32) KL_SC(float, float);
    else if (out_f32) KL_SC(bf16, float);
    else KL_SC(bf16, bf16);
#undef KL_SC
    KL_LAUNCH_CHECK();
    if (update_state && taps > 1) {
        dim3 g2((channels + threads - 1) / threads, n_seqs);
        if (dtype == KL_F32)
            launch_kernel(short_conv_state_kernel<float>, g2, threads, 0, stream, (const float*)x, ld_x, taps, state, ld_state, cu_tokens, seq_slots, channels);
        else
            launch_kernel(short_conv_state_kernel<bf16>, g2, threads, 0, stream, (const bf16*)x, ld_x, taps, state, ld_state, cu_tokens, seq_slots, channels);
        KL_LAUNCH_CHECK();
    }
    return KL_OK;
}
