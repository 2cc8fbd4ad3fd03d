// Routing for a mixture of experts: who goes where, and the weighted sum at the end.
//
//   moe_route_kernel    a warp per token: s = softmax(z) over all experts in 32 bits (z plus a bias per expert
//                       where one is given), the `top` largest (the lower index among equals), their scores
//                       as weights (divided by their sum if asked, which is the softmax over the chosen
//                       logits alone).
//   moe_plan_kernel     one CTA: counts per expert, a list of (token, choice) pairs sorted by expert in
//                       which every expert's run is padded to whole tiles, the expert of every tile, and
//                       each pair's place in the list.  Everything stays on the device, so a step with
//                       experts needs no answer from the host and can be captured in a graph.
//   moe_combine_kernel  out[t] = sum over the token's choices, in the order of the choices, of
//                       weight * (the expert's result at the pair's place), in 32 bits.
//
// The order of the pairs inside an expert's run is whatever the counters gave; no result depends on it,
// because the grouped product computes every row by itself.  ExiledOfCode/KuiperLLama has dense
// feed-forwards alone (kuiper/source/model/llama3.cpp:692-718).
#include "common.cuh"

namespace kl {

constexpr int MOE_MAX_PER_LANE = 8;      // experts <= 256
constexpr int MOE_PLAN_THREADS = 1024;
constexpr int MOE_MAX_EXPERTS = 32 * MOE_MAX_PER_LANE;

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ bias, int tokens, int experts, int top, int renormalise,
                 int groups, int keep_groups, float renorm_eps, int* __restrict__ choice, float* __restrict__ weight) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float group_best[4][MOE_MAX_EXPERTS];
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const float* z = logits + (size_t)t * ld;
    float s[MOE_MAX_PER_LANE];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < experts ? (bias ? z[e] + bias[e] : z[e]) : -INFINITY;
        m = fmaxf(m, s[i]);
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < experts ? expf(s[i] - m) : -1.f;          // taken and absent experts hold -1: below every score
        sum += e < experts ? s[i] : 0.f;
    }
    sum = warp_sum(sum);
    if (groups > 1 && keep_groups < groups) {
        // Experts form `groups` equal groups of neighbours; a group's score is its largest score, and only the experts
        // of the `keep_groups` best groups (the lower index among equals) stay in the choice.
        float* gb = group_best[threadIdx.x >> 5];
        const int per = experts / groups;
        for (int g = lane; g < groups; g += 32) gb[g] = -1.f;
        __syncwarp();
        for (int g = 0; g < groups; ++g) {
            float b = -1.f;
#pragma unroll
            for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
                const int e = lane + 32 * i;
                if (e < experts && e / per == g) b = fmaxf(b, s[i]);
            }
            b = warp_max(b);
            if (lane == 0) gb[g] = b;
        }
        __syncwarp();
        // rank of every group: how many groups come before it (a larger score, or an equal one with a lower index)
#pragma unroll
        for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < experts) {
                const int g = e / per;
                const float mine_b = gb[g];
                int before = 0;
                for (int o = 0; o < groups; ++o) before += (gb[o] > mine_b || (gb[o] == mine_b && o < g)) ? 1 : 0;
                if (before >= keep_groups) s[i] = -1.f;
            }
        }
    }
    float chosen_sum = 0.f, mine = 0.f;
    int mine_e = 0;
    for (int k = 0; k < top; ++k) {
        float best = -1.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MOE_MAX_PER_LANE; ++i)
            if (s[i] > best) { best = s[i]; best_e = lane + 32 * i; }    // ascending e inside a lane: the lower index wins
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
#pragma unroll
        for (int i = 0; i < MOE_MAX_PER_LANE; ++i)
            if (lane + 32 * i == best_e) s[i] = -1.f;
        chosen_sum += best;
        if (lane == k % 32) { mine = best; mine_e = best_e; }
        if (k % 32 == 31 || k == top - 1) {
            const int kk = (k / 32) * 32 + lane;
            if (kk <= k) { choice[(size_t)t * top + kk] = mine_e; weight[(size_t)t * top + kk] = mine; }
        }
    }
    // weights: the softmax scores, or those divided by the chosen ones' sum
    __syncwarp();
    const float denom = renormalise ? chosen_sum + renorm_eps * sum : sum;      // scores s = exp / sum: s_k / (sum of chosen s + eps)
    for (int kk = lane; kk < top; kk += 32) weight[(size_t)t * top + kk] = weight[(size_t)t * top + kk] / denom;
}

__global__ void __launch_bounds__(MOE_PLAN_THREADS)
moe_plan_kernel(const int* __restrict__ choice, const int* __restrict__ token_slot, int tokens, int top, int experts, int tile_rows,
                int cap, int tiles, int* __restrict__ rank, int* __restrict__ pair_pos, int* __restrict__ list_rows,
                int* __restrict__ tile_group) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ int count[MOE_MAX_EXPERTS];
    __shared__ int first[MOE_MAX_EXPERTS + 1];
    const int pairs = tokens * top;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < cap; i += blockDim.x) list_rows[i] = -1;
    for (int i = threadIdx.x; i < tiles; i += blockDim.x) tile_group[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int t = p / top;
        const bool live = token_slot == nullptr || token_slot[t] >= 0;
        rank[p] = live ? atomicAdd(&count[choice[p]], 1) : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = at;
            at += (count[e] + tile_rows - 1) / tile_rows * tile_rows;
        }
        first[experts] = at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        for (int tile = first[e] / tile_rows; tile < first[e + 1] / tile_rows; ++tile) tile_group[tile] = e;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int r = rank[p];
        const int pos = r < 0 ? -1 : first[choice[p]] + r;
        pair_pos[p] = pos;
        if (pos >= 0) list_rows[pos] = p / top;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ results, long long ld, const int* __restrict__ pair_pos, const float* __restrict__ weight,
                   int tokens, int top, int hidden, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)tokens * hidden;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / hidden;
        const int c = (int)(idx - t * hidden);
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int pos = pair_pos[t * top + k];
            if (pos >= 0) acc = fmaf(weight[t * top + k], to_f32(results[(size_t)pos * ld + c]), acc);
        }
        out[idx] = acc;
    }
}

// rows[p] = x[list_rows[p]] for every place of the list, zeros at padding places: the operand of a product
// whose loader reads whole tiles of consecutive rows.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T* __restrict__ x, long long ld, const int* __restrict__ list_rows, int cap, int width, T* __restrict__ rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int per = width / 8;                                  // 16-byte pieces per row
    const size_t total = (size_t)cap * per;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t p = idx / per;
        const int c = (int)(idx - p * per) * 8;
        const int src = list_rows[p];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (src >= 0) v = *reinterpret_cast<const uint4*>(x + (size_t)src * ld + c);
        *reinterpret_cast<uint4*>(rows + p * width + c) = v;
    }
}

}  // namespace kl

using namespace kl;

// bfloat16 rows of width % 8 == 0 on 16-byte boundaries.
KL_API int kl_moe_gather(const void* x, long long ld, const int* list_rows, int cap, int width, void* rows, cudaStream_t stream) {
    if (cap <= 0) return KL_OK;
    if (width <= 0 || width % 8 || ld % 8 || (((uintptr_t)x | (uintptr_t)rows) & 15)) return KL_ERR_BAD_ALIGN;
    const int blocks = kl::strided_grid((size_t)cap * (width / 8), 256, 16);
    launch_kernel(moe_gather_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)x, ld, list_rows, cap, width, (bf16*)rows);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_moe_route(const float* logits, long long ld, const float* bias, int tokens, int experts, int top, int renormalise, int groups,
                        int keep_groups, float renorm_eps, int* choice, float* weight, cudaStream_t stream) {
    if (tokens <= 0) return KL_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts) return KL_ERR_BAD_SIZE;
    if (groups < 1 || experts % groups || keep_groups < 1 || keep_groups > groups || top > keep_groups * (experts / groups)) return KL_ERR_BAD_SIZE;
    launch_kernel(moe_route_kernel, (tokens + 3) / 4, 128, 0, stream, logits, ld, bias, tokens, experts, top, renormalise, groups, keep_groups,
                  renorm_eps, choice, weight);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// cap: length of the padded list (at least tokens * top + experts * (tile_rows - 1), a multiple of tile_rows);
// tiles = cap / tile_rows.
KL_API int kl_moe_plan(const int* choice, const int* token_slot, int tokens, int top, int experts, int tile_rows, int cap, int tiles,
                       int* rank, int* pair_pos, int* list_rows, int* tile_group, cudaStream_t stream) {
    if (tokens <= 0) return KL_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || tile_rows <= 0 || cap % tile_rows || tiles * tile_rows != cap) return KL_ERR_BAD_SIZE;
    if ((long long)cap < (long long)tokens * top + (long long)experts * (tile_rows - 1)) return KL_ERR_BAD_SIZE;
    launch_kernel(moe_plan_kernel, 1, MOE_PLAN_THREADS, 0, stream, choice, token_slot, tokens, top, experts, tile_rows, cap, tiles,
                  rank, pair_pos, list_rows, tile_group);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_moe_combine(const void* results, long long ld, const int* pair_pos, const float* weight, int tokens, int top,
                          int hidden, float* out, int dtype, cudaStream_t stream) {
    if (tokens <= 0 || hidden <= 0) return KL_OK;
    const int blocks = kl::strided_grid((size_t)tokens * hidden, 256, 16);
    if (dtype == KL_F32)
        launch_kernel(moe_combine_kernel<float>, blocks, 256, 0, stream, (const float*)results, ld, pair_pos, weight, tokens, top, hidden, out);
    else if (dtype == KL_BF16)
        launch_kernel(moe_combine_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)results, ld, pair_pos, weight, tokens, top, hidden, out);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
