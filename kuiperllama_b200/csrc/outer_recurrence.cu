// A linear recurrence whose state is a matrix per head, fed by outer products:
//
//   S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T        S: [N, P] per head, float32, from the slot's state (zero in a fresh slot)
//   y_t = S_t^T q_t + D v_t                           y: [P] per head, float32
//
// a_t is one number per (token, head) (a state-space layer: exp(-exp(A_log) dt), with c_t = dt, k = B, q = C, v = x
// and the skip D) or one number per (token, head, row of S) (gated linear attention: c = 1, D = 0).  k and q may be
// shared by the heads of a group (head h reads group h / (heads / groups)).  Everything inside the recurrence is
// 32-bit; k, q and v are read in their own type (float32, or the compute dtype straight from a projection), q times
// q_scale.
//
//   outer_recurrence_kernel<TI, NPT>   a CTA per (sequence, head, block of columns of S).  A column of S is cut over
//       L lanes of one warp, lane l holding rows l, l + L, ... (NPT of them, in registers); tokens arrive in tiles
//       through shared memory; per token every thread decays and updates its rows, multiplies them by q and the
//       lanes' sums are added by shuffles.  Tokens are walked in order from the slot's state, so a result does not
//       depend on how a prompt was cut.
//   outer_recurrence_slab_kernel<TI, R, C>   the form that runs where the sizes allow: R x C of S per thread (see there).
//   decay_softplus_kernel     dt = softplus(raw + bias), a = exp(-exp(A_log) dt) per (token, head), 32-bit.
//   decay_lowrank_kernel      a = sigmoid(z)^(1 / tau) = exp(-softplus(-z) / tau), z = W2 r + b with r a short row per
//                             token (the first of two projections, made with the mixer's other projections), 32-bit.
//
// ExiledOfCode/KuiperLLama has no recurrent mixer (its mixer is mha_kernel.cu:61,74-106).
#include "common.cuh"

namespace kl {

constexpr int OR_THREADS = 512;          // the most threads of a CTA; a launch takes 128, 256 or 512
constexpr int OR_TILE = 32;           // tokens per shared-memory tile

struct OuterArgs {
    const void* q; long long ld_q; int q_col;        // [rows, >= q_col + groups * N]
    const void* k; long long ld_k; int k_col;
    const void* v; long long ld_v; int v_col;        // [rows, >= v_col + heads * P]
    const float* a; long long ld_a;                  // [rows, heads] or [rows, heads * N]
    const float* c; long long ld_c;                  // [rows, heads] or null
    const float* skip;                               // [heads] or null
    float* state; long long ld_state;                // the slot's S at state + slot * ld_state, [heads, N, P]
    float* y; long long ld_y;                        // [rows, heads * P]
    const int* cu_tokens; const int* seq_slots;
    int heads, groups, N, P, L, a_per_row;
    int vec_state;                                   // every row piece of four columns of S is 16-byte aligned
    int vec_in;                                      // k, q and a can be read four elements at a time
    float q_scale;
};

template <typename TI, int NPT>
__global__ void __launch_bounds__(OR_THREADS, 1)
outer_recurrence_kernel(const OuterArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int s = blockIdx.z, h = blockIdx.y;
    const int row0 = A.cu_tokens[s], n_new = A.cu_tokens[s + 1] - row0;
    if (n_new <= 0) return;
    const int N = A.N, P = A.P, L = A.L;
    const int threads = blockDim.x;
    const int cols_per_cta = threads / L;
    const int lane = threadIdx.x % L;
    const int col = blockIdx.x * cols_per_cta + threadIdx.x / L;
    const bool live = col < P;
    const int g = h / (A.heads / A.groups);
    // shared: per tile token: k [N] (times c), q [N] (times q_scale), a [N or 1], v [cols_per_cta]
    const int a_len = A.a_per_row ? N : 1;
    const int per_tok = 2 * N + a_len + cols_per_cta;
    float* S_slot = A.state + (size_t)A.seq_slots[s] * A.ld_state + (size_t)h * N * P;
    float S[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = i * L + lane;
        S[i] = (live && n < N) ? S_slot[(size_t)n * P + col] : 0.f;
    }
    const TI* qp = (const TI*)A.q; const TI* kp = (const TI*)A.k; const TI* vp = (const TI*)A.v;
    const float skip = A.skip != nullptr ? A.skip[h] : 0.f;
    for (int t0 = 0; t0 < n_new; t0 += OR_TILE) {
        const int nt = min(OR_TILE, n_new - t0);
        __syncthreads();
        // the tile's k (times c), q (times q_scale), a and v, each in a loop of its own so that the loads of several
        // turns are in flight together
#pragma unroll 4
        for (int idx = threadIdx.x; idx < nt * N; idx += threads) {
            const int tt = idx / N, j = idx - tt * N;
            const size_t row = (size_t)(row0 + t0 + tt);
            float val = to_f32(kp[row * A.ld_k + A.k_col + (size_t)g * N + j]);
            if (A.c != nullptr) val *= A.c[row * A.ld_c + h];
            sm[tt * per_tok + j] = val;
        }
#pragma unroll 4
        for (int idx = threadIdx.x; idx < nt * N; idx += threads) {
            const int tt = idx / N, j = idx - tt * N;
            const size_t row = (size_t)(row0 + t0 + tt);
            sm[tt * per_tok + N + j] = to_f32(qp[row * A.ld_q + A.q_col + (size_t)g * N + j]) * A.q_scale;
        }
#pragma unroll 4
        for (int idx = threadIdx.x; idx < nt * a_len; idx += threads) {
            const int tt = idx / a_len, j = idx - tt * a_len;
            const size_t row = (size_t)(row0 + t0 + tt);
            sm[tt * per_tok + 2 * N + j] = A.a_per_row ? A.a[row * A.ld_a + (size_t)h * N + j] : A.a[row * A.ld_a + h];
        }
        for (int idx = threadIdx.x; idx < nt * cols_per_cta; idx += threads) {
            const int tt = idx / cols_per_cta, j = idx - tt * cols_per_cta;
            const size_t row = (size_t)(row0 + t0 + tt);
            const int cc = blockIdx.x * cols_per_cta + j;
            sm[tt * per_tok + 2 * N + a_len + j] = cc < P ? to_f32(vp[row * A.ld_v + A.v_col + (size_t)h * P + cc]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* kk = sm + tt * per_tok;
            const float* qq = kk + N;
            const float* aa = qq + N;
            const float vv = aa[a_len + threadIdx.x / L];
            float acc = 0.f;
            if (A.a_per_row) {
#pragma unroll
                for (int i = 0; i < NPT; ++i) {
                    const int n = i * L + lane;
                    if (n < N) {
                        S[i] = fmaf(aa[n], S[i], kk[n] * vv);
                        acc = fmaf(S[i], qq[n], acc);
                    }
                }
            } else {
                const float a0 = aa[0];
#pragma unroll
                for (int i = 0; i < NPT; ++i) {
                    const int n = i * L + lane;
                    if (n < N) {
                        S[i] = fmaf(a0, S[i], kk[n] * vv);
                        acc = fmaf(S[i], qq[n], acc);
                    }
                }
            }
            for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0 && live) A.y[(size_t)(row0 + t0 + tt) * A.ld_y + (size_t)h * P + col] = fmaf(skip, vv, acc);
        }
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = i * L + lane;
        if (live && n < N) S_slot[(size_t)n * P + col] = S[i];
    }
}

__device__ __forceinline__ void or_ld4(const float* p, float (&x)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void or_ld4(const bf16* p, float (&x)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
}

// The same recurrence with R rows x C columns of S in a thread's registers: per token a thread reads R values each of
// k, q (and a) and C of v for 3 R C multiply-adds, and only the column sums cross lanes.  A warp holds LR = 32 / CGW lanes
// along the rows (lane = column group + CGW * row group; row n = row group + LR * i), so neighbouring lanes hold
// neighbouring columns of a row.  Rows from N to LR * R are zero in shared memory and change nothing.
template <typename TI, int R, int C>
__global__ void __launch_bounds__(256)
outer_recurrence_slab_kernel(const OuterArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    const int s = blockIdx.z, h = blockIdx.y;
    const int row0 = A.cu_tokens[s], n_new = A.cu_tokens[s + 1] - row0;
    if (n_new <= 0) return;
    const int N = A.N, P = A.P, LR = A.L, Np = LR * R;
    const int threads = blockDim.x;
    const int cgw = 32 / LR;                                   // column groups per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rg = lane / cgw, cg = warp * cgw + lane % cgw;   // the thread's row group, and its column group in the CTA
    const int cols_per_cta = (threads / LR) * C;
    const int col0 = blockIdx.x * cols_per_cta + cg * C;
    const bool live = col0 < P;                                // P is a multiple of C
    const int g = h / (A.heads / A.groups);
    const int a_len = A.a_per_row ? Np : 4;                    // one decay per head: a piece of four, so that rows stay aligned
    const int per_tok = 2 * Np + a_len + cols_per_cta;         // k (times c), q (times q_scale), a, v
    float* S_slot = A.state + (size_t)A.seq_slots[s] * A.ld_state + (size_t)h * N * P;
    float S[R][C];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int n = rg + LR * i;
        if (C == 4 && A.vec_state && live && n < N) {                         // P and col0 are multiples of 4
            const float4 v4 = *reinterpret_cast<const float4*>(S_slot + (size_t)n * P + col0);
            S[i][0] = v4.x; S[i][1] = v4.y; S[i][2] = v4.z; S[i][C - 1] = v4.w;
        } else {
#pragma unroll
            for (int j = 0; j < C; ++j) S[i][j] = (live && n < N) ? S_slot[(size_t)n * P + col0 + j] : 0.f;
        }
    }
    const TI* qp = (const TI*)A.q; const TI* kp = (const TI*)A.k; const TI* vp = (const TI*)A.v;
    const float skip = A.skip != nullptr ? A.skip[h] : 0.f;
    // one tile's tokens: decay, update, multiply by q, add the lanes' column sums
    auto compute = [&](int t0, int nt) {
        for (int tt = 0; tt < nt; ++tt) {
            const float* kk = sm + tt * per_tok;
            const float* qq = kk + Np;
            const float* aa = qq + Np;
            float v[C], acc[C];
#pragma unroll
            for (int j = 0; j < C; ++j) { v[j] = aa[a_len + cg * C + j]; acc[j] = 0.f; }
            const float a0 = aa[0];
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int n = rg + LR * i;
                const float kn = kk[n], qn = qq[n], an = A.a_per_row ? aa[n] : a0;
#pragma unroll
                for (int j = 0; j < C; ++j) {
                    S[i][j] = fmaf(an, S[i][j], kn * v[j]);
                    acc[j] = fmaf(S[i][j], qn, acc[j]);
                }
            }
            for (int o = cgw; o < 32; o <<= 1) {
#pragma unroll
                for (int j = 0; j < C; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
            }
            if (rg == 0 && live) {
                float* y = A.y + (size_t)(row0 + t0 + tt) * A.ld_y + (size_t)h * P + col0;
#pragma unroll
                for (int j = 0; j < C; ++j) y[j] = fmaf(skip, v[j], acc[j]);
            }
        }
    };
    for (int t0 = 0; t0 < n_new; t0 += OR_TILE) {
        const int nt = min(OR_TILE, n_new - t0);
        __syncthreads();
        if (A.vec_in) {                                        // four elements a turn; N, Np and per_tok are multiples of 4
            const int quads = Np / 4;
#pragma unroll 4
            for (int idx = threadIdx.x; idx < nt * quads; idx += threads) {
                const int tt = idx / quads, j = (idx - tt * quads) * 4;
                const size_t row = (size_t)(row0 + t0 + tt);
                float kv[4] = {0.f, 0.f, 0.f, 0.f}, qv[4] = {0.f, 0.f, 0.f, 0.f}, av[4] = {0.f, 0.f, 0.f, 0.f};
                if (j < N) {
                    or_ld4(kp + row * A.ld_k + A.k_col + (size_t)g * N + j, kv);
                    or_ld4(qp + row * A.ld_q + A.q_col + (size_t)g * N + j, qv);
                    const float cc = A.c != nullptr ? A.c[row * A.ld_c + h] : 1.0f;
#pragma unroll
                    for (int e = 0; e < 4; ++e) { kv[e] *= cc; qv[e] *= A.q_scale; }
                    if (A.a_per_row) or_ld4(A.a + row * A.ld_a + (size_t)h * N + j, av);
                }
                float* dst = sm + tt * per_tok + j;
                *reinterpret_cast<float4*>(dst) = make_float4(kv[0], kv[1], kv[2], kv[3]);
                *reinterpret_cast<float4*>(dst + Np) = make_float4(qv[0], qv[1], qv[2], qv[3]);
                if (A.a_per_row) *reinterpret_cast<float4*>(dst + 2 * Np) = make_float4(av[0], av[1], av[2], av[3]);
            }
        } else
#pragma unroll 8
        for (int idx = threadIdx.x; idx < nt * Np; idx += threads) {
            const int tt = idx / Np, j = idx - tt * Np;
            const size_t row = (size_t)(row0 + t0 + tt);
            float kv = 0.f, qv = 0.f;
            if (j < N) {
                kv = to_f32(kp[row * A.ld_k + A.k_col + (size_t)g * N + j]);
                if (A.c != nullptr) kv *= A.c[row * A.ld_c + h];
                qv = to_f32(qp[row * A.ld_q + A.q_col + (size_t)g * N + j]) * A.q_scale;
            }
            sm[tt * per_tok + j] = kv;
            sm[tt * per_tok + Np + j] = qv;
            if (A.a_per_row) sm[tt * per_tok + 2 * Np + j] = j < N ? A.a[row * A.ld_a + (size_t)h * N + j] : 0.f;
        }
        for (int idx = threadIdx.x; idx < nt * cols_per_cta; idx += threads) {
            const int tt = idx / cols_per_cta, j = idx - tt * cols_per_cta;
            const size_t row = (size_t)(row0 + t0 + tt);
            const int cc = blockIdx.x * cols_per_cta + j;
            sm[tt * per_tok + 2 * Np + a_len + j] = cc < P ? to_f32(vp[row * A.ld_v + A.v_col + (size_t)h * P + cc]) : 0.f;
        }
        if (!A.a_per_row)
            for (int tt = threadIdx.x; tt < nt; tt += threads) sm[tt * per_tok + 2 * Np] = A.a[(size_t)(row0 + t0 + tt) * A.ld_a + h];
        __syncthreads();
        compute(t0, nt);
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int n = rg + LR * i;
        if (!(live && n < N)) continue;
        if (C == 4 && A.vec_state) {
            *reinterpret_cast<float4*>(S_slot + (size_t)n * P + col0) = make_float4(S[i][0], S[i][1], S[i][2], S[i][C - 1]);
        } else {
#pragma unroll
            for (int j = 0; j < C; ++j) S_slot[(size_t)n * P + col0 + j] = S[i][j];
        }
    }
}

__global__ void decay_softplus_kernel(const void* __restrict__ raw, long long ld_raw, int col, int bf, const float* __restrict__ bias,
                                      const float* __restrict__ A_log, int rows, int heads, float* __restrict__ dt,
                                      float* __restrict__ a) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * heads) return;
    const int t = idx / heads, h = idx - t * heads;
    const size_t at = (size_t)t * ld_raw + col + h;
    float z = (bf ? __bfloat162float(((const bf16*)raw)[at]) : ((const float*)raw)[at]) + bias[h];
    const float d = z > 20.f ? z : log1pf(expf(z));
    dt[idx] = d;
    a[idx] = expf(-expf(A_log[h]) * d);
}

// a[t, c] = exp(-softplus(-z) / tau), z = b[c] + sum_r W2[c, r] * r1[t, r]
template <typename T>
__global__ void __launch_bounds__(256)
decay_lowrank_kernel(const T* __restrict__ r1, long long ld_r1, int col, int rank, const float* __restrict__ W2,
                     const float* __restrict__ b, float inv_tau, int rows, int channels, float* __restrict__ a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row[];
    const int t = blockIdx.x;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) row[r] = to_f32(r1[(size_t)t * ld_r1 + col + r]);
    __syncthreads();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float z = 0.f;
        for (int r = 0; r < rank; ++r) z = fmaf(W2[(size_t)c * rank + r], row[r], z);
        z += b != nullptr ? b[c] : 0.f;
        const float nz = -z;
        const float sp = nz > 20.f ? nz : log1pf(expf(nz));
        a[(size_t)t * channels + c] = expf(-sp * inv_tau);
    }
}

}  // namespace kl

using namespace kl;

// in_dtype: the type of q, k and v (KL_F32 or KL_BF16).  a_per_row != 0: a is [rows, heads * N].
KL_API int kl_outer_recurrence(const void* q, long long ld_q, int q_col, const void* k, long long ld_k, int k_col, const void* v,
                               long long ld_v, int v_col, const float* a, long long ld_a, int a_per_row, const float* c,
                               long long ld_c, const float* skip, float* state, long long ld_state, float* y, long long ld_y,
                               const int* cu_tokens, const int* seq_slots, int n_seqs, int max_new, int heads, int groups, int N, int P,
                               float q_scale, int in_dtype, cudaStream_t stream) {
    if (n_seqs <= 0) return KL_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0 || N > 1024) return KL_ERR_BAD_SIZE;
    if (in_dtype != KL_F32 && in_dtype != KL_BF16) return KL_ERR_BAD_DTYPE;
    int sms = 0, dev = 0;
    KL_CUDA(cudaGetDevice(&dev));
    KL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    OuterArgs A;
    A.q = q; A.ld_q = ld_q; A.q_col = q_col; A.k = k; A.ld_k = ld_k; A.k_col = k_col; A.v = v; A.ld_v = ld_v; A.v_col = v_col;
    A.a = a; A.ld_a = ld_a; A.c = c; A.ld_c = ld_c; A.skip = skip; A.state = state; A.ld_state = ld_state; A.y = y; A.ld_y = ld_y;
    A.cu_tokens = cu_tokens; A.seq_slots = seq_slots; A.heads = heads; A.groups = groups; A.N = N; A.P = P;
    A.a_per_row = a_per_row ? 1 : 0; A.q_scale = q_scale;
    A.vec_state = ((uintptr_t)state % 16 == 0 && ld_state % 4 == 0 && P % 4 == 0) ? 1 : 0;
    {   // slabs of R x C in registers: the largest slab that still gives every SM eight warps, else the smallest that fits
        const int slabs[3][2] = {{8, 4}, {4, 4}, {2, 2}};
        int pick = -1, pick_lr = 0;
        for (int z = 0; z < 3; ++z) {
            const int R = slabs[z][0], C = slabs[z][1];
            if (P % C) continue;
            int LR = 1;
            while (LR * R < N) LR <<= 1;
            if (LR > 32) continue;
            pick = z; pick_lr = LR;
            if ((long long)n_seqs * heads * LR * (P / C) / 32 >= 8LL * sms) break;
        }
        if (pick >= 0) {
            const int R = slabs[pick][0], C = slabs[pick][1], LR = pick_lr;
            int threads = LR * (P / C);
            threads = threads > 256 ? 256 : ((threads + 31) & ~31);
            auto ctas = [&](int th) { return (long long)((P / C + th / LR - 1) / (th / LR)) * heads * n_seqs; };
            // short runs (decode): smaller CTAs until every SM has two.  Long runs: a CTA's threads share the loading of
            // each tile of tokens, which is the same for every column of a head, so the CTA stays wide
            while (max_new <= 16 && threads > 32 && (threads / 2) % 32 == 0 && ctas(threads) < 2LL * sms) threads >>= 1;
            A.L = LR;
            const int cols = (threads / LR) * C;
            dim3 grid((P + cols - 1) / cols, heads, n_seqs);
            const int per_tok = 2 * LR * R + (a_per_row ? LR * R : 4) + cols;
            const size_t smem = (size_t)OR_TILE * per_tok * sizeof(float);
            const int es = in_dtype == KL_F32 ? 4 : 2;
            auto quad = [&](const void* p, long long ld, int col) { return (uintptr_t)p % (4 * es) == 0 && ld % 4 == 0 && col % 4 == 0; };
            A.vec_in = (N % 4 == 0 && (LR * R) % 4 == 0 && per_tok % 4 == 0 && quad(q, ld_q, q_col) && quad(k, ld_k, k_col) &&
                        (!a_per_row || ((uintptr_t)a % 16 == 0 && ld_a % 4 == 0))) ? 1 : 0;
            if (smem <= 200 * 1024) {
#define KL_SLAB(TI, R_, C_)                                                                                          \
    do {                                                                                                            \
        if (smem > 48 * 1024)                                                                                       \
            KL_CUDA(cudaFuncSetAttribute(outer_recurrence_slab_kernel<TI, R_, C_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        launch_kernel(outer_recurrence_slab_kernel<TI, R_, C_>, grid, threads, smem, stream, A);                    \
    } while (0)
#define KL_SLAB_BY(TI)                                                                                              \
    do {                                                                                                            \
        if (R == 8) KL_SLAB(TI, 8, 4); else if (R == 4) KL_SLAB(TI, 4, 4); else KL_SLAB(TI, 2, 2);                  \
    } while (0)
                if (in_dtype == KL_F32) KL_SLAB_BY(float); else KL_SLAB_BY(bf16);
#undef KL_SLAB_BY
#undef KL_SLAB
                KL_LAUNCH_CHECK();
                return KL_OK;
            }
        }
    }
    // any other size: a column of S over L lanes, rows of S in registers per thread at most 16 where 32 lanes allow it
    int L = 1;
    while (L < 32 && (N + L - 1) / L > 16) L <<= 1;
    // and more lanes (fewer rows per thread) while the launch would leave the SMs short of warps: a prompt of one sequence
    // is a chain of dependent steps per thread, and only other warps hide its latency
    long long warps = (long long)n_seqs * heads * P * L / 32;
    while (L < 32 && (N + L - 1) / L > 2 && warps < 24LL * sms) { L <<= 1; warps <<= 1; }
    const int npt = (N + L - 1) / L;
    A.L = L; A.vec_in = 0;
    // the largest CTA that still leaves two CTAs per SM (a CTA loads a tile of tokens, waits, and computes: another one
    // fills the wait), and no wider than the columns of S
    int threads = OR_THREADS;
    while (threads > 128 && (threads / 2 >= P * L || (long long)((P * L + threads - 1) / threads) * heads * n_seqs < 2LL * sms)) threads >>= 1;
    const int cols = threads / L;
    dim3 grid((P + cols - 1) / cols, heads, n_seqs);
    const size_t smem = (size_t)OR_TILE * (2 * N + (a_per_row ? N : 1) + cols) * sizeof(float);
    if (smem > 200 * 1024) return KL_ERR_BAD_SIZE;
#define KL_OR(TI, NPT)                                                                                              \
    do {                                                                                                            \
        if (smem > 48 * 1024)                                                                                       \
            KL_CUDA(cudaFuncSetAttribute(outer_recurrence_kernel<TI, NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        launch_kernel(outer_recurrence_kernel<TI, NPT>, grid, threads, smem, stream, A);                         \
    } while (0)
#define KL_OR_BY_NPT(TI)                                                                                            \
    do {                                                                                                            \
        if (npt <= 2) KL_OR(TI, 2); else if (npt <= 4) KL_OR(TI, 4); else if (npt <= 8) KL_OR(TI, 8); else if (npt <= 16) KL_OR(TI, 16); else KL_OR(TI, 32); \
    } while (0)
    if (in_dtype == KL_F32) KL_OR_BY_NPT(float); else KL_OR_BY_NPT(bf16);
#undef KL_OR_BY_NPT
#undef KL_OR
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_decay_softplus(const void* raw, long long ld_raw, int col, int dtype, const float* bias, const float* A_log, int rows,
                             int heads, float* dt, float* a, cudaStream_t stream) {
    if (rows <= 0 || heads <= 0) return KL_OK;
    if (dtype != KL_F32 && dtype != KL_BF16) return KL_ERR_BAD_DTYPE;
    const int total = rows * heads;
    launch_kernel(decay_softplus_kernel, (total + 255) / 256, 256, 0, stream, raw, ld_raw, col, (int)(dtype == KL_BF16), bias, A_log, rows,
                  heads, dt, a);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_decay_lowrank(const void* r1, long long ld_r1, int col, int rank, const float* W2, const float* b, float tau, int rows,
                            int channels, float* a, int dtype, cudaStream_t stream) {
    if (rows <= 0 || channels <= 0) return KL_OK;
    if (rank <= 0 || rank > 4096 || !(tau > 0.f)) return KL_ERR_BAD_SIZE;
    int yblocks = (channels + 255) / 256;
    if (yblocks > 64) yblocks = 64;
    dim3 grid(rows, yblocks);
    if (dtype == KL_F32)
        launch_kernel(decay_lowrank_kernel<float>, grid, 256, rank * sizeof(float), stream, (const float*)r1, ld_r1, col, rank, W2, b, 1.0f / tau,
                      rows, channels, a);
    else if (dtype == KL_BF16)
        launch_kernel(decay_lowrank_kernel<bf16>, grid, 256, rank * sizeof(float), stream, (const bf16*)r1, ld_r1, col, rank, W2, b, 1.0f / tau,
                      rows, channels, a);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
