// The mixed-head attention of attention_mixed.cu for whole prompts, portions and decode steps, tiled so that a chunk of
// keys and values is read once for several queries and all heads, and a sequence's keys can be cut over several CTAs:
//
//   s_h(i, j) = scale * q_h(i) . k_kv(h)(j);   s <- cap * tanh(s / cap);   s <- s - r1_h * ln(1 + r2_h * (i - j))
//   visible:    j <= i and (i - j < window or j < keep_first)
//   p_h(i, .) = softmax over the visible keys;   w_h(i, j) = sum_g talk[h, g] p_g(i, j);   out_h(i) = gate * sum_j w_h(i, j) v(j)
//
// w mixes NORMALISED weights of all heads at one key, so every head's maximum and sum must be known before the first
// product with the values.  The work is two launches of one kernel and, where the keys were cut, a third:
//
//   phase 0   every head's maximum and sum over the visible keys of its split           -> ml [rows, heads, splits, 2]
//   phase 1   merges the splits' maxima and sums, computes the scores once more, p = exp(s - m) / l, the mix through
//             shared memory, and O += W V in registers; one split writes `out`, several write float32 pieces
//   reduce    adds the pieces in the order of the splits, multiplies by the gate and rounds
//
// A CTA of 16 warps holds TQ consecutive tokens of one sequence with ALL heads and walks the keys in chunks of 32 by
// absolute position: a chunk lies in one page, and the chunks, the masks and the order of the sums depend on
// positions only.  Chunks that neither the window nor the kept first keys reach are skipped; the visible ones are dealt
// to the splits in turn.  In the scores a warp takes a head and a lane a key (the key's row in registers four
// elements at a time, the TQ query rows broadcast from shared memory); in the mix a thread takes a (query, key) pair
// and eight heads at a time; in W V a warp takes a head and 64 value columns, a lane two of them for all TQ queries.
// All arithmetic is 32-bit FMA: the weights after the mix are 32-bit numbers of either sign.
//
// ExiledOfCode/KuiperLLama's attention is mha_kernel.cu:61,74-106 (one sequence, one query, no window, no bias).
#include "common.cuh"

namespace kl {

constexpr int MT_WARPS = 16;
constexpr int MT_THREADS = MT_WARPS * 32;
constexpr int MT_CH = 32;             // keys per chunk
constexpr int MT_PS = 36;             // row stride of the weights in shared memory (16-byte rows, 4 mod 32 banks)

struct MixedTiledArgs {
    const void* q; long long q_stride;               // [rows, >= heads * dim]
    const void* gate; long long gate_stride;         // [rows, >= heads] or null
    void* out; long long out_stride;                 // [rows, >= heads * vdim]
    const void* k_cache; const void* v_cache;        // [pages, kv_heads, PAGE, dim] and [pages, kv_heads, PAGE, vdim]
    const int* block_table; int blocks_per_seq;
    const int* cu_tokens; const int* seq_slots; const int* seq_starts;
    const float* r1; const float* r2; const float* talk;
    float* ml;                                       // [rows, heads, splits, 2]
    float* part;                                     // [rows, splits, heads * vdim] (splits > 1)
    int heads, kv_heads, dim, vdim, window, keep_first, splits;
    int qp, kvp, vp;                                 // row strides in shared memory: queries, keys, values (elements)
    int pipelined;                                   // two key buffers and one of values, filled by asynchronous copies
    float scale, softcap, out_scale;
};

__device__ __forceinline__ void mt_ld4(const float* p, float (&x)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void mt_ld4(const bf16* p, float (&x)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
}
__device__ __forceinline__ void mt_ld2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
}
__device__ __forceinline__ void mt_ld2(const bf16* p, float& a, float& b) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
    a = __uint_as_float(v << 16); b = __uint_as_float(v & 0xffff0000u);
}

// rows of `width` elements from the cache (row r of key head g of the chunk at `src + (g * PAGE + r) * width`) into
// shared memory rows of stride `sp`; rows past `n_valid` and the columns from `width` to `sp` become zero
template <typename T>
__device__ __forceinline__ void mt_load_chunk(T* dst, const T* src, int G, int width, int sp, int n_valid) {
    if (width % 4 == 0) {
        const int quads = sp / 4;
        for (int idx = threadIdx.x; idx < G * MT_CH * quads; idx += MT_THREADS) {
            const int row = idx / quads, e = (idx - row * quads) * 4;
            const int g = row / MT_CH, j = row - g * MT_CH;
            T* d4 = dst + (size_t)row * sp + e;
            if (j < n_valid && e < width) {
                if (sizeof(T) == 4) *reinterpret_cast<float4*>(d4) = *reinterpret_cast<const float4*>(src + ((size_t)g * PAGE + j) * width + e);
                else *reinterpret_cast<uint2*>(d4) = *reinterpret_cast<const uint2*>(src + ((size_t)g * PAGE + j) * width + e);
            } else {
                if (sizeof(T) == 4) *reinterpret_cast<float4*>(d4) = make_float4(0.f, 0.f, 0.f, 0.f);
                else *reinterpret_cast<uint2*>(d4) = make_uint2(0u, 0u);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < G * MT_CH * sp; idx += MT_THREADS) {
            const int row = idx / sp, e = idx - row * sp;
            const int g = row / MT_CH, j = row - g * MT_CH;
            dst[idx] = (j < n_valid && e < width) ? src[((size_t)g * PAGE + j) * width + e] : from_f32<T>(0.f);
        }
    }
}

// the same chunk by asynchronous copies (rows of a multiple of four elements): 8 bytes a piece for bfloat16, 16 for float32
template <typename T>
__device__ __forceinline__ void mt_copy_chunk_async(T* dst, const T* src, int G, int width, int sp, int n_valid) {
    const int quads = sp / 4;
    for (int idx = threadIdx.x; idx < G * MT_CH * quads; idx += MT_THREADS) {
        const int row = idx / quads, e = (idx - row * quads) * 4;
        const int g = row / MT_CH, j = row - g * MT_CH;
        const bool valid = j < n_valid && e < width;
        const T* from = valid ? src + ((size_t)g * PAGE + j) * width + e : src;
        const uint32_t to = (uint32_t)__cvta_generic_to_shared(dst + (size_t)row * sp + e);
        const int bytes = valid ? 4 * (int)sizeof(T) : 0;                  // nothing read: the piece becomes zero
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(to), "l"(from), "n"(4 * (int)sizeof(T)), "r"(bytes) : "memory");
    }
}
__device__ __forceinline__ void mt_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void mt_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// UMAX: (head, 64 value columns) pieces of O per warp, TQ * UMAX <= 32 (phase 0 has none)
template <typename T, int TQ, int UMAX, int PHASE>
__global__ void __launch_bounds__(MT_THREADS, 1)
attention_mixed_tiled_kernel(const MixedTiledArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char mt_smem[];
    const int s = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x, split = blockIdx.z;       // late tiles see the most keys: they start first
    const int row0 = A.cu_tokens[s] + tile * TQ;
    const int nrows = min(TQ, A.cu_tokens[s + 1] - row0);
    if (nrows <= 0) return;
    const int H = A.heads, G = A.kv_heads, d = A.dim, dv = A.vdim, per = H / G;
    const int H8 = (H + 7) & ~7;
    const int i0 = A.seq_starts[s] + tile * TQ;
    const int i_last = i0 + nrows - 1;
    const int lo_tile = A.window > 0 ? max(0, i0 - A.window + 1) : 0;
    const int keep = A.window > 0 ? A.keep_first : 0;
    const int n_chunks = i_last / MT_CH + 1;
    const int* table = A.block_table + (size_t)A.seq_slots[s] * A.blocks_per_seq;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool mix = A.talk != nullptr;

    const int stat = (H * TQ + 3) & ~3;
    float* Pb = reinterpret_cast<float*>(mt_smem);                         // [H][TQ][MT_PS]
    float* Wb = Pb + (size_t)H * TQ * MT_PS;                               // the mixed weights (phase 1 with talk)
    float* talkT = Wb + ((PHASE == 1 && mix) ? (size_t)H * TQ * MT_PS : 0);    // talkT[g][h], rows of H8
    float* msm = talkT + ((PHASE == 1 && mix) ? (size_t)H * H8 : 0);
    float* lsm = msm + stat;
    float* bias_tab = lsm + stat + warp * (TQ + MT_CH);                    // the warp's distance biases of a chunk (after Qs, see below)
    T* Qs = reinterpret_cast<T*>(lsm + stat + MT_WARPS * (TQ + MT_CH));    // [H][TQ][qp]
    // keys [G][32][kvp] and values [G][32][vp]: one buffer for both in turn, or (pipelined) two of keys and one of values
    T* Kb = Qs + (size_t)H * TQ * A.qp;
    const size_t k_elems = (size_t)G * MT_CH * A.kvp;
    T* Vb = A.pipelined ? Kb + 2 * k_elems : Kb;

    // ---- prologue: the tile's queries; the maxima and sums
    {
        const T* q = (const T*)A.q;
        for (int idx = threadIdx.x; idx < H * TQ * A.qp; idx += MT_THREADS) {
            const int hr = idx / A.qp, e = idx - hr * A.qp;
            const int h = hr / TQ, r = hr - h * TQ;
            Qs[idx] = (r < nrows && e < d) ? q[(size_t)(row0 + r) * A.q_stride + (size_t)h * d + e] : from_f32<T>(0.f);
        }
    }
    if (PHASE == 0) {
        for (int idx = threadIdx.x; idx < H * TQ; idx += MT_THREADS) { msm[idx] = -INFINITY; lsm[idx] = 0.f; }
    } else {
        for (int idx = warp; idx < H * TQ; idx += MT_WARPS) {              // a (head, query) per warp, a split per lane
            const int h = idx / TQ, r = idx - h * TQ;
            float mz = -INFINITY, lz = 0.f;
            if (r < nrows && lane < A.splits) {
                const float* p = A.ml + (((size_t)(row0 + r) * H + h) * A.splits + lane) * 2;
                mz = p[0];
                lz = p[1];
            }
            const float m = warp_max(mz);
            const float l = warp_sum(mz == -INFINITY ? 0.f : lz * expf(mz - m));
            if (lane == 0) {
                msm[idx] = m;
                lsm[idx] = l > 0.f ? 1.0f / l : 0.f;       // the inverse of the sum
            }
        }
        if (mix)
            for (int idx = threadIdx.x; idx < H * H8; idx += MT_THREADS) {
                const int g = idx / H8, h = idx - g * H8;
                talkT[idx] = h < H ? A.talk[(size_t)h * H + g] : 0.f;
            }
    }

    const int slices = (dv + 63) / 64;
    const int n_units = H * slices;
    float acc[UMAX][TQ][2];
    if (PHASE == 1) {
#pragma unroll
        for (int u = 0; u < UMAX; ++u)
#pragma unroll
            for (int r = 0; r < TQ; ++r) { acc[u][r][0] = 0.f; acc[u][r][1] = 0.f; }
    }
    const int d4 = (d + 3) & ~3;

    // visible chunks are dealt to the splits in turn
    int mine = 0, c_next = -1;
    auto advance = [&]() {
        for (++c_next; c_next < n_chunks; ++c_next) {
            const int j = c_next * MT_CH;
            if (!(j + MT_CH - 1 >= lo_tile || j < keep)) continue;
            if ((mine++) % A.splits == split) break;
        }
    };
    auto chunk_src = [&](const void* cache, int c, int width) {
        const int j = c * MT_CH;
        return (const T*)cache + ((size_t)table[j / PAGE] * G * PAGE + j % PAGE) * width;
    };
    advance();
    if (A.pipelined) {
        if (c_next < n_chunks) mt_copy_chunk_async<T>(Kb, chunk_src(A.k_cache, c_next, d), G, d, A.kvp, min(MT_CH, i_last - c_next * MT_CH + 1));
        mt_commit();
    }
    int buf = 0;
    while (c_next < n_chunks) {
        const int c = c_next;
        advance();
        const int j0 = c * MT_CH;
        const int n_valid = min(MT_CH, i_last - j0 + 1);
        const T* Kc = Kb;
        if (A.pipelined) {
            Kc = Kb + buf * k_elems;
            mt_wait<0>();
            __syncthreads();                               // this chunk's keys are here; the chunk before is done with the buffers
            if (PHASE == 1) {
                mt_copy_chunk_async<T>(Vb, chunk_src(A.v_cache, c, dv), G, dv, A.vp, n_valid);
                mt_commit();
            }
            if (c_next < n_chunks)
                mt_copy_chunk_async<T>(Kb + (buf ^ 1) * k_elems, chunk_src(A.k_cache, c_next, d), G, d, A.kvp, min(MT_CH, i_last - c_next * MT_CH + 1));
            mt_commit();
            buf ^= 1;
        } else {
            __syncthreads();                               // the chunk before is done with the buffers
            mt_load_chunk<T>(Kb, chunk_src(A.k_cache, c, d), G, d, A.kvp, n_valid);
            __syncthreads();
        }

        // ---- scores: a head per warp, a key per lane, TQ queries in registers
        for (int h = warp; h < H; h += MT_WARPS) {
            float sc[TQ];
#pragma unroll
            for (int r = 0; r < TQ; ++r) sc[r] = 0.f;
            const T* kr = Kc + ((size_t)(h / per) * MT_CH + lane) * A.kvp;
            const T* qr = Qs + (size_t)h * TQ * A.qp;
            for (int e = 0; e < d4; e += 4) {
                float kx[4];
                mt_ld4(kr + e, kx);
#pragma unroll
                for (int r = 0; r < TQ; ++r) {
                    float qx[4];
                    mt_ld4(qr + r * A.qp + e, qx);
                    sc[r] = fmaf(qx[0], kx[0], sc[r]); sc[r] = fmaf(qx[1], kx[1], sc[r]);
                    sc[r] = fmaf(qx[2], kx[2], sc[r]); sc[r] = fmaf(qx[3], kx[3], sc[r]);
                }
            }
            const int pos = j0 + lane;
            if (A.r1 != nullptr) {                         // the bias depends on i - j alone: TQ + 31 values for the chunk
                const float r1 = A.r1[h], r2 = A.r2[h];
                __syncwarp();
                for (int x = lane; x < TQ + MT_CH - 1; x += 32) bias_tab[x] = r1 * log1pf(r2 * (float)max(0, i0 - j0 - (MT_CH - 1) + x));
                __syncwarp();
            }
#pragma unroll
            for (int r = 0; r < TQ; ++r) {
                const int i = i0 + r;
                const bool vis = r < nrows && pos <= i && (A.window == 0 || i - pos < A.window || pos < keep);
                float v = -INFINITY;
                if (vis) {
                    v = sc[r] * A.scale;
                    if (A.softcap > 0.f) v = A.softcap * tanhf(v / A.softcap);
                    if (A.r1 != nullptr) v -= bias_tab[r + (MT_CH - 1) - lane];
                }
                if (PHASE == 0) {
                    const float m_old = msm[h * TQ + r];
                    const float m_new = fmaxf(m_old, warp_max(v));
                    const float sum = warp_sum(vis ? expf(v - m_new) : 0.f);
                    __syncwarp();
                    if (lane == 0 && m_new != -INFINITY) {
                        lsm[h * TQ + r] = lsm[h * TQ + r] * (m_old == -INFINITY ? 0.f : expf(m_old - m_new)) + sum;
                        msm[h * TQ + r] = m_new;
                    }
                } else {
                    Pb[((size_t)h * TQ + r) * MT_PS + lane] = vis ? expf(v - msm[h * TQ + r]) * lsm[h * TQ + r] : 0.f;
                }
            }
        }
        if (PHASE == 0) continue;
        if (A.pipelined) {
            mt_wait<1>();                                  // the values are here (the next keys may still be on their way)
            __syncthreads();                               // every head's p of the chunk is written
        } else {
            __syncthreads();                               // every head's p of the chunk is written; the keys are free
            mt_load_chunk<T>(Vb, chunk_src(A.v_cache, c, dv), G, dv, A.vp, n_valid);
        }
        if (mix) {                                         // a (query, key) pair per thread, eight heads at a time
            constexpr int COLS = TQ * MT_CH;
            const int col = threadIdx.x % COLS, grp = threadIdx.x / COLS;
            const int r = col / MT_CH, j = col - r * MT_CH;
            for (int hb = grp; hb < H8 / 8; hb += MT_THREADS / COLS) {
                float w[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) w[u] = 0.f;
#pragma unroll 4
                for (int g = 0; g < H; ++g) {
                    const float p = Pb[((size_t)g * TQ + r) * MT_PS + j];
                    const float4 t0 = *reinterpret_cast<const float4*>(talkT + (size_t)g * H8 + hb * 8);
                    const float4 t1 = *reinterpret_cast<const float4*>(talkT + (size_t)g * H8 + hb * 8 + 4);
                    w[0] = fmaf(t0.x, p, w[0]); w[1] = fmaf(t0.y, p, w[1]); w[2] = fmaf(t0.z, p, w[2]); w[3] = fmaf(t0.w, p, w[3]);
                    w[4] = fmaf(t1.x, p, w[4]); w[5] = fmaf(t1.y, p, w[5]); w[6] = fmaf(t1.z, p, w[6]); w[7] = fmaf(t1.w, p, w[7]);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (hb * 8 + u < H) Wb[((size_t)(hb * 8 + u) * TQ + r) * MT_PS + j] = w[u];
            }
        }
        __syncthreads();

        // ---- O += W V: a (head, 64 columns) piece per warp and turn, two columns per lane, TQ queries
        const float* Ws = mix ? Wb : Pb;
#pragma unroll
        for (int u = 0; u < UMAX; ++u) {
            const int unit = warp + MT_WARPS * u;
            if (unit < n_units) {
                const int h = unit / slices, c0 = (unit - h * slices) * 64 + lane * 2;
                const T* vcol = Vb + (size_t)(h / per) * MT_CH * A.vp + min(c0, A.vp - 2);
                const float* wr = Ws + (size_t)h * TQ * MT_PS;
                for (int j = 0; j < MT_CH; j += 4) {
                    float va[4], vb[4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) mt_ld2(vcol + (size_t)(j + jj) * A.vp, va[jj], vb[jj]);
#pragma unroll
                    for (int r = 0; r < TQ; ++r) {
                        const float4 w = *reinterpret_cast<const float4*>(wr + r * MT_PS + j);
                        float x = acc[u][r][0], y = acc[u][r][1];
                        x = fmaf(w.x, va[0], x); y = fmaf(w.x, vb[0], y);
                        x = fmaf(w.y, va[1], x); y = fmaf(w.y, vb[1], y);
                        x = fmaf(w.z, va[2], x); y = fmaf(w.z, vb[2], y);
                        x = fmaf(w.w, va[3], x); y = fmaf(w.w, vb[3], y);
                        acc[u][r][0] = x; acc[u][r][1] = y;
                    }
                }
            }
        }
    }

    if (PHASE == 0) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < H * TQ; idx += MT_THREADS) {
            const int h = idx / TQ, r = idx - h * TQ;
            if (r < nrows) {
                float* p = A.ml + (((size_t)(row0 + r) * H + h) * A.splits + split) * 2;
                p[0] = msm[idx];
                p[1] = lsm[idx];
            }
        }
        return;
    }
    const T* gate = (const T*)A.gate;
#pragma unroll
    for (int u = 0; u < UMAX; ++u) {
        const int unit = warp + MT_WARPS * u;
        if (unit < n_units) {
            const int h = unit / slices, c0 = (unit - h * slices) * 64 + lane * 2;
#pragma unroll
            for (int r = 0; r < TQ; ++r) {
                if (r >= nrows) continue;
                const size_t row = (size_t)(row0 + r);
                if (A.splits > 1) {
                    float* p = A.part + (row * A.splits + split) * ((size_t)H * dv) + (size_t)h * dv;
                    if (c0 < dv) p[c0] = acc[u][r][0];
                    if (c0 + 1 < dv) p[c0 + 1] = acc[u][r][1];
                } else {
                    float f = A.out_scale;
                    if (gate != nullptr) f *= 1.0f / (1.0f + expf(-to_f32(gate[row * A.gate_stride + h])));
                    T* o = (T*)A.out + row * A.out_stride + (size_t)h * dv;
                    if (c0 < dv) o[c0] = from_f32<T>(acc[u][r][0] * f);
                    if (c0 + 1 < dv) o[c0 + 1] = from_f32<T>(acc[u][r][1] * f);
                }
            }
        }
    }
}

// out[t, h, :] = out_scale * sigmoid(gate[t, h]) * sum over the splits of part[t, z, h, :], in the order of the splits
template <typename T>
__global__ void attention_mixed_reduce_kernel(const float* __restrict__ part, int splits, const T* __restrict__ gate, long long gate_stride,
                                              T* __restrict__ out, long long out_stride, const int* __restrict__ token_slot, int rows,
                                              int heads, int vdim, float out_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int width = heads * vdim;
    const size_t total = (size_t)rows * width;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / width), o = (int)(idx - (size_t)t * width);
        if (token_slot[t] < 0) continue;
        const float* p = part + (size_t)t * splits * width + o;
        float y = 0.f;
        for (int z = 0; z < splits; ++z) y += p[(size_t)z * width];
        y *= out_scale;
        if (gate != nullptr) y *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + o / vdim])));
        out[(size_t)t * out_stride + o] = from_f32<T>(y);
    }
}

struct MixedTiledPlan { int tq, qp, kvp, vp, pipelined; size_t smem; };

// the largest tile of queries whose registers (pieces of O per warp) and shared memory fit; tq 0: none does
static MixedTiledPlan mixed_tiled_plan(int heads, int kv_heads, int dim, int vdim, int elem, bool mix, int max_new) {
    MixedTiledPlan P;
    P.qp = (dim + 3) & ~3;
    P.kvp = P.qp;
    if ((P.kvp / 4) % 2 == 0) P.kvp += 4;                  // an odd number of 16-byte (8-byte) pieces per row: no bank conflicts
    P.vp = vdim % 4 == 0 ? vdim : ((vdim + 1) & ~1);
    const int H8 = (heads + 7) & ~7;
    const int units = heads * ((vdim + 63) / 64);
    const int order[3] = {8, 4, 1};
    for (int pipelined = (dim % 4 == 0 && vdim % 4 == 0) ? 1 : 0; pipelined >= 0; --pipelined)
        for (int k = 0; k < 3; ++k) {
            const int tq = order[k];
            if (tq > 1 && max_new <= 1) continue;
            if (tq == 8 && max_new <= 4) continue;
            if (units > MT_WARPS * (32 / tq)) continue;
            const size_t stat = ((size_t)heads * tq + 3) & ~(size_t)3;
            const size_t words = (size_t)heads * tq * MT_PS * (mix ? 2 : 1) + (mix ? (size_t)heads * H8 : 0) + 2 * stat + MT_WARPS * (tq + MT_CH);
            const size_t k_elems = (size_t)kv_heads * MT_CH * P.kvp, v_elems = (size_t)kv_heads * MT_CH * P.vp;
            const size_t kv = pipelined ? 2 * k_elems + v_elems : (k_elems > v_elems ? k_elems : v_elems);
            P.smem = words * 4 + ((size_t)heads * tq * P.qp + kv) * elem;
            P.pipelined = pipelined;
            if (P.smem <= 226 * 1024) { P.tq = tq; return P; }
        }
    P.tq = 0; P.smem = 0; P.pipelined = 0;
    return P;
}

}  // namespace kl

using namespace kl;

// Queries per tile that kl_attention_mixed_tiled would use for these sizes, 0 where it cannot run them.
KL_API int kl_attention_mixed_tiled_fits(int heads, int kv_heads, int dim, int vdim, int dtype, int has_talk, int max_new) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0) return 0;
    if (dtype != KL_F32 && dtype != KL_BF16) return 0;
    return mixed_tiled_plan(heads, kv_heads, dim, vdim, dtype == KL_F32 ? 4 : 2, has_talk != 0, max_new).tq;
}

// ml: float32 [rows, heads, splits, 2]; part: float32 [rows, splits, heads * vdim] where splits > 1, else null.
KL_API int kl_attention_mixed_tiled(const void* q, long long q_stride, const void* gate, long long gate_stride, void* out,
                                    long long out_stride, const void* k_cache, const void* v_cache, const int* block_table,
                                    int blocks_per_seq, const int* cu_tokens, const int* seq_slots, const int* seq_starts,
                                    const int* token_slot, int rows, int n_seqs, int max_new, int heads, int kv_heads, int dim, int vdim,
                                    float scale, float softcap, const float* r1, const float* r2, const float* talk, int window,
                                    int keep_first, float out_scale, int splits, float* ml, float* part, int dtype, cudaStream_t stream) {
    if (rows <= 0 || n_seqs <= 0 || max_new <= 0) return KL_OK;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || window < 0 || keep_first < 0 || splits < 1 || splits > 32) return KL_ERR_BAD_SIZE;
    if ((r1 == nullptr) != (r2 == nullptr) || ml == nullptr || (splits > 1 && part == nullptr)) return KL_ERR_BAD_SIZE;
    if (dtype != KL_F32 && dtype != KL_BF16) return KL_ERR_BAD_DTYPE;
    const MixedTiledPlan P = mixed_tiled_plan(heads, kv_heads, dim, vdim, dtype == KL_F32 ? 4 : 2, talk != nullptr, max_new);
    if (P.tq == 0) return KL_ERR_BAD_SIZE;
    MixedTiledArgs A;
    A.q = q; A.q_stride = q_stride; A.gate = gate; A.gate_stride = gate_stride; A.out = out; A.out_stride = out_stride;
    A.k_cache = k_cache; A.v_cache = v_cache; A.block_table = block_table; A.blocks_per_seq = blocks_per_seq;
    A.cu_tokens = cu_tokens; A.seq_slots = seq_slots; A.seq_starts = seq_starts; A.r1 = r1; A.r2 = r2; A.talk = talk;
    A.ml = ml; A.part = part; A.heads = heads; A.kv_heads = kv_heads; A.dim = dim; A.vdim = vdim; A.window = window;
    A.keep_first = keep_first; A.splits = splits; A.qp = P.qp; A.kvp = P.kvp; A.vp = P.vp; A.pipelined = P.pipelined;
    A.scale = scale; A.softcap = softcap; A.out_scale = out_scale;
    const dim3 grid((max_new + P.tq - 1) / P.tq, n_seqs, splits);
    const int per_warp = (heads * ((vdim + 63) / 64) + MT_WARPS - 1) / MT_WARPS;
#define KL_MT(T, TQ, U)                                                                                                            \
    do {                                                                                                                           \
        KL_CUDA(cudaFuncSetAttribute(attention_mixed_tiled_kernel<T, TQ, 1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P.smem)); \
        KL_CUDA(cudaFuncSetAttribute(attention_mixed_tiled_kernel<T, TQ, U, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P.smem)); \
        launch_kernel(attention_mixed_tiled_kernel<T, TQ, 1, 0>, grid, MT_THREADS, P.smem, stream, A);                             \
        launch_kernel(attention_mixed_tiled_kernel<T, TQ, U, 1>, grid, MT_THREADS, P.smem, stream, A);                             \
    } while (0)
#define KL_MT_BY_TQ(T)                                                                                                             \
    do {                                                                                                                           \
        if (P.tq == 8) { if (per_warp <= 2) KL_MT(T, 8, 2); else KL_MT(T, 8, 4); }                                                 \
        else if (P.tq == 4) { if (per_warp <= 2) KL_MT(T, 4, 2); else KL_MT(T, 4, 8); }                                            \
        else { if (per_warp <= 2) KL_MT(T, 1, 2); else if (per_warp <= 8) KL_MT(T, 1, 8); else KL_MT(T, 1, 32); }                  \
    } while (0)
    if (dtype == KL_F32) KL_MT_BY_TQ(float); else KL_MT_BY_TQ(bf16);
#undef KL_MT_BY_TQ
#undef KL_MT
    KL_LAUNCH_CHECK();
    if (splits > 1) {
        const int blocks = kl::strided_grid((size_t)rows * heads * vdim, 256, 4);
        if (dtype == KL_F32)
            launch_kernel(attention_mixed_reduce_kernel<float>, blocks, 256, 0, stream, (const float*)part, splits, (const float*)gate, gate_stride,
                          (float*)out, out_stride, token_slot, rows, heads, vdim, out_scale);
        else
            launch_kernel(attention_mixed_reduce_kernel<bf16>, blocks, 256, 0, stream, (const float*)part, splits, (const bf16*)gate, gate_stride,
                          (bf16*)out, out_stride, token_slot, rows, heads, vdim, out_scale);
        KL_LAUNCH_CHECK();
    }
    return KL_OK;
}
