// Attention over a compressed cache: every token keeps ONE row [c (rank) | r (rot)] for all heads, c a normed
// low-rank latent and r a rotated key part.  Per head the key is [W_uk,h c | r] and the value W_uv,h c, so with
//
//     qa_h = [W_uk,h^T q_h,unrotated | q_h,rotated]          (rank + rot numbers)
//
// the score is qa_h . [c | r] and the head's output is W_uv,h (sum_j p_j c_j): the heads share the cached rows as
// keys, and the values are the keys' first `rank` elements.  Nothing but c and r is cached or rebuilt.
//
//   * latent_prepare: from a token's projections, the root-mean-square norm of c (with a weight), the rotation of
//     r and of the queries' rotated parts (element i of the rotated part pairs with i + rot/2), the row into its page;
//   * head_product: y[n, h, :] = W_h x[n, h, :] (or W_h^T), one small matrix per head: q -> qa and the output's way back
//     (there with sigmoid(gate) on the result);
//   * latent_attention: every query token on its own over its sequence's rows, causal, with a sliding window and a
//     sink (a learned number per head whose exponential joins the softmax's denominator, with no value).
// Scores, softmax, norms and angles are 32-bit; the cache is in the model's dtype.
//
// Cache layout of one layer's page: [row][rank + rot].
#include "common.cuh"

#define LA_MAX_ROT 512

// ---------------------------------------------------------------------------------------------------- prepare
// proj: 32-bit rows with stride ld; q at column q0: [head][dim unrotated | rot rotated]; the latent at column c0:
// [rank | rot].  qa: 32-bit [N, nh, rank + rot]; its last rot columns are written here.  Of the rot elements the
// first rot_dims turn (element i with i + rot_dims/2), the others pass unchanged.
template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, int ld, int q0, int c0, const float* __restrict__ wc, float eps,
                      const float* __restrict__ inv_freq, const int* __restrict__ positions,
                      const int* __restrict__ seq_of, const int* __restrict__ page_table, int table_stride,
                      int page_shift, T* __restrict__ pool, long long page_stride, float* __restrict__ qa, int nh, int dim,
                      int rot, int rank, int rot_dims) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    __shared__ float rot_sn[LA_MAX_ROT / 2], rot_cs[LA_MAX_ROT / 2];
    const int n = blockIdx.x;
    const float* row = proj + (size_t)n * ld;
    const int pos = positions[n];
    const int half = rot_dims >> 1;            // the first rot_dims of the rot elements turn, the rest pass unchanged
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        rot_sn[i] = sn;
        rot_cs[i] = cs;
    }
    const float* c = row + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(c[i], c[i], ss);
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)rank + eps);      // (its barriers also publish the table)
    const int page_size = 1 << page_shift;
    const int page = page_table[(size_t)seq_of[n] * table_stride + (pos >> page_shift)];
    const int w = rank + rot;
    if (mv_page_ok(page)) {
        T* dst = pool + (size_t)page * page_stride + (size_t)(pos & (page_size - 1)) * w;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = mv_from_f32<T>(c[i] * scale * wc[i]);
        const float* r = c + rank;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float u = r[i], v = r[i + half];
            dst[rank + i] = mv_from_f32<T>(u * rot_cs[i] - v * rot_sn[i]);
            dst[rank + half + i] = mv_from_f32<T>(v * rot_cs[i] + u * rot_sn[i]);
        }
        for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = mv_from_f32<T>(r[i]);
    }
    if (!qa) return;                       // the queries are prepared elsewhere
    for (int e = threadIdx.x; e < nh * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const float* qr = row + q0 + (size_t)h * (dim + rot) + dim;
        const float u = qr[i], v = qr[i + half];
        float* dst = qa + ((size_t)n * nh + h) * w + rank;
        dst[i] = u * rot_cs[i] - v * rot_sn[i];
        dst[half + i] = v * rot_cs[i] + u * rot_sn[i];
    }
    for (int e = threadIdx.x; e < nh * (rot - rot_dims); e += blockDim.x) {
        const int h = e / (rot - rot_dims), i = rot_dims + e - h * (rot - rot_dims);
        qa[((size_t)n * nh + h) * w + rank + i] = row[q0 + (size_t)h * (dim + rot) + dim + i];
    }
}

MV_GUARD_SETTER(latent_attention)

MV_API int mv_latent_prepare(const float* proj, int ld, int q0, int c0, const float* wc, float eps, const float* inv_freq,
                             const int* positions, const int* seq_of, const int* page_table, int table_stride,
                             int page_size, void* pool, long long page_stride, int dtype, float* qa, int N, int nh,
                             int dim, int rot, int rank, int rot_dims, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (rot < 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > rot || rot > LA_MAX_ROT || rank < 1 || page_size < 1 || (page_size & (page_size - 1)))
        return (int)cudaErrorInvalidValue;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    if (dtype == MV_DT_BF16)
        mv_launch(latent_prepare_kernel<__nv_bfloat16>, N, 256, 0, stream, proj, ld, q0, c0, wc, eps, inv_freq, positions,
                  seq_of, page_table, table_stride, shift, (__nv_bfloat16*)pool, page_stride, qa, nh, dim, rot, rank, rot_dims);
    else
        mv_launch(latent_prepare_kernel<float>, N, 256, 0, stream, proj, ld, q0, c0, wc, eps, inv_freq, positions, seq_of,
                  page_table, table_stride, shift, (float*)pool, page_stride, qa, nh, dim, rot, rank, rot_dims);
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------ a small matrix per head
// y[n, h, o] = sum_i W_h[o, i] x[n, h, i]  with W stored [nh * O, I] (head h owns rows h O .. (h + 1) O), or, with
// `transposed`, W stored [nh * I, O] and y[n, h, o] = sum_i W_h[i, o] x[n, h, i].  x: 32-bit, element (n, h, i) at
// x[n ldx + h hx + i]; y likewise with ldy, hy.  `gate` (or null): 32-bit logits, element (n, h, o) at
// gate[n ldg + h O + o]; the result is multiplied by sigmoid of it.  Sums are 32-bit.
// A block is 32 tokens x 64 outputs of one head; a thread has 2 tokens x 4 outputs.
#define HP_TN 32
#define HP_TO 64
#define HP_TK 32

template <typename TW, typename TY>
__global__ void __launch_bounds__(256)
head_product_kernel(const float* __restrict__ x, long long ldx, int hx, const TW* __restrict__ w, int transposed,
                    const float* __restrict__ gate, long long ldg, TY* __restrict__ y, long long ldy, int hy, int N, int I,
                    int O) {
    mv_pdl_begin();
    __shared__ float xs[HP_TN][HP_TK + 1];
    __shared__ float ws[HP_TK][HP_TO + 1];
    const int h = blockIdx.z, n0 = blockIdx.y * HP_TN, o0 = blockIdx.x * HP_TO;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;       // outputs 4 tx .. 4 tx + 3, tokens 2 ty, 2 ty + 1
    float acc[2][4] = {};
    for (int k0 = 0; k0 < I; k0 += HP_TK) {
        __syncthreads();
        for (int e = tid; e < HP_TN * HP_TK; e += 256) {
            const int r = e / HP_TK, c = e - r * HP_TK;
            const int n = n0 + r, i = k0 + c;
            xs[r][c] = (n < N && i < I) ? x[(size_t)n * ldx + (size_t)h * hx + i] : 0.f;
        }
        if (transposed) {
            for (int e = tid; e < HP_TK * HP_TO; e += 256) {
                const int r = e / HP_TO, c = e - r * HP_TO;           // consecutive threads: consecutive o
                const int i = k0 + r, o = o0 + c;
                ws[r][c] = (i < I && o < O) ? mv_to_f32(w[((size_t)h * I + i) * O + o]) : 0.f;
            }
        } else {
            for (int e = tid; e < HP_TK * HP_TO; e += 256) {
                const int c = e / HP_TK, r = e - c * HP_TK;           // consecutive threads: consecutive i
                const int i = k0 + r, o = o0 + c;
                ws[r][c] = (i < I && o < O) ? mv_to_f32(w[((size_t)h * O + o) * I + i]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < HP_TK; ++k) {
            const float a0 = xs[2 * ty][k], a1 = xs[2 * ty + 1][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = ws[k][4 * tx + j];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int n = n0 + 2 * ty + t;
        if (n >= N) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + 4 * tx + j;
            if (o >= O) continue;
            float v = acc[t][j];
            if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)n * ldg + (size_t)h * O + o]));
            y[(size_t)n * ldy + (size_t)h * hy + o] = mv_from_f32<TY>(v);
        }
    }
}

MV_API int mv_head_product(const float* x, long long ldx, int hx, const void* w, int w_dtype, int transposed,
                           const float* gate, long long ldg, void* y, int y_dtype, long long ldy, int hy, int N, int nh,
                           int I, int O, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (nh < 1 || I < 1 || O < 1) return (int)cudaErrorInvalidValue;
    const dim3 grid((O + HP_TO - 1) / HP_TO, (N + HP_TN - 1) / HP_TN, nh);
#define HP_LAUNCH(TW, TY)                                                                                              \
    mv_launch(head_product_kernel<TW, TY>, grid, 256, 0, stream, x, ldx, hx, (const TW*)w, transposed, gate, ldg, (TY*)y, \
              ldy, hy, N, I, O)
    if (w_dtype == MV_DT_BF16) {
        if (y_dtype == MV_DT_BF16) HP_LAUNCH(__nv_bfloat16, __nv_bfloat16); else HP_LAUNCH(__nv_bfloat16, float);
    } else {
        if (y_dtype == MV_DT_BF16) HP_LAUNCH(float, __nv_bfloat16); else HP_LAUNCH(float, float);
    }
#undef HP_LAUNCH
    return mv_launch_status();
}

// ---------------------------------------------------------------------------------------------------- attention
// One block a (token, tile of up to LA_HEADS heads); a warp a head.  The block brings LA_KEYS rows of the cache into
// shared memory at a time; a lane scores one key for its warp's head (a dot product over rank + rot), the warp keeps the
// running maximum and denominator, then every lane adds the rows' first `rank` elements, weighted, into the output
// columns it owns (lane, lane + 32, ...).  The maximum starts at the sink and the denominator at 1 where there is one,
// so the sink counts once and has no value.
#define LA_HEADS 8
#define LA_KEYS 32
#define LA_AHEAD 5             // 16-byte copies a thread has on their way at a time
#define LA_MAX_OUT 32          // output columns a lane (the template's R) at most: rank <= 1024

template <typename T, int R>
__global__ void __launch_bounds__(LA_HEADS * 32)
latent_attention_kernel(const float* __restrict__ qa, const T* __restrict__ pool, long long page_stride,
                        const int* __restrict__ page_table, int table_stride, int page_shift,
                        const int* __restrict__ positions, const int* __restrict__ seq_of,
                        const float* __restrict__ sinks, float* __restrict__ out, int nh, int rank, int rot, float scale,
                        int window, int splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    mv_pdl_begin();
    extern __shared__ __align__(16) float la_smem[];
    const int w = rank + rot;
    const int wp = w | 1;                                       // odd row pitch: a lane a row without bank conflicts
    float* qs = la_smem;                                        // [LA_HEADS][w]
    float* ks = qs + LA_HEADS * w;                              // [LA_KEYS][wp]
    const int n = blockIdx.x, h0 = blockIdx.y * LA_HEADS;
    const int heads = min(LA_HEADS, nh - h0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[n];
    const int* table = page_table + (size_t)seq_of[n] * table_stride;
    const int page_mask = (1 << page_shift) - 1;
    // rows of the cache start on 16 bytes and are whole 16-byte pieces
    const bool wide = (w * sizeof(T)) % 16 == 0 && (page_stride * sizeof(T)) % 16 == 0 && ((uintptr_t)pool & 15) == 0;
    for (int e = threadIdx.x; e < heads * w; e += blockDim.x) qs[e] = qa[((size_t)n * nh + h0) * w + e];
    int j_lo = window > 0 ? max(0, pos - window + 1) : 0;
    int j_hi = pos;
    const int split = blockIdx.z;
    if (splits > 1) {                                           // this block's share of the keys, whole tiles of LA_KEYS
        const int per = ((pos - j_lo + splits) / splits + LA_KEYS - 1) / LA_KEYS * LA_KEYS;
        j_lo += split * per;
        j_hi = min(pos, j_lo + per - 1);
    }
    const bool active = warp < heads;
    const int h = h0 + warp;
    const bool with_sink = active && sinks && split == 0;       // the sink counts once: in the first share
    float m = with_sink ? sinks[h] : -INFINITY;
    float l = with_sink ? 1.f : 0.f;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    const float* q = qs + warp * w;
    for (int j0 = j_lo; j0 <= j_hi; j0 += LA_KEYS) {
        const int nk = min(LA_KEYS, j_hi - j0 + 1);
        __syncthreads();
        if (wide) {
            // 16 bytes a copy, LA_AHEAD of them on their way before the first is unpacked: a thread that waited for
            // every element by itself spent the tile waiting
            constexpr int V = 16 / (int)sizeof(T);
            const int cpr = w / V, total = nk * cpr;
            for (int e0 = threadIdx.x; e0 < total; e0 += LA_AHEAD * LA_HEADS * 32) {
                uint4 got[LA_AHEAD];
#pragma unroll
                for (int u = 0; u < LA_AHEAD; ++u) {
                    const int e = e0 + u * LA_HEADS * 32;
                    if (e < total) {
                        const int r = e / cpr, c = e - r * cpr;
                        const int j = j0 + r;
                        const int page = mv_read_page(table[j >> page_shift]);
                        got[u] = *reinterpret_cast<const uint4*>(pool + (size_t)page * page_stride +
                                                                 (size_t)(j & page_mask) * w + c * V);
                    }
                }
#pragma unroll
                for (int u = 0; u < LA_AHEAD; ++u) {
                    const int e = e0 + u * LA_HEADS * 32;
                    if (e < total) {
                        const int r = e / cpr, c = e - r * cpr;
                        float f[V];
                        mv_unpack16(got[u], f, (const T*)nullptr);
#pragma unroll
                        for (int i = 0; i < V; ++i) ks[r * wp + c * V + i] = f[i];
                    }
                }
            }
        } else {
            for (int e = threadIdx.x; e < nk * w; e += blockDim.x) {
                const int r = e / w, c = e - r * w;
                const int j = j0 + r;
                const int page = mv_read_page(table[j >> page_shift]);
                ks[r * wp + c] = mv_to_f32(pool[(size_t)page * page_stride + (size_t)(j & page_mask) * w + c]);
            }
        }
        __syncthreads();
        if (!active) continue;
        float s = -INFINITY;
        if (lane < nk) {
            const float* kr = ks + lane * wp;
            float d = 0.f;
            int c = 0;
            if ((w & 3) == 0) {                     // q four elements a load (a row of qs then starts on 16 bytes)
                float d1 = 0.f, d2 = 0.f, d3 = 0.f;
                for (; c < w; c += 4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(q + c);
                    d = fmaf(q4.x, kr[c], d);
                    d1 = fmaf(q4.y, kr[c + 1], d1);
                    d2 = fmaf(q4.z, kr[c + 2], d2);
                    d3 = fmaf(q4.w, kr[c + 3], d3);
                }
                d = (d + d1) + (d2 + d3);
            }
            for (; c < w; ++c) d = fmaf(q[c], kr[c], d);
            s = d * scale;
        }
        const float m_new = fmaxf(m, mv_warp_max(s));
        const float p = lane < nk ? expf(s - m_new) : 0.f;
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * corr + mv_warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] *= corr;
        for (int t = 0; t < nk; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const float* kr = ks + t * wp;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int c = lane + 32 * r;
                if (c < rank) acc[r] = fmaf(pt, kr[c], acc[r]);
            }
        }
    }
    if (active && splits > 1) {                                 // unnormalised sums, maximum and denominator of the share
        const size_t at = ((size_t)n * nh + h) * splits + split;
        float* o = part_o + at * rank;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int c = lane + 32 * r;
            if (c < rank) o[c] = acc[r];
        }
        if (lane == 0) {
            part_ml[2 * at] = m;
            part_ml[2 * at + 1] = l;
        }
    } else if (active) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        float* o = out + ((size_t)n * nh + h) * rank;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int c = lane + 32 * r;
            if (c < rank) o[c] = acc[r] * inv;
        }
    }
}

// The shares of one (token, head) put together: out = sum_z acc_z exp(m_z - M) / sum_z l_z exp(m_z - M), M = max m_z.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, float* __restrict__ out,
                              int rank, int splits) {
    mv_pdl_begin();
    const size_t at = (size_t)blockIdx.x * splits;
    float M = -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, part_ml[2 * (at + z)]);
    float L = 0.f;
    for (int z = 0; z < splits; ++z) {
        const float mz = part_ml[2 * (at + z)];
        if (mz != -INFINITY) L += part_ml[2 * (at + z) + 1] * expf(mz - M);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float a = 0.f;
        for (int z = 0; z < splits; ++z) {
            const float mz = part_ml[2 * (at + z)];
            if (mz != -INFINITY) a = fmaf(part_o[(at + z) * rank + c], expf(mz - M), a);
        }
        out[(size_t)blockIdx.x * rank + c] = a * inv;
    }
}

// qa [N, nh, rank + rot] and out [N, nh, rank], 32-bit; pool: pages of [row][rank + rot] in `dtype`; sinks [nh] or null.
// splits > 1: every (token, head tile) is `splits` blocks, each over its share of the keys, and a second kernel puts
// the shares together; part_o [N, nh, splits, rank] and part_ml [N, nh, splits, 2] are their scratch.
MV_API int mv_latent_attention(const float* qa, const void* pool, long long page_stride, int dtype, const int* page_table,
                               int table_stride, int page_size, const int* positions, const int* seq_of,
                               const float* sinks, float* out, int N, int nh, int rank, int rot, float scale, int window,
                               int splits, float* part_o, float* part_ml, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (rank < 1 || rank > 32 * LA_MAX_OUT || rot < 0 || page_size < 1 || (page_size & (page_size - 1)) || window < 0 ||
        splits < 1 || splits > 65535 || (splits > 1 && (!part_o || !part_ml)))
        return (int)cudaErrorInvalidValue;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    const int w = rank + rot;
    const size_t smem = sizeof(float) * ((size_t)LA_HEADS * w + (size_t)LA_KEYS * (w | 1));
    const dim3 grid(N, (nh + LA_HEADS - 1) / LA_HEADS, splits);
#define LA_LAUNCH(T, R)                                                                                                   \
    do {                                                                                                                  \
        if (smem > 48 * 1024) {                                                                                           \
            const cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<T, R>,                                     \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
            if (e != cudaSuccess) return (int)e;                                                                          \
        }                                                                                                                 \
        mv_launch(latent_attention_kernel<T, R>, grid, LA_HEADS * 32, smem, stream, qa, (const T*)pool, page_stride,      \
                  page_table, table_stride, shift, positions, seq_of, sinks, out, nh, rank, rot, scale, window, splits,  \
                  part_o, part_ml);                                                                                       \
    } while (0)
#define LA_BY_RANK(T)                                                                                                     \
    do {                                                                                                                  \
        if (rank <= 128) LA_LAUNCH(T, 4);                                                                                 \
        else if (rank <= 256) LA_LAUNCH(T, 8);                                                                            \
        else if (rank <= 512) LA_LAUNCH(T, 16);                                                                           \
        else LA_LAUNCH(T, 32);                                                                                            \
    } while (0)
    if (dtype == MV_DT_BF16) LA_BY_RANK(__nv_bfloat16); else LA_BY_RANK(float);
#undef LA_BY_RANK
#undef LA_LAUNCH
    if (splits > 1) {
        const int e = mv_launch_status();
        if (e) return e;
        mv_launch(latent_attention_merge_kernel, N * nh, 128, 0, stream, (const float*)part_o, (const float*)part_ml, out,
                  rank, splits);
    }
    return mv_launch_status();
}
