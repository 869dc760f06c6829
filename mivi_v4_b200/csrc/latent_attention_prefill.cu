// Attention over a compressed cache (see latent_attention.cu) for steps with many query tokens, bfloat16, on the
// tensor cores.  Where a few query tokens fold W_uk into the query and read the cached rows as they are, many query
// tokens pay for building every head's keys and values once: the cached rows a step can see are copied out of their
// pages side by side, one product with [W_uk; W_uv] turns them into keys and values for all heads, and the attention
// itself is attention_sink_prefill.cu's plan: a block is 64 consecutive query tokens of one sequence for one head, 4
// warps of 16 queries; keys and values stream through shared memory in blocks of 64 (cp.async, double-buffered); both
// products are mma.sync m16n8k16 with float32 accumulation and the running-maximum softmax in float32 registers
// between them.  A head's key is [its unrotated part | the rotated part that all heads share]; the sink starts every
// row's maximum and denominator; the output is multiplied element by element by the sigmoid of a gate.
//
//   * latent_query:  q [N, nh, dim + rot] bfloat16 from the 32-bit projections, the last rot elements turned;
//   * latent_gather: the rows [lo_b, end_b) of every sequence b of the step, lo_b = max(0, start_b - window + 1),
//                    out of the pages into c [rows, rank] and r [rows, rot];
//   * latent_attention_prefill: q against kx [rows, nh dim | nh vdim] (the product's result) and r.
// Row r of sequence b's position t is  sum_{b' < b} (end_b' - lo_b') + t - lo_b  in all three.
#include "common.cuh"

namespace {

constexpr int QT = 64;          // queries per block
constexpr int KB = 64;          // keys per block of the stream
constexpr int NWARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

// first position a step's tokens of a sequence that starts the step at `start` can see
__device__ __forceinline__ int first_seen(int start, int window) { return window > 0 ? max(0, start - window + 1) : 0; }

// ------------------------------------------------------------------------------------------------------ queries
__global__ void __launch_bounds__(256)
latent_query_kernel(const float* __restrict__ proj, int ld, int q0, const float* __restrict__ inv_freq,
                    const int* __restrict__ positions, __nv_bfloat16* __restrict__ q, int nh, int dim, int rot,
                    int rot_dims) {
    mv_pdl_begin();
    const int n = blockIdx.x;
    const int dk = dim + rot, half = rot_dims >> 1;
    const float* row = proj + (size_t)n * ld + q0;
    const float pos = (float)positions[n];
    __nv_bfloat16* dst = q + (size_t)n * nh * dk;
    for (int e = threadIdx.x; e < nh * dk; e += blockDim.x) {
        const int c = e % dk;
        const int i = c - dim;
        float x = row[e];
        if (i >= 0 && i < rot_dims) {
            const int f = i < half ? i : i - half;
            float sn, cs;
            sincosf(pos * inv_freq[f], &sn, &cs);
            x = i < half ? x * cs - row[e + half] * sn : x * cs + row[e - half] * sn;
        }
        dst[e] = __float2bfloat16(x);
    }
}

// ------------------------------------------------------------------------------------------------------- gather
__global__ void __launch_bounds__(64)
latent_gather_kernel(const __nv_bfloat16* __restrict__ pool, long long page_stride, const int* __restrict__ page_table,
                     int table_stride, int page_shift, const int* __restrict__ cu, const int* __restrict__ starts, int B,
                     int window, int rank, int rot, __nv_bfloat16* __restrict__ c, __nv_bfloat16* __restrict__ r) {
    mv_pdl_begin();
    int b = 0, left = blockIdx.x, lo = 0;
    for (; b < B; ++b) {
        lo = first_seen(starts[b], window);
        const int rows = starts[b] + cu[b + 1] - cu[b] - lo;
        if (left < rows) break;
        left -= rows;
    }
    if (b >= B) return;
    const int t = lo + left;
    const int page = mv_read_page(page_table[(size_t)b * table_stride + (t >> page_shift)]);
    const uint4* src = reinterpret_cast<const uint4*>(pool + (size_t)page * page_stride +
                                                      (size_t)(t & ((1 << page_shift) - 1)) * (rank + rot));
    uint4* dc = reinterpret_cast<uint4*>(c + (size_t)blockIdx.x * rank);
    uint4* dr = reinterpret_cast<uint4*>(r + (size_t)blockIdx.x * rot);
    const int nc = rank >> 3, nr = rot >> 3;
    for (int i = threadIdx.x; i < nc + nr; i += blockDim.x) {
        const uint4 v = src[i];
        if (i < nc) dc[i] = v; else dr[i - nc] = v;
    }
}

// ---------------------------------------------------------------------------------------------------- attention
// q [N, nh, dim + rot]; kx [rows, ld_kx]: head h's unrotated keys at column h dim, its values at v0 + h dv; r [rows, rot];
// gate: 32-bit logits [N, >= nh dv] with row stride ld_gate, or null; o [N, nh dv].  The softmax weights enter the
// second product as two bfloat16 numbers each (the rounded weight and what the rounding left), so the sum over the
// values carries the weights to 16 bits of mantissa although the tensor cores read bfloat16.
template <int DKM, int DVM>
__global__ void __launch_bounds__(NWARPS * 32)
latent_attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kx, int ld_kx,
                                int v0, const __nv_bfloat16* __restrict__ rk, const int* __restrict__ cu,
                                const int* __restrict__ starts, const float* __restrict__ sinks,
                                const float* __restrict__ gate, int ld_gate, __nv_bfloat16* __restrict__ o, int B, int nh,
                                int dim, int rot, int dv, float scale, int window) {
    mv_pdl_begin();
    const int dk = dim + rot;
    const int ldk = dk + 8, ldv = dv + 8;             // padded rows: conflict-free fragment loads
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [2][KB][ldk]
    __nv_bfloat16* vs = ks + 2 * KB * ldk;                              // [2][KB][ldv]

    int b = 0, tile = blockIdx.x, base = 0;           // base: the gathered row of this sequence's first seen position
    for (; b < B; ++b) {
        const int len = cu[b + 1] - cu[b];
        const int tiles = (len + QT - 1) / QT;
        if (tile < tiles) break;
        tile -= tiles;
        base += starts[b] + len - first_seen(starts[b], window);
    }
    if (b >= B) return;
    const int h = blockIdx.y;
    const int lo = first_seen(starts[b], window);
    const int row0 = cu[b] + tile * QT;
    const int nq = min(QT, cu[b + 1] - cu[b] - tile * QT);
    const int pos0 = starts[b] + tile * QT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, t4 = lane & 3;

    const int qi0 = warp * 16 + gq, qi1 = qi0 + 8;
    const int p0 = pos0 + qi0, p1 = pos0 + qi1;
    unsigned qf[DKM / 16][4];
    {
        const __nv_bfloat16* r0 = q + ((size_t)(row0 + min(qi0, nq - 1)) * nh + h) * dk;
        const __nv_bfloat16* r1 = q + ((size_t)(row0 + min(qi1, nq - 1)) * nh + h) * dk;
#pragma unroll
        for (int kk = 0; kk < DKM / 16; ++kk) {
            if (kk * 16 < dk) {
                qf[kk][0] = *reinterpret_cast<const unsigned*>(r0 + kk * 16 + 2 * t4);
                qf[kk][1] = *reinterpret_cast<const unsigned*>(r1 + kk * 16 + 2 * t4);
                qf[kk][2] = *reinterpret_cast<const unsigned*>(r0 + kk * 16 + 2 * t4 + 8);
                qf[kk][3] = *reinterpret_cast<const unsigned*>(r1 + kk * 16 + 2 * t4 + 8);
            }
        }
    }

    float oacc[DVM / 8][4];
#pragma unroll
    for (int j = 0; j < DVM / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
    // the sink starts the running maximum and the denominator (its own term, exp(sink - max), is 1 now); a row's
    // denominator is summed over the four lanes of its quad at the end, so one of them holds the sink's 1
    float m0 = sinks ? sinks[h] : -INFINITY, m1 = m0;
    float l0 = (sinks && t4 == 0) ? 1.f : 0.f, l1 = l0;

    const int last_pos = pos0 + nq - 1;
    const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kb_begin = first_key / KB, n_iter = last_pos / KB + 1 - kb_begin;

    auto load_block = [&](int kb, int buf) {
        const int kc = dim >> 3, rc = rot >> 3, vc = dv >> 3, all = kc + rc + vc;
        for (int idx = threadIdx.x; idx < KB * all; idx += NWARPS * 32) {
            const int r = idx / all, c = idx - r * all;
            const int t = min(max(kb * KB + r, lo), last_pos);           // rows outside repeat a row that is there
            const size_t row = (size_t)(base + t - lo);
            if (c < kc)
                cp_async16(ks + ((size_t)buf * KB + r) * ldk + c * 8, kx + row * ld_kx + (size_t)h * dim + c * 8);
            else if (c < kc + rc)
                cp_async16(ks + ((size_t)buf * KB + r) * ldk + dim + (c - kc) * 8, rk + row * rot + (c - kc) * 8);
            else
                cp_async16(vs + ((size_t)buf * KB + r) * ldv + (c - kc - rc) * 8,
                           kx + row * ld_kx + v0 + (size_t)h * dv + (c - kc - rc) * 8);
        }
    };

    load_block(kb_begin, 0);
    cp_async_commit();
    for (int it = 0; it < n_iter; ++it) {
        const int kb = kb_begin + it, buf = it & 1;
        if (it + 1 < n_iter) load_block(kb + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const __nv_bfloat16* kt = ks + (size_t)buf * KB * ldk;
        const __nv_bfloat16* vt = vs + (size_t)buf * KB * ldv;
        float s[KB / 8][4];
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
            const __nv_bfloat16* krow = kt + (size_t)(j * 8 + gq) * ldk + 2 * t4;
#pragma unroll
            for (int kk = 0; kk < DKM / 16; ++kk) {
                if (kk * 16 < dk) {
                    const unsigned b0 = *reinterpret_cast<const unsigned*>(krow + kk * 16);
                    const unsigned b1 = *reinterpret_cast<const unsigned*>(krow + kk * 16 + 8);
                    mma_bf16(s[j], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
                }
            }
        }
        const int key0 = kb * KB;
        const bool need_mask = key0 + KB - 1 > pos0 + warp * 16 || (window > 0 && key0 <= pos0 + warp * 16 + 15 - window);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sc = s[j][e] * scale;
                if (need_mask) {
                    const int t = key0 + j * 8 + 2 * t4 + (e & 1);
                    const int p = (e < 2) ? p0 : p1;
                    if (t > p || (window > 0 && t <= p - window)) sc = -INFINITY;
                }
                s[j][e] = sc;
            }
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a row whose keys are all masked so far (and that has no sink) keeps m = -inf; use 0 as its reference
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = m0 == -INFINITY ? 0.f : exp2f((m0 - ref0) * LOG2E);
        const float c1 = m1 == -INFINITY ? 0.f : exp2f((m1 - ref1) * LOG2E);
        m0 = mn0; m1 = mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
            s[j][0] = exp2f((s[j][0] - ref0) * LOG2E);
            s[j][1] = exp2f((s[j][1] - ref0) * LOG2E);
            s[j][2] = exp2f((s[j][2] - ref1) * LOG2E);
            s[j][3] = exp2f((s[j][3] - ref1) * LOG2E);
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        l0 = l0 * c0 + sum0;
        l1 = l1 * c1 + sum1;
#pragma unroll
        for (int j = 0; j < DVM / 8; ++j) {
            oacc[j][0] *= c0; oacc[j][1] *= c0;
            oacc[j][2] *= c1; oacc[j][3] *= c1;
        }
        // O += P V, 16 keys at a time; P = hi + lo
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
            unsigned hi[4], lw[4];
#pragma unroll
            for (int f = 0; f < 4; ++f) {
                const float x = s[2 * kk + (f >> 1)][(f & 1) * 2], y = s[2 * kk + (f >> 1)][(f & 1) * 2 + 1];
                const __nv_bfloat162 hv = __floats2bfloat162_rn(x, y);
                hi[f] = *reinterpret_cast<const unsigned*>(&hv);
                lw[f] = pack_bf16(x - __low2float(hv), y - __high2float(hv));
            }
#pragma unroll
            for (int dj = 0; dj < DVM / 16; ++dj) {
                if (dj * 16 < dv) {
                    unsigned vb[4];
                    const int mi = lane >> 3, r = lane & 7;
                    ldmatrix_x4_trans(vb, vt + (size_t)(kk * 16 + (mi & 1) * 8 + r) * ldv + dj * 16 + (mi >> 1) * 8);
                    mma_bf16(oacc[2 * dj], hi[0], hi[1], hi[2], hi[3], vb[0], vb[1]);
                    mma_bf16(oacc[2 * dj + 1], hi[0], hi[1], hi[2], hi[3], vb[2], vb[3]);
                    mma_bf16(oacc[2 * dj], lw[0], lw[1], lw[2], lw[3], vb[0], vb[1]);
                    mma_bf16(oacc[2 * dj + 1], lw[0], lw[1], lw[2], lw[3], vb[2], vb[3]);
                }
            }
        }
        __syncthreads();
    }

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv[2] = {l0 > 0.f ? 1.f / l0 : 0.f, l1 > 0.f ? 1.f / l1 : 0.f};
    const int qi[2] = {qi0, qi1};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        if (qi[half] >= nq) continue;
        const size_t n = (size_t)(row0 + qi[half]);
        const float* g = gate ? gate + n * ld_gate + (size_t)h * dv + 2 * t4 : nullptr;
        __nv_bfloat16* dst = o + (n * nh + h) * dv + 2 * t4;
#pragma unroll
        for (int j = 0; j < DVM / 8; ++j) {
            if (j * 8 < dv) {
                float x = oacc[j][2 * half] * inv[half], y = oacc[j][2 * half + 1] * inv[half];
                if (g) {
                    x *= 1.0f / (1.0f + expf(-g[j * 8]));
                    y *= 1.0f / (1.0f + expf(-g[j * 8 + 1]));
                }
                *reinterpret_cast<unsigned*>(dst + j * 8) = pack_bf16(x, y);
            }
        }
    }
}

template <int DKM, int DVM>
int launch(const void* q, const void* kx, int ld_kx, int v0, const void* rk, const int* cu, const int* starts,
           const float* sinks, const float* gate, int ld_gate, void* o, int N, int B, int nh, int dim, int rot, int dv,
           float scale, int window, cudaStream_t stream) {
    const size_t smem = (size_t)2 * KB * (dim + rot + 8 + dv + 8) * sizeof(__nv_bfloat16);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(latent_attention_prefill_kernel<DKM, DVM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)((size_t)2 * KB * (DKM + 8 + DVM + 8) * sizeof(__nv_bfloat16)));
        attr_set = true;
    }
    const dim3 grid((N + QT - 1) / QT + B, nh);       // an upper bound of the tiles; spare blocks return at once
    mv_launch(latent_attention_prefill_kernel<DKM, DVM>, grid, NWARPS * 32, smem, stream, (const __nv_bfloat16*)q,
              (const __nv_bfloat16*)kx, ld_kx, v0, (const __nv_bfloat16*)rk, cu, starts, sinks, gate, ld_gate,
              (__nv_bfloat16*)o, B, nh, dim, rot, dv, scale, window);
    return mv_launch_status();
}

}  // namespace

MV_GUARD_SETTER(latent_attention_prefill)

// q [N, nh, dim + rot] bfloat16 from 32-bit rows `proj` (row stride ld, the queries from column q0), the first
// rot_dims of every head's last rot elements turned by the angle positions[n] inv_freq[i] (i with i + rot_dims / 2).
MV_API int mv_latent_query(const float* proj, int ld, int q0, const float* inv_freq, const int* positions, void* q, int N,
                           int nh, int dim, int rot, int rot_dims, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || (rot_dims && !inv_freq)) return (int)cudaErrorInvalidValue;
    mv_launch(latent_query_kernel, N, 256, 0, stream, proj, ld, q0, inv_freq, positions, (__nv_bfloat16*)q, nh, dim, rot,
              rot_dims);
    return mv_launch_status();
}

// The cached rows [rank | rot] (bfloat16) that the step's tokens can see, sequence after sequence, into c [rows, rank]
// and r [rows, rot]; `rows` is their number, sum_b (starts[b] + cu[b + 1] - cu[b] - first_seen(starts[b], window)).
MV_API int mv_latent_gather(const void* pool, long long page_stride, const int* page_table, int table_stride,
                            int page_size, const int* cu, const int* starts, int B, int window, int rank, int rot,
                            void* c, void* r, int rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (page_size < 1 || (page_size & (page_size - 1)) || rank % 8 || rot % 8 || window < 0) return (int)cudaErrorInvalidValue;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    mv_launch(latent_gather_kernel, rows, 64, 0, stream, (const __nv_bfloat16*)pool, page_stride, page_table, table_stride,
              shift, cu, starts, B, window, rank, rot, (__nv_bfloat16*)c, (__nv_bfloat16*)r);
    return mv_launch_status();
}

// bfloat16; dim and rot multiples of 8 whose sum is a multiple of 16 up to 192; dv a multiple of 16 up to 128.
MV_API int mv_latent_attention_prefill(const void* q, const void* kx, int ld_kx, int v0, const void* r, const int* cu,
                                       const int* starts, const float* sinks, const float* gate, int ld_gate, void* o,
                                       int N, int B, int nh, int dim, int rot, int dv, float scale, int window,
                                       cudaStream_t stream) {
    if (N <= 0) return 0;
    const int dk = dim + rot;
    if (dim % 8 || rot % 8 || dk % 16 || dv % 16 || dk < 16 || dv < 16 || dk > 192 || dv > 128 || ld_kx % 8 || v0 % 8 ||
        window < 0)
        return (int)cudaErrorInvalidValue;
#define LP_GO(A, C)                                                                                                        \
    return launch<A, C>(q, kx, ld_kx, v0, r, cu, starts, sinks, gate, ld_gate, o, N, B, nh, dim, rot, dv, scale, window, \
                        stream)
    if (dk <= 128 && dv <= 64) LP_GO(128, 64);
    if (dk <= 128) LP_GO(128, 128);
    if (dv <= 64) LP_GO(192, 64);
    LP_GO(192, 128);
#undef LP_GO
}
