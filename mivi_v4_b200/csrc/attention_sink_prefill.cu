// Attention with a sink, capped scores, a window that keeps the first tokens, a gate per head, and keys and
// values of different sizes (see attention_sink.cu for the formulas) for steps with many query tokens,
// bfloat16, over the paged cache.  The plan is attention_prefill.cu's: a block is 64 consecutive query tokens
// of one sequence for one query head, 4 warps of 16 queries; the keys and values the tile may see stream
// through shared memory in blocks of 64 (cp.async, double-buffered); both products run on the tensor cores
// (mma.sync m16n8k16, float32 accumulation) with the running-maximum softmax in float32 registers between
// them.  What differs: the key blocks a tile walks are the blocks of the kept first tokens followed by the
// blocks of its window; the scores are scaled and capped in float32 before the maximum is taken; the sink
// starts every row's maximum and denominator; the output is multiplied by the sigmoid of the row's gate;
// with a chunked mask the walk starts at the first query's chunk and keys before a row's own chunk are masked.
// Key and value sizes are run-time multiples of 16 up to the template's bounds.  Further parameters, as in
// attention_sink.cu: a distance bias r1_h ln(1 + r2_h (i - j)) taken off the scores; values that are the keys' first dv
// elements; a gate per element instead of per head; every head's weights applied to every kv head's values (32-bit
// results, for weights that are mixed between the heads afterwards).  SPLIT: a softmax weight enters the value
// product as two bfloat16 numbers, the rounded weight and the rounding's remainder (two mma a tile), which
// carries 16 bits of its mantissa.
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
// the remainders of two values after their rounding to the bfloat16 pair `rounded`, as a bfloat16 pair
__device__ __forceinline__ unsigned pack_rest(float lo, float hi, unsigned rounded) {
    return pack_bf16(lo - __uint_as_float(rounded << 16), hi - __uint_as_float(rounded & 0xffff0000u));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

template <int DKM, int DVM, bool SPLIT>
__global__ void __launch_bounds__(NWARPS * 32)
attention_sink_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                              long long page_stride, const int* __restrict__ page_table, int table_stride,
                              int page_shift, const int* __restrict__ cu, const int* __restrict__ starts,
                              const float* __restrict__ sinks, const float* __restrict__ gate, int ld_gate,
                              __nv_bfloat16* __restrict__ o, int B, int nh, int nkv, int dk, int dv, float scale,
                              float cap, int window, int keep_first, int chunk, const float* __restrict__ r1,
                              const float* __restrict__ r2, int v_in_k, int gate_wide, float* __restrict__ o_all) {
    const int ldk = dk + 8, ldv = dv + 8;             // padded rows: conflict-free fragment loads
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [2][KB][ldk]
    __nv_bfloat16* vs = ks + 2 * KB * ldk;                              // [2][KB][ldv]

    int b = 0, tile = blockIdx.x;
    for (; b < B; ++b) {
        const int tiles = (cu[b + 1] - cu[b] + QT - 1) / QT;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (b >= B) return;
    // with o_all the grid's y counts (head, kv head whose values are read)
    const int h = o_all ? blockIdx.y / nkv : blockIdx.y, g = h / (nh / nkv);
    const int vg = o_all ? blockIdx.y - h * nkv : g;
    const float db1 = r1 ? r1[h] : 0.f, db2 = r1 ? r2[h] : 0.f;
    const int row0 = cu[b] + tile * QT;
    const int rows_in_seq = cu[b + 1] - cu[b];
    const int nq = min(QT, rows_in_seq - tile * QT);
    const int pos0 = starts[b] + tile * QT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, t4 = lane & 3;
    const int page_size = 1 << page_shift;
    const int* table = page_table + (size_t)b * table_stride;
    const size_t v_base = v_in_k ? 0 : (size_t)nkv * page_size * dk;
    const int v_ld = v_in_k ? dk : dv;

    const int qi0 = warp * 16 + gq, qi1 = qi0 + 8;
    const int p0 = pos0 + qi0, p1 = pos0 + qi1;
    const int cs0 = chunk > 0 ? p0 - p0 % chunk : 0, cs1 = chunk > 0 ? p1 - p1 % chunk : 0;    // where the rows' chunks start
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
    // the sink starts the running maximum and the denominator (its own term, exp(sink - max), is 1 now); the
    // denominator of a row is summed over the four lanes of its quad at the end, so one of them holds it
    float m0 = sinks ? sinks[h] : -INFINITY, m1 = m0;
    float l0 = (sinks && t4 == 0) ? 1.f : 0.f, l1 = l0;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    // key blocks this tile walks: the blocks that hold kept first tokens and lie before the window's
    // blocks, then from the first query's window start to the last query's position
    const int last_pos = pos0 + nq - 1;
    // with a chunked mask (chunk > 0: a query reads only the keys of its own chunk of positions) the first
    // query's chunk starts the walk
    const int first_key = chunk > 0 ? pos0 - pos0 % chunk : (window > 0 ? max(0, pos0 - window + 1) : 0);
    const int kb_begin = first_key / KB, kb_end = last_pos / KB + 1;
    const int n_kept = (chunk == 0 && window > 0 && keep_first > 0) ? min((keep_first + KB - 1) / KB, kb_begin) : 0;
    const int n_iter = n_kept + kb_end - kb_begin;

    auto load_block = [&](int kb, int buf) {
        const int kchunks = dk >> 3, vchunks = dv >> 3;
        for (int idx = threadIdx.x; idx < KB * (kchunks + vchunks); idx += NWARPS * 32) {
            const int r = idx / (kchunks + vchunks), c = idx - r * (kchunks + vchunks);
            const int t = min(kb * KB + r, last_pos);                    // rows past the end repeat the last key
            const int page = mv_read_page(table[t >> page_shift]);
            const __nv_bfloat16* pbase = pool + (size_t)page * page_stride;
            const size_t prow = (size_t)g * page_size + (t & (page_size - 1));
            if (c < kchunks)
                cp_async16(ks + ((size_t)buf * KB + r) * ldk + c * 8, pbase + prow * dk + c * 8);
            else
                cp_async16(vs + ((size_t)buf * KB + r) * ldv + (c - kchunks) * 8,
                           pbase + v_base + ((size_t)vg * page_size + (t & (page_size - 1))) * v_ld + (c - kchunks) * 8);
        }
    };
    auto block_of = [&](int it) { return it < n_kept ? it : kb_begin + (it - n_kept); };

    load_block(block_of(0), 0);
    cp_async_commit();
    for (int it = 0; it < n_iter; ++it) {
        const int kb = block_of(it), buf = it & 1;
        if (it + 1 < n_iter) load_block(block_of(it + 1), buf ^ 1);
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
        // scale and cap, mask, then the running maximum of the two rows
        const int key0 = kb * KB;
        const bool need_mask = r1 != nullptr || it < n_kept || key0 + KB - 1 > pos0 + warp * 16 ||
                               (chunk > 0 ? key0 < cs1 : (window > 0 && key0 <= pos0 + warp * 16 + 15 - window));
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sc = s[j][e] * scale;
                if (cap > 0.f) {
                    // tanh(x) = (1 - e^-2|x|) / (1 + e^-2|x|) with the fast exponential: within 1e-6 of the capped
                    // score's size, far below the bfloat16 rounding of the weights that follows
                    const float x = sc * inv_cap, e2 = __expf(-2.0f * fabsf(x));
                    sc = copysignf(cap * __fdividef(1.0f - e2, 1.0f + e2), x);
                }
                if (need_mask) {
                    const int t = key0 + j * 8 + 2 * t4 + (e & 1);
                    const int p = (e < 2) ? p0 : p1;
                    if (t > p || (chunk > 0 ? t < ((e < 2) ? cs0 : cs1)
                                            : (window > 0 && t <= p - window && t >= keep_first))) sc = -INFINITY;
                    else if (r1) sc -= db1 * __logf(1.0f + db2 * (float)(p - t));
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
        // O += P V, 16 keys at a time
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
            const unsigned a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            const unsigned a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            const unsigned a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            const unsigned a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            unsigned c0r = 0, c1r = 0, c2r = 0, c3r = 0;                   // what the rounding left of each weight
            if (SPLIT) {
                c0r = pack_rest(s[2 * kk][0], s[2 * kk][1], a0);
                c1r = pack_rest(s[2 * kk][2], s[2 * kk][3], a1);
                c2r = pack_rest(s[2 * kk + 1][0], s[2 * kk + 1][1], a2);
                c3r = pack_rest(s[2 * kk + 1][2], s[2 * kk + 1][3], a3);
            }
#pragma unroll
            for (int dj = 0; dj < DVM / 16; ++dj) {
                if (dj * 16 < dv) {
                    unsigned vb[4];
                    const int mi = lane >> 3, r = lane & 7;
                    ldmatrix_x4_trans(vb, vt + (size_t)(kk * 16 + (mi & 1) * 8 + r) * ldv + dj * 16 + (mi >> 1) * 8);
                    mma_bf16(oacc[2 * dj], a0, a1, a2, a3, vb[0], vb[1]);
                    mma_bf16(oacc[2 * dj + 1], a0, a1, a2, a3, vb[2], vb[3]);
                    if (SPLIT) {
                        mma_bf16(oacc[2 * dj], c0r, c1r, c2r, c3r, vb[0], vb[1]);
                        mma_bf16(oacc[2 * dj + 1], c0r, c1r, c2r, c3r, vb[2], vb[3]);
                    }
                }
            }
        }
        __syncthreads();
    }

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.f / l0, i1 = 1.f / l1;
    auto finish = [&](int qi, float inv, int e0) {
        if (qi >= nq) return;
        const size_t row = (size_t)(row0 + qi);
        const float* grow = gate ? gate + row * ld_gate + (gate_wide ? (size_t)h * dv : (size_t)h) : nullptr;
        if (grow && !gate_wide) inv *= 1.0f / (1.0f + expf(-grow[0]));
#pragma unroll
        for (int j = 0; j < DVM / 8; ++j) {
            if (j * 8 < dv) {
                const int d = j * 8 + 2 * t4;
                float x = oacc[j][e0] * inv, y = oacc[j][e0 + 1] * inv;
                if (grow && gate_wide) {
                    x *= 1.0f / (1.0f + expf(-grow[d]));
                    y *= 1.0f / (1.0f + expf(-grow[d + 1]));
                }
                if (o_all)
                    *reinterpret_cast<float2*>(o_all + ((row * nh + h) * nkv + vg) * dv + d) = make_float2(x, y);
                else
                    *reinterpret_cast<unsigned*>(o + (row * nh + h) * dv + d) = pack_bf16(x, y);
            }
        }
    };
    finish(qi0, i0, 0);
    finish(qi1, i1, 2);
}

template <int DKM, int DVM, bool SPLIT>
int launch(const void* q, const void* pool, long long page_stride, const int* page_table, int table_stride,
           int page_shift, const int* cu, const int* starts, const float* sinks, const float* gate, int ld_gate, void* o,
           int N, int B, int nh, int nkv, int dk, int dv, float scale, float cap, int window, int keep_first,
           int chunk, const float* r1, const float* r2, int v_in_k, int gate_wide, float* o_all, cudaStream_t stream) {
    const size_t smem = (size_t)2 * KB * (dk + 8 + dv + 8) * sizeof(__nv_bfloat16);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(attention_sink_prefill_kernel<DKM, DVM, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)((size_t)2 * KB * (DKM + 8 + DVM + 8) * sizeof(__nv_bfloat16)));
        attr_set = true;
    }
    dim3 grid((N + QT - 1) / QT + B, o_all ? nh * nkv : nh);         // an upper bound of the tiles; spare blocks return at once
    attention_sink_prefill_kernel<DKM, DVM, SPLIT><<<grid, NWARPS * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, page_stride, page_table, table_stride, page_shift, cu,
        starts, sinks, gate, ld_gate, (__nv_bfloat16*)o, B, nh, nkv, dk, dv, scale, cap, window, keep_first, chunk, r1, r2,
        v_in_k, gate_wide, o_all);
    return mv_launch_status();
}

}  // namespace

MV_GUARD_SETTER(attention_sink_prefill)

// bfloat16 only; key and value sizes that are multiples of 16 up to 128.  Other sizes and float32 take the
// kernel of attention_sink.cu.
MV_API int mv_attention_sink_prefill(const void* q, const void* pool, long long page_stride, const int* page_table,
                                     int table_stride, int page_size, const int* cu, const int* starts,
                                     const float* sinks, const float* gate, int ld_gate, void* o, int N, int B, int nh,
                                     int nkv, int dk, int dv, float scale, float cap, int window, int keep_first,
                                     int chunk, const float* r1, const float* r2, int v_in_k, int gate_wide, float* o_all,
                                     int split, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (nkv < 1 || nh % nkv || (page_size & (page_size - 1)) || dk % 16 || dv % 16 || dk < 16 || dv < 16 || dk > 128 ||
        dv > 128 || (v_in_k && dv > dk) || (r1 && !r2))
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
#define AS_GO(A, C)                                                                                                  \
    do {                                                                                                             \
        if (split)                                                                                                   \
            return launch<A, C, true>(q, pool, page_stride, page_table, table_stride, page_shift, cu, starts, sinks, gate, \
                                      ld_gate, o, N, B, nh, nkv, dk, dv, scale, cap, window, keep_first, chunk, r1, r2, \
                                      v_in_k, gate_wide, o_all, stream);                                             \
        return launch<A, C, false>(q, pool, page_stride, page_table, table_stride, page_shift, cu, starts, sinks, gate, \
                                   ld_gate, o, N, B, nh, nkv, dk, dv, scale, cap, window, keep_first, chunk, r1, r2,    \
                                   v_in_k, gate_wide, o_all, stream);                                                \
    } while (0)
    if (dk <= 64 && dv <= 64) AS_GO(64, 64);
    if (dk <= 64) AS_GO(64, 128);
    if (dv <= 64) AS_GO(128, 64);
    AS_GO(128, 128);
#undef AS_GO
}
