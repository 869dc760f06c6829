// Softmax attention over the paged cache with the variations that a grouped-query layer may carry:
//   * keys and values of different sizes (dk, dv);
//   * a root-mean-square norm over the WHOLE q projection and the whole k projection (all heads
//     at once), before the rotation;
//   * a rotation of the first rot_dims elements of every head only, element i paired with
//     i + rot_dims/2;
//   * capped scores: s <- cap * tanh(s / cap);
//   * a sliding window that keeps the first tokens: query i reads key j <= i if i - j < window or
//     j < keep_first;
//   * a sink: a learned number per head whose exponential joins the softmax's denominator, with no
//     value of its own;
//   * a gate per token and head, sigmoid of a logit, on the head's output;
//   * the q and k norm per head instead (one weight of the head's size, shared by all heads);
//   * a factor on the rotation's cos and sin (a rotation whose stretched frequencies are made up for
//     by longer vectors);
//   * a chunked mask: query i reads key j <= i only if both lie in the same chunk of `chunk` positions,
//     counted from the sequence's position 0.
//   * a distance bias: r1_h ln(1 + r2_h (i - j)) is taken off the score of query i and key j, two numbers a head;
//   * values that are the keys (the first dv elements of a key row): a page then holds key rows only;
//   * a gate per token and ELEMENT of the concatenated heads instead of one per head;
//   * every query head's weights applied to the values of EVERY kv head (32-bit results [token][head][kv head][dv]),
//     from which mv_mix_heads forms  out_h = sum_g talk[h][g] O[g][kv head of h]: softmax weights mixed between the
//     heads after the softmax, each head reading the values of its own kv head.
// Each is a parameter (0 or null turns it off).
//
// Cache layout of one layer's page: [kv head][row][dk] keys, then [kv head][row][dv] values; with
// dk == dv this is the layout [2][kv head][row][hd] of the library's other attention kernels.
#include "common.cuh"

#define AS_MAX_DIM 256

// ------------------------------------------------ prepare q, k, v of a step's tokens
// A token is shared by gridDim.y blocks: each works out the two sums of squares over the whole of q and of k
// (a few thousand values) and then finishes its share of the elements.  proj: 32-bit rows [q (nh*dk) | k (nkv*dk) | v (nkv*dv) | ...] with row
// stride ld.  q goes to q_out in the model's dtype, k and v into the token's row of its page.
template <typename T>
__global__ void __launch_bounds__(256)
qkv_prepare_wide_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ wq,
                        const float* __restrict__ wk, float eps, int rot_dims, const float* __restrict__ inv_freq,
                        const int* __restrict__ positions, const int* __restrict__ seq_of,
                        const int* __restrict__ page_table, int table_stride, int page_shift, T* __restrict__ pool,
                        long long page_stride, T* __restrict__ q_out, int nh, int nkv, int dk, int dv, int per_head,
                        float amplitude) {
    mv_pdl_begin();
    extern __shared__ float head_scale[];           // [nh + nkv] with per_head
    __shared__ float scratch[33];
    __shared__ float rot_sn[AS_MAX_DIM / 2], rot_cs[AS_MAX_DIM / 2];
    const int n = blockIdx.x;
    const float* row = proj + (size_t)n * ld;
    const int nq = nh * dk, nk = nkv * dk, nv = nkv * dv;
    // the rotation of pair i at this token's position is the same for every head: worked out once
    for (int i = threadIdx.x; i < (rot_dims >> 1); i += blockDim.x)
    {
        float sn, cs;
        sincosf((float)positions[n] * inv_freq[i], &sn, &cs);
        rot_sn[i] = sn * amplitude;
        rot_cs[i] = cs * amplitude;
    }
    const float* qr = row;
    const float* kr = row + nq;
    const float* vr = kr + nk;
    float sq = 0.f, sk = 0.f;
    float q_scale = 1.f, k_scale = 1.f;
    if (per_head) {
        // a warp a head: q's heads, then k's (they follow q in the row)
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int hh = warp; hh < nh + nkv; hh += (blockDim.x >> 5)) {
            const float* hr = row + (size_t)hh * dk;
            float ss = 0.f;
            for (int d = lane; d < dk; d += 32) ss = fmaf(hr[d], hr[d], ss);
            ss = mv_warp_sum(ss);
            if (lane == 0) head_scale[hh] = 1.0f / sqrtf(ss / (float)dk + eps);
        }
        __syncthreads();
    } else {
        for (int e = threadIdx.x; e < nq; e += blockDim.x) sq = fmaf(qr[e], qr[e], sq);
        for (int e = threadIdx.x; e < nk; e += blockDim.x) sk = fmaf(kr[e], kr[e], sk);
        q_scale = wq ? 1.0f / sqrtf(mv_block_sum(sq, scratch) / (float)nq + eps) : 1.f;
        k_scale = wk ? 1.0f / sqrtf(mv_block_sum(sk, scratch) / (float)nk + eps) : 1.f;
    }
    __syncthreads();                                 // the rotation's table is complete whatever norm ran
    const int pos = positions[n];
    const int page_size = 1 << page_shift;
    const int page = page_table[(size_t)seq_of[n] * table_stride + (pos >> page_shift)];
    const int prow = pos & (page_size - 1);
    T* kpage = pool + (size_t)page * page_stride;
    T* vpage = kpage + (size_t)nkv * page_size * dk;
    const bool page_ok = mv_page_ok(page);
    const int half = rot_dims >> 1;
    const int per = (nq + nk + nv + gridDim.y - 1) / gridDim.y;         // elements of q, k and v a block finishes
    const int e_lo = blockIdx.y * per, e_hi = min(e_lo + per, nq + nk + nv);
    for (int e = e_lo + threadIdx.x; e < min(e_hi, nq + nk); e += blockDim.x) {
        const bool is_q = e < nq;
        const int f = is_q ? e : e - nq;
        const float* src = is_q ? qr : kr;
        const float* w = is_q ? wq : wk;
        const int head = f / dk, d = f - head * dk;
        const float sc = per_head ? (w ? head_scale[is_q ? head : nh + head] : 1.f) : (is_q ? q_scale : k_scale);
        const int wo = per_head ? head * dk : 0;           // a per-head weight is indexed inside the head
        float a = src[f] * sc * (w ? w[f - wo] : 1.f);
        if (d < rot_dims) {
            // element d < half pairs with d + half: (u, v) -> (u cos - v sin, v cos + u sin)
            const int i = d < half ? d : d - half;
            const int fp = d < half ? f + half : f - half;
            const float b = src[fp] * sc * (w ? w[fp - wo] : 1.f);
            const float sn = rot_sn[i], cs = rot_cs[i];
            a = d < half ? a * cs - b * sn : a * cs + b * sn;
        }
        if (is_q)
            q_out[(size_t)n * nq + f] = mv_from_f32<T>(a);
        else if (page_ok)
            kpage[((size_t)head * page_size + prow) * dk + d] = mv_from_f32<T>(a);
    }
    if (page_ok)
        for (int e = max(e_lo, nq + nk) - (nq + nk) + threadIdx.x; e < e_hi - (nq + nk); e += blockDim.x) {
            const int head = e / dv, d = e - head * dv;
            vpage[((size_t)head * page_size + prow) * dv + d] = mv_from_f32<T>(vr[e]);
        }
}

MV_GUARD_SETTER(attention_sink)

MV_API int mv_qkv_prepare_wide(const float* proj, int ld, const float* wq, const float* wk, float eps, int rot_dims,
                               const float* inv_freq, const int* positions, const int* seq_of, const int* page_table,
                               int table_stride, int page_size, void* pool, long long page_stride, void* q_out,
                               int dtype, int N, int nh, int nkv, int dk, int dv, int per_head, float amplitude,
                               cudaStream_t stream) {
    if (N <= 0) return 0;
    const size_t smem = per_head ? sizeof(float) * (size_t)(nh + nkv) : 0;
    if ((page_size & (page_size - 1)) || rot_dims % 2 || rot_dims > dk || (rot_dims && !inv_freq) || smem > 32768)
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    // few tokens: several blocks a token, so that the step still spreads over the device
    const int parts = N >= 256 ? 1 : (N >= 64 ? 2 : 6);
    const dim3 grid(N, parts);
    if (dtype == MV_DT_BF16)
        mv_launch(qkv_prepare_wide_kernel<__nv_bfloat16>, grid, 256, smem, stream, proj, ld, wq, wk, eps, rot_dims, inv_freq,
                  positions, seq_of, page_table, table_stride, page_shift, (__nv_bfloat16*)pool, page_stride,
                  (__nv_bfloat16*)q_out, nh, nkv, dk, dv, per_head, amplitude);
    else
        mv_launch(qkv_prepare_wide_kernel<float>, grid, 256, smem, stream, proj, ld, wq, wk, eps, rot_dims, inv_freq,
                  positions, seq_of, page_table, table_stride, page_shift, (float*)pool, page_stride, (float*)q_out, nh,
                  nkv, dk, dv, per_head, amplitude);
    return mv_launch_status();
}

// ------------------------------------------------------------------ attention
// One block of eight warps per (token, kv head, tile of GT query heads of that kv head): the heads of a group
// read the same keys and values, so a key row and a value row are loaded once for all of them.  The keys a
// query reads are the kept first ones [0, keep) and the window [lo, pos], walked as one run, 32 at a time; the
// runs are dealt out to the eight warps in turn.  In a run each lane scores one key (against every head of the
// tile), the warp agrees on each head's running maximum, then the lanes split the value's elements for the
// weighted sums.  The sink starts the first warp's running maximum and denominator (its own term is
// exp(sink - max)), so it is counted once and needs no key.  The eight partial results are merged in a fixed
// order, so a position's result depends on nothing but its keys.
#define AS_WARPS 8
#define AS_ACC (AS_MAX_DIM / 32)
// Which element of a value row a lane's r-th sum belongs to: lane + 32 r, or with PAIR (rows of an even length on even
// offsets) the lane's r/2-th PAIR of neighbours, 2 lane + 64 (r / 2) + (r mod 2), which it loads with one instruction.
template <bool PAIR> __device__ __forceinline__ int as_dim(int lane, int r) {
    return PAIR ? 2 * lane + 64 * (r >> 1) + (r & 1) : lane + 32 * r;
}
__device__ __forceinline__ void as_load2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
}
__device__ __forceinline__ void as_load2(const __nv_bfloat16* p, float& a, float& b) {
    const unsigned v = *reinterpret_cast<const unsigned*>(p);
    a = __uint_as_float(v << 16); b = __uint_as_float(v & 0xffff0000u);
}
template <typename T, bool VEC, int GT, bool PAIR>
__global__ void __launch_bounds__(AS_WARPS * 32)
attention_sink_kernel(const T* __restrict__ q, const T* __restrict__ pool, long long page_stride,
                      const int* __restrict__ page_table, int table_stride, int page_shift,
                      const int* __restrict__ positions, const int* __restrict__ seq_of,
                      const float* __restrict__ sinks, const float* __restrict__ gate, int ld_gate,
                      T* __restrict__ o, int N, int nh, int nkv, int dk, int dv, float scale, float cap, int window,
                      int keep_first, int chunk, const float* __restrict__ r1, const float* __restrict__ r2, int v_in_k,
                      int gate_wide, float* __restrict__ o_all) {
    mv_pdl_begin();
    extern __shared__ __align__(16) float as_smem[];
    float* qs = as_smem;                            // [GT][dk]
    float* part_acc = qs + GT * dk;                 // [AS_WARPS][GT][dv]
    float* part_m = part_acc + AS_WARPS * GT * dv;  // [AS_WARPS][GT]
    float* part_l = part_m + AS_WARPS * GT;
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = nh / nkv, tiles = (G + GT - 1) / GT;
    // with o_all a block is one of nkv that share (token, kv head, tile): each applies the weights to another kv head's values
    const int vm = o_all ? nkv : 1;
    const int bid = blockIdx.x / vm, vg_all = blockIdx.x - bid * vm;
    const int n = bid / (nkv * tiles), rest = bid - n * nkv * tiles;
    const int g = rest / tiles, h0 = g * G + (rest - g * tiles) * GT;        // the tile's first query head
    const int vg = o_all ? vg_all : g;                                       // the kv head whose values are read
    const int n_heads = min(GT, (g + 1) * G - h0);
    const int pos = positions[n];
    const int page_size = 1 << page_shift;
    const int* table = page_table + (size_t)seq_of[n] * table_stride;
    const size_t v_base = v_in_k ? 0 : (size_t)nkv * page_size * dk;
    const int v_ld = v_in_k ? dk : dv;

    for (int idx = threadIdx.x; idx < GT * dk; idx += AS_WARPS * 32) {
        const int i = idx / dk, d = idx - i * dk;
        qs[idx] = i < n_heads ? mv_to_f32(q[((size_t)n * nh + h0 + i) * dk + d]) : 0.f;
    }
    __syncthreads();

    float acc[GT][AS_ACC], m[GT], l[GT];
#pragma unroll
    for (int i = 0; i < GT; ++i) {
#pragma unroll
        for (int r = 0; r < AS_ACC; ++r) acc[i][r] = 0.f;
        const bool first = sinks && wib == 0 && i < n_heads;
        m[i] = first ? sinks[h0 + i] : -INFINITY;
        l[i] = first ? 1.f : 0.f;
    }
    // a chunked mask: the keys from the start of the query's own chunk on
    const int lo = chunk > 0 ? pos - pos % chunk : (window > 0 ? max(0, pos - window + 1) : 0);
    const int keep = chunk > 0 ? 0 : min(keep_first, lo);
    const int total = keep + (pos - lo + 1);
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    for (int u0 = wib * 32; u0 < total; u0 += AS_WARPS * 32) {
        const int u = u0 + lane;
        const bool valid = u < total;
        const int t = u < keep ? u : lo + (u - keep);
        float s[GT], p[GT];
#pragma unroll
        for (int i = 0; i < GT; ++i) s[i] = -INFINITY;
        unsigned long long vaddr = 0;
        if (valid) {
            const int page = mv_read_page(table[t >> page_shift]);
            const T* pbase = pool + (size_t)page * page_stride;
            const size_t r = (size_t)g * page_size + (t & (page_size - 1));
            const T* krow = pbase + r * dk;
            vaddr = (unsigned long long)(pbase + v_base + ((size_t)vg * page_size + (t & (page_size - 1))) * v_ld);
            float dot[GT];
#pragma unroll
            for (int i = 0; i < GT; ++i) dot[i] = 0.f;
            if (VEC) {
#pragma unroll 4
                for (int d = 0; d < dk; d += 8) {
                    float kv[8];
                    mv_load8(krow + d, kv);
#pragma unroll
                    for (int i = 0; i < GT; ++i) {
                        // dk is a multiple of 8 here: the head's row in shared memory is read four values at a time
                        const float4 qa = *reinterpret_cast<const float4*>(qs + i * dk + d);
                        const float4 qb = *reinterpret_cast<const float4*>(qs + i * dk + d + 4);
                        dot[i] = fmaf(qa.x, kv[0], dot[i]); dot[i] = fmaf(qa.y, kv[1], dot[i]);
                        dot[i] = fmaf(qa.z, kv[2], dot[i]); dot[i] = fmaf(qa.w, kv[3], dot[i]);
                        dot[i] = fmaf(qb.x, kv[4], dot[i]); dot[i] = fmaf(qb.y, kv[5], dot[i]);
                        dot[i] = fmaf(qb.z, kv[6], dot[i]); dot[i] = fmaf(qb.w, kv[7], dot[i]);
                    }
                }
            } else {
                for (int d = 0; d < dk; ++d) {
                    const float kv = mv_to_f32(krow[d]);
#pragma unroll
                    for (int i = 0; i < GT; ++i) dot[i] = fmaf(qs[i * dk + d], kv, dot[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < GT; ++i) {
                s[i] = dot[i] * scale;
                if (r1 && i < n_heads) s[i] -= r1[h0 + i] * log1pf(r2[h0 + i] * (float)(pos - t));
                if (cap > 0.f) {
                    if (sizeof(T) == 2) {
                        // a bfloat16 run: tanh(x) = (1 - e^-2|x|) / (1 + e^-2|x|) with the fast exponential, as in the
                        // kernel of long steps (within 1e-6 of the cap; the operands were rounded to 2^-9)
                        const float x = s[i] * inv_cap, e2 = __expf(-2.0f * fabsf(x));
                        s[i] = copysignf(cap * __fdividef(1.0f - e2, 1.0f + e2), x);
                    } else {
                        s[i] = cap * tanhf(s[i] * inv_cap);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < GT; ++i) {
            const float m_new = fmaxf(m[i], mv_warp_max(s[i]));
            p[i] = valid ? expf(s[i] - m_new) : 0.f;
            const float corr = m[i] == -INFINITY ? 0.f : expf(m[i] - m_new);
            l[i] = l[i] * corr + mv_warp_sum(p[i]);
#pragma unroll
            for (int r = 0; r < AS_ACC; ++r) acc[i][r] *= corr;
            m[i] = m_new;
        }
        // the values of the run's keys, eight rows requested before any is used (a row beyond the run is not read)
        const int cnt = min(32, total - u0);
        for (int j0 = 0; j0 < cnt; j0 += 8) {
            const T* vrow[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) vrow[e] = (const T*)__shfl_sync(0xffffffffu, vaddr, j0 + e);
            float pj[GT][8];
#pragma unroll
            for (int i = 0; i < GT; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) pj[i][e] = __shfl_sync(0xffffffffu, p[i], j0 + e);
            if (PAIR) {
#pragma unroll
                for (int r = 0; r < AS_ACC; r += 2) {
                    const int d = as_dim<true>(lane, r);
                    if (d < dv) {
                        float x0[8], x1[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            x0[e] = x1[e] = 0.f;
                            if (j0 + e < cnt) as_load2(vrow[e] + d, x0[e], x1[e]);
                        }
#pragma unroll
                        for (int i = 0; i < GT; ++i)
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                acc[i][r] = fmaf(pj[i][e], x0[e], acc[i][r]);
                                acc[i][r + 1] = fmaf(pj[i][e], x1[e], acc[i][r + 1]);
                            }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < AS_ACC; ++r) {
                    const int d = lane + 32 * r;
                    if (d < dv) {
                        float x[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) x[e] = (j0 + e < cnt) ? mv_to_f32(vrow[e][d]) : 0.f;
#pragma unroll
                        for (int i = 0; i < GT; ++i)
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[i][r] = fmaf(pj[i][e], x[e], acc[i][r]);
                    }
                }
            }
        }
    }
    // merge the warps' partial results (with no sink a warp that saw no key holds m = -inf and weighs nothing;
    // the query's own key lies in some warp's run, so a head's denominator is never empty)
#pragma unroll
    for (int i = 0; i < GT; ++i) {
        if (lane == 0) { part_m[wib * GT + i] = m[i]; part_l[wib * GT + i] = l[i]; }
#pragma unroll
        for (int r = 0; r < AS_ACC; ++r) {
            const int d = as_dim<PAIR>(lane, r);
            if (d < dv) part_acc[(wib * GT + i) * dv + d] = acc[i][r];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_heads * dv; idx += AS_WARPS * 32) {
        const int i = idx / dv, d = idx - i * dv;
        float M = part_m[i];
#pragma unroll
        for (int w = 1; w < AS_WARPS; ++w) M = fmaxf(M, part_m[w * GT + i]);
        float L = 0.f, v = 0.f;
#pragma unroll
        for (int w = 0; w < AS_WARPS; ++w) {
            const float pm = part_m[w * GT + i];
            const float wgt = pm == -INFINITY ? 0.f : expf(pm - M);
            L = fmaf(part_l[w * GT + i], wgt, L);
            v = fmaf(part_acc[(w * GT + i) * dv + d], wgt, v);
        }
        float mul = 1.0f / L;
        if (gate) mul *= 1.0f / (1.0f + expf(-gate[(size_t)n * ld_gate + (gate_wide ? (size_t)(h0 + i) * dv + d : (size_t)(h0 + i))]));
        if (o_all)
            o_all[(((size_t)n * nh + h0 + i) * nkv + vg) * dv + d] = v * mul;
        else
            o[((size_t)n * nh + h0 + i) * dv + d] = mv_from_f32<T>(v * mul);
    }
}

// head_tile: see below.  q [N, nh * dk]; o [N, nh * dv]; sinks [nh] or null; gate: 32-bit logits, gate[n * ld_gate + h]
// (with gate_wide gate[n * ld_gate + h * dv + d]), or null; r1, r2 [nh] or null; v_in_k: the values are the keys' first dv
// elements; o_all: 32-bit [N, nh, nkv, dv] or null (then o is not written).
MV_API int mv_attention_sink(const void* q, const void* pool, long long page_stride, const int* page_table,
                             int table_stride, int page_size, const int* positions, const int* seq_of,
                             const float* sinks, const float* gate, int ld_gate, void* o, int dtype, int N, int nh,
                             int nkv, int dk, int dv, float scale, float cap, int window, int keep_first,
                             int head_tile, int chunk, const float* r1, const float* r2, int v_in_k, int gate_wide,
                             float* o_all, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (dk < 1 || dk > AS_MAX_DIM || dv < 1 || dv > AS_MAX_DIM || nkv < 1 || nh % nkv || (page_size & (page_size - 1)) ||
        (v_in_k && dv > dk) || (r1 && !r2))
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    const int G = nh / nkv;
    // head_tile query heads of a kv head share a block (their keys and values are loaded once): 1, 2 or 4, or 0
    // for the kernel's own choice.  Measured at 8 and 64 sequences of 1,088 visible keys (32 heads on 8 kv heads),
    // a block a head was as fast or faster (more blocks in flight hide the loads' latency; the shared rows
    // come from L2 anyway), so tiles are chosen only for steps of thousands of (token, head) pairs.
    int gt = head_tile > 0 ? head_tile : ((long long)N * nh >= 4096 && G >= 2 ? 2 : 1);
    if (gt != 1 && gt != 2 && gt != 4) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((long long)N * nkv * ((G + gt - 1) / gt) * (o_all ? nkv : 1));
    const int esize = dtype == MV_DT_BF16 ? 2 : 4;
    const bool vec = dk % 8 == 0 && ((uintptr_t)pool % 16) == 0 && (page_stride * esize) % 16 == 0;
    const size_t smem = sizeof(float) * ((size_t)gt * dk + (size_t)AS_WARPS * gt * (dv + 2));
    // value rows of an even length on even offsets: a lane takes pairs of neighbours, one load each
    const bool pair = dv % 2 == 0 && (v_in_k ? dk : dv) % 2 == 0 && page_stride % 2 == 0 && ((uintptr_t)pool % 8) == 0 &&
                      ((long long)nkv * page_size * dk) % 2 == 0;
#define AS_LAUNCH(T, V, GTV)                                                                                         \
    do {                                                                                                             \
    if (pair)                                                                                                        \
        mv_launch(attention_sink_kernel<T, V, GTV, true>, blocks, AS_WARPS * 32, smem, stream, (const T*)q,          \
                  (const T*)pool, page_stride, page_table, table_stride, page_shift, positions, seq_of, sinks, gate, \
                  ld_gate, (T*)o, N, nh, nkv, dk, dv, scale, cap, window, keep_first, chunk, r1, r2, v_in_k,         \
                  gate_wide, o_all);                                                                                 \
    else                                                                                                             \
    mv_launch(attention_sink_kernel<T, V, GTV, false>, blocks, AS_WARPS * 32, smem, stream, (const T*)q, (const T*)pool,    \
              page_stride, page_table, table_stride, page_shift, positions, seq_of, sinks, gate, ld_gate, (T*)o, N,  \
              nh, nkv, dk, dv, scale, cap, window, keep_first, chunk, r1, r2, v_in_k, gate_wide, o_all);             \
    } while (0)
#define AS_PICK(T, V)                                                                                                \
    do {                                                                                                             \
        if (gt == 4) AS_LAUNCH(T, V, 4); else if (gt == 2) AS_LAUNCH(T, V, 2); else AS_LAUNCH(T, V, 1);             \
    } while (0)
    if (dtype == MV_DT_BF16) {
        if (vec) AS_PICK(__nv_bfloat16, true); else AS_PICK(__nv_bfloat16, false);
    } else {
        if (vec) AS_PICK(float, true); else AS_PICK(float, false);
    }
#undef AS_PICK
#undef AS_LAUNCH
    return mv_launch_status();
}

// ------------------------------------------------------------------ softmax weights mixed between the heads
// out[n][h][:] = sum_g talk[h][g] * o_all[n][g][kv head of h][:]: what  sum_j (sum_g talk[h][g] w_g(i, j)) v_(kv(h))(j)
// is once every head's weights have been applied to every kv head's values.  32-bit sums; out in the model's dtype.
template <typename T>
__global__ void __launch_bounds__(256)
mix_heads_kernel(const float* __restrict__ o_all, const float* __restrict__ talk, T* __restrict__ out, long long total,
                 int nh, int nkv, int dv) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int d = (int)(idx % dv);
    const long long nhh = idx / dv;
    const int h = (int)(nhh % nh);
    const long long n = nhh / nh;
    const int m = h / (nh / nkv);
    const float* src = o_all + ((size_t)n * nh * nkv + m) * dv + d;
    float acc = 0.f;
    for (int g = 0; g < nh; ++g) acc = fmaf(talk[(size_t)h * nh + g], src[(size_t)g * nkv * dv], acc);
    out[idx] = mv_from_f32<T>(acc);
}

// The same with a block a token: the token's nh * nkv * dv values and the mixing matrix lie in shared memory, so that
// every value is read from memory once although nh / nkv heads sum it.
template <typename T>
__global__ void __launch_bounds__(256)
mix_heads_token_kernel(const float* __restrict__ o_all, const float* __restrict__ talk, T* __restrict__ out, int nh,
                       int nkv, int dv) {
    mv_pdl_begin();
    extern __shared__ __align__(16) float mh_smem[];
    float* vals = mh_smem;                                  // [nh][nkv][dv]
    float* tk = vals + (size_t)nh * nkv * dv;               // [nh][nh]
    const size_t n = blockIdx.x;
    const int per = nh * nkv * dv;
    const float* src = o_all + n * per;
    for (int i = threadIdx.x; i < per; i += blockDim.x) vals[i] = src[i];
    for (int i = threadIdx.x; i < nh * nh; i += blockDim.x) tk[i] = talk[i];
    __syncthreads();
    const int G = nh / nkv;
    for (int i = threadIdx.x; i < nh * dv; i += blockDim.x) {
        const int h = i / dv, d = i - h * dv, m = h / G;
        const float* col = vals + (size_t)m * dv + d;
        const float* row = tk + (size_t)h * nh;
        float acc = 0.f;
        for (int g = 0; g < nh; ++g) acc = fmaf(row[g], col[(size_t)g * nkv * dv], acc);
        out[n * nh * dv + i] = mv_from_f32<T>(acc);
    }
}

MV_API int mv_mix_heads(const float* o_all, const float* talk, void* out, int dtype, int N, int nh, int nkv, int dv,
                        cudaStream_t stream) {
    const long long total = (long long)N * nh * dv;
    if (total <= 0) return 0;
    if (nkv < 1 || nh % nkv) return (int)cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * ((size_t)nh * nkv * dv + (size_t)nh * nh);
    // (few tokens: a thread an element fills the device better than a block a token)
    if (smem <= 96 * 1024 && N >= 128) {
        if (dtype == MV_DT_BF16) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(mix_heads_token_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            mv_launch(mix_heads_token_kernel<__nv_bfloat16>, N, 256, smem, stream, o_all, talk, (__nv_bfloat16*)out, nh, nkv, dv);
        } else {
            if (smem > 48 * 1024) cudaFuncSetAttribute(mix_heads_token_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            mv_launch(mix_heads_token_kernel<float>, N, 256, smem, stream, o_all, talk, (float*)out, nh, nkv, dv);
        }
        return mv_launch_status();
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == MV_DT_BF16)
        mv_launch(mix_heads_kernel<__nv_bfloat16>, blocks, 256, 0, stream, o_all, talk, (__nv_bfloat16*)out, total, nh, nkv, dv);
    else
        mv_launch(mix_heads_kernel<float>, blocks, 256, 0, stream, o_all, talk, (float*)out, total, nh, nkv, dv);
    return mv_launch_status();
}
