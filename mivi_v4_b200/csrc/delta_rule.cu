// The gated delta rule with a decay per key channel, one head at a time:
//
//     S  <- diag(g_t) S                        (S: dk x dv; g_t: a factor in (0, 1] per key channel)
//     u_t = beta_t (v_t - S^T k_t)             (what the state does not yet say about v_t)
//     S  <- S + k_t u_t^T
//     o_t = S^T q_t                            (the read-out sees the token's own write)
//
// with q and k made unit vectors per head first (x / sqrt(sum x^2 + norm_eps), q also times q_scale),
// beta_t = sigmoid(b_t) per head, and g = exp(-exp(A_log_h) softplus(a + dt_bias)) per head and key channel
// (with head_decay: a and dt_bias hold one number a head, and all key channels of a head share its decay).
// Head h reads q and k of head h / (heads / kv_heads).  The state lives in 32-bit floats per sequence slot and
// is carried from step to step; a step brings any number of next tokens for each of its sequences.  Everything
// here is 32-bit.
//
// Work: a block is (16 value columns, head, sequence) and walks the sequence's tokens in order.  A value column
// is owned by 8 lanes, lane p holding the state's rows p, p + 8, ... of that column in registers; the state is
// stored [slot][head][dv][dk], so these 8 lanes read 32 contiguous bytes.  Tokens come through shared memory
// eight at a time.  The order of every sum depends on nothing but dk, so a prompt gives the same numbers
// however it is cut into steps.
#include "common.cuh"

#define DR_COLS 16
#define DR_PART 8
#define DR_CHUNK 8

__device__ __forceinline__ float dr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <int R>
__global__ void __launch_bounds__(DR_COLS * DR_PART)
delta_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                  const float* __restrict__ v, int ldv, const float* __restrict__ b, int ldb,
                  const float* __restrict__ a, int lda, const float* __restrict__ dt_bias,
                  const float* __restrict__ a_log, float q_scale, float norm_eps, float* __restrict__ state,
                  const int* __restrict__ slots, const int* __restrict__ cu, float* __restrict__ o, int n_heads,
                  int kv_heads, int dk, int dv, int head_decay) {
    mv_pdl_begin();
    extern __shared__ float smem[];
    float* qs = smem;                           // [DR_CHUNK][dk]
    float* ks = qs + DR_CHUNK * dk;
    float* gs = ks + DR_CHUNK * dk;
    float* vs = gs + DR_CHUNK * dk;             // [DR_CHUNK][DR_COLS]
    float* bs = vs + DR_CHUNK * DR_COLS;        // [DR_CHUNK]
    float* ns = bs + DR_CHUNK;                  // [DR_CHUNK][2]: what q and k are multiplied by
    const int tile = blockIdx.x, h = blockIdx.y, sq = blockIdx.z;
    const int tid = threadIdx.x, p = tid & (DR_PART - 1), jl = tid >> 3;
    const int j = tile * DR_COLS + jl;
    const int row0 = cu[sq], len = cu[sq + 1] - row0;
    if (len <= 0) return;
    const int hk = h / (n_heads / kv_heads);
    const int slot = mv_read_slot(slots[sq]);
    float* srow = state + (((size_t)slot * n_heads + h) * dv + (j < dv ? j : 0)) * dk;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = p + DR_PART * r;
        S[r] = (j < dv && i < dk) ? srow[i] : 0.f;
    }
    const float rate = expf(a_log[h]);
    for (int c0 = 0; c0 < len; c0 += DR_CHUNK) {
        const int nt = min(DR_CHUNK, len - c0);
        __syncthreads();
        for (int idx = tid; idx < nt * dk; idx += DR_COLS * DR_PART) {
            const int t = idx / dk, i = idx - t * dk;
            const size_t row = (size_t)(row0 + c0 + t);
            qs[idx] = q[row * ldq + (size_t)hk * dk + i];
            ks[idx] = k[row * ldk + (size_t)hk * dk + i];
            // one decay logit a head (head_decay) or one a head and key channel
            const size_t ai = head_decay ? (size_t)h : (size_t)h * dk + i;
            gs[idx] = expf(-rate * dr_softplus(a[row * lda + ai] + dt_bias[ai]));
        }
        for (int idx = tid; idx < nt * DR_COLS; idx += DR_COLS * DR_PART) {
            const int t = idx / DR_COLS, c = idx - t * DR_COLS, col = tile * DR_COLS + c;
            vs[idx] = col < dv ? v[(size_t)(row0 + c0 + t) * ldv + (size_t)h * dv + col] : 0.f;
        }
        if (tid < nt) bs[tid] = 1.0f / (1.0f + expf(-b[(size_t)(row0 + c0 + tid) * ldb + h]));
        __syncthreads();
        {
            // sixteen groups of eight lanes: group (t, which) sums the squares of token t's q or k
            const int t = jl >> 1, which = jl & 1;
            const float* src = (which ? ks : qs) + t * dk;
            float ss = 0.f;
            if (t < nt)
                for (int i = p; i < dk; i += DR_PART) ss = fmaf(src[i], src[i], ss);
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            ss += __shfl_xor_sync(0xffffffffu, ss, 4);
            if (p == 0 && t < nt) ns[2 * t + which] = (which ? 1.f : q_scale) / sqrtf(ss + norm_eps);
        }
        __syncthreads();
        for (int idx = tid; idx < nt * dk; idx += DR_COLS * DR_PART) {
            const int t = idx / dk;
            qs[idx] *= ns[2 * t];
            ks[idx] *= ns[2 * t + 1];
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vj = vs[t * DR_COLS + jl], bt = bs[t];
            const float* qt = qs + t * dk;
            const float* kt = ks + t * dk;
            const float* gt = gs + t * dk;
            float said = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = p + DR_PART * r;
                if (i < dk) {
                    S[r] *= gt[i];
                    said = fmaf(S[r], kt[i], said);
                }
            }
            said += __shfl_xor_sync(0xffffffffu, said, 1);
            said += __shfl_xor_sync(0xffffffffu, said, 2);
            said += __shfl_xor_sync(0xffffffffu, said, 4);
            const float u = bt * (vj - said);
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = p + DR_PART * r;
                if (i < dk) {
                    S[r] = fmaf(kt[i], u, S[r]);
                    acc = fmaf(S[r], qt[i], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (p == 0 && j < dv) o[(size_t)(row0 + c0 + t) * n_heads * dv + (size_t)h * dv + j] = acc;
        }
    }
    if (j < dv && mv_slot_ok(slots[sq])) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = p + DR_PART * r;
            if (i < dk) srow[i] = S[r];
        }
    }
}

MV_GUARD_SETTER(delta_rule)

// q, k [N, >= kv_heads * dk], v [N, >= n_heads * dv], b [N, >= n_heads] (beta's logits), a [N, >= n_heads * dk] (the
// decay's logits) with row strides ldq, ldk, ldv, ldb, lda (elements); dt_bias [n_heads * dk]; a_log [n_heads];
// state [slots][n_heads][dv][dk]; slots [n_seqs]; cu [n_seqs + 1]; o [N, n_heads * dv] dense.
MV_API int mv_delta_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* b, int ldb,
                         const float* a, int lda, const float* dt_bias, const float* a_log, float q_scale, float norm_eps,
                         float* state, const int* slots, const int* cu, float* o, int n_seqs, int n_heads, int kv_heads,
                         int dk, int dv, int head_decay, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || kv_heads < 1 || n_heads % kv_heads) return (int)cudaErrorInvalidValue;
    const dim3 grid((dv + DR_COLS - 1) / DR_COLS, n_heads, n_seqs);
    const size_t smem = (size_t)DR_CHUNK * (3 * dk + DR_COLS + 3) * sizeof(float);
#define DR_LAUNCH(R)                                                                                                   \
    mv_launch(delta_scan_kernel<R>, grid, DR_COLS * DR_PART, smem, stream, q, ldq, k, ldk, v, ldv, b, ldb, a, lda, dt_bias, \
              a_log, q_scale, norm_eps, state, slots, cu, o, n_heads, kv_heads, dk, dv, head_decay)
    if (dk <= 32) DR_LAUNCH(4);
    else if (dk <= 64) DR_LAUNCH(8);
    else if (dk <= 128) DR_LAUNCH(16);
    else DR_LAUNCH(32);
#undef DR_LAUNCH
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------- steps of many tokens
// Two kernels.  delta_prepare does, once per token, what does not depend on the state: q and k as unit vectors
// (q also times q_scale), k . q of each q/k head, the decays g, and beta; one row of `prep` a token:
//     [q: kv_heads dk | k: kv_heads dk | g: heads dk | beta: heads | k.q: kv_heads]      (row stride ldp, 32-bit)
// delta_scan_long then walks a sequence with nothing but the recurrence in its loop.  The tokens come through
// shared memory sixteen at a time, the next sixteen on their way (cp.async) while these are worked on.  In the
// loop  S' = diag(g) S  is read twice at once, a = S'^T k and b = S'^T q, so that one round of shuffles serves
// both; u = beta (v - a); o = b + u (k . q), which is (S' + k u^T)^T q; S = S' + k u^T.
#define DL_CHUNK 16

__global__ void __launch_bounds__(256)
delta_prepare_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                     const float* __restrict__ b, int ldb, const float* __restrict__ a, int lda,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log, float q_scale, float norm_eps,
                     float* __restrict__ prep, int ldp, int n_heads, int kv_heads, int dk, int head_decay) {
    mv_pdl_begin();
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* row = prep + (size_t)n * ldp;
    const int qk = kv_heads * dk, hk = n_heads * dk;
    for (int h = warp; h < kv_heads; h += nwarps) {
        const float* qh = q + (size_t)n * ldq + (size_t)h * dk;
        const float* kh = k + (size_t)n * ldk + (size_t)h * dk;
        float sq = 0.f, sk = 0.f, dot = 0.f;
        for (int i = lane; i < dk; i += 32) {
            const float x = qh[i], y = kh[i];
            sq = fmaf(x, x, sq);
            sk = fmaf(y, y, sk);
            dot = fmaf(x, y, dot);
        }
        sq = mv_warp_sum(sq);
        sk = mv_warp_sum(sk);
        dot = mv_warp_sum(dot);
        const float fq = q_scale / sqrtf(sq + norm_eps), fk = 1.0f / sqrtf(sk + norm_eps);
        for (int i = lane; i < dk; i += 32) {
            row[(size_t)h * dk + i] = qh[i] * fq;
            row[qk + (size_t)h * dk + i] = kh[i] * fk;
        }
        if (lane == 0) row[2 * qk + hk + n_heads + h] = dot * fq * fk;
    }
    for (int e = threadIdx.x; e < hk; e += blockDim.x) {
        const int h = e / dk;
        const int ai = head_decay ? h : e;
        row[2 * qk + e] = expf(-expf(a_log[h]) * dr_softplus(a[(size_t)n * lda + ai] + dt_bias[ai]));
    }
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x)
        row[2 * qk + hk + h] = 1.0f / (1.0f + expf(-b[(size_t)n * ldb + h]));
}

__device__ __forceinline__ void dl_copy4(float* smem, const float* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void dl_copy16(float* smem, const float* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void dl_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void dl_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The rows of q, k and g, DR_COLS columns of v, beta and k.q of up to DL_CHUNK tokens from token c0 of a sequence on
// their way into one buffer of shared memory.
__device__ __forceinline__ void dl_stage(float* buf, const float* __restrict__ prep, int ldp, const float* __restrict__ v,
                                         int ldv, int row0, int c0, int len, int h, int hk, int qk, int n_heads, int dk,
                                         int dv, int col0, int wide, int tid, int nthreads) {
        const int nt = min(DL_CHUNK, len - c0);
        float* qs = buf;
        float* ks = qs + DL_CHUNK * dk;
        float* gs = ks + DL_CHUNK * dk;
        float* vs = gs + DL_CHUNK * dk;
        float* bs = vs + DL_CHUNK * DR_COLS;
        float* ds = bs + DL_CHUNK;
        if (wide) {
            const int dk4 = dk >> 2;
            for (int idx = tid; idx < nt * dk4; idx += nthreads) {
                const int t = idx / dk4, i = (idx - t * dk4) << 2;
                const float* src = prep + (size_t)(row0 + c0 + t) * ldp;
                dl_copy16(qs + t * dk + i, src + (size_t)hk * dk + i);
                dl_copy16(ks + t * dk + i, src + qk + (size_t)hk * dk + i);
                dl_copy16(gs + t * dk + i, src + 2 * qk + (size_t)h * dk + i);
            }
        } else {
            for (int idx = tid; idx < nt * dk; idx += nthreads) {
                const int t = idx / dk, i = idx - t * dk;
                const float* src = prep + (size_t)(row0 + c0 + t) * ldp;
                dl_copy4(qs + idx, src + (size_t)hk * dk + i);
                dl_copy4(ks + idx, src + qk + (size_t)hk * dk + i);
                dl_copy4(gs + idx, src + 2 * qk + (size_t)h * dk + i);
            }
        }
        for (int idx = tid; idx < nt * DR_COLS; idx += nthreads) {
            const int t = idx / DR_COLS, c = idx - t * DR_COLS;
            if (col0 + c < dv) dl_copy4(vs + idx, v + (size_t)(row0 + c0 + t) * ldv + (size_t)h * dv + col0 + c);
        }
        if (tid < nt) {
            const float* src = prep + (size_t)(row0 + c0 + tid) * ldp + 2 * qk + (size_t)n_heads * dk;
            dl_copy4(bs + tid, src + h);
            dl_copy4(ds + tid, src + n_heads + hk);
        }
    }

// One buffer of shared memory: [q: CHUNK dk | k: CHUNK dk | g: CHUNK dk | v: CHUNK DR_COLS | beta: CHUNK | k.q: CHUNK]
// PART lanes share a column of the state (element i of it with lane i % PART).  Keys under 64 channels run here with 8
// lanes a column; from 64 channels on delta_scan_warp_kernel below takes over.  (A whole warp a column, 16 warps a
// block, was measured issue-bound: 740 us for 2,048 tokens of 128 x 128 against 696 for the kernel below.)
template <int R, int PART>
__global__ void __launch_bounds__(DR_COLS * PART)
delta_scan_long_kernel(const float* __restrict__ prep, int ldp, const float* __restrict__ v, int ldv,
                       float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu,
                       float* __restrict__ o, int n_heads, int kv_heads, int dk, int dv, int wide) {
    mv_pdl_wait();                          // the successor is let go when the last token is done
    extern __shared__ __align__(16) float dl_smem[];
    const int per = DL_CHUNK * (3 * dk + DR_COLS + 2);
    const int tile = blockIdx.x, h = blockIdx.y, sq = blockIdx.z;
    const int tid = threadIdx.x, p = tid & (PART - 1), jl = tid / PART;
    const int j = tile * DR_COLS + jl;
    const int row0 = cu[sq], len = cu[sq + 1] - row0;
    if (len <= 0) return;
    const int hk = h / (n_heads / kv_heads);
    const int qk = kv_heads * dk;
    const int slot = mv_read_slot(slots[sq]);
    float* srow = state + (((size_t)slot * n_heads + h) * dv + (j < dv ? j : 0)) * dk;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = p + PART * r;
        S[r] = (j < dv && i < dk) ? srow[i] : 0.f;
    }
    const int col0 = tile * DR_COLS;

    auto stage = [&](int c0, float* buf) {
        dl_stage(buf, prep, ldp, v, ldv, row0, c0, len, h, hk, qk, n_heads, dk, dv, col0, wide, tid, DR_COLS * PART);
    };

    stage(0, dl_smem);
    dl_commit();
    int which = 0;
    for (int c0 = 0; c0 < len; c0 += DL_CHUNK, which ^= 1) {
        float* buf = dl_smem + which * per;
        if (c0 + DL_CHUNK < len) {
            stage(c0 + DL_CHUNK, dl_smem + (which ^ 1) * per);
            dl_commit();
            dl_wait<1>();
        } else {
            dl_wait<0>();
        }
        __syncthreads();
        const int nt = min(DL_CHUNK, len - c0);
        const float* qs = buf;
        const float* ks = qs + DL_CHUNK * dk;
        const float* gs = ks + DL_CHUNK * dk;
        const float* vs = gs + DL_CHUNK * dk;
        const float* bs = vs + DL_CHUNK * DR_COLS;
        const float* ds = bs + DL_CHUNK;
        for (int t = 0; t < nt; ++t) {
            const float* qt = qs + t * dk;
            const float* kt = ks + t * dk;
            const float* gt = gs + t * dk;
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int r = 0; r < R; r += 2) {
                const int i0 = p + PART * r, i1 = i0 + PART;
                if (i0 < dk) {
                    S[r] *= gt[i0];
                    a0 = fmaf(S[r], kt[i0], a0);
                    b0 = fmaf(S[r], qt[i0], b0);
                }
                if (r + 1 < R && i1 < dk) {
                    S[r + 1] *= gt[i1];
                    a1 = fmaf(S[r + 1], kt[i1], a1);
                    b1 = fmaf(S[r + 1], qt[i1], b1);
                }
            }
            float said = a0 + a1, read = b0 + b1;
#pragma unroll
            for (int d = 1; d < PART; d <<= 1) {
                said += __shfl_xor_sync(0xffffffffu, said, d);
                read += __shfl_xor_sync(0xffffffffu, read, d);
            }
            const float u = bs[t] * ((j < dv ? vs[t * DR_COLS + jl] : 0.f) - said);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = p + PART * r;
                if (i < dk) S[r] = fmaf(kt[i], u, S[r]);
            }
            if (p == 0 && j < dv) o[(size_t)(row0 + c0 + t) * n_heads * dv + (size_t)h * dv + j] = fmaf(u, ds[t], read);
        }
        __syncthreads();
    }
    mv_pdl_launch_dependents();
    if (j < dv && mv_slot_ok(slots[sq])) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = p + PART * r;
            if (i < dk) srow[i] = S[r];
        }
    }
}

// From 64 key channels on: a warp carries TWO columns of the state, lane l the channels l, l + 32, ...  A token's q, k and
// g are read once for both columns, and the four sums of a token (what the state says for k and what it reads out
// for q, in each column) are folded while they are added up: lanes exchange the half they do not keep, so 4 + 2 + 1
// values go round instead of 4 x 5, and lanes 0, 8, 16 and 24 end up with one whole sum each.
template <int R>
__global__ void __launch_bounds__(DR_COLS * 16)
delta_scan_warp_kernel(const float* __restrict__ prep, int ldp, const float* __restrict__ v, int ldv,
                       float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu,
                       float* __restrict__ o, int n_heads, int kv_heads, int dk, int dv, int wide) {
    mv_pdl_wait();                          // the successor is let go when the last token is done
    extern __shared__ __align__(16) float dl_smem[];
    const int per = DL_CHUNK * (3 * dk + DR_COLS + 2);
    const int tile = blockIdx.x, h = blockIdx.y, sq = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, jl = (tid >> 5) * 2;
    const int col0 = tile * DR_COLS;
    const int j0 = col0 + jl, j1 = j0 + 1;
    const int row0 = cu[sq], len = cu[sq + 1] - row0;
    if (len <= 0) return;
    const int hk = h / (n_heads / kv_heads);
    const int qk = kv_heads * dk;
    const int slot = mv_read_slot(slots[sq]);
    float* srow0 = state + (((size_t)slot * n_heads + h) * dv + (j0 < dv ? j0 : 0)) * dk;
    float* srow1 = state + (((size_t)slot * n_heads + h) * dv + (j1 < dv ? j1 : 0)) * dk;
    float S0[R], S1[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        S0[r] = (j0 < dv && i < dk) ? srow0[i] : 0.f;
        S1[r] = (j1 < dv && i < dk) ? srow1[i] : 0.f;
    }
    const bool hi16 = lane & 16, hi8 = lane & 8;

    dl_stage(dl_smem, prep, ldp, v, ldv, row0, 0, len, h, hk, qk, n_heads, dk, dv, col0, wide, tid, DR_COLS * 16);
    dl_commit();
    int which = 0;
    for (int c0 = 0; c0 < len; c0 += DL_CHUNK, which ^= 1) {
        float* buf = dl_smem + which * per;
        if (c0 + DL_CHUNK < len) {
            dl_stage(dl_smem + (which ^ 1) * per, prep, ldp, v, ldv, row0, c0 + DL_CHUNK, len, h, hk, qk, n_heads, dk, dv,
                     col0, wide, tid, DR_COLS * 16);
            dl_commit();
            dl_wait<1>();
        } else {
            dl_wait<0>();
        }
        __syncthreads();
        const int nt = min(DL_CHUNK, len - c0);
        const float* qs = buf;
        const float* ks = qs + DL_CHUNK * dk;
        const float* gs = ks + DL_CHUNK * dk;
        const float* vs = gs + DL_CHUNK * dk;
        const float* bs = vs + DL_CHUNK * DR_COLS;
        const float* ds = bs + DL_CHUNK;
        for (int t = 0; t < nt; ++t) {
            const float* qt = qs + t * dk;
            const float* kt = ks + t * dk;
            const float* gt = gs + t * dk;
            float kr[R];
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = lane + 32 * r;
                kr[r] = 0.f;
                if (i < dk) {
                    const float g = gt[i], q = qt[i];
                    kr[r] = kt[i];
                    S0[r] *= g;
                    S1[r] *= g;
                    a0 = fmaf(S0[r], kr[r], a0);
                    a1 = fmaf(S1[r], kr[r], a1);
                    b0 = fmaf(S0[r], q, b0);
                    b1 = fmaf(S1[r], q, b1);
                }
            }
            // lanes 0..15 keep what the state says for k, lanes 16..31 what it reads for q; then lanes with bit 3 clear
            // keep the first column and the others the second
            const float x0 = (hi16 ? b0 : a0) + __shfl_xor_sync(0xffffffffu, hi16 ? a0 : b0, 16);
            const float x1 = (hi16 ? b1 : a1) + __shfl_xor_sync(0xffffffffu, hi16 ? a1 : b1, 16);
            float y = (hi8 ? x1 : x0) + __shfl_xor_sync(0xffffffffu, hi8 ? x0 : x1, 8);
            y += __shfl_xor_sync(0xffffffffu, y, 4);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            const float said0 = __shfl_sync(0xffffffffu, y, 0), said1 = __shfl_sync(0xffffffffu, y, 8);
            const float beta = bs[t];
            const float u0 = beta * ((j0 < dv ? vs[t * DR_COLS + jl] : 0.f) - said0);
            const float u1 = beta * ((j1 < dv ? vs[t * DR_COLS + jl + 1] : 0.f) - said1);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                S0[r] = fmaf(kr[r], u0, S0[r]);
                S1[r] = fmaf(kr[r], u1, S1[r]);
            }
            float* orow = o + (size_t)(row0 + c0 + t) * n_heads * dv + (size_t)h * dv;
            if (lane == 16 && j0 < dv) orow[j0] = fmaf(u0, ds[t], y);
            if (lane == 24 && j1 < dv) orow[j1] = fmaf(u1, ds[t], y);
        }
        __syncthreads();
    }
    mv_pdl_launch_dependents();
    if (mv_slot_ok(slots[sq])) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = lane + 32 * r;
            if (i < dk) {
                if (j0 < dv) srow0[i] = S0[r];
                if (j1 < dv) srow1[i] = S1[r];
            }
        }
    }
}

// Row width of `prep` for these sizes (a multiple of 4 floats, so that rows start on 16 bytes).
static inline int mv_delta_prep_width(int n_heads, int kv_heads, int dk) {
    const int w = 2 * kv_heads * dk + n_heads * dk + n_heads + kv_heads;
    return (w + 3) & ~3;
}

// As mv_delta_scan, for steps of many tokens a sequence; prep [N, mv_delta_prep_width()] is scratch.
MV_API int mv_delta_scan_long(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* b,
                              int ldb, const float* a, int lda, const float* dt_bias, const float* a_log, float q_scale,
                              float norm_eps, float* prep, float* state, const int* slots, const int* cu, float* o, int N,
                              int n_seqs, int n_heads, int kv_heads, int dk, int dv, int head_decay, cudaStream_t stream) {
    if (n_seqs <= 0 || N <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || kv_heads < 1 || n_heads % kv_heads) return (int)cudaErrorInvalidValue;
    const int ldp = mv_delta_prep_width(n_heads, kv_heads, dk);
    mv_launch(delta_prepare_kernel, N, 256, 0, stream, q, ldq, k, ldk, b, ldb, a, lda, dt_bias, a_log, q_scale, norm_eps, prep,
              ldp, n_heads, kv_heads, dk, head_decay);
    // The walk is launched as an ordinary successor, not a programmatic one.  Started while the preparing kernel's blocks
    // still hold the multiprocessors, its few blocks (one sequence of 16 heads x 128 values: 128) went where room came
    // up first, several to a multiprocessor, and the walk, bound by what ONE multiprocessor issues, took 1.75 times as
    // long as when they are dealt out over an idle device (measured: 1.26 ms against 0.72 for 2,048 tokens).
    const dim3 grid((dv + DR_COLS - 1) / DR_COLS, n_heads, n_seqs);
    const size_t smem = 2 * (size_t)DL_CHUNK * (3 * dk + DR_COLS + 2) * sizeof(float);
    // 16-byte copies: every row of q, k and g of a head starts on 16 bytes (ldp is a multiple of 4 floats)
    const int wide = dk % 4 == 0 && (((uintptr_t)prep) & 15) == 0;
#define DL_LAUNCH(R, PART)                                                                                                   \
    do {                                                                                                                 \
        if (smem > 48 * 1024) {                                                                                          \
            const cudaError_t e = cudaFuncSetAttribute(delta_scan_long_kernel<R, PART>,                                  \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (e != cudaSuccess) return (int)e;                                                                         \
        }                                                                                                                \
        delta_scan_long_kernel<R, PART><<<grid, DR_COLS * PART, smem, stream>>>((const float*)prep, ldp, v, ldv, state,  \
                                                                                slots, cu, o, n_heads, kv_heads, dk, dv, \
                                                                                wide);                                   \
    } while (0)
#define DW_LAUNCH(R)                                                                                                     \
    do {                                                                                                                 \
        if (smem > 48 * 1024) {                                                                                          \
            const cudaError_t e = cudaFuncSetAttribute(delta_scan_warp_kernel<R>,                                        \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (e != cudaSuccess) return (int)e;                                                                         \
        }                                                                                                                \
        delta_scan_warp_kernel<R><<<grid, DR_COLS * 16, smem, stream>>>((const float*)prep, ldp, v, ldv, state, slots,  \
                                                                        cu, o, n_heads, kv_heads, dk, dv, wide);         \
    } while (0)
    if (dk <= 32) DL_LAUNCH(4, 8);
    else if (dk < 64) DL_LAUNCH(8, 8);
    else if (dk == 64) DW_LAUNCH(2);
    else if (dk <= 128) DW_LAUNCH(4);
    else DW_LAUNCH(8);
#undef DW_LAUNCH
#undef DL_LAUNCH
    return mv_launch_status();
}
