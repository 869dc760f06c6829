// The gated delta rule with a decay per key channel, one head at a time:
//
//     S  <- diag(g_t) S                        (S: dk x dv; g_t: a factor in (0, 1] per key channel)
//     u_t = beta_t (v_t - S^T k_t)             (what the state does not yet say about v_t)
//     S  <- S + k_t u_t^T
//     o_t = S^T q_t                            (the read-out sees the token's own write)
//
// with q and k made unit vectors per head first (x / sqrt(sum x^2 + norm_eps), q also times q_scale),
// beta_t = sigmoid(b_t) per head, and g = exp(-exp(A_log_h) softplus(a + dt_bias)) per head and key channel.
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
                  int kv_heads, int dk, int dv) {
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
            gs[idx] = expf(-rate * dr_softplus(a[row * lda + (size_t)h * dk + i] + dt_bias[(size_t)h * dk + i]));
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
                         int dk, int dv, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || kv_heads < 1 || n_heads % kv_heads) return (int)cudaErrorInvalidValue;
    const dim3 grid((dv + DR_COLS - 1) / DR_COLS, n_heads, n_seqs);
    const size_t smem = (size_t)DR_CHUNK * (3 * dk + DR_COLS + 3) * sizeof(float);
#define DR_LAUNCH(R)                                                                                                   \
    mv_launch(delta_scan_kernel<R>, grid, DR_COLS * DR_PART, smem, stream, q, ldq, k, ldk, v, ldv, b, ldb, a, lda, dt_bias, \
              a_log, q_scale, norm_eps, state, slots, cu, o, n_heads, kv_heads, dk, dv)
    if (dk <= 32) DR_LAUNCH(4);
    else if (dk <= 64) DR_LAUNCH(8);
    else if (dk <= 128) DR_LAUNCH(16);
    else DR_LAUNCH(32);
#undef DR_LAUNCH
    return mv_launch_status();
}
