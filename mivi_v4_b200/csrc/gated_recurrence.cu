// A linear recurrence per channel with gates that depend on the input (the real-gated linear recurrent unit
// of De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models"):
//
//     r_t = sigmoid(A_b u_t,b + a_b),  i_t = sigmoid(B_b u_t,b + b_b)      (u cut into equal parts b; A_b, B_b square)
//     log a_t = -c r_t softplus(lambda),  a_t = exp(log a_t)
//     S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t                           (per channel, S = 0 before a sequence)
//     out_t = S_t * gelu_tanh(y_t)                                          (y: the block's other branch)
//
// The state S lives in 32-bit floats per sequence slot and is carried from step to step; a step brings any
// number of next tokens for each of its sequences.  Everything here is 32-bit; only `out` is in the model's
// dtype.  Two kernels: the gates (a small dense product per part, then the scalar functions), and the walk
// along the sequence.
#include "common.cuh"

#define GR_TOK 16            // tokens a block of the gate kernel holds
#define GR_THREADS 1024      // channels a block x the most pieces a long sequence is cut into for the walk

__device__ __forceinline__ float gr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// u [N, C] dense; wa_t, wi_t [nb][bs (in)][bs (out)]: the parts' matrices transposed, so that the threads of a
// block read consecutive outputs; ba, bi, lam [C].  a_out, x_out [N, C]: the decay and the gated input
// sqrt(1 - a^2) i u.  A block is (16 tokens, 128 outputs of one part): the tokens' inputs of that part lie in
// shared memory as [in][token], a thread keeps one output of all 16 tokens in registers.
__global__ void __launch_bounds__(128)
block_gates_kernel(const float* __restrict__ u, const float* __restrict__ wa_t, const float* __restrict__ wi_t,
                   const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ lam, float c,
                   float* __restrict__ a_out, float* __restrict__ x_out, int N, int C, int bs) {
    mv_pdl_begin();
    extern __shared__ __align__(16) float gr_us[];           // [bs][GR_TOK]
    const int n0 = blockIdx.x * GR_TOK, b = blockIdx.y;
    const int o = blockIdx.z * blockDim.x + threadIdx.x;
    const int nt = min(GR_TOK, N - n0);
    for (int idx = threadIdx.x; idx < bs * GR_TOK; idx += blockDim.x) {
        const int t = idx / bs, in = idx - t * bs;           // consecutive threads read consecutive inputs
        gr_us[in * GR_TOK + t] = t < nt ? u[(size_t)(n0 + t) * C + (size_t)b * bs + in] : 0.f;
    }
    __syncthreads();
    if (o >= bs) return;
    float ar[GR_TOK], ai[GR_TOK];
#pragma unroll
    for (int t = 0; t < GR_TOK; ++t) ar[t] = ai[t] = 0.f;
    const float* wa = wa_t + (size_t)b * bs * bs + o;
    const float* wi = wi_t + (size_t)b * bs * bs + o;
#pragma unroll 8
    for (int in = 0; in < bs; ++in) {
        const float x = wa[(size_t)in * bs], y = wi[(size_t)in * bs];
        const float4* row = reinterpret_cast<const float4*>(gr_us + in * GR_TOK);
#pragma unroll
        for (int q = 0; q < GR_TOK / 4; ++q) {
            const float4 v = row[q];
            ar[4 * q] = fmaf(x, v.x, ar[4 * q]);         ai[4 * q] = fmaf(y, v.x, ai[4 * q]);
            ar[4 * q + 1] = fmaf(x, v.y, ar[4 * q + 1]); ai[4 * q + 1] = fmaf(y, v.y, ai[4 * q + 1]);
            ar[4 * q + 2] = fmaf(x, v.z, ar[4 * q + 2]); ai[4 * q + 2] = fmaf(y, v.z, ai[4 * q + 2]);
            ar[4 * q + 3] = fmaf(x, v.w, ar[4 * q + 3]); ai[4 * q + 3] = fmaf(y, v.w, ai[4 * q + 3]);
        }
    }
    const int ch = b * bs + o;
    const float rate = c * gr_softplus(lam[ch]), bra = ba[ch], bri = bi[ch];
#pragma unroll
    for (int t = 0; t < GR_TOK; ++t) {
        if (t < nt) {
            const float r = 1.0f / (1.0f + expf(-(ar[t] + bra)));
            const float ig = 1.0f / (1.0f + expf(-(ai[t] + bri)));
            const float log_a = -rate * r;
            const size_t at = (size_t)(n0 + t) * C + ch;
            a_out[at] = expf(log_a);
            // 1 - a^2 = -expm1(2 log a): exact also where a is close to 1
            x_out[at] = sqrtf(-expm1f(2.0f * log_a)) * ig * gr_us[o * GR_TOK + t];
        }
    }
}

// The same for steps of few tokens, where the matrices' bytes are the work: a block is (16 tokens, 32 outputs of one
// part) and its 8 warps share the part's inputs among them, lane l keeping output l of all 16 tokens for its warp's
// inputs; the 8 partial sums meet in shared memory and are added in the warps' order.
#define GR_SPLIT 8
__global__ void __launch_bounds__(32 * GR_SPLIT)
block_gates_few_kernel(const float* __restrict__ u, const float* __restrict__ wa_t, const float* __restrict__ wi_t,
                       const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ lam, float c,
                       float* __restrict__ a_out, float* __restrict__ x_out, int N, int C, int bs) {
    mv_pdl_begin();
    extern __shared__ __align__(16) float gr_us[];           // [bs][GR_TOK], then [GR_SPLIT][2][GR_TOK][32]
    float* part = gr_us + (size_t)bs * GR_TOK;
    const int n0 = blockIdx.x * GR_TOK, b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int o = blockIdx.z * 32 + lane;
    const int nt = min(GR_TOK, N - n0);
    for (int idx = threadIdx.x; idx < bs * GR_TOK; idx += blockDim.x) {
        const int t = idx / bs, in = idx - t * bs;
        gr_us[in * GR_TOK + t] = t < nt ? u[(size_t)(n0 + t) * C + (size_t)b * bs + in] : 0.f;
    }
    __syncthreads();
    float ar[GR_TOK], ai[GR_TOK];
#pragma unroll
    for (int t = 0; t < GR_TOK; ++t) ar[t] = ai[t] = 0.f;
    const int per = (bs + GR_SPLIT - 1) / GR_SPLIT;
    const int in0 = warp * per, in1 = min(in0 + per, bs);
    if (o < bs) {
        const float* wa = wa_t + (size_t)b * bs * bs + o;
        const float* wi = wi_t + (size_t)b * bs * bs + o;
#pragma unroll 8
        for (int in = in0; in < in1; ++in) {
            const float x = wa[(size_t)in * bs], y = wi[(size_t)in * bs];
            const float4* row = reinterpret_cast<const float4*>(gr_us + in * GR_TOK);
#pragma unroll
            for (int q = 0; q < GR_TOK / 4; ++q) {
                const float4 v = row[q];
                ar[4 * q] = fmaf(x, v.x, ar[4 * q]);         ai[4 * q] = fmaf(y, v.x, ai[4 * q]);
                ar[4 * q + 1] = fmaf(x, v.y, ar[4 * q + 1]); ai[4 * q + 1] = fmaf(y, v.y, ai[4 * q + 1]);
                ar[4 * q + 2] = fmaf(x, v.z, ar[4 * q + 2]); ai[4 * q + 2] = fmaf(y, v.z, ai[4 * q + 2]);
                ar[4 * q + 3] = fmaf(x, v.w, ar[4 * q + 3]); ai[4 * q + 3] = fmaf(y, v.w, ai[4 * q + 3]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < GR_TOK; ++t) {
        part[((warp * 2 + 0) * GR_TOK + t) * 32 + lane] = ar[t];
        part[((warp * 2 + 1) * GR_TOK + t) * 32 + lane] = ai[t];
    }
    __syncthreads();
    // a thread a (token, output): 16 x 32 pairs over 256 threads
    for (int idx = threadIdx.x; idx < GR_TOK * 32; idx += blockDim.x) {
        const int t = idx >> 5, l = idx & 31, oo = blockIdx.z * 32 + l;
        if (t >= nt || oo >= bs) continue;
        float sr = 0.f, si = 0.f;
#pragma unroll
        for (int w = 0; w < GR_SPLIT; ++w) {
            sr += part[((w * 2 + 0) * GR_TOK + t) * 32 + l];
            si += part[((w * 2 + 1) * GR_TOK + t) * 32 + l];
        }
        const int ch = b * bs + oo;
        const float r = 1.0f / (1.0f + expf(-(sr + ba[ch])));
        const float ig = 1.0f / (1.0f + expf(-(si + bi[ch])));
        const float log_a = -c * gr_softplus(lam[ch]) * r;
        const size_t at = (size_t)(n0 + t) * C + ch;
        a_out[at] = expf(log_a);
        x_out[at] = sqrtf(-expm1f(2.0f * log_a)) * ig * gr_us[oo * GR_TOK + t];
    }
}

MV_API int mv_block_gates(const float* u, const float* wa_t, const float* wi_t, const float* ba, const float* bi,
                          const float* lam, float c, float* a_out, float* x_out, int N, int C, int n_blocks,
                          cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_blocks < 1 || C % n_blocks) return (int)cudaErrorInvalidValue;
    const int bs = C / n_blocks;
    const size_t smem = (size_t)bs * GR_TOK * sizeof(float);
    if (smem > 160 * 1024) return (int)cudaErrorInvalidValue;
    if (N <= 256) {
        // few tokens: more and smaller blocks, the inputs of a part shared among a block's warps
        const size_t smem_few = smem + (size_t)GR_SPLIT * 2 * GR_TOK * 32 * sizeof(float);
        if (smem_few > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(block_gates_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                       (int)smem_few);
            if (e != cudaSuccess) return (int)e;
        }
        const dim3 grid_few((N + GR_TOK - 1) / GR_TOK, n_blocks, (bs + 31) / 32);
        mv_launch(block_gates_few_kernel, grid_few, 32 * GR_SPLIT, smem_few, stream, u, wa_t, wi_t, ba, bi, lam, c, a_out,
                  x_out, N, C, bs);
        return mv_launch_status();
    }
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(block_gates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = bs >= 128 ? 128 : ((bs + 31) / 32) * 32;
    const dim3 grid((N + GR_TOK - 1) / GR_TOK, n_blocks, (bs + threads - 1) / threads);
    mv_launch(block_gates_kernel, grid, threads, smem, stream, u, wa_t, wi_t, ba, bi, lam, c, a_out, x_out, N, C, bs);
    return mv_launch_status();
}

__device__ __forceinline__ float gr_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// a, x [N, C] dense; y [N, C] with row stride ldy (the other branch before its activation); state [slots][C];
// out [N, C] in the model's dtype.  A block is (blockDim.x channels, a sequence): 32, or 16 where that is what gives
// every multiprocessor a block; its blockDim.y rows of threads each walk one piece of
// the sequence's tokens: first from a zero state, keeping the product of the piece's decays, then, once every
// piece's (product, end state) is known, again from the state that the pieces before leave.  With one row
// (steps of few tokens a sequence) the walk is done once.
template <typename T>
__global__ void __launch_bounds__(GR_THREADS)
gated_recurrence_kernel(const float* __restrict__ a, const float* __restrict__ x, const float* __restrict__ y, int ldy,
                        float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu,
                        T* __restrict__ out, int C) {
    mv_pdl_begin();
    __shared__ float sp[GR_THREADS], ss[GR_THREADS];          // [piece][channel of the block]
    const int CH = blockDim.x;
    const int ch = blockIdx.x * CH + threadIdx.x, sq = blockIdx.y, w = threadIdx.y, W = blockDim.y;
    const int row0 = cu[sq], len = cu[sq + 1] - row0;
    if (len <= 0) return;
    const bool live = ch < C;
    const int per = (len + W - 1) / W;
    const int t0 = min(w * per, len), t1 = min(t0 + per, len);
    const bool slot_ok = mv_slot_ok(slots[sq]);
    float* st = state + (size_t)mv_read_slot(slots[sq]) * C;
    float carry = live ? st[ch] : 0.f;          // read before the barrier: the warp of the last piece writes it at its end
    if (W > 1) {
        float P = 1.f, S = 0.f;
        if (live)
#pragma unroll 8
            for (int t = t0; t < t1; ++t) {
                const size_t at = (size_t)(row0 + t) * C + ch;
                const float d = a[at];
                S = fmaf(d, S, x[at]);
                P *= d;
            }
        sp[w * CH + threadIdx.x] = P;
        ss[w * CH + threadIdx.x] = S;
        __syncthreads();
        if (live)
            for (int v = 0; v < w; ++v) carry = fmaf(sp[v * CH + threadIdx.x], carry, ss[v * CH + threadIdx.x]);
    }
    if (!live) return;
    float S = carry;
#pragma unroll 8
    for (int t = t0; t < t1; ++t) {
        const size_t row = (size_t)(row0 + t);
        S = fmaf(a[row * C + ch], S, x[row * C + ch]);
        out[row * C + ch] = mv_from_f32<T>(S * gr_gelu_tanh(y[row * ldy + ch]));
    }
    if (t1 == len && t1 > t0 && slot_ok) st[ch] = S;
}

MV_GUARD_SETTER(gated_recurrence)

MV_API int mv_gated_recurrence(const float* a, const float* x, const float* y, int ldy, float* state, const int* slots,
                               const int* cu, void* out, int dtype, int n_seqs, int C, int max_len, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (C < 1) return (int)cudaErrorInvalidValue;
    // pieces of 16 tokens at least; 32 channels a block and up to 32 pieces, or, where that leaves multiprocessors
    // without a block in a long step, 16 channels and up to 64 pieces
    const int ch = (max_len >= 1024 && (long long)((C + 31) / 32) * n_seqs < 120) ? 16 : 32;
    const dim3 grid((C + ch - 1) / ch, n_seqs), block(ch, max_len >= 64 ? min(GR_THREADS / ch, max_len / 16) : 1);
    if (dtype == MV_DT_BF16)
        mv_launch(gated_recurrence_kernel<__nv_bfloat16>, grid, block, 0, stream, a, x, y, ldy, state, slots, cu,
                  (__nv_bfloat16*)out, C);
    else
        mv_launch(gated_recurrence_kernel<float>, grid, block, 0, stream, a, x, y, ldy, state, slots, cu, (float*)out, C);
    return mv_launch_status();
}
