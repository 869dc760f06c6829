// What a selective state space layer does to its projection before the recurrence:
//   * a causal convolution along the sequence, one filter of `taps` taps per channel, with a bias, then
//     silu; the last tap is the current token's, and before a sequence's start the input is zero.  The last
//     taps - 1 inputs of a sequence are kept per slot, so a prompt may be cut anywhere;
//   * the step size dt = softplus(raw + bias) per token and head, from which the recurrence's two
//     scalars follow: log a = -e^(A_log) dt and b = dt.
// Input: 32-bit rows of the projection, [.. | conv channels | dt heads] at given column offsets.
// Everything is computed in 32-bit.
#include "common.cuh"

#define SP_MAX_TAPS 16

// conv state [slot][taps - 1][C], oldest first.  One thread a (token, channel).  ACT: silu on the result (else none).
template <bool ACT>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const float* __restrict__ u, int ld, const float* __restrict__ taps,
                        const float* __restrict__ bias, const float* __restrict__ state,
                        const int* __restrict__ seq_of, const int* __restrict__ cu, const int* __restrict__ slots,
                        float* __restrict__ out, long long total, int C, int K) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int n = (int)(idx / C), c = (int)(idx - (long long)n * C);
    const int b = seq_of[n];
    const int li = n - cu[b];                               // place among the step's tokens of its sequence
    const float* st = state + (size_t)mv_read_slot(slots[b]) * (K - 1) * C;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < K; ++j) {
        const int back = K - 1 - j;                          // tap j reads the input `back` tokens ago
        const float x = li >= back ? u[(size_t)(n - back) * ld + c] : st[(size_t)(li + j) * C + c];
        acc = fmaf(taps[(size_t)c * K + j], x, acc);
    }
    out[idx] = ACT ? acc / (1.0f + expf(-acc)) : acc;
}

// The same with four consecutive channels a thread (16-byte loads): C, ld and the pointers allow it.
template <bool ACT>
__global__ void __launch_bounds__(256)
causal_conv_silu_vec_kernel(const float* __restrict__ u, int ld, const float* __restrict__ taps,
                            const float* __restrict__ bias, const float* __restrict__ state,
                            const int* __restrict__ seq_of, const int* __restrict__ cu, const int* __restrict__ slots,
                            float* __restrict__ out, long long total4, int C, int K) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int C4 = C >> 2;
    const int n = (int)(idx / C4), c = (int)(idx - (long long)n * C4) << 2;
    const int b = seq_of[n];
    const int li = n - cu[b];
    const float* st = state + (size_t)mv_read_slot(slots[b]) * (K - 1) * C;
    float4 acc = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float* tp = taps + (size_t)c * K;                  // the four channels' taps: 4 K consecutive values
    if (K == 4) {
        // four taps a channel: a channel's taps are one 16-byte load
        const float4 t0 = *reinterpret_cast<const float4*>(tp), t1 = *reinterpret_cast<const float4*>(tp + 4);
        const float4 t2 = *reinterpret_cast<const float4*>(tp + 8), t3 = *reinterpret_cast<const float4*>(tp + 12);
        const float w0[4] = {t0.x, t0.y, t0.z, t0.w}, w1[4] = {t1.x, t1.y, t1.z, t1.w};
        const float w2[4] = {t2.x, t2.y, t2.z, t2.w}, w3[4] = {t3.x, t3.y, t3.z, t3.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int back = 3 - j;
            const float4 x = li >= back ? *reinterpret_cast<const float4*>(u + (size_t)(n - back) * ld + c)
                                        : *reinterpret_cast<const float4*>(st + (size_t)(li + j) * C + c);
            acc.x = fmaf(w0[j], x.x, acc.x); acc.y = fmaf(w1[j], x.y, acc.y);
            acc.z = fmaf(w2[j], x.z, acc.z); acc.w = fmaf(w3[j], x.w, acc.w);
        }
    } else {
        for (int j = 0; j < K; ++j) {
            const int back = K - 1 - j;
            const float4 x = li >= back ? *reinterpret_cast<const float4*>(u + (size_t)(n - back) * ld + c)
                                        : *reinterpret_cast<const float4*>(st + (size_t)(li + j) * C + c);
            acc.x = fmaf(tp[j], x.x, acc.x); acc.y = fmaf(tp[K + j], x.y, acc.y);
            acc.z = fmaf(tp[2 * K + j], x.z, acc.z); acc.w = fmaf(tp[3 * K + j], x.w, acc.w);
        }
    }
    if (ACT) {
        acc.x = acc.x / (1.0f + expf(-acc.x)); acc.y = acc.y / (1.0f + expf(-acc.y));
        acc.z = acc.z / (1.0f + expf(-acc.z)); acc.w = acc.w / (1.0f + expf(-acc.w));
    }
    *reinterpret_cast<float4*>(out + (size_t)n * C + c) = acc;
}

// After the step the kept inputs are the last taps - 1 of (kept inputs, the step's inputs).  One thread a
// (sequence, channel) reads all it needs before it writes.
__global__ void __launch_bounds__(256)
causal_conv_state_kernel(const float* __restrict__ u, int ld, float* __restrict__ state, const int* __restrict__ cu,
                         const int* __restrict__ slots, int C, int K) {
    mv_pdl_begin();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C || !mv_slot_ok(slots[b])) return;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    float* st = state + (size_t)slots[b] * (K - 1) * C;
    float keep[SP_MAX_TAPS];
    for (int s = 0; s < K - 1; ++s) {
        const int src = s + len;                             // index into (kept inputs, step's inputs)
        keep[s] = src < K - 1 ? st[(size_t)src * C + c] : u[(size_t)(row0 + src - (K - 1)) * ld + c];
    }
    for (int s = 0; s < K - 1; ++s) st[(size_t)s * C + c] = keep[s];
}

__global__ void __launch_bounds__(256)
step_size_kernel(const float* __restrict__ raw, int ld, const float* __restrict__ dt_bias,
                 const float* __restrict__ a_log, float* __restrict__ log_a, float* __restrict__ b_out, long long total,
                 int H) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int n = (int)(idx / H), h = (int)(idx - (long long)n * H);
    const float z = raw[(size_t)n * ld + h] + dt_bias[h];
    const float dt = z > 20.f ? z : log1pf(expf(z));
    b_out[idx] = dt;
    log_a[idx] = -expf(a_log[h]) * dt;
}

// A step of one token a sequence: the convolution's output, the kept inputs' shift and the step size in ONE
// kernel.  A thread is a (sequence, channel): it alone reads and writes that channel's kept inputs, so nothing
// races; the threads after the channels take the heads' step sizes.  Row b of the step is sequence b's token.
__global__ void __launch_bounds__(256)
ssm_decode_prepare_kernel(const float* __restrict__ u, int ld, const float* __restrict__ taps,
                          const float* __restrict__ bias, float* __restrict__ state, const int* __restrict__ slots,
                          float* __restrict__ out, int C, int K, const float* __restrict__ raw, int ld_raw,
                          const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ log_a,
                          float* __restrict__ b_out, int H) {
    mv_pdl_begin();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C + H) return;
    if (c >= C) {
        const int h = c - C;
        const float z = raw[(size_t)b * ld_raw + h] + dt_bias[h];
        const float dt = z > 20.f ? z : log1pf(expf(z));
        b_out[(size_t)b * H + h] = dt;
        log_a[(size_t)b * H + h] = -expf(a_log[h]) * dt;
        return;
    }
    const bool ok = mv_slot_ok(slots[b]);
    float* st = state + (size_t)mv_read_slot(slots[b]) * (K - 1) * C;
    const float x = u[(size_t)b * ld + c];
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < K - 1; ++j) {
        const float kept = st[(size_t)j * C + c];
        acc = fmaf(taps[(size_t)c * K + j], kept, acc);
        if (j > 0 && ok) st[(size_t)(j - 1) * C + c] = kept;
    }
    if (K > 1 && ok) st[(size_t)(K - 2) * C + c] = x;
    acc = fmaf(taps[(size_t)c * K + K - 1], x, acc);
    out[(size_t)b * C + c] = acc / (1.0f + expf(-acc));
}

// The convolution alone for a step of one token a sequence (row b is sequence b's token): output and the kept inputs'
// shift in ONE kernel.  A thread is a (sequence, channel): it alone reads and writes that channel's kept inputs.
template <bool ACT>
__global__ void __launch_bounds__(256)
causal_conv_decode_kernel(const float* __restrict__ u, int ld, const float* __restrict__ taps,
                          const float* __restrict__ bias, float* __restrict__ state, const int* __restrict__ slots,
                          float* __restrict__ out, int C, int K) {
    mv_pdl_begin();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float x = u[(size_t)b * ld + c];
    float acc = bias ? bias[c] : 0.f;
    if (K > 1) {
        const bool ok = mv_slot_ok(slots[b]);
        float* st = state + (size_t)mv_read_slot(slots[b]) * (K - 1) * C;
        for (int j = 0; j < K - 1; ++j) {
            const float kept = st[(size_t)j * C + c];
            acc = fmaf(taps[(size_t)c * K + j], kept, acc);
            if (j > 0 && ok) st[(size_t)(j - 1) * C + c] = kept;
        }
        if (ok) st[(size_t)(K - 2) * C + c] = x;
    }
    acc = fmaf(taps[(size_t)c * K + K - 1], x, acc);
    out[(size_t)b * C + c] = ACT ? acc / (1.0f + expf(-acc)) : acc;
}

MV_GUARD_SETTER(state_space)

// One token a sequence (row b belongs to slots[b]): mv_causal_conv_silu and mv_step_size together.
MV_API int mv_ssm_decode_prepare(const float* u, int ld, const float* taps, const float* bias, float* state,
                                 const int* slots, float* out, int n_seqs, int C, int K, const float* raw, int ld_raw,
                                 const float* dt_bias, const float* a_log, float* log_a, float* b_out, int H,
                                 cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (K < 1 || K > SP_MAX_TAPS || C < 1 || H < 1) return (int)cudaErrorInvalidValue;
    mv_launch(ssm_decode_prepare_kernel, dim3((C + H + 255) / 256, n_seqs), 256, 0, stream, u, ld, taps, bias, state, slots,
              out, C, K, raw, ld_raw, dt_bias, a_log, log_a, b_out, H);
    return mv_launch_status();
}

// u: the convolution's input columns [N, C] with row stride ld; taps [C, K]; bias [C] or null; state
// [slots][K - 1][C]; out [N, C] dense; act: 1 silu on the result, 0 none.  Two kernels: the outputs (which read
// the kept inputs), then the kept inputs' update.  one_each: the caller says that every sequence brings one token and
// that row b is sequence b's (a decode step); both then happen in one kernel.
MV_API int mv_causal_conv(const float* u, int ld, const float* taps, const float* bias, float* state,
                          const int* seq_of, const int* cu, const int* slots, float* out, int N, int n_seqs,
                          int C, int K, int act, int one_each, cudaStream_t stream) {
    if (N <= 0 || n_seqs <= 0) return 0;
    if (K < 1 || K > SP_MAX_TAPS || C < 1) return (int)cudaErrorInvalidValue;
    if (one_each && N == n_seqs) {
        // one token a sequence, row b sequence b's: one kernel
        if (act)
            mv_launch(causal_conv_decode_kernel<true>, dim3((C + 255) / 256, n_seqs), 256, 0, stream, u, ld, taps, bias, state,
                      slots, out, C, K);
        else
            mv_launch(causal_conv_decode_kernel<false>, dim3((C + 255) / 256, n_seqs), 256, 0, stream, u, ld, taps, bias, state,
                      slots, out, C, K);
        return mv_launch_status();
    }
    const long long total = (long long)N * C;
    const bool wide = C % 4 == 0 && ld % 4 == 0 && N >= 64 &&
                      (((uintptr_t)u | (uintptr_t)bias | (uintptr_t)state | (uintptr_t)out | (uintptr_t)taps) & 15) == 0;
#define SP_CONV(KERNEL, COUNT)                                                                                      \
    do {                                                                                                            \
        if (act)                                                                                                    \
            mv_launch(KERNEL<true>, (unsigned)(((COUNT) + 255) / 256), 256, 0, stream, u, ld, taps, bias,           \
                      (const float*)state, seq_of, cu, slots, out, (COUNT), C, K);                                  \
        else                                                                                                        \
            mv_launch(KERNEL<false>, (unsigned)(((COUNT) + 255) / 256), 256, 0, stream, u, ld, taps, bias,          \
                      (const float*)state, seq_of, cu, slots, out, (COUNT), C, K);                                  \
    } while (0)
    if (wide) SP_CONV(causal_conv_silu_vec_kernel, total / 4);
    else SP_CONV(causal_conv_silu_kernel, total);
#undef SP_CONV
    if (K > 1)
        mv_launch(causal_conv_state_kernel, dim3((C + 255) / 256, n_seqs), 256, 0, stream, u, ld, state, cu, slots, C, K);
    return mv_launch_status();
}

// The same with silu, under the name it had first.
MV_API int mv_causal_conv_silu(const float* u, int ld, const float* taps, const float* bias, float* state,
                               const int* seq_of, const int* cu, const int* slots, float* out, int N, int n_seqs,
                               int C, int K, cudaStream_t stream) {
    return mv_causal_conv(u, ld, taps, bias, state, seq_of, cu, slots, out, N, n_seqs, C, K, 1, 0, stream);
}

// raw [N, H] with row stride ld; dt_bias, a_log [H]; log_a, b_out [N, H] dense.
MV_API int mv_step_size(const float* raw, int ld, const float* dt_bias, const float* a_log, float* log_a,
                        float* b_out, int N, int H, cudaStream_t stream) {
    if (N <= 0) return 0;
    const long long total = (long long)N * H;
    mv_launch(step_size_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, raw, ld, dt_bias, a_log, log_a, b_out,
              total, H);
    return mv_launch_status();
}
