// Row-wise pieces that sit between matrix products: a layer norm (with or without a bias), a root-mean-square
// norm over groups of a row followed by a gate, a root-mean-square norm whose result is added to
// the residual stream, a clamped gated activation, a gate by a per-token table row, and the
// rounding of 32-bit rows to the model's dtype.  Statistics and activations are 32-bit whatever
// the output type.
#include "common.cuh"

// ---------------------------------------------------------------- layer norm
// y[i, :] = (x[r, :] - mean) / sqrt(mean((x - mean)^2) + eps) * w (+ b), r = rows ? rows[i] : i.  Two passes
// over the row for the statistics (the variance is the mean of the squared deviations).
template <typename TO>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                 TO* __restrict__ y, const int* __restrict__ rows, int H, float eps) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float* xr = x + (size_t)r * H;
    float s = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) s += xr[h];
    const float mean = mv_block_sum(s, scratch) / (float)H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float d = xr[h] - mean;
        ss = fmaf(d, d, ss);
    }
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)H + eps);
    TO* yr = y + (size_t)i * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        yr[h] = mv_from_f32<TO>(fmaf((xr[h] - mean) * scale, w[h], b ? b[h] : 0.f));
}

// b: the bias [H], or null for none
MV_API int mv_layernorm(const float* x, const float* w, const float* b, void* y, int y_dtype, const int* rows, int n_rows,
                        int H, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (y_dtype == MV_DT_BF16)
        mv_launch(layernorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, x, w, b, (__nv_bfloat16*)y, rows, H, eps);
    else
        mv_launch(layernorm_kernel<float>, n_rows, threads, 0, stream, x, w, b, (float*)y, rows, H, eps);
    return mv_launch_status();
}

// ------------------------------------------------- grouped rms norm with a gate
// A row of C values is cut into groups of ``group``; each group is divided by its root mean
// square (eps inside the root), multiplied by w[c mod w_len] and by act(gate[n, c]) with act =
// silu (0) or sigmoid (1).  One warp per (row, group).  The gate has its own row stride.
// act = 2: the gate comes BEFORE the norm: the values x * silu(gate) are divided by THEIR root mean
// square and multiplied by w.
__device__ __forceinline__ float gn_gated_first(float x, float g) { return x * (g / (1.0f + expf(-g))); }
template <typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gate, int ld_gate,
                     const float* __restrict__ w, int w_len, TO* __restrict__ y, long long n_groups, int C, int group,
                     float eps, int act) {
    mv_pdl_begin();
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (wid >= n_groups) return;
    const int per_row = C / group;
    const long long n = wid / per_row;
    const int c0 = (int)(wid - n * per_row) * group;
    const float* xr = x + (size_t)n * C + c0;
    const float* gr = gate + (size_t)n * ld_gate + c0;
    float ss = 0.f;
    if (act == 2)
        for (int d = lane; d < group; d += 32) { const float v = gn_gated_first(xr[d], gr[d]); ss = fmaf(v, v, ss); }
    else
        for (int d = lane; d < group; d += 32) ss = fmaf(xr[d], xr[d], ss);
    ss = mv_warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)group + eps);
    TO* yr = y + (size_t)n * C + c0;
    for (int d = lane; d < group; d += 32) {
        const float g = gr[d];
        const float sg = 1.0f / (1.0f + expf(-g));
        const float wv = w[(c0 + d) % w_len];
        yr[d] = mv_from_f32<TO>(act == 2 ? gn_gated_first(xr[d], g) * scale * wv
                                         : xr[d] * scale * wv * (act == 0 ? g * sg : sg));
    }
}

// The same with one block per (row, group), for groups of many values (a norm over all heads of a wide layer).
template <typename TO>
__global__ void __launch_bounds__(1024)
gated_rmsnorm_block_kernel(const float* __restrict__ x, const float* __restrict__ gate, int ld_gate,
                           const float* __restrict__ w, int w_len, TO* __restrict__ y, int C, int group, float eps,
                           int act) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const int per_row = C / group;
    const long long n = blockIdx.x / per_row;
    const int c0 = (int)(blockIdx.x - n * per_row) * group;
    const float* xr = x + (size_t)n * C + c0;
    const float* gr = gate + (size_t)n * ld_gate + c0;
    float ss = 0.f;
    if (act == 2)
        for (int d = threadIdx.x; d < group; d += blockDim.x) { const float v = gn_gated_first(xr[d], gr[d]); ss = fmaf(v, v, ss); }
    else
        for (int d = threadIdx.x; d < group; d += blockDim.x) ss = fmaf(xr[d], xr[d], ss);
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)group + eps);
    TO* yr = y + (size_t)n * C + c0;
    for (int d = threadIdx.x; d < group; d += blockDim.x) {
        const float g = gr[d];
        const float sg = 1.0f / (1.0f + expf(-g));
        const float wv = w[(c0 + d) % w_len];
        yr[d] = mv_from_f32<TO>(act == 2 ? gn_gated_first(xr[d], g) * scale * wv
                                         : xr[d] * scale * wv * (act == 0 ? g * sg : sg));
    }
}

MV_API int mv_gated_rmsnorm(const float* x, const float* gate, int ld_gate, const float* w, int w_len, void* y,
                            int y_dtype, int N, int C, int group, float eps, int act, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (group < 1 || C % group || w_len < 1) return (int)cudaErrorInvalidValue;
    const long long n_groups = (long long)N * (C / group);
    if (group >= 512) {
        // few (row, group) pairs of many values each (a decode step of a wide layer): more threads a block
        const int threads = (n_groups < 1024 && group >= 4096) ? 1024 : ((n_groups < 2048 && group >= 2048) ? 512 : 256);
        if (y_dtype == MV_DT_BF16)
            mv_launch(gated_rmsnorm_block_kernel<__nv_bfloat16>, (unsigned)n_groups, threads, 0, stream, x, gate, ld_gate, w,
                      w_len, (__nv_bfloat16*)y, C, group, eps, act);
        else
            mv_launch(gated_rmsnorm_block_kernel<float>, (unsigned)n_groups, threads, 0, stream, x, gate, ld_gate, w, w_len,
                      (float*)y, C, group, eps, act);
        return mv_launch_status();
    }
    const unsigned blocks = (unsigned)((n_groups + 7) / 8);
    if (y_dtype == MV_DT_BF16)
        mv_launch(gated_rmsnorm_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, gate, ld_gate, w, w_len,
                  (__nv_bfloat16*)y, n_groups, C, group, eps, act);
    else
        mv_launch(gated_rmsnorm_kernel<float>, blocks, 256, 0, stream, x, gate, ld_gate, w, w_len, (float*)y, n_groups,
                  C, group, eps, act);
    return mv_launch_status();
}

// ----------------------------------------------- rms norm added to the residual stream
// resid[n, :] += y[n, :] / sqrt(mean(y[n, :]^2) + eps) * w
__global__ void rmsnorm_add_kernel(const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ resid,
                                   int H, float eps) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const float* yr = y + (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) ss = fmaf(yr[h], yr[h], ss);
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)H + eps);
    float* rr = resid + (size_t)blockIdx.x * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) rr[h] += yr[h] * scale * w[h];
}

MV_API int mv_rmsnorm_add(const float* y, const float* w, float* resid, int N, int H, float eps, cudaStream_t stream) {
    if (N <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    mv_launch(rmsnorm_add_kernel, N, threads, 0, stream, y, w, resid, H, eps);
    return mv_launch_status();
}

// The same for a sublayer whose norm sits on its OUTPUT (x += norm(f(x))), where the output may be the
// weighted sum of two branches, y = s1 y1 + s2 y2 (y2 null: y = s1 y1), and where the next sublayer reads
// the completed row rounded to the model's dtype (rounded null: not written).
template <typename TO>
__global__ void rmsnorm_add_sum_kernel(const float* __restrict__ y1, float s1, const float* __restrict__ y2, float s2,
                                       const float* __restrict__ w, float* __restrict__ resid, TO* __restrict__ rounded,
                                       int H, float eps) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float v = y2 ? fmaf(s2, y2[base + h], s1 * y1[base + h]) : s1 * y1[base + h];
        ss = fmaf(v, v, ss);
    }
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)H + eps);
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float v = y2 ? fmaf(s2, y2[base + h], s1 * y1[base + h]) : s1 * y1[base + h];
        const float r = resid[base + h] + v * scale * w[h];
        resid[base + h] = r;
        if (rounded) rounded[base + h] = mv_from_f32<TO>(r);
    }
}

// The same with four values a load, a row's values kept in registers between the two passes: for rows of a
// multiple of 4 and at most 8 values a thread, 16-byte aligned.
template <typename TO>
__global__ void __launch_bounds__(512)
rmsnorm_add_sum_vec_kernel(const float* __restrict__ y1, float s1, const float* __restrict__ y2, float s2,
                           const float* __restrict__ w, float* __restrict__ resid, TO* __restrict__ rounded, int H,
                           float eps) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * H;
    const int H4 = H >> 2;
    float4 v[2];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int h4 = threadIdx.x + i * blockDim.x;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (h4 < H4) {
            const float4 a = reinterpret_cast<const float4*>(y1 + base)[h4];
            v[i] = make_float4(s1 * a.x, s1 * a.y, s1 * a.z, s1 * a.w);
            if (y2) {
                const float4 b = reinterpret_cast<const float4*>(y2 + base)[h4];
                v[i] = make_float4(fmaf(s2, b.x, v[i].x), fmaf(s2, b.y, v[i].y), fmaf(s2, b.z, v[i].z), fmaf(s2, b.w, v[i].w));
            }
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)H + eps);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int h4 = threadIdx.x + i * blockDim.x;
        if (h4 < H4) {
            const float4 ww = reinterpret_cast<const float4*>(w)[h4];
            float4 r = reinterpret_cast<float4*>(resid + base)[h4];
            r.x += v[i].x * scale * ww.x; r.y += v[i].y * scale * ww.y;
            r.z += v[i].z * scale * ww.z; r.w += v[i].w * scale * ww.w;
            reinterpret_cast<float4*>(resid + base)[h4] = r;
            if (rounded) mv_store4(rounded + base + 4 * (size_t)h4, r.x, r.y, r.z, r.w);
        }
    }
}

MV_API int mv_rmsnorm_add_sum(const float* y1, float s1, const float* y2, float s2, const float* w, float* resid,
                              void* rounded, int rounded_dtype, int N, int H, float eps, cudaStream_t stream) {
    if (N <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const bool aligned = (((uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)w | (uintptr_t)resid | (uintptr_t)rounded) & 15) == 0;
    if (H % 4 == 0 && H / 4 <= 2 * threads && aligned) {
        if (rounded && rounded_dtype == MV_DT_BF16)
            mv_launch(rmsnorm_add_sum_vec_kernel<__nv_bfloat16>, N, threads, 0, stream, y1, s1, y2, s2, w, resid,
                      (__nv_bfloat16*)rounded, H, eps);
        else
            mv_launch(rmsnorm_add_sum_vec_kernel<float>, N, threads, 0, stream, y1, s1, y2, s2, w, resid, (float*)rounded, H, eps);
        return mv_launch_status();
    }
    if (rounded && rounded_dtype == MV_DT_BF16)
        mv_launch(rmsnorm_add_sum_kernel<__nv_bfloat16>, N, threads, 0, stream, y1, s1, y2, s2, w, resid,
                  (__nv_bfloat16*)rounded, H, eps);
    else
        mv_launch(rmsnorm_add_sum_kernel<float>, N, threads, 0, stream, y1, s1, y2, s2, w, resid, (float*)rounded, H, eps);
    return mv_launch_status();
}

// ------------------------- a sublayer's result times a vector, added to the stream; then the next norm
// resid[n, :] += vec * (s1 y1 + s2 y2) (y2 null: s1 y1): a layer whose sublayers' results are multiplied element by
// element by a learned vector (and a constant, folded into it) before they join the stream.  With w the row it
// has just completed is normed for the next sublayer: out[n, :] = resid / sqrt(mean(resid^2) + eps) * w.  A thread
// reads back only elements that it wrote itself.
template <typename TO>
__global__ void scaled_add_norm_kernel(const float* __restrict__ y1, float s1, const float* __restrict__ y2, float s2,
                                       const float* __restrict__ vec, float* __restrict__ resid,
                                       const float* __restrict__ w, float eps, TO* __restrict__ out, int H) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float v = y2 ? fmaf(s2, y2[base + h], s1 * y1[base + h]) : s1 * y1[base + h];
        const float r = fmaf(vec[h], v, resid[base + h]);
        resid[base + h] = r;
        ss = fmaf(r, r, ss);
    }
    if (!w) return;
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)H + eps);
    for (int h = threadIdx.x; h < H; h += blockDim.x) out[base + h] = mv_from_f32<TO>(resid[base + h] * scale * w[h]);
}

// The same with four values a load, a row's values kept in registers between the two passes: for rows of a
// multiple of 4 and at most 8 values a thread, 16-byte aligned.
template <typename TO>
__global__ void __launch_bounds__(512)
scaled_add_norm_vec_kernel(const float* __restrict__ y1, float s1, const float* __restrict__ y2, float s2,
                           const float* __restrict__ vec, float* __restrict__ resid, const float* __restrict__ w, float eps,
                           TO* __restrict__ out, int H) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * H;
    const int H4 = H >> 2;
    float4 r[2];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int h4 = threadIdx.x + i * blockDim.x;
        r[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (h4 < H4) {
            const float4 a = reinterpret_cast<const float4*>(y1 + base)[h4];
            float4 v = make_float4(s1 * a.x, s1 * a.y, s1 * a.z, s1 * a.w);
            if (y2) {
                const float4 b = reinterpret_cast<const float4*>(y2 + base)[h4];
                v = make_float4(fmaf(s2, b.x, v.x), fmaf(s2, b.y, v.y), fmaf(s2, b.z, v.z), fmaf(s2, b.w, v.w));
            }
            const float4 c = reinterpret_cast<const float4*>(vec)[h4];
            const float4 x = reinterpret_cast<const float4*>(resid + base)[h4];
            r[i] = make_float4(fmaf(c.x, v.x, x.x), fmaf(c.y, v.y, x.y), fmaf(c.z, v.z, x.z), fmaf(c.w, v.w, x.w));
            reinterpret_cast<float4*>(resid + base)[h4] = r[i];
            ss = fmaf(r[i].x, r[i].x, ss); ss = fmaf(r[i].y, r[i].y, ss);
            ss = fmaf(r[i].z, r[i].z, ss); ss = fmaf(r[i].w, r[i].w, ss);
        }
    }
    if (!w) return;
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)H + eps);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int h4 = threadIdx.x + i * blockDim.x;
        if (h4 < H4) {
            const float4 ww = reinterpret_cast<const float4*>(w)[h4];
            mv_store4(out + base + 4 * (size_t)h4, r[i].x * scale * ww.x, r[i].y * scale * ww.y, r[i].z * scale * ww.z,
                      r[i].w * scale * ww.w);
        }
    }
}

MV_API int mv_scaled_add_norm(const float* y1, float s1, const float* y2, float s2, const float* vec, float* resid,
                              const float* w, float eps, void* out, int out_dtype, int N, int H, cudaStream_t stream) {
    if (N <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const bool aligned = (((uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)vec | (uintptr_t)resid | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (H % 4 == 0 && H / 4 <= 2 * threads && aligned) {
        if (out_dtype == MV_DT_BF16)
            mv_launch(scaled_add_norm_vec_kernel<__nv_bfloat16>, N, threads, 0, stream, y1, s1, y2, s2, vec, resid, w, eps,
                      (__nv_bfloat16*)out, H);
        else
            mv_launch(scaled_add_norm_vec_kernel<float>, N, threads, 0, stream, y1, s1, y2, s2, vec, resid, w, eps, (float*)out, H);
        return mv_launch_status();
    }
    if (out_dtype == MV_DT_BF16)
        mv_launch(scaled_add_norm_kernel<__nv_bfloat16>, N, threads, 0, stream, y1, s1, y2, s2, vec, resid, w, eps,
                  (__nv_bfloat16*)out, H);
    else
        mv_launch(scaled_add_norm_kernel<float>, N, threads, 0, stream, y1, s1, y2, s2, vec, resid, w, eps, (float*)out, H);
    return mv_launch_status();
}

// ------------------------- the same, followed by the layer norm of the row it has just completed
// resid[n, :] += y / rms(y) * w, then out[n, :] = layer_norm(resid[n, :]) * ln_w: the last kernel of a layer and the
// first of the next in one, for layers that end with a normed input added to the residual stream.  A thread reads
// back only elements that it wrote itself.
template <typename TO>
__global__ void rmsnorm_add_layernorm_kernel(const float* __restrict__ y, const float* __restrict__ w, float eps,
                                             float* __restrict__ resid, const float* __restrict__ ln_w, float ln_eps,
                                             TO* __restrict__ out, int H) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const float* yr = y + (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) ss = fmaf(yr[h], yr[h], ss);
    const float scale = 1.0f / sqrtf(mv_block_sum(ss, scratch) / (float)H + eps);
    float* rr = resid + (size_t)blockIdx.x * H;
    float sum = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float v = rr[h] + yr[h] * scale * w[h];
        rr[h] = v;
        sum += v;
    }
    const float mean = mv_block_sum(sum, scratch) / (float)H;
    float dev = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float d = rr[h] - mean;
        dev = fmaf(d, d, dev);
    }
    const float rstd = 1.0f / sqrtf(mv_block_sum(dev, scratch) / (float)H + ln_eps);
    TO* orow = out + (size_t)blockIdx.x * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) orow[h] = mv_from_f32<TO>((rr[h] - mean) * rstd * ln_w[h]);
}

MV_API int mv_rmsnorm_add_layernorm(const float* y, const float* w, float eps, float* resid, const float* ln_w,
                                    float ln_eps, void* out, int out_dtype, int N, int H, cudaStream_t stream) {
    if (N <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (out_dtype == MV_DT_BF16)
        mv_launch(rmsnorm_add_layernorm_kernel<__nv_bfloat16>, N, threads, 0, stream, y, w, eps, resid, ln_w, ln_eps,
                  (__nv_bfloat16*)out, H);
    else
        mv_launch(rmsnorm_add_layernorm_kernel<float>, N, threads, 0, stream, y, w, eps, resid, ln_w, ln_eps, (float*)out, H);
    return mv_launch_status();
}

// ------------------------------------------------------ clamped gated activation
// h[n, f] = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit);
// gate = gu[n, f], up = gu[n, F + f].
template <typename TO>
__global__ void glu_clamped_kernel(const float* __restrict__ gu, TO* __restrict__ h, long long total, int F, float limit,
                                   float alpha) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / F;
    const int f = (int)(i - n * F);
    const float g = fminf(gu[n * 2 * F + f], limit);
    const float u = fminf(fmaxf(gu[n * 2 * F + F + f], -limit), limit);
    h[i] = mv_from_f32<TO>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

// The same with four consecutive features a thread (16-byte loads): F a multiple of 4, 16-byte aligned rows.
template <typename TO>
__global__ void __launch_bounds__(256)
glu_clamped_vec_kernel(const float* __restrict__ gu, TO* __restrict__ h, long long total4, int F, float limit, float alpha) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int F4 = F >> 2;
    const long long n = i / F4;
    const int f = (int)(i - n * F4) << 2;
    const float4 g4 = *reinterpret_cast<const float4*>(gu + n * 2 * F + f);
    const float4 u4 = *reinterpret_cast<const float4*>(gu + n * 2 * F + F + f);
    const float gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w};
    float y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float g = fminf(gs[j], limit);
        const float u = fminf(fmaxf(us[j], -limit), limit);
        y[j] = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    }
    mv_store4(h + n * F + f, y[0], y[1], y[2], y[3]);
}

MV_API int mv_glu_clamped(const float* gu, void* h, int h_dtype, int N, int F, float limit, float alpha,
                          cudaStream_t stream) {
    const long long total = (long long)N * F;
    if (total <= 0) return 0;
    if (F % 4 == 0 && (((uintptr_t)gu | (uintptr_t)h) & 15) == 0) {
        const unsigned blocks4 = (unsigned)((total / 4 + 255) / 256);
        if (h_dtype == MV_DT_BF16)
            mv_launch(glu_clamped_vec_kernel<__nv_bfloat16>, blocks4, 256, 0, stream, gu, (__nv_bfloat16*)h, total / 4, F, limit,
                      alpha);
        else
            mv_launch(glu_clamped_vec_kernel<float>, blocks4, 256, 0, stream, gu, (float*)h, total / 4, F, limit, alpha);
        return mv_launch_status();
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (h_dtype == MV_DT_BF16)
        mv_launch(glu_clamped_kernel<__nv_bfloat16>, blocks, 256, 0, stream, gu, (__nv_bfloat16*)h, total, F, limit, alpha);
    else
        mv_launch(glu_clamped_kernel<float>, blocks, 256, 0, stream, gu, (float*)h, total, F, limit, alpha);
    return mv_launch_status();
}

// --------------------------------------------------- gate by a row of a token table
// out[n, d] = gelu_tanh(p[n, d]) * table[tokens[n], col0 + d], d < D; the table's rows have ld_table elements.
template <typename TT, typename TO>
__global__ void table_gate_kernel(const float* __restrict__ p, const TT* __restrict__ table, int ld_table, int col0,
                                  const int* __restrict__ tokens, TO* __restrict__ out, long long total, int D) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / D;
    const int d = (int)(i - n * D);
    const float zv = p[i];
    const float gelu = 0.5f * zv * (1.0f + tanhf(0.7978845608028654f * (zv + 0.044715f * zv * zv * zv)));
    out[i] = mv_from_f32<TO>(gelu * mv_to_f32(table[(size_t)tokens[n] * ld_table + col0 + d]));
}

MV_API int mv_table_gate(const float* p, const void* table, int table_dtype, int ld_table, int col0, const int* tokens,
                         void* out, int out_dtype, int N, int D, cudaStream_t stream) {
    const long long total = (long long)N * D;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (table_dtype == MV_DT_BF16 && out_dtype == MV_DT_BF16)
        mv_launch(table_gate_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 256, 0, stream, p, (const __nv_bfloat16*)table,
                  ld_table, col0, tokens, (__nv_bfloat16*)out, total, D);
    else if (table_dtype == MV_DT_F32 && out_dtype == MV_DT_F32)
        mv_launch(table_gate_kernel<float, float>, blocks, 256, 0, stream, p, (const float*)table, ld_table, col0, tokens,
                  (float*)out, total, D);
    else if (table_dtype == MV_DT_F32)
        mv_launch(table_gate_kernel<float, __nv_bfloat16>, blocks, 256, 0, stream, p, (const float*)table, ld_table, col0,
                  tokens, (__nv_bfloat16*)out, total, D);
    else
        return (int)cudaErrorInvalidValue;
    return mv_launch_status();
}

// ------------------------------------------------------------------- rounding
// out = x rounded to the output type (the residual stream as a product's operand)
template <typename TO>
__global__ void round_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long total) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = mv_from_f32<TO>(x[i]);
}

MV_API int mv_round_rows(const float* x, void* out, int out_dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == MV_DT_BF16)
        mv_launch(round_rows_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, (__nv_bfloat16*)out, total);
    else
        mv_launch(round_rows_kernel<float>, blocks, 256, 0, stream, x, (float*)out, total);
    return mv_launch_status();
}

// ------------------------------------- a narrow projection of the residual stream, gated by a table row
// out[n, d] = gelu_tanh(G[d, :] . x) * table[tokens[n], col0 + d] with x = resid[n, :] rounded to the matrix's
// type: ``round_rows``, the product with G [D, H] and ``table_gate`` in one kernel, for steps of few tokens
// (every block reads its rows of G once a token).  One warp per (token, d); sums in float32.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
table_gate_proj_kernel(const float* __restrict__ resid, const TW* __restrict__ G, const TW* __restrict__ table,
                       int ld_table, int col0, const int* __restrict__ tokens, TO* __restrict__ out, int N, int H, int D) {
    mv_pdl_begin();
    const int lane = threadIdx.x & 31;
    const int d = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), n = blockIdx.x;
    if (d >= D) return;
    const float* x = resid + (size_t)n * H;
    const TW* g = G + (size_t)d * H;
    float dot = 0.f;
    if (H % 8 == 0 && (((uintptr_t)g | (uintptr_t)x) & 31) == 0) {
        for (int h = lane * 8; h < H; h += 256) {
            float gv[8], xv[8];
            mv_load8(g + h, gv);
            mv_load8(x + h, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) dot = fmaf(mv_to_f32(mv_from_f32<TW>(xv[e])), gv[e], dot);
        }
    } else {
        for (int h = lane; h < H; h += 32) dot = fmaf(mv_to_f32(mv_from_f32<TW>(x[h])), mv_to_f32(g[h]), dot);
    }
    dot = mv_warp_sum(dot);
    if (lane == 0) {
        const float gelu = 0.5f * dot * (1.0f + tanhf(0.7978845608028654f * (dot + 0.044715f * dot * dot * dot)));
        out[(size_t)n * D + d] = mv_from_f32<TO>(gelu * mv_to_f32(table[(size_t)tokens[n] * ld_table + col0 + d]));
    }
}

MV_API int mv_table_gate_proj(const float* resid, const void* G, const void* table, int dtype, int ld_table, int col0,
                              const int* tokens, void* out, int N, int H, int D, cudaStream_t stream) {
    if (N <= 0 || D <= 0) return 0;
    const dim3 grid(N, (D + 7) / 8);
    if (dtype == MV_DT_BF16)
        mv_launch(table_gate_proj_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, resid,
                  (const __nv_bfloat16*)G, (const __nv_bfloat16*)table, ld_table, col0, tokens, (__nv_bfloat16*)out, N, H, D);
    else
        mv_launch(table_gate_proj_kernel<float, float>, grid, 256, 0, stream, resid, (const float*)G, (const float*)table,
                  ld_table, col0, tokens, (float*)out, N, H, D);
    return mv_launch_status();
}
