// Routing of a mixture of experts, and the gated activation of the chosen experts.
//
// Router: s_e = sigmoid(z_e) from 32-bit logits, or softmax over all of them; a correction per expert may be added
// for the choice alone; some of the routed entries may be identity experts (no matrices: their output is their input).  The experts form `n_groups` equal groups of neighbours; a
// group's score is the sum of its two largest s (of its only one, in groups of one); only experts of the
// `keep` best groups can be chosen; the `top` largest s among those are chosen; their weights are s divided
// by the sum of the chosen s (+ 1e-20).  Ties go to the lower index.  A shared expert's gate, sigmoid of one
// more logit, is written as one more column.  All of it is 32-bit.
//
// Output: a dense row of weights per token, [experts (+ 1)], zero for the experts that were not chosen, and
// the chosen experts with their weights as lists [top].
#include "common.cuh"

#define RE_MAX_EXPERTS 1024

__device__ __forceinline__ void re_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// one warp a token.  mode 0: scores sigmoid(z); mode 1: scores softmax(z) over all E routed entries.  `correction`
// (or null) is added to the scores for the CHOICE only; the weights are the chosen entries' own scores over their sum
// (+ 1e-20), times out_scale.  The last n_identity of the E entries are identity experts: the dense row is laid out
// [E - n_identity experts | the shared gate, if any | n_identity identity weights].
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ z, int ld, float* __restrict__ dense, int* __restrict__ pick,
             float* __restrict__ pick_w, int N, int E, int n_groups, int keep, int top, int shared_gate, int mode,
             const float* __restrict__ correction, float out_scale, int n_identity) {
    mv_pdl_begin();
    extern __shared__ float re_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= N) return;
    const float NEG = -3.0e38f;
    float* s = re_smem + (size_t)warp * (2 * E + n_groups);   // scores
    float* ch = s + E;                                        // choice scores; NEG once taken or not allowed
    float* gs = ch + E;                                       // group scores
    const float* zr = z + (size_t)n * ld;
    const int n_real = E - n_identity, sg = shared_gate ? 1 : 0;
    const int cols = E + sg;
    float* dr = dense + (size_t)n * cols;
    if (mode == 1) {
        float mx = NEG;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
        mx = mv_warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(zr[e] - mx);
            s[e] = v;
            sum += v;
        }
        sum = mv_warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) s[e] *= inv;
    } else {
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-zr[e]));
    }
    for (int e = lane; e < E; e += 32) ch[e] = s[e] + (correction ? correction[e] : 0.f);
    for (int c = lane; c < cols; c += 32) dr[c] = 0.f;
    __syncwarp();
    if (shared_gate && lane == 0) dr[n_real] = 1.0f / (1.0f + expf(-zr[E]));
    const int per = E / n_groups;
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float a = NEG, b = NEG;                            // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = ch[e];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = a + (per > 1 ? b : 0.f);
        }
        __syncwarp();
        // the best `keep` groups are marked; then the others' experts are struck out
        for (int r = 0; r < keep; ++r) {
            float v = NEG; int i = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32)
                if (gs[g] > v) { v = gs[g]; i = g; }
            re_argmax(v, i);
            if (lane == 0) gs[i] = 2.f * NEG;                  // chosen
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != 2.f * NEG) ch[e] = NEG;
        __syncwarp();
    }
    float sum = 0.f;
    for (int r = 0; r < top; ++r) {
        float v = NEG; int i = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (ch[e] > v) { v = ch[e]; i = e; }
        re_argmax(v, i);
        const float sc = s[i];
        sum += sc;
        if (lane == 0) {
            pick[(size_t)n * top + r] = i;
            pick_w[(size_t)n * top + r] = sc;
            ch[i] = NEG;
        }
        __syncwarp();
    }
    const float inv = out_scale / (sum + 1e-20f);
    if (lane < top) {
        // (top <= 32 is checked by the host)
        const float w = pick_w[(size_t)n * top + lane] * inv;
        pick_w[(size_t)n * top + lane] = w;
        const int i = pick[(size_t)n * top + lane];
        dr[i < n_real ? i : i + sg] = w;
    }
}

// z [N, >= E (+ 1)] with row stride ld; dense [N, E (+ 1)]; pick, pick_w [N, top]; correction [E] or null.
MV_API int mv_route(const float* z, int ld, float* dense, int* pick, float* pick_w, int N, int E, int n_groups,
                    int keep, int top, int shared_gate, int mode, const float* correction, float out_scale,
                    int n_identity, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (E < 1 || E > RE_MAX_EXPERTS || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups || top < 1 ||
        top > 32 || top > keep * (E / n_groups) || n_identity < 0 || n_identity > E || mode < 0 || mode > 1)
        return (int)cudaErrorInvalidValue;
    const int warps = 4;
    const size_t smem = sizeof(float) * warps * (size_t)(2 * E + n_groups);
    mv_launch(route_kernel, (N + warps - 1) / warps, warps * 32, smem, stream, z, ld, dense, pick, pick_w, N, E,
              n_groups, keep, top, shared_gate, mode, correction, out_scale, n_identity);
    return mv_launch_status();
}

// resid[n, :] += (sum of dense[n, col0 .. col0 + n_cols)) * h[n, :]: experts whose output is their input.
template <typename T>
__global__ void __launch_bounds__(256)
identity_experts_kernel(const T* __restrict__ h, const float* __restrict__ dense, int ld, int col0, int n_cols,
                        float* __restrict__ resid, long long total, int H, int accumulate) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long n = idx / H;
    float w = 0.f;
    for (int c = 0; c < n_cols; ++c) w += dense[n * ld + col0 + c];
    const float v = w * mv_to_f32(h[idx]);
    resid[idx] = accumulate ? resid[idx] + v : v;
}

MV_API int mv_identity_experts(const void* h, int dtype, const float* dense, int ld, int col0, int n_cols, float* resid,
                               int N, int H, int accumulate, cudaStream_t stream) {
    if (N <= 0 || n_cols <= 0) return 0;
    const long long total = (long long)N * H;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == MV_DT_BF16)
        mv_launch(identity_experts_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)h, dense, ld, col0,
                  n_cols, resid, total, H, accumulate);
    else
        mv_launch(identity_experts_kernel<float>, blocks, 256, 0, stream, (const float*)h, dense, ld, col0, n_cols, resid,
                  total, H, accumulate);
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------------
// hid[n, c] = w[n, expert(c)] * silu(gate[n, c]) * up[n, c] over the columns of all experts laid end to end
// (expert e owns [e * ff, (e + 1) * ff), a shared expert the `shared_ff` columns after them, with the weight of
// column E).  gu [N, 2 * F] holds an expert's gates and ups together, [e * 2 ff, (e + 1) * 2 ff): alternating in
// groups of 16 columns (16 gates, their 16 ups, ...) where `group` says so, else the gates, then the ups; the
// shared expert's block follows with `shared_group`.  Where the weight is zero nothing is computed.
template <typename TO>
__global__ void __launch_bounds__(256)
routed_glu_kernel(const float* __restrict__ gu, const float* __restrict__ dense, TO* __restrict__ hid, long long total,
                  int F, int E, int ff, int shared_ff, int cols, int group, int shared_group) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long n = idx / F;
    const int c = (int)(idx - n * F);
    const int e = c < E * ff ? c / ff : E;
    const float w = dense[n * cols + e];
    float out = 0.f;
    if (w != 0.f) {
        const int cc = c - e * ff, width = e < E ? ff : shared_ff, grp = e < E ? group : shared_group;
        const float* blk = gu + n * 2 * F + (size_t)e * 2 * ff;
        const int gi = grp ? (cc / grp) * 2 * grp + cc % grp : cc;
        const float g = blk[gi], u = blk[gi + (grp ? grp : width)];
        out = w * (g / (1.0f + expf(-g))) * u;
    }
    hid[idx] = mv_from_f32<TO>(out);
}

// extra_cols: columns of a dense row after the experts' (and the shared gate's) that belong to others
MV_API int mv_routed_glu(const float* gu, const float* dense, void* hid, int hid_dtype, int N, int E, int ff,
                         int shared_ff, int group, int shared_group, int extra_cols, cudaStream_t stream) {
    if (N <= 0) return 0;
    const int F = E * ff + shared_ff, cols = E + (shared_ff ? 1 : 0) + extra_cols;
    if ((group && ff % group) || (shared_group && shared_ff % shared_group)) return (int)cudaErrorInvalidValue;
    const long long total = (long long)N * F;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (hid_dtype == MV_DT_BF16)
        mv_launch(routed_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, gu, dense, (__nv_bfloat16*)hid, total, F, E,
                  ff, shared_ff, cols, group, shared_group);
    else
        mv_launch(routed_glu_kernel<float>, blocks, 256, 0, stream, gu, dense, (float*)hid, total, F, E, ff, shared_ff, cols,
                  group, shared_group);
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------------
// For steps of many tokens: the (token, choice) entries sorted by expert, so that every expert multiplies its own
// tokens' rows only.  The sort is a stable counting sort: a block an expert walks the entries in order and ranks
// its own; the ranks depend on the entries alone, not on which block ran first.
__global__ void __launch_bounds__(256)
expert_rank_kernel(const int* __restrict__ pick, int total, int* __restrict__ rank, int* __restrict__ counts) {
    mv_pdl_begin();
    __shared__ int warp_sum[8];
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int base = 0;
    for (int t0 = 0; t0 < total; t0 += 256) {
        const int idx = t0 + tid;
        const bool mine = idx < total && pick[idx] == e;
        const unsigned votes = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_sum[warp] = __popc(votes);
        __syncthreads();
        int before = 0, all = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            before += w < warp ? warp_sum[w] : 0;
            all += warp_sum[w];
        }
        if (mine) rank[idx] = base + before + __popc(votes & ((1u << lane) - 1u));
        base += all;
        __syncthreads();
    }
    if (tid == 0) counts[e] = base;
}

// place[entry] = (entries of the experts before its own) + its rank; the token's row is copied there.
template <typename T>
__global__ void __launch_bounds__(128)
expert_gather_kernel(const int* __restrict__ pick, const int* __restrict__ rank, const int* __restrict__ counts,
                     const int* __restrict__ offsets, const T* __restrict__ x, int top, int H, int* __restrict__ place,
                     T* __restrict__ xs) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const int idx = blockIdx.x;
    const int e = pick[idx];
    int p;
    if (offsets) {
        p = offsets[e] + rank[idx];                // where the expert's (padded) run of rows starts
    } else {
        int before = 0;
        for (int i = threadIdx.x; i < e; i += blockDim.x) before += counts[i];
        p = (int)(mv_block_sum((float)before, scratch) + 0.5f) + rank[idx];       // exact: counts are far below 2^24
    }
    if (threadIdx.x == 0) place[idx] = p;
    const T* src = x + (size_t)(idx / top) * H;
    T* dst = xs + (size_t)p * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) dst[h] = src[h];
}

// out[n, :] (+)= sum_k w[n, k] ys[place[n * top + k], :] + gate[n] shared[n, :], the choices in their order
__global__ void __launch_bounds__(256)
expert_combine_kernel(const float* __restrict__ ys, const int* __restrict__ place, const float* __restrict__ pick_w,
                      const float* __restrict__ shared, const float* __restrict__ gate, int ld_gate,
                      float* __restrict__ out, int top, int H, int accumulate) {
    mv_pdl_begin();
    const int n = blockIdx.x;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k)
            sum = fmaf(pick_w[(size_t)n * top + k], ys[(size_t)place[(size_t)n * top + k] * H + h], sum);
        if (shared) sum = fmaf(gate ? gate[(size_t)n * ld_gate] : 1.f, shared[(size_t)n * H + h], sum);
        float* o = out + (size_t)n * H + h;
        *o = accumulate ? *o + sum : sum;
    }
}

// pick [N, top] -> rank [N * top], counts [E]
MV_API int mv_expert_rank(const int* pick, int total, int E, int* rank, int* counts, cudaStream_t stream) {
    if (total <= 0 || E <= 0) return 0;
    mv_launch(expert_rank_kernel, E, 256, 0, stream, pick, total, rank, counts);
    return mv_launch_status();
}

// x [N, H] in `dtype` -> xs [N * top, H] sorted by expert; place [N * top] says where each entry went
// offsets (or null): where every expert's run of rows starts (mv_expert_tiles), instead of the plain sums of counts
MV_API int mv_expert_gather(const int* pick, const int* rank, const int* counts, const int* offsets, const void* x,
                            int dtype, int N, int top, int H, int* place, void* xs, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (dtype == MV_DT_BF16)
        mv_launch(expert_gather_kernel<__nv_bfloat16>, N * top, 128, 0, stream, pick, rank, counts, offsets,
                  (const __nv_bfloat16*)x, top, H, place, (__nv_bfloat16*)xs);
    else
        mv_launch(expert_gather_kernel<float>, N * top, 128, 0, stream, pick, rank, counts, offsets, (const float*)x, top, H,
                  place, (float*)xs);
    return mv_launch_status();
}

// Every expert's run of rows padded to whole tiles of `tile_rows`, so that a grouped product's tile never holds two
// experts: offsets[e] = where expert e's run starts, tile_group[t] = the expert of tile t, -1 for the spare tiles
// after the last run.  One block; the host needs to know nothing (n_tiles is an upper bound:
// (entries + E * (tile_rows - 1)) / tile_rows).
__global__ void __launch_bounds__(256)
expert_tiles_kernel(const int* __restrict__ counts, int E, int tile_rows, int* __restrict__ offsets,
                    int* __restrict__ tile_group, int n_tiles) {
    mv_pdl_begin();
    __shared__ int first_tile[RE_MAX_EXPERTS + 1];
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < E; ++e) {
            first_tile[e] = t;
            offsets[e] = t * tile_rows;
            t += (counts[e] + tile_rows - 1) / tile_rows;
        }
        first_tile[E] = t;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) {
        int g = -1;
        if (t < first_tile[E]) {
            int lo = 0, hi = E;                    // the last expert whose first tile is <= t and that has tiles
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (first_tile[mid] <= t) lo = mid; else hi = mid;
            }
            g = lo;
        }
        tile_group[t] = g;
    }
}

MV_API int mv_expert_tiles(const int* counts, int E, int tile_rows, int* offsets, int* tile_group, int n_tiles,
                           cudaStream_t stream) {
    if (E <= 0 || n_tiles <= 0) return 0;
    if (E > RE_MAX_EXPERTS || tile_rows < 1) return (int)cudaErrorInvalidValue;
    mv_launch(expert_tiles_kernel, 1, 256, 0, stream, counts, E, tile_rows, offsets, tile_group, n_tiles);
    return mv_launch_status();
}

MV_API int mv_expert_combine(const float* ys, const int* place, const float* pick_w, const float* shared,
                             const float* gate, int ld_gate, float* out, int N, int top, int H, int accumulate,
                             cudaStream_t stream) {
    if (N <= 0) return 0;
    mv_launch(expert_combine_kernel, N, 256, 0, stream, ys, place, pick_w, shared, gate, ld_gate, out, top, H, accumulate);
    return mv_launch_status();
}

// h[n, c] *= w[n, expert(c)] in place, for activations that a product's epilogue has already gated: eight
// columns a thread (ff and shared_ff are multiples of 8 then), or one.
template <typename T, int V>
__global__ void __launch_bounds__(256)
scale_expert_columns_kernel(T* __restrict__ h, const float* __restrict__ dense, long long total, int F, int E, int ff,
                            int cols) {
    mv_pdl_begin();
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (idx >= total) return;
    const long long n = idx / F;
    const int c = (int)(idx - n * F);
    const float w = dense[n * cols + (c < E * ff ? c / ff : E)];
    if (V == 8) {
        float x[8];
        mv_load8(h + idx, x);
        mv_store4(h + idx, x[0] * w, x[1] * w, x[2] * w, x[3] * w);
        mv_store4(h + idx + 4, x[4] * w, x[5] * w, x[6] * w, x[7] * w);
    } else {
        h[idx] = mv_from_f32<T>(mv_to_f32(h[idx]) * w);
    }
}

MV_API int mv_scale_expert_columns(void* h, int dtype, const float* dense, int N, int E, int ff, int shared_ff,
                                   int extra_cols, cudaStream_t stream) {
    if (N <= 0) return 0;
    const int F = E * ff + shared_ff, cols = E + (shared_ff ? 1 : 0) + extra_cols;
    const long long total = (long long)N * F;
    const bool wide = ff % 8 == 0 && shared_ff % 8 == 0 && ((uintptr_t)h % 16) == 0;
    const unsigned blocks = (unsigned)((total / (wide ? 8 : 1) + 255) / 256);
#define SE_LAUNCH(T, V) mv_launch(scale_expert_columns_kernel<T, V>, blocks, 256, 0, stream, (T*)h, dense, total, F, E, ff, cols)
    if (dtype == MV_DT_BF16) { if (wide) SE_LAUNCH(__nv_bfloat16, 8); else SE_LAUNCH(__nv_bfloat16, 1); }
    else { if (wide) SE_LAUNCH(float, 8); else SE_LAUNCH(float, 1); }
#undef SE_LAUNCH
    return mv_launch_status();
}
