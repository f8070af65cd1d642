// Routed experts: which experts a token uses, the order that puts every expert's tokens side by side for the
// grouped products, and the weighted sum that brings the experts' outputs back to the tokens.
//
//   moe_choose   per token (one warp): the router's logits (a product of the token rows with the router matrix, summed
//                in float32) plus the bias, the `top` largest (the lower index wins a tie), their weights = softmax
//                over the chosen logits only; optionally one more number per token, sigmoid of one more column of
//                that product (w_gate . h), for a shared expert.  A second rule (`rule` 1): scores = softmax of the
//                logits over all experts, the `top` largest of score + bias are chosen, the weights are the chosen
//                scores themselves, divided by their sum and multiplied by `weight_scale`.  A third rule (`rule` 2):
//                scores = sigmoid of every logit by itself, the `top` largest of score + bias are chosen, the weights
//                are the chosen scores as they are, times `weight_scale`
//   moe_sort     one CTA: (token, choice) pairs counted per expert, every expert's stretch padded to a multiple of
//                the products' row tile, so that a row tile belongs to one expert; writes for every place of the
//                padded order its token (-1: padding), for every pair its place, for every row tile its expert
//                (-1: unused).  Sizes are upper bounds known on the host, so nothing has to come back from the device
//   moe_combine  per token: sum_k weight_k * expert_out[place of (token, k)] + gate * shared_out; a chosen expert
//                beyond the ones that have weights (an identity expert) hands the token's own input on
#include "common.cuh"

constexpr int MOE_MAX_LOGITS_PER_LANE = 16;            // 512 experts at most

template <typename TW>
__global__ void __launch_bounds__(128)
moe_choose_kernel(const float* __restrict__ z_in, long z_stride, int n_partials, long partial_stride,
                  const TW* __restrict__ br, int gate_col, int n, int E, int K, int* __restrict__ chosen,
                  float* __restrict__ share, float* __restrict__ gate, int rule, float weight_scale) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= n) return;
    const float* zr = z_in + (size_t)row * z_stride;
    auto logit = [&](int c) { return fb_slab_sum(zr, c, n_partials, partial_stride); };
    float z[MOE_MAX_LOGITS_PER_LANE];                  // lane l keeps the logits of experts l, l + 32, ...
    if (rule == 1 || rule == 2) {
        // scores over all experts first; the bias only moves the choice
        float s[MOE_MAX_LOGITS_PER_LANE];
        float top = -INFINITY;
#pragma unroll
        for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r) {
            const int e = lane + 32 * r;
            s[r] = e < E ? logit(e) : -INFINITY;
            top = fmaxf(top, s[r]);
        }
        if (rule == 1) {
            top = fb_warp_max(top);
            float sum = 0.0f;
#pragma unroll
            for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r) {
                s[r] = lane + 32 * r < E ? expf(s[r] - top) : 0.0f;
                sum += s[r];
            }
            sum = fb_warp_sum(sum);
#pragma unroll
            for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r) s[r] = s[r] / sum;
        } else {
#pragma unroll
            for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r)
                s[r] = lane + 32 * r < E ? 1.0f / (1.0f + expf(-s[r])) : 0.0f;
        }
#pragma unroll
        for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r) {
            const int e = lane + 32 * r;
            z[r] = e < E ? s[r] + (br ? fb_to_float(br[e]) : 0.0f) : -INFINITY;
        }
        float total = 0.0f, mine = 0.0f;               // lane k keeps the k-th chosen score
        for (int k = 0; k < K; ++k) {
            float best = -INFINITY, best_s = 0.0f;
            int best_e = 0x7fffffff;
#pragma unroll
            for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r) {
                const int e = lane + 32 * r;
                if (e < E && (z[r] > best)) { best = z[r]; best_e = e; best_s = s[r]; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, off);
                const float os = __shfl_xor_sync(0xffffffffu, best_s, off);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
                if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; best_s = os; }
            }
#pragma unroll
            for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r)
                if (best_e == lane + 32 * r) z[r] = -INFINITY;           // taken
            total += best_s;
            if (lane == k) mine = best_s;
            if (lane == 0) chosen[(size_t)row * K + k] = best_e;
        }
        if (lane < K) share[(size_t)row * K + lane] = (rule == 1 ? mine / (total + 1e-20f) : mine) * weight_scale;
        if (gate_col >= 0 && lane == 0) gate[row] = 1.0f / (1.0f + expf(-logit(gate_col)));
        return;
    }
#pragma unroll
    for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r) {
        const int e = lane + 32 * r;
        z[r] = e < E ? logit(e) + (br ? fb_to_float(br[e]) : 0.0f) : -INFINITY;
    }
    if (gate_col >= 0 && lane == 0) gate[row] = 1.0f / (1.0f + expf(-logit(gate_col)));
    float first = 0.0f, total = 0.0f, mine = 0.0f;     // lane k keeps the k-th chosen logit (K <= 32)
    for (int k = 0; k < K; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r) {
            const int e = lane + 32 * r;
            if (e < E && (z[r] > best)) { best = z[r]; best_e = e; }     // ascending e: the lower index stays on a tie
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
#pragma unroll
        for (int r = 0; r < MOE_MAX_LOGITS_PER_LANE; ++r)
            if (best_e == lane + 32 * r) z[r] = -INFINITY;               // taken
        if (k == 0) first = best;
        const float p = expf(best - first);            // the first chosen logit is the largest
        total += p;
        if (lane == k) mine = p;
        if (lane == 0) chosen[(size_t)row * K + k] = best_e;
    }
    if (lane < K) share[(size_t)row * K + lane] = mine / total;
}

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ chosen, int pairs, int K, int E, int tile, int max_tiles,
                int* __restrict__ place_token, int* __restrict__ pair_place, int* __restrict__ tile_expert,
                int* __restrict__ place_pair) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ int shi[];                       // [E] counts, then [E] cursors
    int* count = shi;
    int* cursor = shi + E;
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) count[e] = 0;
    for (int i = tid; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
    for (int i = tid; i < max_tiles * tile; i += blockDim.x) place_token[i] = -1;
    __syncthreads();
    for (int p = tid; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = at;
            const int tiles = (count[e] + tile - 1) / tile;
            for (int t = 0; t < tiles; ++t) tile_expert[at / tile + t] = e;
            at += tiles * tile;
        }
    }
    __syncthreads();
    for (int p = tid; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < 0 || e >= E) { pair_place[p] = -1; continue; }
        const int at = atomicAdd(&cursor[e], 1);
        place_token[at] = p / K;
        pair_place[p] = at;
        if (place_pair) place_pair[at] = p;
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ expert_out, long expert_stride,
                                   const int* __restrict__ pair_place, const float* __restrict__ share, int K,
                                   const float* __restrict__ shared_out, int shared_partials, long shared_partial_stride,
                                   const float* __restrict__ gate, float* __restrict__ out, int n, int D,
                                   const T* __restrict__ pass_on, long pass_stride) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * D) return;
    const int row = (int)(idx / D), c = (int)(idx - (size_t)row * D);
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) {
        const int at = pair_place[(size_t)row * K + k];
        const float w = share ? share[(size_t)row * K + k] : 1.0f;
        if (at >= 0) acc = fmaf(w, expert_out[(size_t)at * expert_stride + c], acc);
        else if (pass_on) acc = fmaf(w, fb_to_float(pass_on[(size_t)row * pass_stride + c]), acc);
    }
    if (shared_out) {
        float s = 0.0f;
        for (int p = 0; p < shared_partials; ++p) s += shared_out[(size_t)p * shared_partial_stride + idx];
        acc = fmaf(gate ? gate[row] : 1.0f, s, acc);
    }
    out[idx] = acc;
}

// out[place] = h[place_token[place]] (a row of zeros where the place is padding): the tokens side by side in expert
// order, for the products that fetch their rows by tensor-map copies.  With `share` and `place_pair` the row is
// multiplied by the share of the pair that the place stands for (experts whose weight scales what they read).
template <typename T>
__global__ void moe_gather_rows_kernel(const T* __restrict__ h, long h_stride, const int* __restrict__ place_token,
                                       T* __restrict__ out, int rows, int D, const float* __restrict__ share,
                                       const int* __restrict__ place_pair) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int chunks = D / 8;                          // 16 bytes of bfloat16, 32 of float32
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * chunks) return;
    const int r = (int)(idx / chunks), c = (int)(idx - (size_t)r * chunks);
    const int src = place_token[r];
    struct alignas(sizeof(T) * 8) Chunk { T v[8]; };
    Chunk z;
#pragma unroll
    for (int i = 0; i < 8; ++i) z.v[i] = fb_from_float<T>(0.0f);
    if (src >= 0) {
        z = *reinterpret_cast<const Chunk*>(h + (size_t)src * h_stride + (size_t)c * 8);
        if (share) {
            const float w = share[place_pair[r]];
#pragma unroll
            for (int i = 0; i < 8; ++i) z.v[i] = fb_from_float<T>(fb_to_float(z.v[i]) * w);
        }
    }
    *reinterpret_cast<Chunk*>(out + (size_t)r * D + (size_t)c * 8) = z;
}

// Any width and alignment, one number a thread.
template <typename T>
__global__ void moe_gather_rows_scalar_kernel(const T* __restrict__ h, long h_stride, const int* __restrict__ place_token,
                                              T* __restrict__ out, int rows, int D, const float* __restrict__ share,
                                              const int* __restrict__ place_pair) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * D) return;
    const int r = (int)(idx / D), c = (int)(idx - (size_t)r * D);
    const int src = place_token[r];
    float v = 0.0f;
    if (src >= 0) v = fb_to_float(h[(size_t)src * h_stride + c]) * (share ? share[place_pair[r]] : 1.0f);
    out[idx] = fb_from_float<T>(v);
}

FB_API int fb_moe_gather_rows(const void* h, long long h_stride, int dtype, const int* place_token, void* out,
                              int rows, int D, const float* share, const int* place_pair, cudaStream_t stream) {
    FB_REQUIRE(!share || place_pair, "moe_gather_rows: shares need the pair of every place");
    FB_REQUIRE(rows >= 0 && D > 0, "moe_gather_rows: bad sizes");
    if (rows == 0) return 0;
    if (D % 8 == 0 && h_stride % 8 == 0 && ((uintptr_t)h & 31) == 0 && ((uintptr_t)out & 31) == 0) {
        const size_t total = (size_t)rows * (D / 8);
        FB_DISPATCH_DTYPE(dtype, T,
            (fb_launch((moe_gather_rows_kernel<T>), dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                       (const T*)h, (long)h_stride, place_token, (T*)out, rows, D, share, place_pair)));
    } else {
        const size_t total = (size_t)rows * D;
        FB_DISPATCH_DTYPE(dtype, T,
            (fb_launch((moe_gather_rows_scalar_kernel<T>), dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                       (const T*)h, (long)h_stride, place_token, (T*)out, rows, D, share, place_pair)));
    }
    return fb_check_launch("moe_gather_rows");
}

// rule 0: the `top` largest logits + bias, weights = softmax over the chosen; rule 1: scores = softmax over all E, the
// `top` largest of score + bias, weights = chosen scores / their sum * weight_scale; rule 2: scores = sigmoid of each
// logit, the `top` largest of score + bias, weights = chosen scores * weight_scale.
// z: float32 router logits [n, >= E (+1)] (possibly split-K shares), as a product of the token rows with the stacked
// router matrix left them; br: the router's bias or nullptr; gate_col: the column that holds w_gate . h (negative: none).
FB_API int fb_moe_choose(const float* z, long long z_stride, int n_partials, long long partial_stride, const void* br,
                         int w_dtype, int gate_col, int n, int E, int K, int* chosen, float* share, float* gate,
                         int rule, float weight_scale, cudaStream_t stream) {
    FB_REQUIRE(rule >= 0 && rule <= 2, "router: unknown rule %d", rule);
    FB_REQUIRE(n >= 0 && E > 0 && K > 0 && K <= E, "router: bad sizes n=%d experts=%d top=%d", n, E, K);
    FB_REQUIRE(E <= 32 * MOE_MAX_LOGITS_PER_LANE, "router: %d experts are more than %d", E, 32 * MOE_MAX_LOGITS_PER_LANE);
    FB_REQUIRE(K <= 32, "router: top = %d is more than 32", K);
    FB_REQUIRE(gate_col < 0 || gate, "router: a gate column without a place for the gate");
    FB_REQUIRE(z_stride >= E && z_stride > gate_col, "router: logit rows are too short");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    FB_DISPATCH_DTYPE(w_dtype, TW,
        (fb_launch((moe_choose_kernel<TW>), dim3((n + 3) / 4), dim3(128), 0, stream, z, (long)z_stride, n_partials,
                   (long)partial_stride, (const TW*)br, gate_col, n, E, K, chosen, share, gate, rule, weight_scale)));
    return fb_check_launch("moe_choose");
}

// Row tiles the padded order can take at most: every full tile of pairs, and one ragged tile per expert that has any.
FB_API int fb_moe_max_tiles(int pairs, int E, int tile) {
    return pairs / tile + (E < pairs ? E : pairs);
}

// place_pair (optional, [max_tiles * tile]): for every place that holds a token, the (token, choice) pair it stands for.
FB_API int fb_moe_sort(const int* chosen, int pairs, int K, int E, int tile, int max_tiles, int* place_token,
                       int* pair_place, int* tile_expert, int* place_pair, cudaStream_t stream) {
    FB_REQUIRE(pairs >= 0 && K > 0 && E > 0 && tile > 0, "moe_sort: bad sizes");
    FB_REQUIRE(max_tiles >= fb_moe_max_tiles(pairs, E, tile), "moe_sort: %d row tiles are too few", max_tiles);
    if (pairs == 0) return 0;
    fb_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, chosen, pairs, K, E, tile,
              max_tiles, place_token, pair_place, tile_expert, place_pair);
    return fb_check_launch("moe_sort");
}

// Four columns a thread (D a multiple of 4, rows 16-byte aligned): a token's places and shares are fetched once per
// four outputs and every row is read 16 bytes at a time.
template <typename T>
__global__ void moe_combine_vec_kernel(const float* __restrict__ expert_out, long expert_stride,
                                       const int* __restrict__ pair_place, const float* __restrict__ share, int K,
                                       const float* __restrict__ shared_out, int shared_partials,
                                       long shared_partial_stride, const float* __restrict__ gate,
                                       float* __restrict__ out, int n, int D, const T* __restrict__ pass_on,
                                       long pass_stride) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int nvec = D >> 2;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * nvec) return;
    const int row = (int)(idx / nvec), c = (int)(idx - (size_t)row * nvec) * 4;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int k = 0; k < K; ++k) {
        const int at = pair_place[(size_t)row * K + k];
        if (at < 0 && !pass_on) continue;
        const float w = share ? share[(size_t)row * K + k] : 1.0f;
        float4 v;
        if (at < 0) {                                  // an expert without weights: the token's own input
            const T* src = pass_on + (size_t)row * pass_stride + c;
            v = make_float4(fb_to_float(src[0]), fb_to_float(src[1]), fb_to_float(src[2]), fb_to_float(src[3]));
        } else {
            v = *reinterpret_cast<const float4*>(expert_out + (size_t)at * expert_stride + c);
        }
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    if (shared_out) {
        float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int p = 0; p < shared_partials; ++p) {
            const float4 v = *reinterpret_cast<const float4*>(shared_out + (size_t)p * shared_partial_stride +
                                                              (size_t)row * D + c);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        const float gt = gate ? gate[row] : 1.0f;
        acc.x = fmaf(gt, s.x, acc.x); acc.y = fmaf(gt, s.y, acc.y); acc.z = fmaf(gt, s.z, acc.z); acc.w = fmaf(gt, s.w, acc.w);
    }
    *reinterpret_cast<float4*>(out + (size_t)row * D + c) = acc;
}

// pass_on (optional, [n, D] rows `pass_stride` apart, dtype code `pass_dtype`): what a pair without a place (a chosen
// expert that has no weights) contributes, times its share.  share = nullptr: every pair counts once (the shares
// have scaled the experts' inputs already).
FB_API int fb_moe_combine(const float* expert_out, long long expert_stride, const int* pair_place, const float* share,
                          int K, const float* shared_out, int shared_partials, long long shared_partial_stride,
                          const float* gate, float* out, int n, int D, const void* pass_on, int pass_dtype,
                          long long pass_stride, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && D > 0 && K > 0, "moe_combine: bad sizes");
    if (n == 0) return 0;
    if (!pass_on) pass_dtype = FB_F32;
    if (D % 4 == 0 && expert_stride % 4 == 0 && shared_partial_stride % 4 == 0 && (uintptr_t)expert_out % 16 == 0 &&
        (uintptr_t)out % 16 == 0 && (!shared_out || (uintptr_t)shared_out % 16 == 0)) {
        const size_t total4 = (size_t)n * (D / 4);
        FB_DISPATCH_DTYPE(pass_dtype, T,
            (fb_launch((moe_combine_vec_kernel<T>), dim3((unsigned)((total4 + 255) / 256)), dim3(256), 0, stream,
                       expert_out, (long)expert_stride, pair_place, share, K, shared_out,
                       shared_partials < 1 ? 1 : shared_partials, (long)shared_partial_stride, gate, out, n, D,
                       (const T*)pass_on, (long)pass_stride)));
        return fb_check_launch("moe_combine");
    }
    const size_t total = (size_t)n * D;
    FB_DISPATCH_DTYPE(pass_dtype, T,
        (fb_launch((moe_combine_kernel<T>), dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, expert_out,
                   (long)expert_stride, pair_place, share, K, shared_out, shared_partials < 1 ? 1 : shared_partials,
                   (long)shared_partial_stride, gate, out, n, D, (const T*)pass_on, (long)pass_stride)));
    return fb_check_launch("moe_combine");
}
