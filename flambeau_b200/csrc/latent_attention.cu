// Attention whose keys and values are kept as one narrow latent row per token.
//
// A token's cache row is [c : Rc | kr : r]: c is the RMS-normed latent from which every head's unrotated key
// (Wuk_h c) and value (Wuv_h c) follow, kr one rotated key part that all heads share.  Nothing per head is cached.
// Queries meet the latent directly: with q_h = [qn : d | qr : r],
//
//     score = (Wuk_h^T qn) . c + rot(qr) . kr          and          out_h = Wuv_h (sum_j p_j c_j),
//
// so the attention itself runs as one key/value head of size Rc + r that all query heads share, with the cache rows as
// keys and as values (the last r columns of its output are not used), and two small maps per head stand around it.
//
// Kernels:
//   mla_latents   per token: the query's latent RMS-normed and rounded for the product that expands it; the
//                 key/value latent RMS-normed, the shared key part rotated, both written into the token's cache row.
//                 Inputs are the float32 split-K shares of the stacked down-projection.
//   head_linear   out[t, h, :N] = W_h [N, K] . a[t, h, :K] for every head, float32 accumulation on the CUDA cores;
//                 `a` may be float32 shares (added first).  Two optional extras: K..K+r of the input row rotated into
//                 N..N+r of the output row (the query side), and the result multiplied by sigmoid of a gate taken
//                 from another product's shares (the output side).
// Rotation pairs neighbours: (x[2i], x[2i+1]) -> (x[2i] cos - x[2i+1] sin, x[2i+1] cos + x[2i] sin), i < half, with
// per-token tables; dimensions from 2 half on pass unchanged.
#include "common.cuh"

__device__ __forceinline__ float mla_slab_sum(const float* row, int c, int n_partials, long partial_stride) {
    float v = row[c];
    for (int p = 1; p < n_partials; ++p) v += row[(size_t)p * partial_stride + c];
    return v;
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
mla_latents_kernel(const float* __restrict__ proj, long proj_stride, int n_partials, long partial_stride, int Rq,
                   const TW* __restrict__ wq, TO* __restrict__ cq, int kv_off, int Rc, int r,
                   const TW* __restrict__ wkv, float eps, const float* __restrict__ cos_t,
                   const float* __restrict__ sin_t, int half, const int* __restrict__ positions,
                   const int* __restrict__ row_seq, const int* __restrict__ block_table, int table_stride,
                   const int* __restrict__ table_base, TO* __restrict__ pool, int page_size, int n_pages, int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ float lat[];
    __shared__ float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* pr = proj + (size_t)t * proj_stride;
    if (blockIdx.y == 0) {                             // block-uniform
        float ss = 0.0f;
        for (int i = tid; i < Rq; i += blockDim.x) {
            const float v = mla_slab_sum(pr, i, n_partials, partial_stride);
            lat[i] = v;
            ss = fmaf(v, v, ss);
        }
        const float inv = 1.0f / sqrtf(fb_block_sum(ss, red) / (float)Rq + eps);
        for (int i = tid; i < Rq; i += blockDim.x)
            cq[(size_t)t * Rq + i] = fb_from_float<TO>(lat[i] * inv * fb_to_float(wq[i]));
        return;
    }
    const int pos = positions[t], seq = row_seq[t];
    const int entry = pos / page_size - (table_base ? table_base[seq] : 0);
    const int page = (entry >= 0 && entry < table_stride) ? block_table[(size_t)seq * table_stride + entry] : -1;
    if (page < 0 || page >= n_pages) {
        if (tid == 0) atomicOr(status, FB_STATUS_BAD_PAGE);
        return;
    }
    TO* dst = pool + ((size_t)page * page_size + pos % page_size) * (size_t)(Rc + r);
    float ss = 0.0f;
    for (int i = tid; i < Rc; i += blockDim.x) {
        const float v = mla_slab_sum(pr, kv_off + i, n_partials, partial_stride);
        lat[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(fb_block_sum(ss, red) / (float)Rc + eps);
    for (int i = tid; i < Rc; i += blockDim.x) dst[i] = fb_from_float<TO>(lat[i] * inv * fb_to_float(wkv[i]));
    const float* kr = pr + kv_off + Rc;
    for (int i = tid; i < r - half; i += blockDim.x) {
        if (i < half) {
            const float u = mla_slab_sum(kr, 2 * i, n_partials, partial_stride);
            const float v = mla_slab_sum(kr, 2 * i + 1, n_partials, partial_stride);
            const float c = cos_t[(size_t)t * half + i], s = sin_t[(size_t)t * half + i];
            dst[Rc + 2 * i] = fb_from_float<TO>(u * c - v * s);
            dst[Rc + 2 * i + 1] = fb_from_float<TO>(v * c + u * s);
        } else {
            dst[Rc + half + i] = fb_from_float<TO>(mla_slab_sum(kr, half + i, n_partials, partial_stride));
        }
    }
}

constexpr int HL_TM = 32, HL_TN = 64, HL_KC = 16;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_linear_kernel(const TA* __restrict__ a, long a_stride, long a_head, int n_partials, long partial_stride,
                   const TW* __restrict__ w, TO* __restrict__ out, long o_stride, long o_head,
                   const float* __restrict__ gate, long gate_stride, int gate_partials, long gate_partial_stride,
                   int gate_off, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int half, int r,
                   int n, int N, int K) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    __shared__ float As[HL_KC][HL_TM + 1];
    __shared__ float Ws[HL_KC][HL_TN + 1];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.x * HL_TM, n0 = blockIdx.y * HL_TN, h = blockIdx.z;
    const TA* ah = a + (size_t)h * a_head;
    const TW* wh = w + (size_t)h * N * K;
    float acc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += HL_KC) {
#pragma unroll
        for (int u = 0; u < (HL_TM * HL_KC) / 256; ++u) {
            const int idx = tid + 256 * u, m = idx / HL_KC, k = idx - m * HL_KC;
            float v = 0.0f;
            if (m0 + m < n && k0 + k < K) {
                const TA* p = ah + (size_t)(m0 + m) * a_stride + k0 + k;
                v = fb_to_float(p[0]);
                for (int q = 1; q < n_partials; ++q) v += fb_to_float(p[(size_t)q * partial_stride]);
            }
            As[k][m] = v;
        }
#pragma unroll
        for (int u = 0; u < (HL_TN * HL_KC) / 256; ++u) {
            const int idx = tid + 256 * u, nn = idx / HL_KC, k = idx - nn * HL_KC;
            Ws[k][nn] = (n0 + nn < N && k0 + k < K) ? fb_to_float(wh[(size_t)(n0 + nn) * K + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HL_KC; ++k) {
            const float a0 = As[k][ty], a1 = As[k][ty + 16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float b = Ws[k][tx + 16 * i];
                acc[0][i] = fmaf(a0, b, acc[0][i]);
                acc[1][i] = fmaf(a1, b, acc[1][i]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int m = m0 + ty + 16 * j;
        if (m >= n) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = n0 + tx + 16 * i;
            if (c >= N) continue;
            float v = acc[j][i];
            if (gate) {
                const float g = mla_slab_sum(gate + (size_t)m * gate_stride, gate_off + h * N + c, gate_partials,
                                             gate_partial_stride);
                v = v / (1.0f + expf(-g));
            }
            out[(size_t)m * o_stride + (size_t)h * o_head + c] = fb_from_float<TO>(v);
        }
    }
    if (r > 0 && blockIdx.y == 0) {
        // the rotated tail: columns K .. K+r of the input row go, turned, to columns N .. N+r of the output row
        const int per = r - half;
        for (int e = tid; e < HL_TM * per; e += 256) {
            const int mm = e / per, i = e - mm * per, m = m0 + mm;
            if (m >= n) break;
            const TA* src = ah + (size_t)m * a_stride + K;
            TO* dst = out + (size_t)m * o_stride + (size_t)h * o_head + N;
            auto in = [&](int c) {
                float v = fb_to_float(src[c]);
                for (int q = 1; q < n_partials; ++q) v += fb_to_float(src[(size_t)q * partial_stride + c]);
                return v;
            };
            if (i < half) {
                const float u = in(2 * i), v = in(2 * i + 1);
                const float c = cos_t[(size_t)m * half + i], s = sin_t[(size_t)m * half + i];
                dst[2 * i] = fb_from_float<TO>(u * c - v * s);
                dst[2 * i + 1] = fb_from_float<TO>(v * c + u * s);
            } else {
                dst[half + i] = fb_from_float<TO>(in(half + i));
            }
        }
    }
}

// proj: float32 shares [n, >= max(Rq, kv_off + Rc + r)].  cq: [n, Rq] in the engine's dtype.  With `pool` the token's
// cache row is written as well ([pages][1][page size][Rc + r], engine dtype); without it only the query's latent.
FB_API int fb_mla_latents(const float* proj, long long proj_stride, int n_partials, long long partial_stride, int Rq,
                          const void* wq, void* cq, int kv_off, int Rc, int r, const void* wkv, int w_dtype, float eps,
                          const float* cos_t, const float* sin_t, int half, const int* positions, const int* row_seq,
                          const int* block_table, int table_stride, const int* table_base, void* pool, int out_dtype,
                          int page_size, int n_pages, int n, int* status, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && Rq > 0 && Rc > 0 && r >= 0 && half >= 0 && 2 * half <= r, "latent attention: bad sizes");
    FB_REQUIRE(eps > 0.0f, "latent attention: eps must be positive");
    FB_REQUIRE(half == 0 || (cos_t && sin_t), "latent attention: a rotation needs its tables");
    FB_REQUIRE(!pool || (block_table && positions && row_seq && wkv), "latent attention: a cache write needs the step's tables");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    const size_t smem = (size_t)(Rq > Rc ? Rq : Rc) * sizeof(float);
    FB_REQUIRE(smem <= 48 * 1024, "latent attention: a latent of more than 12288 numbers");
    FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, TO,
        (fb_launch((mla_latents_kernel<TW, TO>), dim3(n, pool ? 2 : 1), dim3(256), smem, stream, proj, (long)proj_stride,
                   n_partials, (long)partial_stride, Rq, (const TW*)wq, (TO*)cq, kv_off, Rc, r, (const TW*)wkv, eps,
                   cos_t, sin_t, half, positions, row_seq, block_table, table_stride, table_base, (TO*)pool, page_size,
                   n_pages, status))));
    return fb_check_launch("mla_latents");
}

// out[t*o_stride + h*o_head + c] = sum_k w[h][c][k] * a[t*a_stride + h*a_head + k]   (c < N, k < K)
FB_API int fb_head_linear(const void* a, int a_dtype, long long a_stride, long long a_head, int n_partials,
                          long long partial_stride, const void* w, int w_dtype, void* out, int out_dtype,
                          long long o_stride, long long o_head, const float* gate, long long gate_stride,
                          int gate_partials, long long gate_partial_stride, int gate_off, const float* cos_t,
                          const float* sin_t, int half, int r, int n, int H, int N, int K, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && H > 0 && N > 0 && K > 0 && r >= 0 && half >= 0 && 2 * half <= r, "head_linear: bad sizes");
    FB_REQUIRE(n_partials <= 1 || a_dtype == FB_F32, "head_linear: only float32 inputs come as shares");
    FB_REQUIRE(half == 0 || (cos_t && sin_t), "head_linear: a rotation needs its tables");
    FB_REQUIRE(H <= 65535 && (N + HL_TN - 1) / HL_TN <= 65535, "head_linear: too many heads or outputs");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    if (gate_partials < 1) gate_partials = 1;
    const dim3 grid((n + HL_TM - 1) / HL_TM, (N + HL_TN - 1) / HL_TN, H);
    FB_DISPATCH_DTYPE(a_dtype, TA, FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, TO,
        (fb_launch((head_linear_kernel<TA, TW, TO>), grid, dim3(256), 0, stream, (const TA*)a, (long)a_stride,
                   (long)a_head, n_partials, (long)partial_stride, (const TW*)w, (TO*)out, (long)o_stride, (long)o_head,
                   gate, (long)gate_stride, gate_partials, (long)gate_partial_stride, gate_off, cos_t, sin_t, half, r,
                   n, N, K)))));
    return fb_check_launch("head_linear");
}

// x[t, h, 0 .. 2 half) turned in place by the tables' angles, neighbours paired (float32 rows [n, heads * head_dim]).
__global__ void rope_neighbours_kernel(float* __restrict__ x, long stride, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int half, int heads, int head_dim, int n) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * heads * half) return;
    const int i = (int)(idx % half);
    const int h = (int)((idx / half) % heads);
    const int t = (int)(idx / ((size_t)half * heads));
    float* p = x + (size_t)t * stride + (size_t)h * head_dim + 2 * i;
    const float u = p[0], v = p[1], c = cos_t[(size_t)t * half + i], s = sin_t[(size_t)t * half + i];
    p[0] = u * c - v * s;
    p[1] = v * c + u * s;
}

FB_API int fb_rope_neighbours(float* x, long long stride, const float* cos_t, const float* sin_t, int half, int heads,
                              int head_dim, int n, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && heads > 0 && half >= 0 && 2 * half <= head_dim, "rope_neighbours: bad sizes");
    if (n == 0 || half == 0) return 0;
    const size_t total = (size_t)n * heads * half;
    fb_launch(rope_neighbours_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, (long)stride, cos_t,
              sin_t, half, heads, head_dim, n);
    return fb_check_launch("rope_neighbours");
}
