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
// Rotation turns pair i < half of the rotated part, (u, v) -> (u cos - v sin, v cos + u sin), with per-token tables;
// `pairing` says which dimensions form pair i: 0 neighbours (2i, 2i + 1), 1 halves (i, i + half).  Dimensions from
// 2 half on pass unchanged.
#include "common.cuh"
#include "attention_common.cuh"

__device__ __forceinline__ float mla_slab_sum(const float* row, int c, int n_partials, long partial_stride) {
    return fb_slab_sum(row, c, n_partials, partial_stride);
}
// The two dimensions of pair i of a rotated vector with `half` pairs.
__device__ __forceinline__ int rot_first(int pairing, int i) { return pairing ? i : 2 * i; }
__device__ __forceinline__ int rot_second(int pairing, int i, int half) { return pairing ? i + half : 2 * i + 1; }

template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
mla_latents_kernel(const float* __restrict__ proj, long proj_stride, int n_partials, long partial_stride, int Rq,
                   const TW* __restrict__ wq, TO* __restrict__ cq, int kv_off, int Rc, int r,
                   const TW* __restrict__ wkv, float eps, const float* __restrict__ cos_t,
                   const float* __restrict__ sin_t, int half, int pairing, const int* __restrict__ positions,
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
            const int iu = rot_first(pairing, i), iv = rot_second(pairing, i, half);
            const float u = mla_slab_sum(kr, iu, n_partials, partial_stride);
            const float v = mla_slab_sum(kr, iv, n_partials, partial_stride);
            const float c = cos_t[(size_t)t * half + i], s = sin_t[(size_t)t * half + i];
            dst[Rc + iu] = fb_from_float<TO>(u * c - v * s);
            dst[Rc + iv] = fb_from_float<TO>(v * c + u * s);
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
                   int pairing, int n, int N, int K) {
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
                const int iu = rot_first(pairing, i), iv = rot_second(pairing, i, half);
                const float u = in(iu), v = in(iv);
                const float c = cos_t[(size_t)m * half + i], s = sin_t[(size_t)m * half + i];
                dst[iu] = fb_from_float<TO>(u * c - v * s);
                dst[iv] = fb_from_float<TO>(v * c + u * s);
            } else {
                dst[half + i] = fb_from_float<TO>(in(half + i));
            }
        }
    }
}

// The same map on the tensor cores, for bfloat16 weights and outputs: a CTA of four warps takes 64 tokens x 64
// outputs of one head, every warp 16 tokens (mma.sync m16n8k16, float32 accumulation).  Inputs that come as float32
// shares are added in float32 and rounded once to bfloat16 on their way into shared memory.  Rows of both tiles lie
// 72 numbers apart, so that the eight rows a fragment load touches fall into different banks.
constexpr int HM_TM = 64, HM_TN = 64, HM_KC = 64, HM_LD = HM_KC + 8;

template <typename TA>
__global__ void __launch_bounds__(128, 4)
head_linear_mma_kernel(const TA* __restrict__ a, long a_stride, long a_head, int n_partials, long partial_stride,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long o_stride, long o_head,
                       const float* __restrict__ gate, long gate_stride, int gate_partials, long gate_partial_stride,
                       int gate_off, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int half, int r,
                       int pairing, int n, int N, int K, int a_vec, int w_vec) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    __shared__ __align__(16) __nv_bfloat16 As[HM_TM][HM_LD];
    __shared__ __align__(16) __nv_bfloat16 Ws[HM_TN][HM_LD];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.x * HM_TM, n0 = blockIdx.y * HM_TN, h = blockIdx.z;
    const TA* ah = a + (size_t)h * a_head;
    const __nv_bfloat16* wh = w + (size_t)h * N * K;
    float acc[HM_TN / 8][4];
#pragma unroll
    for (int j = 0; j < HM_TN / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += HM_KC) {
        // Both tiles' loads are issued before anything is stored, so that a thread has all of them in flight at once.
        constexpr int PER = 16 / sizeof(TA);           // numbers in 16 bytes
        constexpr int A_GROUPS = HM_TM * (HM_KC / PER) / 128, W_GROUPS = HM_TN * (HM_KC / 8) / 128;
        uint4 wraw[W_GROUPS];
        if (w_vec) {
#pragma unroll
            for (int u = 0; u < W_GROUPS; ++u) {
                const int idx = tid + 128 * u, nn = idx / (HM_KC / 8), k = (idx - nn * (HM_KC / 8)) * 8;
                wraw[u] = make_uint4(0u, 0u, 0u, 0u);
                if (n0 + nn < N && k0 + k < K) wraw[u] = *reinterpret_cast<const uint4*>(wh + (size_t)(n0 + nn) * K + k0 + k);
            }
        }
        if (a_vec) {                                   // (uniform) rows and heads start on 16-byte borders, K % 8 == 0
            float v[A_GROUPS][PER];
            if (n_partials == 1) {
                uint4 raw[A_GROUPS];
#pragma unroll
                for (int u = 0; u < A_GROUPS; ++u) {
                    const int idx = tid + 128 * u, m = idx / (HM_KC / PER), k = (idx - m * (HM_KC / PER)) * PER;
                    raw[u] = make_uint4(0u, 0u, 0u, 0u);       // (all bits clear is zero in both types)
                    if (m0 + m < n && k0 + k < K)
                        raw[u] = *reinterpret_cast<const uint4*>(ah + (size_t)(m0 + m) * a_stride + k0 + k);
                }
#pragma unroll
                for (int u = 0; u < A_GROUPS; ++u) {
                    const TA* x = reinterpret_cast<const TA*>(&raw[u]);
#pragma unroll
                    for (int e = 0; e < PER; ++e) v[u][e] = fb_to_float(x[e]);
                }
            } else {
                // shares (few rows as a rule): per group up to eight shares in flight, added in their order
#pragma unroll
                for (int u = 0; u < A_GROUPS; ++u) {
                    const int idx = tid + 128 * u, m = idx / (HM_KC / PER), k = (idx - m * (HM_KC / PER)) * PER;
#pragma unroll
                    for (int e = 0; e < PER; ++e) v[u][e] = 0.0f;
                    if (m0 + m >= n || k0 + k >= K) continue;
                    const TA* p = ah + (size_t)(m0 + m) * a_stride + k0 + k;
                    for (int q0 = 0; q0 < n_partials; q0 += 8) {
                        uint4 raw[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            raw[q] = q0 + q < n_partials ? *reinterpret_cast<const uint4*>(p + (size_t)(q0 + q) * partial_stride)
                                                         : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const TA* x = reinterpret_cast<const TA*>(&raw[q]);
                            if (q0 + q < n_partials) {
#pragma unroll
                                for (int e = 0; e < PER; ++e) v[u][e] += fb_to_float(x[e]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < A_GROUPS; ++u) {
                const int idx = tid + 128 * u, m = idx / (HM_KC / PER), k = (idx - m * (HM_KC / PER)) * PER;
#pragma unroll
                for (int e = 0; e < PER; e += 2)
                    *reinterpret_cast<uint32_t*>(&As[m][k + e]) = fb_attn::pack_bf16(v[u][e], v[u][e + 1]);
            }
        } else {
            for (int idx = tid; idx < HM_TM * HM_KC; idx += 128) {
                const int m = idx / HM_KC, k = idx - m * HM_KC;
                float v = 0.0f;
                if (m0 + m < n && k0 + k < K) {
                    const TA* p = ah + (size_t)(m0 + m) * a_stride + k0 + k;
                    v = fb_to_float(p[0]);
                    for (int q = 1; q < n_partials; ++q) v += fb_to_float(p[(size_t)q * partial_stride]);
                }
                As[m][k] = __float2bfloat16(v);
            }
        }
        // the head's weights
        if (w_vec) {
#pragma unroll
            for (int u = 0; u < W_GROUPS; ++u) {
                const int idx = tid + 128 * u, nn = idx / (HM_KC / 8), k = (idx - nn * (HM_KC / 8)) * 8;
                *reinterpret_cast<uint4*>(&Ws[nn][k]) = wraw[u];
            }
        } else {
            for (int idx = tid; idx < HM_TN * HM_KC; idx += 128) {
                const int nn = idx / HM_KC, k = idx - nn * HM_KC;
                Ws[nn][k] = (n0 + nn < N && k0 + k < K) ? wh[(size_t)(n0 + nn) * K + k0 + k] : __float2bfloat16(0.0f);
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HM_KC; kk += 16) {
            uint32_t af[4];
            af[0] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g][kk + 2 * t]);
            af[1] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g + 8][kk + 2 * t]);
            af[2] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g][kk + 8 + 2 * t]);
            af[3] = *reinterpret_cast<const uint32_t*>(&As[warp * 16 + g + 8][kk + 8 + 2 * t]);
#pragma unroll
            for (int j = 0; j < HM_TN / 8; ++j) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&Ws[j * 8 + g][kk + 2 * t]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&Ws[j * 8 + g][kk + 8 + 2 * t]);
                fb_attn::mma_bf16(acc[j], af, b0, b1);
            }
        }
        __syncthreads();
    }
    // An accumulator pair (two neighbouring outputs of a row) leaves as one 4-byte store, and its gates arrive as
    // 8-byte loads, where the rows' and heads' places allow it.
    const bool pairs = ((o_stride | o_head | N) & 1) == 0 && ((uintptr_t)out & 3) == 0;
    const bool gate_pairs = gate && ((gate_stride | gate_partial_stride | gate_off | N) & 1) == 0 && ((uintptr_t)gate & 7) == 0;
#pragma unroll
    for (int j = 0; j < HM_TN / 8; ++j)
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            const int m = m0 + warp * 16 + g + hi * 8, c = n0 + j * 8 + 2 * t;
            if (m >= n || c >= N) continue;
            float v0 = acc[j][2 * hi], v1 = acc[j][2 * hi + 1];
            const bool both = c + 1 < N;
            if (gate) {
                float g0, g1 = 0.0f;
                const float* gr = gate + (size_t)m * gate_stride;
                const int gc = gate_off + h * N + c;
                if (gate_pairs && both) {
                    float2 sum = *reinterpret_cast<const float2*>(gr + gc);
                    for (int q = 1; q < gate_partials; ++q) {
                        const float2 more = *reinterpret_cast<const float2*>(gr + (size_t)q * gate_partial_stride + gc);
                        sum.x += more.x; sum.y += more.y;
                    }
                    g0 = sum.x; g1 = sum.y;
                } else {
                    g0 = mla_slab_sum(gr, gc, gate_partials, gate_partial_stride);
                    if (both) g1 = mla_slab_sum(gr, gc + 1, gate_partials, gate_partial_stride);
                }
                v0 = v0 / (1.0f + expf(-g0));
                v1 = v1 / (1.0f + expf(-g1));
            }
            __nv_bfloat16* dst = out + (size_t)m * o_stride + (size_t)h * o_head + c;
            if (pairs && both) {
                *reinterpret_cast<uint32_t*>(dst) = fb_attn::pack_bf16(v0, v1);
            } else {
                dst[0] = __float2bfloat16(v0);
                if (both) dst[1] = __float2bfloat16(v1);
            }
        }
    if (r > 0 && blockIdx.y == 0) {
        // the rotated tail: columns K .. K+r of the input row go, turned, to columns N .. N+r of the output row
        const int per = r - half;
        for (int e = tid; e < HM_TM * per; e += 128) {
            const int mm = e / per, i = e - mm * per, m = m0 + mm;
            if (m >= n) break;
            const TA* src = ah + (size_t)m * a_stride + K;
            __nv_bfloat16* dst = out + (size_t)m * o_stride + (size_t)h * o_head + N;
            auto in = [&](int c) {
                float v = fb_to_float(src[c]);
                for (int q = 1; q < n_partials; ++q) v += fb_to_float(src[(size_t)q * partial_stride + c]);
                return v;
            };
            if (i < half) {
                const int iu = rot_first(pairing, i), iv = rot_second(pairing, i, half);
                const float u = in(iu), v = in(iv);
                const float c = cos_t[(size_t)m * half + i], s = sin_t[(size_t)m * half + i];
                dst[iu] = __float2bfloat16(u * c - v * s);
                dst[iv] = __float2bfloat16(v * c + u * s);
            } else {
                dst[half + i] = __float2bfloat16(in(half + i));
            }
        }
    }
}

// proj: float32 shares [n, >= max(Rq, kv_off + Rc + r)].  cq: [n, Rq] in the engine's dtype.  With `pool` the token's
// cache row is written as well ([pages][1][page size][Rc + r], engine dtype); without it only the query's latent.
FB_API int fb_mla_latents(const float* proj, long long proj_stride, int n_partials, long long partial_stride, int Rq,
                          const void* wq, void* cq, int kv_off, int Rc, int r, const void* wkv, int w_dtype, float eps,
                          const float* cos_t, const float* sin_t, int half, int pairing, const int* positions,
                          const int* row_seq, const int* block_table, int table_stride, const int* table_base, void* pool, int out_dtype,
                          int page_size, int n_pages, int n, int* status, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && Rq > 0 && Rc > 0 && r >= 0 && half >= 0 && 2 * half <= r, "latent attention: bad sizes");
    FB_REQUIRE(eps > 0.0f, "latent attention: eps must be positive");
    FB_REQUIRE(half == 0 || (cos_t && sin_t), "latent attention: a rotation needs its tables");
    FB_REQUIRE(pairing == 0 || pairing == 1, "latent attention: pairs are neighbours (0) or halves (1)");
    FB_REQUIRE(!pool || (block_table && positions && row_seq && wkv), "latent attention: a cache write needs the step's tables");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    const size_t smem = (size_t)(Rq > Rc ? Rq : Rc) * sizeof(float);
    FB_REQUIRE(smem <= 48 * 1024, "latent attention: a latent of more than 12288 numbers");
    FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, TO,
        (fb_launch((mla_latents_kernel<TW, TO>), dim3(n, pool ? 2 : 1), dim3(256), smem, stream, proj, (long)proj_stride,
                   n_partials, (long)partial_stride, Rq, (const TW*)wq, (TO*)cq, kv_off, Rc, r, (const TW*)wkv, eps,
                   cos_t, sin_t, half, pairing, positions, row_seq, block_table, table_stride, table_base, (TO*)pool, page_size,
                   n_pages, status))));
    return fb_check_launch("mla_latents");
}

// out[t*o_stride + h*o_head + c] = sum_k w[h][c][k] * a[t*a_stride + h*a_head + k]   (c < N, k < K)
FB_API int fb_head_linear(const void* a, int a_dtype, long long a_stride, long long a_head, int n_partials,
                          long long partial_stride, const void* w, int w_dtype, void* out, int out_dtype,
                          long long o_stride, long long o_head, const float* gate, long long gate_stride,
                          int gate_partials, long long gate_partial_stride, int gate_off, const float* cos_t,
                          const float* sin_t, int half, int r, int pairing, int n, int H, int N, int K, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && H > 0 && N > 0 && K > 0 && r >= 0 && half >= 0 && 2 * half <= r, "head_linear: bad sizes");
    FB_REQUIRE(n_partials <= 1 || a_dtype == FB_F32, "head_linear: only float32 inputs come as shares");
    FB_REQUIRE(half == 0 || (cos_t && sin_t), "head_linear: a rotation needs its tables");
    FB_REQUIRE(pairing == 0 || pairing == 1, "head_linear: pairs are neighbours (0) or halves (1)");
    FB_REQUIRE(H <= 65535 && (N + HL_TN - 1) / HL_TN <= 65535, "head_linear: too many heads or outputs");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    if (gate_partials < 1) gate_partials = 1;
    if (w_dtype == FB_BF16 && out_dtype == FB_BF16) {
        // 16-byte loads where every row, head and share starts on such a border
        const int per = a_dtype == FB_F32 ? 4 : 8;
        const int a_vec = K % 8 == 0 && a_stride % per == 0 && a_head % per == 0 && partial_stride % per == 0 &&
                          (uintptr_t)a % 16 == 0;
        const int w_vec = K % 8 == 0 && (uintptr_t)w % 16 == 0;
        const dim3 tiles((n + HM_TM - 1) / HM_TM, (N + HM_TN - 1) / HM_TN, H);
        FB_DISPATCH_DTYPE(a_dtype, TA,
            (fb_launch((head_linear_mma_kernel<TA>), tiles, dim3(128), 0, stream, (const TA*)a, (long)a_stride,
                       (long)a_head, n_partials, (long)partial_stride, (const __nv_bfloat16*)w, (__nv_bfloat16*)out,
                       (long)o_stride, (long)o_head, gate, (long)gate_stride, gate_partials, (long)gate_partial_stride,
                       gate_off, cos_t, sin_t, half, r, pairing, n, N, K, a_vec, w_vec)));
        return fb_check_launch("head_linear");
    }
    const dim3 grid((n + HL_TM - 1) / HL_TM, (N + HL_TN - 1) / HL_TN, H);
    FB_DISPATCH_DTYPE(a_dtype, TA, FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, TO,
        (fb_launch((head_linear_kernel<TA, TW, TO>), grid, dim3(256), 0, stream, (const TA*)a, (long)a_stride,
                   (long)a_head, n_partials, (long)partial_stride, (const TW*)w, (TO*)out, (long)o_stride, (long)o_head,
                   gate, (long)gate_stride, gate_partials, (long)gate_partial_stride, gate_off, cos_t, sin_t, half, r,
                   pairing, n, N, K)))));
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
