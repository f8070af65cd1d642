// Several residual streams (hyper-connections): a sublayer reads a learned mix of S copies of the stream and writes
// its output back into all of them through learned weights.
//
// With streams x_1 .. x_S (float32 [S][n][D]), the output y of the sublayer before (float32, possibly split-K shares)
// and that sublayer's weights mix [S, S] (indexed [from, to]) and out [S]:
//
//     x_t  <-  sum_s mix[s, t] x_s  +  out[t] y          (every new stream from the old ones)
//     u     =  sum_t in[t] x_t                            (what the next sublayer reads; in = nullptr: all ones)
//     h     =  u / sqrt(mean(u^2) + eps) * (w + offset)   (or u itself, float32, where no norm weight is given)
//
// hc_step does all of it in one pass over a row: the write of the sublayer before, the read of the next one and its
// RMS norm.  Everything is float32; only h is rounded to the engine's type.  Without y the streams stay as they are
// (the first sublayer of a step).  With `rows` only those rows are formed and nothing is written back (the rows whose
// logits are wanted, at the end of a step).
#include "common.cuh"

constexpr int HC_MAX_STREAMS = 8;

// SMAX: the most copies this instance holds in registers (2, 4 or 8), so that a row of few copies does not pay for eight.
template <typename TW, typename TO, int VEC, int SMAX>
__global__ void __launch_bounds__(256)
hc_step_kernel(float* __restrict__ xs, long stream_stride, int S, const float* __restrict__ y, int n_partials,
               long partial_stride, const float* __restrict__ mix, const float* __restrict__ out_w,
               const float* __restrict__ in_w, const TW* __restrict__ norm_w, float eps, float w_offset,
               TO* __restrict__ out, const int* __restrict__ rows, int write_back, int D) {
    fb_pdl_launch_dependents();
    extern __shared__ float hc_u[];                    // [D] the row that the norm reads
    __shared__ float red[32];
    __shared__ float c_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], c_out[HC_MAX_STREAMS], c_in[HC_MAX_STREAMS];
    const int tid = threadIdx.x;
    // (the sublayers' weights do not depend on the kernel before this one)
    for (int i = tid; i < S * S; i += blockDim.x) c_mix[i] = (y && mix) ? mix[i] : ((i / S == i % S) ? 1.0f : 0.0f);
    for (int i = tid; i < S; i += blockDim.x) {
        c_out[i] = (y && out_w) ? out_w[i] : 0.0f;
        c_in[i] = in_w ? in_w[i] : 1.0f;
    }
    __syncthreads();
    fb_pdl_wait();
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    float* xr = xs + (size_t)r * D;
    const float* yr = y ? y + (size_t)r * D : nullptr;
    float ss = 0.0f;
    for (int c = tid * VEC; c < D; c += blockDim.x * VEC) {
        float xv[SMAX][VEC], yv[VEC], u[VEC];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) {
            if (s >= S) break;
            if constexpr (VEC == 4) {
                const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)s * stream_stride + c);
                xv[s][0] = v.x; xv[s][1] = v.y; xv[s][2] = v.z; xv[s][3] = v.w;
            } else {
                xv[s][0] = xr[(size_t)s * stream_stride + c];
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) { yv[e] = 0.0f; u[e] = 0.0f; }
        if (yr) {
            for (int p = 0; p < n_partials; ++p) {
                if constexpr (VEC == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(yr + (size_t)p * partial_stride + c);
                    yv[0] += v.x; yv[1] += v.y; yv[2] += v.z; yv[3] += v.w;
                } else {
                    yv[0] += yr[(size_t)p * partial_stride + c];
                }
            }
        }
#pragma unroll
        for (int t = 0; t < SMAX; ++t) {
            if (t >= S) break;
            float nv[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) nv[e] = c_out[t] * yv[e];
#pragma unroll
            for (int s = 0; s < SMAX; ++s) {
                if (s >= S) break;
                const float m = c_mix[s * S + t];
#pragma unroll
                for (int e = 0; e < VEC; ++e) nv[e] = fmaf(m, xv[s][e], nv[e]);
            }
            if (yr && write_back) {
                if constexpr (VEC == 4) *reinterpret_cast<float4*>(xr + (size_t)t * stream_stride + c) = make_float4(nv[0], nv[1], nv[2], nv[3]);
                else xr[(size_t)t * stream_stride + c] = nv[0];
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) u[e] = fmaf(c_in[t], nv[e], u[e]);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            hc_u[c + e] = u[e];
            ss = fmaf(u[e], u[e], ss);
        }
    }
    if (!out) return;
    TO* dst = out + (size_t)j * D;
    if (!norm_w) {                                     // (uniform) the read alone: float32 rows
        __syncthreads();
        for (int c = tid; c < D; c += blockDim.x) dst[c] = fb_from_float<TO>(hc_u[c]);
        return;
    }
    const float inv = 1.0f / sqrtf(fb_block_sum(ss, red) / (float)D + eps);
    for (int c = tid; c < D; c += blockDim.x)
        dst[c] = fb_from_float<TO>(hc_u[c] * inv * (fb_to_float(norm_w[c]) + w_offset));
}

// xs: float32 [S][n][D], streams `stream_stride` elements apart.  y: float32 [n, D], the first of n_partials slabs
// `partial_stride` apart, or nullptr (nothing to write).  mix [S*S] ([from][to]), out_w [S]: float32, the weights of the
// sublayer that produced y.  in_w [S] float32 or nullptr (ones).  norm_w [D] (dtype w_dtype) or nullptr: then `out`
// receives u itself.  out: [n_out, D] of out_dtype, or nullptr (only the write).  rows: int32 [n_out] or nullptr (row j
// is row j).  write_back: the new streams replace the old ones (must be 0 with `rows`).
FB_API int fb_hc_step(float* xs, long long stream_stride, int S, const float* y, int n_partials, long long partial_stride,
                      const float* mix, const float* out_w, const float* in_w, const void* norm_w, int w_dtype,
                      float eps, float w_offset, void* out, int out_dtype, const int* rows, int write_back, int n_out,
                      int D, cudaStream_t stream) {
    FB_REQUIRE(S >= 1 && S <= HC_MAX_STREAMS, "hyper-connections: %d streams (1 to %d)", S, HC_MAX_STREAMS);
    FB_REQUIRE(n_out >= 0 && D > 0, "hyper-connections: bad sizes");
    FB_REQUIRE(!y || (mix && out_w), "hyper-connections: an output to write needs the weights of its sublayer");
    FB_REQUIRE(!(rows && write_back), "hyper-connections: chosen rows are read, not written back");
    FB_REQUIRE(out || (y && write_back), "hyper-connections: nothing to do");
    FB_REQUIRE(!norm_w || eps > 0.0f, "hyper-connections: eps must be positive");
    if (n_out == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    const size_t smem = (size_t)D * sizeof(float);
    FB_REQUIRE(smem <= 48 * 1024, "hyper-connections: rows of more than 12288 numbers");
    if (!norm_w) w_dtype = FB_F32;
    if (!out) out_dtype = FB_F32;
    const bool vec = D % 4 == 0 && stream_stride % 4 == 0 && partial_stride % 4 == 0 && ((uintptr_t)xs & 15) == 0 &&
                     (!y || ((uintptr_t)y & 15) == 0);
    const int per = vec ? 4 : 1;
    int threads = ((D / per + 31) / 32) * 32;
    threads = threads < 32 ? 32 : threads > 256 ? 256 : threads;
#define HC_LAUNCH(V, M)                                                                                                \
    FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, TO,                                                    \
        (fb_launch((hc_step_kernel<TW, TO, V, M>), dim3(n_out), dim3(threads), smem, stream, xs, (long)stream_stride,  \
                   S, y, n_partials, (long)partial_stride, mix, out_w, in_w, (const TW*)norm_w, eps, w_offset,         \
                   (TO*)out, rows, write_back, D))))
    if (vec) {
        if (S <= 2) HC_LAUNCH(4, 2); else if (S <= 4) HC_LAUNCH(4, 4); else HC_LAUNCH(4, 8);
    } else {
        HC_LAUNCH(1, 8);
    }
#undef HC_LAUNCH
    return fb_check_launch("hc_step");
}
