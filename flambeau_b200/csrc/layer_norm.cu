// A norm that takes the mean off first, with the residual add fused in front of it:
//   r = rows ? rows[j] : j
//   v = x[r] + sum_p delta[p][r]              (float32 slabs: a part's output, or the split-K shares of its last product)
//   if (!rows && delta) x[r] = v              (the stream is updated in place)
//   out[j] = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w          (no bias)
// Mean, deviations, their squares and the product with the weight are float32.  The row waits in shared memory
// between the passes: the variance is taken from the deviations, not from the mean of squares, so that a row whose
// mean is large against its spread keeps its digits.
#include "common.cuh"

template <typename TW, typename TO, bool VEC>
__global__ void __launch_bounds__(1024)
add_layernorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_partials, size_t partial_stride,
                     const TW* __restrict__ w, TO* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ __align__(16) float ln_row[];
    __shared__ float red[32];
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    float* xr = x + (size_t)r * H;
    float sum = 0.0f;
    if (VEC) {
        const int nvec = H >> 2;
        for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
            float4 v = *reinterpret_cast<const float4*>(xr + 4 * c);
            if (delta) {
                for (int p = 0; p < n_partials; ++p) {
                    const float4 d = *reinterpret_cast<const float4*>(delta + (size_t)p * partial_stride + (size_t)r * H + 4 * c);
                    v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                }
                if (!rows) *reinterpret_cast<float4*>(xr + 4 * c) = v;
            }
            *reinterpret_cast<float4*>(ln_row + 4 * c) = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = xr[c];
            if (delta) {
                for (int p = 0; p < n_partials; ++p) v += delta[(size_t)p * partial_stride + (size_t)r * H + c];
                if (!rows) xr[c] = v;
            }
            ln_row[c] = v;
            sum += v;
        }
    }
    // (every thread reads back only what it wrote itself, so the row needs no barrier of its own)
    const float mean = fb_block_sum(sum, red) / (float)H;
    float sq = 0.0f;
    if (VEC) {
        for (int c = threadIdx.x; c < (H >> 2); c += blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(ln_row + 4 * c);
            const float a = v.x - mean, b = v.y - mean, d = v.z - mean, e = v.w - mean;
            sq += (a * a + b * b) + (d * d + e * e);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) { const float a = ln_row[c] - mean; sq = fmaf(a, a, sq); }
    }
    const float inv = 1.0f / sqrtf(fb_block_sum(sq, red) / (float)H + eps);
    TO* o = out + (size_t)j * H;
    const int step = VEC ? 4 : 1;
    for (int c = threadIdx.x * step; c < H; c += blockDim.x * step) {
#pragma unroll
        for (int u = 0; u < step; ++u)
            o[c + u] = fb_from_float<TO>((ln_row[c + u] - mean) * inv * fb_to_float(w[c + u]));
    }
}

FB_API int fb_add_layernorm(float* x, const float* delta, int n_partials, long long partial_stride, const void* w,
                            int w_dtype, void* out, int out_dtype, const int* rows, int n_out, int H, float eps,
                            cudaStream_t stream) {
    FB_REQUIRE(n_out >= 0 && H > 0, "add_layernorm: bad sizes n=%d H=%d", n_out, H);
    FB_REQUIRE(eps > 0.0f, "add_layernorm: eps must be positive");
    if (n_out == 0) return 0;
    if (!delta) n_partials = 0;
    const size_t smem = (size_t)H * sizeof(float);
    FB_REQUIRE(smem <= 200 * 1024, "add_layernorm: width %d does not fit in shared memory", H);
    const bool vec = H % 4 == 0 && ((uintptr_t)x % 16 == 0) &&
                     (!delta || ((uintptr_t)delta % 16 == 0 && partial_stride % 4 == 0));
    const int per = vec ? H / 4 : H;
    const int threads = per >= 1024 ? 1024 : ((per + 31) / 32) * 32;
    FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, TO, {
        if (vec) {
            auto kernel = add_layernorm_kernel<TW, TO, true>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            fb_launch(kernel, dim3(n_out), dim3(threads), smem, stream, x, delta, n_partials, (size_t)partial_stride,
                      (const TW*)w, (TO*)out, rows, H, eps);
        } else {
            auto kernel = add_layernorm_kernel<TW, TO, false>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            fb_launch(kernel, dim3(n_out), dim3(threads), smem, stream, x, delta, n_partials, (size_t)partial_stride,
                      (const TW*)w, (TO*)out, rows, H, eps);
        }
    }));
    return fb_check_launch("add_layernorm");
}

// ---------------------------------------------------------------------------
// A weighted mean over depth.  A model keeps what every layer so far has produced (slot 0: the embedding output) and
// hands on a learned mix of all of them:
//   v = x + sum_p delta[p]                    (the running layer's result: the stream plus what is still pending)
//   hist[count - 1] = v
//   x = sum_{j < count} w[j] * hist[j]
// `hist` is [slots][n * H] float32, `hist_stride` elements apart.  Elementwise, float32.
// ---------------------------------------------------------------------------
template <typename TW, int V>
__global__ void depth_average_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_partials,
                                     size_t partial_stride, float* __restrict__ hist, size_t hist_stride, int count,
                                     const TW* __restrict__ w, size_t groups) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    struct alignas(4 * V) Group { float f[V]; };
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    Group v = reinterpret_cast<const Group*>(x)[i];
    for (int p = 0; p < n_partials; ++p) {
        const Group d = *reinterpret_cast<const Group*>(delta + (size_t)p * partial_stride + V * i);
#pragma unroll
        for (int u = 0; u < V; ++u) v.f[u] += d.f[u];
    }
    *reinterpret_cast<Group*>(hist + (size_t)(count - 1) * hist_stride + V * i) = v;
    const float wl = fb_to_float(w[count - 1]);
    Group acc;
#pragma unroll
    for (int u = 0; u < V; ++u) acc.f[u] = wl * v.f[u];
    for (int j = 0; j < count - 1; ++j) {
        const Group h = *reinterpret_cast<const Group*>(hist + (size_t)j * hist_stride + V * i);
        const float wj = fb_to_float(w[j]);
#pragma unroll
        for (int u = 0; u < V; ++u) acc.f[u] = fmaf(wj, h.f[u], acc.f[u]);
    }
    reinterpret_cast<Group*>(x)[i] = acc;
}

FB_API int fb_depth_average(float* x, const float* delta, int n_partials, long long partial_stride, float* hist,
                            long long hist_stride, int count, const void* w, int w_dtype, long long total,
                            cudaStream_t stream) {
    FB_REQUIRE(total >= 0 && count >= 1 && hist && w, "depth_average: bad arguments");
    if (total == 0) return 0;
    if (!delta) n_partials = 0;
    const bool vec = total % 4 == 0 && hist_stride % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)hist % 16 == 0 &&
                     (!delta || ((uintptr_t)delta % 16 == 0 && partial_stride % 4 == 0));
    const size_t groups = vec ? (size_t)total / 4 : (size_t)total;
    const dim3 grid((unsigned)((groups + 255) / 256));
    FB_DISPATCH_DTYPE(w_dtype, TW, {
        if (vec)
            fb_launch((depth_average_kernel<TW, 4>), grid, dim3(256), 0, stream, x, delta, n_partials,
                      (size_t)partial_stride, hist, (size_t)hist_stride, count, (const TW*)w, groups);
        else
            fb_launch((depth_average_kernel<TW, 1>), grid, dim3(256), 0, stream, x, delta, n_partials,
                      (size_t)partial_stride, hist, (size_t)hist_stride, count, (const TW*)w, groups);
    });
    return fb_check_launch("depth_average");
}
