// What lies between a fused q/k/v projection and the attention when queries and keys pass an RMS norm on the way:
// add the projection's split-K shares, normalise q and k, rotate them, round q once, and put k and v into their
// cache pages.  One CTA per token; the row's q and k live in shared memory between the two passes.
//
// The norm's reach is an argument: over every head alone (FB_QK_NORM_HEAD: width = head size, one weight of
// that size shared by the heads) or over the whole projection at once (FB_QK_NORM_PROJECTION: width = heads * head
// size, a weight of that size), before the rotation in both cases.  The weight enters as (w + weight_offset).
// Rotation: the first 2 * half dimensions of a head, dimension i paired with i + half, angles from the step's
// cos/sin tables [n, half]; the rest of the head passes unchanged.  Value rows have a width of their own.
#include "common.cuh"

enum FbQkNorm : int { FB_QK_NORM_NONE = 0, FB_QK_NORM_HEAD = 1, FB_QK_NORM_PROJECTION = 2 };

__device__ __forceinline__ float qkr_slab_sum(const float* row, int c, int n_partials, long partial_stride) {
    float v = row[c];
    for (int p = 1; p < n_partials; ++p) v += row[(size_t)p * partial_stride + c];
    return v;
}

template <typename TW, typename T>
__global__ void __launch_bounds__(1024)
qk_norm_rope_kv_write_kernel(const float* __restrict__ proj, long proj_stride, int n_partials, long partial_stride,
                             const TW* __restrict__ q_weight, const TW* __restrict__ k_weight, int scope, float eps,
                             float weight_offset, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                             int half, T* __restrict__ q_out, long q_out_stride, const int* __restrict__ positions,
                             const int* __restrict__ row_seq, const int* __restrict__ block_table, int table_stride,
                             const int* __restrict__ table_base, int table_head, T* __restrict__ k_pool,
                             T* __restrict__ v_pool, int page_size, int n_pages, int nh, int nkv, int hd, int vd,
                             int write_kv, int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ float sh[];                      // [qw + kw] the row's q and k; then one factor per head
    __shared__ float red[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const int qw = nh * hd, kw = nkv * hd, vw = nkv * vd;
    const int heads = nh + nkv;
    float* inv = sh + qw + kw;                         // [heads]
    const float* pr = proj + (size_t)row * proj_stride;
    for (int c = tid; c < qw + kw; c += blockDim.x) sh[c] = qkr_slab_sum(pr, c, n_partials, partial_stride);
    __syncthreads();
    if (scope == FB_QK_NORM_PROJECTION) {
        float sq = 0.0f, sk = 0.0f;
        for (int c = tid; c < qw; c += blockDim.x) sq = fmaf(sh[c], sh[c], sq);
        for (int c = tid; c < kw; c += blockDim.x) sk = fmaf(sh[qw + c], sh[qw + c], sk);
        sq = fb_block_sum(sq, red);
        sk = fb_block_sum(sk, red);
        const float iq = 1.0f / sqrtf(sq / (float)qw + eps), ik = 1.0f / sqrtf(sk / (float)kw + eps);
        for (int h = tid; h < heads; h += blockDim.x) inv[h] = h < nh ? iq : ik;
    } else if (scope == FB_QK_NORM_HEAD) {
        const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
        for (int h = warp; h < heads; h += nwarps) {
            const float* x = sh + (size_t)h * hd;
            float s = 0.0f;
            for (int d = lane; d < hd; d += 32) s = fmaf(x[d], x[d], s);
            s = fb_warp_sum(s);
            if (lane == 0) inv[h] = 1.0f / sqrtf(s / (float)hd + eps);
        }
    } else {
        for (int h = tid; h < heads; h += blockDim.x) inv[h] = 1.0f;
    }
    __syncthreads();

    // where this token's key and value rows go
    T* k_dst = nullptr;
    T* v_dst = nullptr;
    if (write_kv) {
        const int p = positions[row], seq = row_seq[row];
        const int entry = fb_table_column(p / page_size, table_base ? table_base[seq] : 0, table_head);
        const int page = (entry >= 0 && entry < table_stride) ? block_table[(size_t)seq * table_stride + entry] : -1;
        if (page < 0 || page >= n_pages) {
            if (tid == 0) atomicOr(status, FB_STATUS_BAD_PAGE);
        } else {
            // pools are [page][kv head][slot][row]: head g's row of this token
            k_dst = k_pool + ((size_t)page * nkv * page_size + (p % page_size)) * hd;
            v_dst = v_pool + ((size_t)page * nkv * page_size + (p % page_size)) * vd;
        }
    }
    const float* cs = half ? cos_t + (size_t)row * half : nullptr;
    const float* sn = half ? sin_t + (size_t)row * half : nullptr;
    const int n_items = write_kv ? heads * hd : qw;
    for (int e = tid; e < n_items; e += blockDim.x) {
        const int h = e / hd, d = e - h * hd;
        const bool is_q = h < nh;
        const TW* w = is_q ? q_weight : k_weight;
        // the weight's index: within the whole projection, or within the head
        const int wbase = scope == FB_QK_NORM_PROJECTION ? (is_q ? h : h - nh) * hd : 0;
        const float f = inv[h];
        auto val = [&](int dd) -> float {
            const float x = sh[(size_t)h * hd + dd] * f;
            return (w && scope != FB_QK_NORM_NONE) ? x * (fb_to_float(w[wbase + dd]) + weight_offset) : x;
        };
        float y;
        if (d < half) {
            y = val(d) * cs[d] - val(d + half) * sn[d];
        } else if (d < 2 * half) {
            y = val(d) * cs[d - half] + val(d - half) * sn[d - half];
        } else {
            y = val(d);
        }
        if (is_q) {
            q_out[(size_t)row * q_out_stride + e] = fb_from_float<T>(y);
        } else if (k_dst) {
            k_dst[(size_t)(h - nh) * page_size * hd + d] = fb_from_float<T>(y);
        }
    }
    if (v_dst) {
        for (int e = tid; e < vw; e += blockDim.x) {
            const int g = e / vd, d = e - g * vd;
            v_dst[(size_t)g * page_size * vd + d] =
                fb_from_float<T>(qkr_slab_sum(pr, qw + kw + e, n_partials, partial_stride));
        }
    }
}

// proj: float32 rows [q: nh*hd | k: nkv*hd | v: nkv*vd], possibly as n_partials shares partial_stride elements apart.
// q_weight / k_weight (dtype w_dtype): [hd] each for FB_QK_NORM_HEAD, [nh*hd] and [nkv*hd] for FB_QK_NORM_PROJECTION.
FB_API int fb_qk_norm_rope_kv_write(const float* proj, long long proj_stride, int n_partials, long long partial_stride,
                                    const void* q_weight, const void* k_weight, int w_dtype, int scope, float eps,
                                    float weight_offset, const float* cos_t, const float* sin_t, int half, void* q_out,
                                    long long q_out_stride, int out_dtype, const int* positions, const int* row_seq,
                                    const int* block_table, int table_stride, const int* table_base, int table_head,
                                    void* k_pool, void* v_pool, int page_size, int n_pages, int n, int nh, int nkv, int hd, int vd,
                                    int write_kv, int* status, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && hd > 0 && vd > 0, "qk_norm_rope_kv_write: bad sizes");
    FB_REQUIRE(scope >= FB_QK_NORM_NONE && scope <= FB_QK_NORM_PROJECTION, "qk_norm_rope_kv_write: unknown reach %d", scope);
    FB_REQUIRE(half >= 0 && 2 * half <= hd, "qk_norm_rope_kv_write: rotary width %d exceeds head size %d", 2 * half, hd);
    FB_REQUIRE(half == 0 || (cos_t && sin_t), "qk_norm_rope_kv_write: rotary tables missing");
    FB_REQUIRE(!write_kv || (positions && row_seq && block_table && k_pool && v_pool && page_size > 0 && n_pages > 0),
               "qk_norm_rope_kv_write: cache arguments missing");
    FB_REQUIRE(proj_stride >= (long long)nh * hd + (long long)nkv * hd + (long long)nkv * vd,
               "qk_norm_rope_kv_write: projection rows are too short");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    const size_t smem = ((size_t)(nh + nkv) * hd + nh + nkv) * sizeof(float);
    FB_REQUIRE(smem <= 200 * 1024, "qk_norm_rope_kv_write: a row of q and k (%zu bytes) does not fit shared memory", smem);
    FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, T, {
        auto kernel = qk_norm_rope_kv_write_kernel<TW, T>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        const int cols = (nh + 2 * nkv) * (hd > vd ? hd : vd);
        fb_launch(kernel, dim3(n), dim3(n > 128 ? 256 : cols >= 4096 ? 1024 : cols >= 1024 ? 512 : 256), smem, stream, proj, (long)proj_stride, n_partials, (long)partial_stride,
                  (const TW*)q_weight, (const TW*)k_weight, scope, eps, weight_offset, cos_t, sin_t, half, (T*)q_out,
                  (long)q_out_stride, positions, row_seq, block_table, table_stride, table_base, table_head, (T*)k_pool,
                  (T*)v_pool, page_size, n_pages, nh, nkv, hd, vd, write_kv, status);
    }));
    return fb_check_launch("qk_norm_rope_kv_write");
}
