// Gated linear attention: a linear recurrence with one matrix of state per head, S [dk, dv] in float32, whose rows
// (one per key channel) decay each by a factor of its own before a token adds its key times its value:
//
//     S <- diag(alpha) S + k v^T;   o = S^T q          (alpha: one number per head, key channel and token)
//     alpha = sigmoid(z)^(1/tau),   z = W2 (W1 h) + b  (a map through a narrow middle, W1 h being part of the
//                                                        mixer's stacked projection)
//
// Every column of S (one value dimension) goes through this on its own, so columns are spread over threads and a
// request's tokens are taken in order.
//
// Kernels, in the order a step runs them:
//   gla_prepare      per (token, head): add the projection's split-K shares; q times `q_scale`, k and v as they are;
//                    z from the narrow middle, log sigmoid(z) / tau and its exponential; all float32
//   gla_recurrent    per (request, head, a few columns): the recurrence over the step's tokens, the column's state in
//                    registers, 16 (or 32) lanes a column; tokens arrive by asynchronous copies in two stages
// The head norm and output gate that follow are those of the gated delta rule (gdr_out_norm).
//
// A request's slot of state holds S as [heads][dv][dk] (a column's dk values side by side) at its start.
// Projection rows are [q: H*dk | k: H*dk | v: H*dv | gate: H*dv | middle: R].
#include "common.cuh"

__device__ __forceinline__ float gla_slab_sum(const float* row, int c, int n_partials, long partial_stride) {
    return fb_slab_sum(row, c, n_partials, partial_stride);
}

template <typename TW>
__global__ void __launch_bounds__(128)
gla_prepare_kernel(const float* __restrict__ proj, long proj_stride, int n_partials, long partial_stride,
                   const TW* __restrict__ w2, const TW* __restrict__ b2, int R, float inv_tau, float q_scale,
                   float* __restrict__ qkv, float* __restrict__ decay, int H, int dk, int dv) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ float mid[];                     // the narrow middle of the decay's map, [R]
    const int row = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int qk = H * dk, C = 2 * qk + H * dv;
    const float* pr = proj + (size_t)row * proj_stride;
    for (int r = tid; r < R; r += blockDim.x) mid[r] = gla_slab_sum(pr, C + H * dv + r, n_partials, partial_stride);
    __syncthreads();
    float* out = qkv + (size_t)row * C;
    for (int d = tid; d < dk; d += blockDim.x) {
        const int c = head * dk + d;
        out[c] = gla_slab_sum(pr, c, n_partials, partial_stride) * q_scale;
        out[qk + c] = gla_slab_sum(pr, qk + c, n_partials, partial_stride);
        float z = fb_to_float(b2[c]);
        const TW* wr = w2 + (size_t)c * R;
        for (int r = 0; r < R; ++r) z = fmaf(fb_to_float(wr[r]), mid[r], z);
        // log sigmoid(z) = min(z, 0) - log(1 + exp(-|z|))
        const float ls = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
        decay[(size_t)row * qk + c] = expf(ls * inv_tau);
    }
    for (int d = tid; d < dv; d += blockDim.x) {
        const int c = 2 * qk + head * dv + d;
        out[c] = gla_slab_sum(pr, c, n_partials, partial_stride);
    }
}

// A 4-byte copy from global to shared memory that does not pass through registers (the thread goes on at once).
__device__ __forceinline__ void gla_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void gla_copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT> __device__ __forceinline__ void gla_copies_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory");
}

// LPC lanes a column, R state values a lane (dk <= LPC R), 256 / LPC columns a CTA.
template <int R, int LPC> struct GlaTile {
    static constexpr int THREADS = 256, COLS = THREADS / LPC, DKP = LPC * R;
    static constexpr int CH = DKP <= 128 ? 32 : DKP <= 256 ? 16 : 8;         // tokens fetched at a time
    static constexpr int STAGE_FLOATS = CH * (3 * DKP + COLS);
};

template <int R, int LPC, bool STATE_BY4>
__global__ void __launch_bounds__(256)
gla_recurrent_kernel(const float* __restrict__ qkv, const float* __restrict__ decay, float* __restrict__ state,
                     long state_stride, const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                     const int* __restrict__ seq_slot, float* __restrict__ o, int H, int dk, int dv) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    using Tile = GlaTile<R, LPC>;
    constexpr int THREADS = Tile::THREADS, COLS = Tile::COLS, CH = Tile::CH, DKP = Tile::DKP;
    extern __shared__ __align__(16) float sh[];
    const int seq = blockIdx.x / H, head = blockIdx.x - seq * H;
    const int tid = threadIdx.x;
    const int li = tid % LPC, col = blockIdx.y * COLS + tid / LPC;
    const bool live = col < dv;
    const int qk = H * dk, C = 2 * qk + H * dv;
    const int start = seq_q_start[seq], L = seq_q_len[seq];
    float* S = state + (size_t)seq_slot[seq] * state_stride + ((size_t)head * dv + (live ? col : 0)) * dk;

    // a stage: q [CH][DKP], k [CH][DKP], alpha [CH][DKP] (rows padded with zeros beyond dk), v [CH][COLS]
    auto fetch = [&](int t0, float* st) {
        const int cnt = min(CH, L - t0);
        float* qs = st;
        float* ks = qs + CH * DKP;
        float* as = ks + CH * DKP;
        float* vs = as + CH * DKP;
        for (int e = tid; e < cnt * DKP; e += THREADS) {
            const int t = e / DKP, d = e - t * DKP;
            if (d < dk) {
                const float* rowp = qkv + (size_t)(start + t0 + t) * C + (size_t)head * dk + d;
                gla_copy4(qs + e, rowp);
                gla_copy4(ks + e, rowp + qk);
                gla_copy4(as + e, decay + (size_t)(start + t0 + t) * qk + (size_t)head * dk + d);
            } else {
                qs[e] = 0.0f;
                ks[e] = 0.0f;
                as[e] = 0.0f;
            }
        }
        for (int e = tid; e < cnt * COLS; e += THREADS) {
            const int t = e / COLS, c2 = blockIdx.y * COLS + (e - t * COLS);
            if (c2 < dv) gla_copy4(vs + e, qkv + (size_t)(start + t0 + t) * C + 2 * qk + (size_t)head * dv + c2);
            else vs[e] = 0.0f;
        }
        gla_copies_commit();
    };

    // Which key channels a lane holds: four neighbouring ones out of every 4 LPC where R allows it (a lane fetches them
    // as one 16-byte vector and neighbouring lanes read neighbouring vectors), else every LPC-th.
    constexpr bool VEC = R % 4 == 0;
    auto channel = [&](int r) { return VEC ? (r / 4) * (4 * LPC) + 4 * li + (r & 3) : li + LPC * r; };
    // (STATE_BY4: the state moves as 16-byte vectors; the launcher asks for it where a lane's groups of four are whole
    // and aligned)
    float s[R];
    if constexpr (STATE_BY4) {
#pragma unroll
        for (int r = 0; r < R; r += 4) {
            const int d = channel(r);
            float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (live && d < dk) x = *reinterpret_cast<const float4*>(S + d);
            s[r] = x.x;
            if (r + 1 < R) s[r + 1] = x.y;
            if (r + 2 < R) s[r + 2] = x.z;
            if (r + 3 < R) s[r + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = channel(r);
            s[r] = (live && d < dk) ? S[d] : 0.0f;
        }
    }
    if (L > 0) fetch(0, sh);
    int buf = 0;
    for (int t0 = 0; t0 < L; t0 += CH, buf ^= 1) {
        const int cnt = min(CH, L - t0);
        float* st = sh + buf * Tile::STAGE_FLOATS;
        const bool more = t0 + CH < L;
        if (more) fetch(t0 + CH, sh + (buf ^ 1) * Tile::STAGE_FLOATS);    // (its last readers passed the barrier below)
        if (more) gla_copies_wait<1>(); else gla_copies_wait<0>();
        __syncthreads();
        const float* qs = st;
        const float* ks = qs + CH * DKP;
        const float* as = ks + CH * DKP;
        const float* vs = as + CH * DKP;
        // (four tokens unrolled: only the state's multiply-adds depend on the token before, so the loads, the sums
        // and the exchanges between lanes of neighbouring tokens overlap)
#pragma unroll 4
        for (int t = 0; t < cnt; ++t) {
            const float v = vs[t * COLS + tid / LPC];
            float qv[R], kv[R], av[R];
            if constexpr (VEC) {
                const float4* q4 = reinterpret_cast<const float4*>(qs + t * DKP) + li;
                const float4* k4 = reinterpret_cast<const float4*>(ks + t * DKP) + li;
                const float4* a4 = reinterpret_cast<const float4*>(as + t * DKP) + li;
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    const float4 a = q4[r * LPC], b = k4[r * LPC], c = a4[r * LPC];
                    qv[4 * r] = a.x; qv[4 * r + 1] = a.y; qv[4 * r + 2] = a.z; qv[4 * r + 3] = a.w;
                    kv[4 * r] = b.x; kv[4 * r + 1] = b.y; kv[4 * r + 2] = b.z; kv[4 * r + 3] = b.w;
                    av[4 * r] = c.x; av[4 * r + 1] = c.y; av[4 * r + 2] = c.z; av[4 * r + 3] = c.w;
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    qv[r] = qs[t * DKP + li + LPC * r];
                    kv[r] = ks[t * DKP + li + LPC * r];
                    av[r] = as[t * DKP + li + LPC * r];
                }
            }
            float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                s[r] = fmaf(av[r], s[r], kv[r] * v);
                if (r & 1) acc1 = fmaf(s[r], qv[r], acc1); else acc0 = fmaf(s[r], qv[r], acc0);
            }
            float acc = acc0 + acc1;
#pragma unroll
            for (int off = LPC / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (live && li == 0) o[(size_t)(start + t0 + t) * H * dv + (size_t)head * dv + col] = acc;
        }
        __syncthreads();                               // the stage may be overwritten by the fetch after next
    }
    if constexpr (STATE_BY4) {
#pragma unroll
        for (int r = 0; r < R; r += 4) {
            const int d = channel(r);
            if (live && d < dk)
                *reinterpret_cast<float4*>(S + d) = make_float4(s[r], r + 1 < R ? s[r + 1] : 0.0f, r + 2 < R ? s[r + 2] : 0.0f,
                                                               r + 3 < R ? s[r + 3] : 0.0f);
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = channel(r);
        if (live && d < dk) S[d] = s[r];
    }
}

FB_API int fb_gla_prepare(const float* proj, long long proj_stride, int n_partials, long long partial_stride,
                          const void* w2, const void* b2, int w_dtype, int R, float tau, float q_scale, float* qkv,
                          float* decay, int n, int H, int dk, int dv, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && H > 0 && dk > 0 && dv > 0 && R > 0, "linear attention: bad sizes");
    FB_REQUIRE(tau > 0.0f, "linear attention: tau must be positive");
    FB_REQUIRE(proj_stride >= 2LL * H * dk + 2LL * H * dv + R, "linear attention: projection rows are too short");
    FB_REQUIRE(H <= 65535 && R <= 8192, "linear attention: too many heads, or a middle wider than 8192");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    FB_DISPATCH_DTYPE(w_dtype, TW,
        (fb_launch((gla_prepare_kernel<TW>), dim3(n, H), dim3(128), (size_t)R * sizeof(float), stream, proj,
                   (long)proj_stride, n_partials, (long)partial_stride, (const TW*)w2, (const TW*)b2, R, 1.0f / tau,
                   q_scale, qkv, decay, H, dk, dv)));
    return fb_check_launch("gla_prepare");
}

template <int R, int LPC>
static int launch_gla_recurrent(const float* qkv, const float* decay, float* state, long state_stride,
                                const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int n_seqs, int rows,
                                float* o, int H, int dk, int dv, cudaStream_t stream) {
    using Tile = GlaTile<R, LPC>;
    const size_t smem = (size_t)2 * Tile::STAGE_FLOATS * sizeof(float);
    const dim3 grid(n_seqs * H, (dv + Tile::COLS - 1) / Tile::COLS);
    // The state as 16-byte vectors where a lane's groups of four are whole and aligned, in steps of few tokens a
    // request, whose time is the state's way in and out; over long portions the variant with plain state loads runs
    // the token loop faster (measured: 475 against 520 us over 2,048 tokens, 16.2 against 12.3 us for one token).
    if (R % 4 == 0 && (dk & 3) == 0 && (state_stride & 3) == 0 && ((uintptr_t)state & 15) == 0 &&
        rows <= 4L * n_seqs) {
        auto kernel = gla_recurrent_kernel<R, LPC, R % 4 == 0>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fb_launch(kernel, grid, dim3(Tile::THREADS), smem, stream, qkv, decay, state, state_stride, seq_q_start,
                  seq_q_len, seq_slot, o, H, dk, dv);
    } else {
        auto kernel = gla_recurrent_kernel<R, LPC, false>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fb_launch(kernel, grid, dim3(Tile::THREADS), smem, stream, qkv, decay, state, state_stride, seq_q_start,
                  seq_q_len, seq_slot, o, H, dk, dv);
    }
    return fb_check_launch("gla_recurrent");
}

FB_API int fb_gla_recurrent(const float* qkv, const float* decay, float* state, long long state_stride,
                            const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int n_seqs, int rows,
                            float* o, int H, int dk, int dv, cudaStream_t stream) {
    FB_REQUIRE(n_seqs >= 0 && rows >= 0 && H > 0 && dk > 0 && dv > 0, "linear attention: bad sizes");
    FB_REQUIRE(dk <= 1024, "linear attention: key size %d is larger than 1024", dk);
    if (n_seqs == 0) return 0;
#define FB_GLA_CASE(R, LPC) return launch_gla_recurrent<R, LPC>(qkv, decay, state, (long)state_stride, seq_q_start, \
        seq_q_len, seq_slot, n_seqs, rows, o, H, dk, dv, stream)
    if (dk <= 16) FB_GLA_CASE(1, 16);
    if (dk <= 32) FB_GLA_CASE(2, 16);
    if (dk <= 64) FB_GLA_CASE(4, 16);
    if (dk <= 128) FB_GLA_CASE(8, 16);
    if (dk <= 256) FB_GLA_CASE(16, 16);
    if (dk <= 512) FB_GLA_CASE(16, 32);
    FB_GLA_CASE(32, 32);
#undef FB_GLA_CASE
}
