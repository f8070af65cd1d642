// A short causal convolution over time that is added to its own input: every channel has `taps` weights of its own,
//
//     out_t = h_t + sum_j w[c][j] * h_(t - taps + 1 + j)          (the last tap is the current token's; zeros before
//                                                                   the request's first token)
//
// for the rows of a step, which hold portions of several requests.  Inputs before a portion's start come from the
// request's kept tail, the last taps - 1 inputs of the step before: `state` is a float32 array per request slot with the
// tail at `tail_off`, laid out [taps - 1][D], oldest first.
//
//   time_conv         per (row, stretch of channels): the sum above in float32, rounded once to the output's dtype
//                     (one channel, four channels, or four channels and four rows a thread)
//   time_conv_tail    per (request, stretch of channels): the step's last taps - 1 inputs become the kept tail (a
//                     portion shorter than that keeps the newest entries of the old tail in front of its own)
//
// The tail kernel runs after the convolution has read the old tail (stream order).
#include "common.cuh"

template <typename TO>
__global__ void __launch_bounds__(256)
time_conv_kernel(const float* __restrict__ h, const float* __restrict__ wt, int taps, const float* __restrict__ state,
                 long state_stride, long tail_off, const int* __restrict__ row_seq,
                 const int* __restrict__ seq_q_start, const int* __restrict__ seq_slot, TO* __restrict__ out, int D) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int row = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= D) return;
    const int seq = row_seq[row];
    const int i = row - seq_q_start[seq];              // place within the step's portion of this request
    const float* tail = state + (size_t)seq_slot[seq] * state_stride + tail_off;
    float acc = h[(size_t)row * D + c];
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float x = i - back >= 0 ? h[(size_t)(row - back) * D + c]
                                      : tail[(size_t)(taps - 1 + i - back) * D + c];
        acc = fmaf(wt[(size_t)j * D + c], x, acc);
    }
    out[(size_t)row * D + c] = fb_from_float<TO>(acc);
}

// Four neighbouring channels a thread (D, the slots' stride and the tail's place multiples of 4): rows, tails and the
// weights of a tap move as 16-byte vectors, so that a thread has four times the bytes in flight.
template <typename TO>
__global__ void __launch_bounds__(256)
time_conv4_kernel(const float* __restrict__ h, const float* __restrict__ wt, int taps, const float* __restrict__ state,
                  long state_stride, long tail_off, const int* __restrict__ row_seq,
                  const int* __restrict__ seq_q_start, const int* __restrict__ seq_slot, TO* __restrict__ out, int D) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int row = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= D) return;
    const int seq = row_seq[row];
    const int i = row - seq_q_start[seq];
    const float* tail = state + (size_t)seq_slot[seq] * state_stride + tail_off;
    float4 acc = *reinterpret_cast<const float4*>(h + (size_t)row * D + c);
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float* src = i - back >= 0 ? h + (size_t)(row - back) * D + c
                                         : tail + (size_t)(taps - 1 + i - back) * D + c;
        const float4 x = *reinterpret_cast<const float4*>(src);
        const float4 wj = *reinterpret_cast<const float4*>(wt + (size_t)j * D + c);
        acc.x = fmaf(wj.x, x.x, acc.x);
        acc.y = fmaf(wj.y, x.y, acc.y);
        acc.z = fmaf(wj.z, x.z, acc.z);
        acc.w = fmaf(wj.w, x.w, acc.w);
    }
    TO* o = out + (size_t)row * D + c;
    o[0] = fb_from_float<TO>(acc.x);
    o[1] = fb_from_float<TO>(acc.y);
    o[2] = fb_from_float<TO>(acc.z);
    o[3] = fb_from_float<TO>(acc.w);
}

// Four channels and four consecutive rows a thread, the number of taps known to the compiler: the rows' inputs are
// fetched once into a window of 4 + TAPS - 1 vectors (a row's earlier inputs are the rows before it, which belong to the
// same request as long as the row is not among its portion's first TAPS - 1), the weights once for the four rows.
// Only a portion's first rows go to the request's kept tail.
constexpr int TC_ROWS = 4;

template <int TAPS, typename TO>
__global__ void __launch_bounds__(256)
time_conv4x4_kernel(const float* __restrict__ h, const float* __restrict__ wt, const float* __restrict__ state,
                    long state_stride, long tail_off, const int* __restrict__ row_seq,
                    const int* __restrict__ seq_q_start, const int* __restrict__ seq_slot, TO* __restrict__ out, int n,
                    int D) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int row0 = blockIdx.x * TC_ROWS;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= D) return;
    float4 win[TC_ROWS + TAPS - 1];                    // win[k]: the inputs of row row0 - (TAPS - 1) + k
#pragma unroll
    for (int k = 0; k < TC_ROWS + TAPS - 1; ++k) {
        const int row = row0 - (TAPS - 1) + k;
        win[k] = (row >= 0 && row < n) ? *reinterpret_cast<const float4*>(h + (size_t)row * D + c)
                                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float4 w[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) w[j] = *reinterpret_cast<const float4*>(wt + (size_t)j * D + c);
#pragma unroll
    for (int r = 0; r < TC_ROWS; ++r) {
        const int row = row0 + r;
        if (row >= n) break;
        const int seq = row_seq[row];
        const int i = row - seq_q_start[seq];          // place within the step's portion of this request
        float4 acc = win[r + TAPS - 1];
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            const int back = TAPS - 1 - j;
            float4 x = win[r + j];
            if (i - back < 0)                          // before the portion: the kept tail, oldest first
                x = *reinterpret_cast<const float4*>(state + (size_t)seq_slot[seq] * state_stride + tail_off +
                                                     (size_t)(TAPS - 1 + i - back) * D + c);
            acc.x = fmaf(w[j].x, x.x, acc.x);
            acc.y = fmaf(w[j].y, x.y, acc.y);
            acc.z = fmaf(w[j].z, x.z, acc.z);
            acc.w = fmaf(w[j].w, x.w, acc.w);
        }
        TO* o = out + (size_t)row * D + c;
        o[0] = fb_from_float<TO>(acc.x);
        o[1] = fb_from_float<TO>(acc.y);
        o[2] = fb_from_float<TO>(acc.z);
        o[3] = fb_from_float<TO>(acc.w);
    }
}

__global__ void __launch_bounds__(256)
time_conv_tail_kernel(const float* __restrict__ h, int taps, float* __restrict__ state, long state_stride, long tail_off,
                      const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                      const int* __restrict__ seq_slot, int D) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= D) return;
    const int L = seq_q_len[seq], start = seq_q_start[seq];
    float* tail = state + (size_t)seq_slot[seq] * state_stride + tail_off;
    // ascending m: an entry taken from the old tail lies above the one being written
    for (int m = 0; m < taps - 1; ++m) {
        const int src = L - (taps - 1) + m;
        tail[(size_t)m * D + c] = src >= 0 ? h[(size_t)(start + src) * D + c] : tail[(size_t)(taps - 1 + src) * D + c];
    }
}

// h: float32 [n, D] contiguous; wt: float32 [taps, D], tap by tap (a warp reads neighbouring channels' weights of one
// tap side by side); out: [n, D] contiguous in the engine's dtype.
FB_API int fb_time_conv(const float* h, const float* wt, int taps, float* state, long long state_stride,
                        long long tail_off, const int* row_seq, const int* seq_q_start, const int* seq_q_len,
                        const int* seq_slot, int n_seqs, void* out, int out_dtype, int n, int D, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && D > 0 && taps >= 1 && n_seqs >= 0, "time_conv: bad sizes");
    FB_REQUIRE(taps == 1 || state, "time_conv: more than one tap needs the requests' kept inputs");
    if (n == 0) return 0;
    const unsigned stretches = (unsigned)((D + 255) / 256);
    FB_REQUIRE(stretches <= 65535, "time_conv: width %d is too large", D);
    const bool by4 = D % 4 == 0 && state_stride % 4 == 0 && tail_off % 4 == 0 && (uintptr_t)h % 16 == 0 &&
                     (uintptr_t)wt % 16 == 0 && (!state || (uintptr_t)state % 16 == 0);
    if (by4 && taps <= 4 && n >= 16) {                 // (few rows: a row a CTA keeps more of the machine busy)
        const unsigned stretches4 = (unsigned)((D / 4 + 255) / 256);
        const dim3 grid((n + TC_ROWS - 1) / TC_ROWS, stretches4);
#define FB_TC_CASE(T)                                                                                               \
        FB_DISPATCH_DTYPE(out_dtype, TO,                                                                            \
            (fb_launch((time_conv4x4_kernel<T, TO>), grid, dim3(256), 0, stream, h, wt, (const float*)state,         \
                       (long)state_stride, (long)tail_off, row_seq, seq_q_start, seq_slot, (TO*)out, n, D)))
        if (taps == 1) FB_TC_CASE(1);
        else if (taps == 2) FB_TC_CASE(2);
        else if (taps == 3) FB_TC_CASE(3);
        else FB_TC_CASE(4);
#undef FB_TC_CASE
    } else if (by4) {
        const unsigned stretches4 = (unsigned)((D / 4 + 255) / 256);
        FB_DISPATCH_DTYPE(out_dtype, TO,
            (fb_launch((time_conv4_kernel<TO>), dim3(n, stretches4), dim3(256), 0, stream, h, wt, taps,
                       (const float*)state, (long)state_stride, (long)tail_off, row_seq, seq_q_start, seq_slot, (TO*)out, D)));
    } else {
        FB_DISPATCH_DTYPE(out_dtype, TO,
            (fb_launch((time_conv_kernel<TO>), dim3(n, stretches), dim3(256), 0, stream, h, wt, taps,
                       (const float*)state, (long)state_stride, (long)tail_off, row_seq, seq_q_start, seq_slot, (TO*)out, D)));
    }
    int rc = fb_check_launch("time_conv");
    if (rc || taps < 2) return rc;
    fb_launch(time_conv_tail_kernel, dim3(n_seqs, stretches), dim3(256), 0, stream, h, taps, state, (long)state_stride,
              (long)tail_off, seq_q_start, seq_q_len, seq_slot, D);
    return fb_check_launch("time_conv_tail");
}
