// Several residual streams mixed by small learned matrices around every sublayer, and the token shift of a recurrent mixer.
//
// streams_step: a model may carry n copies x_1 .. x_n of the residual stream ([rows, n, dim] fp32).  Around a sublayer with
// output y,
//     x_t <- sum_s mix[s, t] x_s + out[t] (y + bias)        (the right-hand side sees only the streams as they were)
// and the next sublayer reads  h = rms_norm(sum_s in[s] x_s) * g  with ONE number g as the norm's weight.  One launch does
// the write of the sublayer that ended and the read of the one that follows: a CTA per row, the n numbers of a column in
// registers, the row's sum of squares by a block reduction, then a second sweep over the row it has just written.  n = 1
// with mix = out = in = 1 is the plain residual sum with its norm.  Either half may be absent (no y: the streams are only
// read; no in: only written), and the streams may start as n copies of one row (x0, the embedding).  Everything is fp32
// but h, which is rounded once to the projections' type.
//
// shift_mix: m_i[t] = h[t] + (h[t-1] - h[t]) * mu_i for i < n learned per-channel vectors mu_i, with h[-1] = 0 at a
// sequence's start and the last row of the previous step (the sequence's slot, fp32 [dim]) otherwise.  The thread that
// reads the slot is the one that writes it, after reading.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kMaxStreams = 8;

template <typename T>
__global__ void __launch_bounds__(256)
streams_step_kernel(float *xs, const float *__restrict__ x0, const float *__restrict__ y, const T *__restrict__ y_bias,
                    const float *__restrict__ write_w /* mix [n, n] (from, to), then out [n] */,
                    const float *__restrict__ read_w /* in [n], then the norm's weight */, float eps, T *__restrict__ h, int n, int dim) {
    __shared__ float scratch[33];
    __shared__ float sw[kMaxStreams * kMaxStreams + 2 * kMaxStreams + 1];
    float *mix = sw, *outw = sw + kMaxStreams * kMaxStreams, *inw = outw + kMaxStreams;
    for (int e = threadIdx.x; e < n * n + n; e += blockDim.x)
        if (write_w) (e < n * n ? mix[e] : outw[e - n * n]) = write_w[e];
    for (int e = threadIdx.x; e <= n; e += blockDim.x)
        if (read_w) inw[e] = read_w[e];
    __syncthreads();
    const size_t row = blockIdx.x;
    float *xr = xs + row * n * dim;
    float ss = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float x[kMaxStreams], nx[kMaxStreams];
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
            if (s < n) x[s] = x0 ? x0[row * dim + d] : xr[(size_t)s * dim + d];
        if (write_w) {
            const float yv = y[row * dim + d] + (y_bias ? to_f(y_bias[d]) : 0.f);
#pragma unroll
            for (int t = 0; t < kMaxStreams; ++t) {
                if (t < n) {
                    float acc = 0.f;
#pragma unroll
                    for (int s = 0; s < kMaxStreams; ++s)
                        if (s < n) acc = fmaf(mix[s * n + t], x[s], acc);
                    nx[t] = fmaf(outw[t], yv, acc);
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s) nx[s] = x[s];
        }
        if (write_w || x0) {
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < n) xr[(size_t)s * dim + d] = nx[s];
        }
        if (read_w) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < n) u = fmaf(inw[s], nx[s], u);
            ss = fmaf(u, u, ss);
        }
    }
    if (!read_w) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps) * inw[n];
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {  // the thread's own columns again (it wrote them itself)
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
            if (s < n) u = fmaf(inw[s], xr[(size_t)s * dim + d], u);
        h[row * dim + d] = from_f<T>(u * inv);
    }
}

constexpr int kShiftChunk = 32;  // tokens per CTA

template <typename T>
__global__ void __launch_bounds__(128)
shift_mix_kernel(const T *__restrict__ h, long long h_token, const T *__restrict__ mu, int n, int dim, const int32_t *__restrict__ seq_info,
                 float *__restrict__ state, long long slot_stride, int num_slots, T *__restrict__ out, long long out_part) {
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    const int first = seq_info[s * 4 + 0], count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    const int lo = blockIdx.z * kShiftChunk, hi = min(count, lo + kShiftChunk);
    if (c >= dim || lo >= count) return;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    float *mine = state + (size_t)(slot_ok ? slot : 0) * slot_stride + c;
    float before;
    if (lo == 0) {
        before = (start > 0 && slot_ok) ? *mine : 0.f;
        if (slot_ok) *mine = to_f(h[(size_t)(first + count - 1) * h_token + c]);
    } else {
        before = to_f(h[(size_t)(first + lo - 1) * h_token + c]);
    }
    float m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = i < n ? to_f(mu[(size_t)i * dim + c]) : 0.f;
    for (int j = lo; j < hi; ++j) {
        const float x = to_f(h[(size_t)(first + j) * h_token + c]);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < n) out[(size_t)i * out_part + (size_t)(first + j) * dim + c] = from_f<T>(fmaf(before - x, m[i], x));
        before = x;
    }
}

}  // namespace tlb

using namespace tlb;

extern "C" {

int tlb_streams_step(float *xs, const float *x0, const float *y, const void *y_bias, const float *write_w, const float *read_w, float eps, void *h,
                     int rows, int streams, int dim, int dtype, void *stream) {
    if (rows <= 0) return TL_OK;
    if (!xs || streams <= 0 || dim <= 0 || (write_w && !y) || (read_w && !h) || (!write_w && !read_w && !x0))
        return tl::fail(TL_EINVAL, "streams_step: bad argument");
    if (streams > kMaxStreams) return tl::fail(TL_EINVAL, "streams_step: %d streams > %d", streams, kMaxStreams);
    TLB_DISPATCH(dtype, "streams_step",
                 streams_step_kernel<T><<<rows, 256, 0, as_stream(stream)>>>(xs, x0, y, (const T *)y_bias, write_w, read_w, eps, (T *)h, streams, dim));
    TL_LAUNCH_CHECK("streams_step");
    return TL_OK;
}

int tlb_shift_mix(const void *h, long long h_token, const void *mu, int parts, int dim, const int32_t *seq_info, int num_seqs, int max_tokens_per_seq,
                  float *state, long long slot_stride, int num_slots, void *out, long long out_part, int dtype, void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (!h || !mu || !seq_info || !state || !out || parts <= 0 || parts > 8 || dim <= 0 || max_tokens_per_seq <= 0 || num_slots <= 0)
        return tl::fail(TL_EINVAL, "shift_mix: bad argument");
    dim3 grid(num_seqs, ceil_div(dim, 128), ceil_div(max_tokens_per_seq, kShiftChunk));
    TLB_DISPATCH(dtype, "shift_mix",
                 shift_mix_kernel<T><<<grid, 128, 0, as_stream(stream)>>>((const T *)h, h_token, (const T *)mu, parts, dim, seq_info, state, slot_stride,
                                                                           num_slots, (T *)out, out_part));
    TL_LAUNCH_CHECK("shift_mix");
    return TL_OK;
}

}  // extern "C"
