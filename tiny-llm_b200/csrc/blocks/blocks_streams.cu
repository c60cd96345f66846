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

template <typename T> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
    static __device__ __forceinline__ float4 load(const float *p) { return *reinterpret_cast<const float4 *>(p); }
};
template <> struct Pack4<bf16> {
    static __device__ __forceinline__ void store(bf16 *p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t *>(&a), u.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(p) = u;
    }
    static __device__ __forceinline__ float4 load(const bf16 *p) {
        uint2 u = *reinterpret_cast<const uint2 *>(p);
        float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

// V = 4: four adjacent columns per thread and step (16-byte accesses; dim % 4 == 0), the sublayer's input kept in registers
// between the two sweeps when the row fits (dim <= 4 * kKeep * 256); V = 1: any dim, the second sweep reads the row again.
// The arithmetic per column is the same in both, so a row's result does not depend on which one ran.
constexpr int kKeep = 4;

template <typename T, int N /* streams, 0 = any number up to kMaxStreams */, int V>
__global__ void __launch_bounds__(256)
streams_step_kernel(float *xs, const float *__restrict__ x0, const float *__restrict__ y, const T *__restrict__ y_bias,
                    const float *__restrict__ write_w /* mix [n, n] (from, to), then out [n] */,
                    const float *__restrict__ read_w /* in [n], then the norm's weight */, float eps, T *__restrict__ h, int n_any, int dim) {
    constexpr int NM = N ? N : kMaxStreams;
    const int n = N ? N : n_any;
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
    float keep[V == 4 ? kKeep : 1][V];
    const bool kept = V == 4 && dim <= 4 * kKeep * 256;
    int step = 0;
    for (int d = threadIdx.x * V; d < dim; d += blockDim.x * V, ++step) {
        float x[NM][V], nx[NM][V], yv[V];
#pragma unroll
        for (int s = 0; s < NM; ++s) {
            if (s < n) {
                const float *src = x0 ? x0 + row * dim + d : xr + (size_t)s * dim + d;
                if (V == 4) {
                    float4 t = *reinterpret_cast<const float4 *>(src);
                    x[s][0] = t.x, x[s][1 % V] = t.y, x[s][2 % V] = t.z, x[s][3 % V] = t.w;
                } else x[s][0] = src[0];
            }
        }
        if (write_w) {
            if (V == 4) {
                float4 t = *reinterpret_cast<const float4 *>(y + row * dim + d);
                yv[0] = t.x, yv[1 % V] = t.y, yv[2 % V] = t.z, yv[3 % V] = t.w;
                if (y_bias) {
                    float4 b = Pack4<T>::load(y_bias + d);
                    yv[0] += b.x, yv[1 % V] += b.y, yv[2 % V] += b.z, yv[3 % V] += b.w;
                }
            } else yv[0] = y[row * dim + d] + (y_bias ? to_f(y_bias[d]) : 0.f);
#pragma unroll
            for (int t = 0; t < NM; ++t) {
                if (t < n) {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        float acc = 0.f;
#pragma unroll
                        for (int s = 0; s < NM; ++s)
                            if (s < n) acc = fmaf(mix[s * n + t], x[s][v], acc);
                        nx[t][v] = fmaf(outw[t], yv[v], acc);
                    }
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < NM; ++s)
#pragma unroll
                for (int v = 0; v < V; ++v) nx[s][v] = x[s][v];
        }
        if (write_w || x0) {
#pragma unroll
            for (int s = 0; s < NM; ++s) {
                if (s < n) {
                    if (V == 4) *reinterpret_cast<float4 *>(xr + (size_t)s * dim + d) = make_float4(nx[s][0], nx[s][1 % V], nx[s][2 % V], nx[s][3 % V]);
                    else xr[(size_t)s * dim + d] = nx[s][0];
                }
            }
        }
        if (read_w) {
#pragma unroll
            for (int v = 0; v < V; ++v) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < NM; ++s)
                    if (s < n) u = fmaf(inw[s], nx[s][v], u);
                ss = fmaf(u, u, ss);
                if (V == 4 && kept) {
#pragma unroll
                    for (int kk = 0; kk < kKeep; ++kk)
                        if (kk == step) keep[kk % (V == 4 ? kKeep : 1)][v] = u;
                }
            }
        }
    }
    if (!read_w) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps) * inw[n];
    step = 0;
    for (int d = threadIdx.x * V; d < dim; d += blockDim.x * V, ++step) {  // the thread's own columns again (it wrote them itself)
        float u[V];
        if (V == 4 && kept) {
#pragma unroll
            for (int kk = 0; kk < kKeep; ++kk)
                if (kk == step) {
#pragma unroll
                    for (int v = 0; v < V; ++v) u[v] = keep[kk % (V == 4 ? kKeep : 1)][v];
                }
        } else {
#pragma unroll
            for (int v = 0; v < V; ++v) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < NM; ++s)
                    if (s < n) a = fmaf(inw[s], xr[(size_t)s * dim + d + v], a);
                u[v] = a;
            }
        }
        if (V == 4) Pack4<T>::store(h + row * dim + d, make_float4(u[0] * inv, u[1 % V] * inv, u[2 % V] * inv, u[3 % V] * inv));
        else h[row * dim + d] = from_f<T>(u[0] * inv);
    }
}

constexpr int kShiftChunk = 32, kShiftSmallChunk = 8;  // tokens per CTA; the small one when the launch would leave SMs idle

template <typename T>
__global__ void __launch_bounds__(128)
shift_mix_kernel(const T *__restrict__ h, long long h_token, const T *__restrict__ mu, int n, int dim, const int32_t *__restrict__ seq_info,
                 float *__restrict__ state, long long slot_stride, int num_slots, T *__restrict__ out, long long out_part, int chunk) {
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    const int first = seq_info[s * 4 + 0], count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    const int lo = blockIdx.z * chunk, hi = min(count, lo + chunk);
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
    // 16-byte accesses when every row of every operand starts on such a boundary
    const bool wide = dim % 4 == 0 && (uintptr_t)xs % 16 == 0 && (uintptr_t)x0 % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)y_bias % 8 == 0 &&
                      (uintptr_t)h % 8 == 0;
#define TLB_SS(NV, VV) streams_step_kernel<T, NV, VV><<<rows, 256, 0, as_stream(stream)>>>(xs, x0, y, (const T *)y_bias, write_w, read_w, eps, (T *)h, streams, dim)
#define TLB_SS_N(VV) do { if (streams == 1) TLB_SS(1, VV); else if (streams == 2) TLB_SS(2, VV); else if (streams == 4) TLB_SS(4, VV); else TLB_SS(0, VV); } while (0)
    TLB_DISPATCH(dtype, "streams_step", if (wide) TLB_SS_N(4); else TLB_SS_N(1));
#undef TLB_SS_N
#undef TLB_SS
    TL_LAUNCH_CHECK("streams_step");
    return TL_OK;
}

int tlb_shift_mix(const void *h, long long h_token, const void *mu, int parts, int dim, const int32_t *seq_info, int num_seqs, int max_tokens_per_seq,
                  float *state, long long slot_stride, int num_slots, void *out, long long out_part, int dtype, void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (!h || !mu || !seq_info || !state || !out || parts <= 0 || parts > 8 || dim <= 0 || max_tokens_per_seq <= 0 || num_slots <= 0)
        return tl::fail(TL_EINVAL, "shift_mix: bad argument");
    const int chunk = (long long)num_seqs * ceil_div(dim, 128) * ceil_div(max_tokens_per_seq, kShiftChunk) < 148 * 8 ? kShiftSmallChunk : kShiftChunk;
    dim3 grid(num_seqs, ceil_div(dim, 128), ceil_div(max_tokens_per_seq, chunk));
    TLB_DISPATCH(dtype, "shift_mix",
                 shift_mix_kernel<T><<<grid, 128, 0, as_stream(stream)>>>((const T *)h, h_token, (const T *)mu, parts, dim, seq_info, state, slot_stride,
                                                                           num_slots, (T *)out, out_part, chunk));
    TL_LAUNCH_CHECK("shift_mix");
    return TL_OK;
}

}  // extern "C"
