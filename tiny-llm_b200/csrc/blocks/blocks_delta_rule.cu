// Gated delta rule (a recurrent mixer with an error-correcting write) over ragged batches, its state kept in fp32
// slots, and the short causal convolution that feeds it.
//
// Per sequence and head a matrix S [dk, dv] is carried from token to token:
//     S <- diag(g_t) S            g_t one decay per key channel, or one per head
//     u  = beta_t (v_t - S^T k_t)   what the state does not yet say about v_t
//     S <- S + k_t u^T
//     o_t = S^T q_t                 the read-out sees the token's own write
//     g_t = exp(-exp(A_log) * softplus(a_t + dt_bias)),   beta_t = sigmoid(b_t)
// q_t and k_t are unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q_t times q_scale; head h reads query/key head
// h / (heads / key_heads).  The columns of S never mix (u_j needs column j only), so a CTA owns 32 of them for one
// (sequence, head) and walks the tokens in order; 4 lanes share a column, each holding every 4th row in registers, and
// the two sums over rows (S^T k, S^T q) close with two shuffles each.  Tokens are staged 16 (8 for dk > 128) at a time
// in shared memory as fp32: decay, unit k, scaled unit q per key channel, all computed there in fp32 from the
// projections.  A sequence that starts at position 0 starts from zero, whatever its slot held; the slot is written back
// after the last token.  Every sum has an order fixed by token and channel indices alone, so a token's result does not
// depend on how the sequence was cut into steps or on what else is in the batch.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kDrCols = 32;   // state columns per CTA
constexpr int kDrLanes = 4;   // lanes per column

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T, int KR /* rows per lane: dk <= 4 * KR */, int kTok /* tokens staged at a time */>
__global__ void __launch_bounds__(kDrCols * kDrLanes)
delta_scan_kernel(const T *__restrict__ q, long long q_token, long long q_head, const T *__restrict__ k, long long k_token, long long k_head,
                  const T *__restrict__ v, long long v_token, long long v_head, const T *__restrict__ beta, long long b_token,
                  const void *__restrict__ a, int a_f32, long long a_token, int per_channel, const T *__restrict__ a_log,
                  const T *__restrict__ dt_bias, float q_scale, float unit_eps, int heads, int group, int dk, int dv,
                  const int32_t *__restrict__ seq_info, float *__restrict__ state, long long slot_stride, int num_slots, float *__restrict__ out) {
    __shared__ float4 sx[kTok * 4 * KR];  // per token and key channel: (decay, k, q, -)
    __shared__ float sv[kTok * kDrCols];
    __shared__ float sbeta[kTok];
    __shared__ float sinv[kTok * 2];
    const int colblocks = (dv + kDrCols - 1) / kDrCols;
    const int s = blockIdx.x, head = blockIdx.y / colblocks, col0 = (blockIdx.y % colblocks) * kDrCols;
    const int first = seq_info[s * 4 + 0], count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    const int cidx = threadIdx.x / kDrLanes, r = threadIdx.x % kDrLanes;
    const int col = col0 + cidx;
    const bool col_ok = col < dv;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    const int khead = head / group;
    float *mine = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)head * dk * dv;
    const float rate = expf(to_f(a_log[head]));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    float S[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        int row = r + kDrLanes * i;
        S[i] = (start > 0 && slot_ok && col_ok && row < dk) ? mine[(size_t)row * dv + col] : 0.f;
    }
    for (int t0 = 0; t0 < count; t0 += kTok) {
        const int n = min(kTok, count - t0);
        __syncthreads();
        for (int e = threadIdx.x; e < n * dk; e += blockDim.x) {
            int j = e / dk, d = e - j * dk;
            size_t tok = (size_t)(first + t0 + j);
            size_t ai = tok * a_token + (per_channel ? (size_t)head * dk + d : (size_t)head);
            float logit = (a_f32 ? ((const float *)a)[ai] : to_f(((const T *)a)[ai])) + to_f(dt_bias[per_channel ? head * dk + d : head]);
            sx[j * 4 * KR + d] = make_float4(expf(-rate * softplus_f(logit)), to_f(k[tok * k_token + (size_t)khead * k_head + d]),
                                             to_f(q[tok * q_token + (size_t)khead * q_head + d]), 0.f);
        }
        for (int e = threadIdx.x; e < n * kDrCols; e += blockDim.x) {
            int j = e / kDrCols, d = e - j * kDrCols;
            sv[e] = col0 + d < dv ? to_f(v[(size_t)(first + t0 + j) * v_token + (size_t)head * v_head + col0 + d]) : 0.f;
        }
        if (threadIdx.x < n) {
            float bl = to_f(beta[(size_t)(first + t0 + threadIdx.x) * b_token + head]);
            sbeta[threadIdx.x] = 1.0f / (1.0f + expf(-bl));
        }
        __syncthreads();
        for (int j = warp; j < n; j += (kDrCols * kDrLanes) / 32) {  // unit vectors: one warp per token, lanes in a fixed order
            float sk = 0.f, sq = 0.f;
            for (int d = lane; d < dk; d += 32) {
                float4 x = sx[j * 4 * KR + d];
                sk = fmaf(x.y, x.y, sk);
                sq = fmaf(x.z, x.z, sq);
            }
            sk = warp_sum(sk);
            sq = warp_sum(sq);
            if (lane == 0) sinv[2 * j] = 1.0f / sqrtf(sk + unit_eps), sinv[2 * j + 1] = q_scale / sqrtf(sq + unit_eps);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n * dk; e += blockDim.x) {
            int j = e / dk, d = e - j * dk;
            float4 x = sx[j * 4 * KR + d];
            x.y *= sinv[2 * j];
            x.z *= sinv[2 * j + 1];
            sx[j * 4 * KR + d] = x;
        }
        __syncthreads();
        for (int j = 0; j < n; ++j) {
            const float4 *xa = sx + j * 4 * KR;
            float p0 = 0.f, p1 = 0.f;
#pragma unroll
            for (int i = 0; i < KR; i += 2) {
                int row = r + kDrLanes * i;
                if (row < dk) {
                    float4 x = xa[row];
                    S[i] *= x.x;
                    p0 = fmaf(x.y, S[i], p0);
                }
                if (row + kDrLanes < dk) {
                    float4 x = xa[row + kDrLanes];
                    S[i + 1] *= x.x;
                    p1 = fmaf(x.y, S[i + 1], p1);
                }
            }
            float p = p0 + p1;
            p += __shfl_xor_sync(0xffffffffu, p, 1);
            p += __shfl_xor_sync(0xffffffffu, p, 2);
            const float u = sbeta[j] * (sv[j * kDrCols + cidx] - p);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int i = 0; i < KR; i += 2) {
                int row = r + kDrLanes * i;
                if (row < dk) {
                    float4 x = xa[row];
                    S[i] = fmaf(x.y, u, S[i]);
                    o0 = fmaf(x.z, S[i], o0);
                }
                if (row + kDrLanes < dk) {
                    float4 x = xa[row + kDrLanes];
                    S[i + 1] = fmaf(x.y, u, S[i + 1]);
                    o1 = fmaf(x.z, S[i + 1], o1);
                }
            }
            float o = o0 + o1;
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (r == 0 && col_ok) out[((size_t)(first + t0 + j) * heads + head) * dv + col] = o;
        }
    }
    if (slot_ok && col_ok) {
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            int row = r + kDrLanes * i;
            if (row < dk) mine[(size_t)row * dv + col] = S[i];
        }
    }
}

// y[t, c] = silu(sum_i taps[c, K-1-i] * x[t - i, c]) along each sequence, inputs before position 0 being zero and the
// K-1 inputs before this step's first token coming from the sequence's slot (hist [C, K-1] fp32, oldest first).  One
// thread per (channel, token of a chunk); the CTA of a sequence's first chunk also leaves the slot holding the last
// K-1 inputs for the next step (it is the only one that reads the slot, so nothing races).
constexpr int kConvMaxTaps = 8;

template <typename T>
__global__ void __launch_bounds__(128)
short_conv_kernel(const T *__restrict__ x, long long x_token, const T *__restrict__ taps, int channels, int K, int act,
                  const int32_t *__restrict__ seq_info, float *__restrict__ state, long long slot_stride, int num_slots, T *__restrict__ y,
                  int chunk) {
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    const int first = seq_info[s * 4 + 0], count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    const int lo = blockIdx.z * chunk, hi = min(count, lo + chunk);
    if (c >= channels || lo >= count) return;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    float *hist = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)c * (K - 1);
    float w[kConvMaxTaps], old[kConvMaxTaps];
#pragma unroll
    for (int i = 0; i < kConvMaxTaps; ++i) {
        w[i] = i < K ? to_f(taps[(size_t)c * K + (K - 1 - i)]) : 0.f;  // w[i] multiplies the input i tokens back
        // old[i] = the input i + 1 tokens before this step's first token
        old[i] = (blockIdx.z == 0 && i < K - 1 && slot_ok && start - 1 - i >= 0) ? hist[K - 2 - i] : 0.f;
    }
    for (int j = lo; j < hi; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < kConvMaxTaps; ++i) {
            if (i < K) {
                int jj = j - i;
                float in = jj >= 0 ? to_f(x[(size_t)(first + jj) * x_token + c]) : old[min(-jj - 1, kConvMaxTaps - 1)];
                acc = fmaf(w[i], in, acc);
            }
        }
        if (act == 1) acc = acc / (1.0f + expf(-acc));
        y[(size_t)(first + j) * channels + c] = from_f<T>(acc);
    }
    if (blockIdx.z == 0 && slot_ok) {
        // hist[m] <- the input K-1-m tokens before the NEXT step's first token, m = 0 .. K-2
#pragma unroll
        for (int i = 0; i < kConvMaxTaps; ++i) {
            if (i < K - 1) {
                int jj = count - 1 - i;  // i tokens before the last one of this step
                hist[K - 2 - i] = jj >= 0 ? to_f(x[(size_t)(first + jj) * x_token + c]) : old[min(-jj - 1, kConvMaxTaps - 1)];
            }
        }
    }
}

// cos / sin of position * base^(-2 i / dims) / factor for every token: tables [rows, dims / 2] fp32 that kernels rotating in
// fp32 (those that feed a recurrence) read instead of evaluating the angle themselves.
__global__ void rope_table_kernel(const int32_t *__restrict__ tok_pos, int dims, double log2_base, double inv_factor, float *__restrict__ cs,
                                  float *__restrict__ sn) {
    const int row = blockIdx.x, half = dims / 2;
    const int pos = tok_pos[row];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double freq = exp2(-2.0 * (double)i / (double)dims * log2_base) * inv_factor;
        double s, c;
        sincos((double)pos * freq, &s, &c);
        cs[(size_t)row * half + i] = (float)c;
        sn[(size_t)row * half + i] = (float)s;
    }
}

}  // namespace tlb

using namespace tlb;

extern "C" {

int tlb_delta_scan(const void *q, long long q_token, long long q_head, const void *k, long long k_token, long long k_head, const void *v,
                   long long v_token, long long v_head, const void *beta, long long b_token, const void *a, int a_is_f32, long long a_token,
                   int per_channel, const void *a_log, const void *dt_bias, float q_scale, float unit_eps, int heads, int key_heads, int dk, int dv,
                   const int32_t *seq_info, int num_seqs, float *state, long long slot_stride, int num_slots, float *out, int dtype, void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (!q || !k || !v || !beta || !a || !a_log || !dt_bias || !seq_info || !state || !out || heads <= 0 || key_heads <= 0 || heads % key_heads ||
        dk <= 0 || dv <= 0 || num_slots <= 0)
        return tl::fail(TL_EINVAL, "delta_scan: bad argument");
    if (dk > 256) return tl::fail(TL_EINVAL, "delta_scan: key size %d > 256", dk);
    const int colblocks = ceil_div(dv, kDrCols), group = heads / key_heads;
    cudaStream_t st = as_stream(stream);
    const int kr = ceil_div(dk, kDrLanes);
#define TLB_DR_K(KRV)                                                                                                                              \
    delta_scan_kernel<T, KRV, (KRV > 32 ? 8 : 16)><<<dim3(num_seqs, heads * colblocks), kDrCols * kDrLanes, 0, st>>>(                               \
        (const T *)q, q_token, q_head, (const T *)k, k_token, k_head, (const T *)v, v_token, v_head, (const T *)beta, b_token, a, a_is_f32, a_token, \
        per_channel, (const T *)a_log, (const T *)dt_bias, q_scale, unit_eps, heads, group, dk, dv, seq_info, state, slot_stride, num_slots, out)
    TLB_DISPATCH(dtype, "delta_scan", if (kr <= 8) TLB_DR_K(8); else if (kr <= 16) TLB_DR_K(16); else if (kr <= 32) TLB_DR_K(32); else TLB_DR_K(64));
#undef TLB_DR_K
    TL_LAUNCH_CHECK("delta_scan");
    return TL_OK;
}

int tlb_short_conv(const void *x, long long x_token, const void *taps, int channels, int num_taps, int act, const int32_t *seq_info, int num_seqs,
                   int max_tokens_per_seq, float *state, long long slot_stride, int num_slots, void *y, int dtype, void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (!x || !taps || !seq_info || !y || channels <= 0 || num_taps <= 0 || max_tokens_per_seq <= 0 || (num_taps > 1 && (!state || num_slots <= 0)) ||
        act < 0 || act > 1)
        return tl::fail(TL_EINVAL, "short_conv: bad argument");
    if (num_taps > kConvMaxTaps) return tl::fail(TL_EINVAL, "short_conv: %d taps > %d", num_taps, kConvMaxTaps);
    const int chunk = 32;
    dim3 grid(num_seqs, ceil_div(channels, 128), ceil_div(max_tokens_per_seq, chunk));
    TLB_DISPATCH(dtype, "short_conv",
                 short_conv_kernel<T><<<grid, 128, 0, as_stream(stream)>>>((const T *)x, x_token, (const T *)taps, channels, num_taps, act, seq_info,
                                                                          state, slot_stride, num_slots, (T *)y, chunk));
    TL_LAUNCH_CHECK("short_conv");
    return TL_OK;
}

int tlb_rope_table(const int32_t *tok_pos, int rows, int dims, double base, double factor, float *cos_out, float *sin_out, void *stream) {
    if (rows <= 0 || dims <= 0) return TL_OK;
    if (!tok_pos || !cos_out || !sin_out || (dims & 1) || base <= 0 || !(factor > 0)) return tl::fail(TL_EINVAL, "rope_table: bad argument");
    rope_table_kernel<<<rows, 64, 0, as_stream(stream)>>>(tok_pos, dims, log2(base), 1.0 / factor, cos_out, sin_out);
    TL_LAUNCH_CHECK("rope_table");
    return TL_OK;
}

}  // extern "C"
