// Linear attention with a decay (a recurrent mixer) over ragged batches, its state kept in fp32 slots.
//
// Per sequence and head a matrix S [dk, dv] is carried from token to token:
//     S <- diag(alpha_t) S + k_t v_t^T,      o_t = S^T (q_scale * q_t),
//     alpha_t = sigmoid(z_t + bias)^(1 / tau) = exp(log_sigmoid(z_t + bias) / tau)        (per key channel)
// or, given head_decay, one fixed alpha per head (retention).  With rotation tables the first rope_dims entries of every
// head of q and k are rotated by the token's tabulated angle while they are staged, in fp32: what enters the recurrence is
// never rounded back to the projections' type.
// The columns of S never mix, so a CTA owns 32 of them for one (sequence, head) and walks tokens in order; 4 lanes share
// a column, each holding every 4th row of it in registers.  The tokens' q, k and decays are staged 16 (8 for dk > 128) at a time in shared
// memory as fp32 (the decay is computed there, in fp32, from the fp32 logits).  A sequence that starts at position 0
// starts from zero, whatever its slot held; otherwise the slot is read, and in both cases written back after the last
// token.  Single tokens and portions of up to 64 tokens are one walk.  A longer portion is cut into segments at the
// multiples of 64 in ABSOLUTE positions, which run side by side: every segment's local end state from zero and the
// product of its decays, then the start state of every segment by walking those in order (S' = decay * S + local), then
// the outputs of every segment from its start state.  Every sum has an order fixed by token, channel and segment
// indices alone; the cuts depend on positions only, so how a prompt was cut into steps changes the result by the
// rounding of the combination at most.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kLaCols = 32;    // state columns per CTA
constexpr int kLaLanes = 4;    // lanes per column
constexpr int kLaSegment = TLB_DECAY_SCAN_SEGMENT;  // positions per segment of a long portion

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// Segment c of a sequence's new tokens [p0, p0 + n): cut at the multiples of kLaSegment in ABSOLUTE positions, so that
// where a prompt was cut into steps does not move the cuts.  Returns false when the sequence has no segment c.
__device__ __forceinline__ bool la_segment(int p0, int n, int c, int &lo, int &hi, int &nseg) {
    const int end = p0 + n, b0 = (p0 / kLaSegment + 1) * kLaSegment;
    nseg = (n <= kLaSegment || end <= b0) ? 1 : 1 + (end - b0 + kLaSegment - 1) / kLaSegment;  // a short portion is never cut
    if (c >= nseg) return false;
    lo = c == 0 ? p0 : b0 + (c - 1) * kLaSegment;
    hi = nseg == 1 ? end : min(end, c == 0 ? b0 : lo + kLaSegment);
    return true;
}

// One kernel, three uses (pass):
//   0  the whole portion of a sequence in one CTA per (head, column block): state from the slot (or zero at position 0),
//      outputs, state back to the slot.  Single tokens and short portions.
//   1  segment c alone from a ZERO state, no outputs: its local end state and the product of its decays go to the
//      workspace (the last segment of a sequence is skipped: nobody needs its local state).
//   3  segment c from the start state that decay_combine_kernel left in the workspace: outputs; the last segment writes
//      the slot.
//
// decay_kind chooses where the decay comes from: 0 = sigmoid(z + bias)^(1/tau) per key channel, or head_decay; 2 = exp(-exp(z + bias))
// per key channel; 3 = one number per head and token, exp(-exp(a_log[h]) dt) with dt = softplus(z[t, h] + bias[h]), and the
// token's key is multiplied by dt (a discretised state-space step).  q and k may have fewer heads than v (qk_heads; head h
// reads query/key head h / (heads / qk_heads)).  skip [heads]: o_t += skip[h] v_t.  BONUS: the read-out comes BEFORE the
// update and sees the token's own k v^T weighted by bonus [heads, dk] instead: o_t = (S + diag(bonus) k_t v_t^T)^T q_t.
template <typename T, int KR /* rows per lane: dk <= 4 * KR */, int kLaTokens /* tokens staged at a time */, bool BONUS>
__global__ void __launch_bounds__(kLaCols * kLaLanes)
decay_scan_kernel(const T *__restrict__ q, long long q_token, long long q_head, const T *__restrict__ k, long long k_token, long long k_head,
                  const T *__restrict__ v, long long v_token, long long v_head, const float *__restrict__ z, long long z_token,
                  const T *__restrict__ z_bias, float inv_tau, const float *__restrict__ head_decay, const float *__restrict__ rope_cos,
                  const float *__restrict__ rope_sin, int rope_dims, int rope_interleaved, float q_scale, int heads, int dk, int dv,
                  const int32_t *__restrict__ seq_info,
                  float *__restrict__ state, long long slot_stride, int num_slots, float *__restrict__ out, int pass, int max_segments,
                  float *__restrict__ seg_state, float *__restrict__ seg_decay, int decay_kind, const T *__restrict__ a_log,
                  const T *__restrict__ bonus, int qk_heads, const T *__restrict__ skip) {
    __shared__ float4 sx[kLaTokens * 4 * KR];  // per token and key channel: (decay, k, scaled q, -), one 16-byte read per row
    __shared__ float sv[kLaTokens * kLaCols];
    __shared__ float sprod[4 * KR];
    __shared__ float2 s_step[kLaTokens];  // decay_kind 3: the token's (decay, step size), worked out once per token
    __shared__ float2 s_chan[4 * KR];     // per key channel of this head: (the decay logit's bias, the bonus), read once
    const int colblocks = (dv + kLaCols - 1) / kLaCols;
    const int s = blockIdx.x, head = blockIdx.y / colblocks, col0 = (blockIdx.y % colblocks) * kLaCols, c = blockIdx.z;
    const int seq_first = seq_info[s * 4 + 0], seq_count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    int lo = start, hi = start + seq_count, nseg = 1;
    if (pass != 0 && !la_segment(start, seq_count, c, lo, hi, nseg)) return;
    if (pass == 1 && c == nseg - 1) return;
    const int first = seq_first + (lo - start), count = hi - lo;
    const int cidx = threadIdx.x / kLaLanes, r = threadIdx.x % kLaLanes;
    const int col = col0 + cidx;
    const bool col_ok = col < dv;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    float *mine = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)head * dk * dv;
    float *seg = seg_state ? seg_state + (((size_t)s * max_segments + c) * heads + head) * dk * dv : nullptr;
    const bool from_slot = pass == 0 || (pass == 3 && c == 0);   // else: zero (pass 1) or the combined start state (pass 3)
    const bool to_slot = pass == 0 || (pass == 3 && c == nseg - 1);

    float S[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        int row = r + kLaLanes * i;
        bool ok = col_ok && row < dk;
        if (from_slot) S[i] = (lo > 0 && slot_ok && ok) ? mine[(size_t)row * dv + col] : 0.f;
        else S[i] = (pass == 3 && ok) ? seg[(size_t)row * dv + col] : 0.f;
    }
    if (pass == 1)
        for (int d = threadIdx.x; d < dk; d += blockDim.x) sprod[d] = 1.f;
    for (int d = threadIdx.x; d < dk; d += blockDim.x)
        s_chan[d] = make_float2((z_bias && decay_kind != 3) ? to_f(z_bias[(size_t)head * dk + d]) : 0.f, BONUS ? to_f(bonus[(size_t)head * dk + d]) : 0.f);
    const int qk_head = head / (heads / qk_heads);
    const float rate = decay_kind == 3 ? expf(to_f(a_log[head])) : 0.f;
    const float skipv = skip ? to_f(skip[head]) : 0.f;
    for (int t0 = 0; t0 < count; t0 += kLaTokens) {
        const int n = min(kLaTokens, count - t0);
        __syncthreads();
        if (decay_kind == 3) {
            if (threadIdx.x < n) {
                const float zz = z[(size_t)(first + t0 + threadIdx.x) * z_token + head] + (z_bias ? to_f(z_bias[head]) : 0.f);
                const float dt = zz > 20.f ? zz : log1pf(expf(zz));
                s_step[threadIdx.x] = make_float2(expf(-rate * dt), dt);
            }
            __syncthreads();
        }
        for (int e = threadIdx.x; e < n * dk; e += blockDim.x) {
            int j = e / dk, d = e - j * dk;
            size_t tok = (size_t)(first + t0 + j);
            float alpha, kmul = 1.f;
            if (head_decay) alpha = head_decay[head];
            else if (decay_kind == 2) alpha = expf(-expf(z[tok * z_token + (size_t)head * dk + d] + s_chan[d].x));
            else if (decay_kind == 3) alpha = s_step[j].x, kmul = s_step[j].y;
            else alpha = expf(log_sigmoid(z[tok * z_token + (size_t)head * dk + d] + s_chan[d].x) * inv_tau);
            const T *kp = k + tok * k_token + (size_t)qk_head * k_head, *qp = q + tok * q_token + (size_t)qk_head * q_head;
            float kd = to_f(kp[d]), qd = to_f(qp[d]);
            if (d < rope_dims) {  // rotate the pair this entry belongs to, in fp32, by the token's tabulated angle
                const int half = rope_dims >> 1;
                const bool low = rope_interleaved ? !(d & 1) : d < half;
                const int i = rope_interleaved ? d >> 1 : (low ? d : d - half);
                const int other = rope_interleaved ? (d ^ 1) : (low ? d + half : d - half);
                const float c = rope_cos[tok * half + i], sn = low ? -rope_sin[tok * half + i] : rope_sin[tok * half + i];
                kd = kd * c + to_f(kp[other]) * sn;
                qd = qd * c + to_f(qp[other]) * sn;
            }
            kd *= kmul;
            sx[j * 4 * KR + d] = make_float4(alpha, kd, qd * q_scale, BONUS ? kd * s_chan[d].y : 0.f);
        }
        for (int e = threadIdx.x; e < n * kLaCols; e += blockDim.x) {
            int j = e / kLaCols, d = e - j * kLaCols;
            sv[e] = col0 + d < dv ? to_f(v[(size_t)(first + t0 + j) * v_token + (size_t)head * v_head + col0 + d]) : 0.f;
        }
        __syncthreads();
        if (pass == 1) {  // the segment's decay product per key channel, in token order
            for (int d = threadIdx.x; d < dk; d += blockDim.x) {
                float p = sprod[d];
                for (int j = 0; j < n; ++j) p *= sx[j * 4 * KR + d].x;
                sprod[d] = p;
            }
        }
        for (int j = 0; j < n; ++j) {
            const float vj = sv[j * kLaCols + cidx];
            const float4 *xa = sx + j * 4 * KR;
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int i = 0; i < KR; i += 2) {
                int row = r + kLaLanes * i;
                if (row < dk) {
                    float4 x = xa[row];
                    if (BONUS) o0 = fmaf(x.z, fmaf(x.w, vj, S[i]), o0);
                    S[i] = fmaf(x.x, S[i], x.y * vj);
                    if (!BONUS) o0 = fmaf(x.z, S[i], o0);
                }
                if (row + kLaLanes < dk) {
                    float4 x = xa[row + kLaLanes];
                    if (BONUS) o1 = fmaf(x.z, fmaf(x.w, vj, S[i + 1]), o1);
                    S[i + 1] = fmaf(x.x, S[i + 1], x.y * vj);
                    if (!BONUS) o1 = fmaf(x.z, S[i + 1], o1);
                }
            }
            if (pass != 1) {
                float o = o0 + o1;
                o += __shfl_xor_sync(0xffffffffu, o, 1);
                o += __shfl_xor_sync(0xffffffffu, o, 2);
                if (r == 0 && col_ok) out[((size_t)(first + t0 + j) * heads + head) * dv + col] = fmaf(skipv, vj, o);
            }
        }
    }
    float *dst = to_slot ? (slot_ok ? mine : nullptr) : (pass == 1 ? seg : nullptr);
    if (dst != nullptr && col_ok) {
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            int row = r + kLaLanes * i;
            if (row < dk) dst[(size_t)row * dv + col] = S[i];
        }
    }
    if (pass == 1 && col0 == 0) {
        __syncthreads();
        float *pd = seg_decay + (((size_t)s * max_segments + c) * heads + head) * dk;
        for (int d = threadIdx.x; d < dk; d += blockDim.x) pd[d] = sprod[d];
    }
}

// Between the two passes: walk a sequence's segments in order, S_start[c + 1] = decay[c] * S_start[c] + local[c], and leave
// every segment's START state where its local end state was.  One thread per state element, (sequence, head) per blockIdx.
__global__ void __launch_bounds__(256)
decay_combine_kernel(const int32_t *__restrict__ seq_info, const float *__restrict__ state, long long slot_stride, int num_slots, int heads, int dk,
                     int dv, int max_segments, float *__restrict__ seg_state, const float *__restrict__ seg_decay) {
    const int s = blockIdx.x, head = blockIdx.y;
    const int count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    int lo, hi, nseg;
    la_segment(start, count, 0, lo, hi, nseg);
    if (nseg <= 1) return;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    const float *mine = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)head * dk * dv;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < dk * dv; e += gridDim.z * blockDim.x) {
        const int row = e / dv;
        float S = (start > 0 && slot_ok) ? mine[e] : 0.f;
        // eight segments' local states and decays are fetched before the first of them is used: the walk is a chain of
        // multiply-adds, not of memory round trips
        constexpr int kAhead = 8;
        for (int c0 = 0; c0 + 1 < nseg; c0 += kAhead) {
            float local[kAhead], decay[kAhead];
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int c = c0 + u;
                if (c + 1 < nseg) {
                    local[u] = seg_state[(((size_t)s * max_segments + c) * heads + head) * dk * dv + e];
                    decay[u] = seg_decay[(((size_t)s * max_segments + c) * heads + head) * dk + row];
                }
            }
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int c = c0 + u;
                if (c + 1 < nseg) {
                    seg_state[(((size_t)s * max_segments + c) * heads + head) * dk * dv + e] = S;
                    S = fmaf(decay[u], S, local[u]);
                }
            }
        }
        seg_state[(((size_t)s * max_segments + (nseg - 1)) * heads + head) * dk * dv + e] = S;
    }
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * act(gate[t, h, :]); one warp per (token, head).  act 0 = none, 1 = silu,
// 2 = sigmoid; w == NULL: no weight; wide_weight: w is [heads * dv] (every head its own part) instead of [dv] shared by the
// heads; gate_first: the gate multiplies o BEFORE the norm, out = n / rms(n) * w with n = o * act(gate).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float *__restrict__ o, const T *__restrict__ w, float eps, const T *__restrict__ gate, long long g_token, int act,
                      T *__restrict__ out, long long rows, int heads, int dv, int wide_weight, int gate_first) {
    long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = row / heads;
    const int head = (int)(row - t * heads);
    const float *src = o + (size_t)row * dv;
    auto gated = [&](int d) {
        float gv = to_f(gate[(size_t)t * g_token + (size_t)head * dv + d]);
        return act == 1 ? gv / (1.0f + expf(-gv)) : act == 2 ? 1.0f / (1.0f + expf(-gv)) : gv;
    };
    const bool first = gate && gate_first;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) {
        float x = first ? src[d] * gated(d) : src[d];
        ss += x * x;
    }
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const T *wr = w ? w + (wide_weight ? (size_t)head * dv : 0) : nullptr;
    for (int d = lane; d < dv; d += 32) {
        float y = src[d] * inv * (wr ? to_f(wr[d]) : 1.f);
        if (gate) y *= gated(d);
        out[(size_t)row * dv + d] = from_f<T>(y);
    }
}

}  // namespace tlb

using namespace tlb;

extern "C" {

size_t tlb_decay_scan_workspace(int num_seqs, int max_tokens_per_seq, int heads, int dk, int dv) {
    if (max_tokens_per_seq <= kLaSegment) return 0;
    size_t segs = (size_t)num_seqs * (2 + (max_tokens_per_seq - 1) / kLaSegment);
    return segs * heads * ((size_t)dk * dv + dk) * sizeof(float);
}

int tlb_decay_scan(const void *q, long long q_token, long long q_head, const void *k, long long k_token, long long k_head, const void *v,
                   long long v_token, long long v_head, const float *z, long long z_token, const void *z_bias, float tau, const float *head_decay,
                   const float *rope_cos, const float *rope_sin, int rope_dims, int rope_interleaved, float q_scale, int heads,
                   int dk, int dv, const int32_t *seq_info, int num_seqs, int max_tokens_per_seq, float *state, long long slot_stride, int num_slots,
                   float *out, void *workspace, size_t workspace_bytes, int decay_kind, const void *a_log, const void *bonus, int qk_heads,
                   const void *skip, int dtype, void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (qk_heads <= 0) qk_heads = heads;
    if ((decay_kind != 0 && decay_kind != 2 && decay_kind != 3) || (decay_kind != 0 && (!z || head_decay)) || (decay_kind == 3 && !a_log) ||
        heads % qk_heads)
        return tl::fail(TL_EINVAL, "decay_scan: bad decay kind or head groups");
    if (!q || !k || !v || (!z && !head_decay) || !seq_info || !state || !out || heads <= 0 || dk <= 0 || dv <= 0 || (z && !(tau > 0.f)) ||
        num_slots <= 0 || max_tokens_per_seq <= 0)
        return tl::fail(TL_EINVAL, "decay_scan: bad argument");
    if (rope_dims < 0 || (rope_dims & 1) || rope_dims > dk || (rope_dims > 0 && (!rope_cos || !rope_sin)))
        return tl::fail(TL_EINVAL, "decay_scan: bad rotation of %d of %d entries", rope_dims, dk);
    if (dk > 256) return tl::fail(TL_EINVAL, "decay_scan: key size %d > 256", dk);
    // portions longer than a segment are cut at absolute multiples of the segment length and run in three passes
    const bool segmented = max_tokens_per_seq > kLaSegment;
    const int max_segments = segmented ? 2 + (max_tokens_per_seq - 1) / kLaSegment : 1;
    float *seg_state = nullptr, *seg_decay = nullptr;
    if (segmented) {
        if (!workspace || workspace_bytes < tlb_decay_scan_workspace(num_seqs, max_tokens_per_seq, heads, dk, dv))
            return tl::fail(TL_EWORKSPACE, "decay_scan: workspace missing or too small");
        seg_state = (float *)workspace;
        seg_decay = seg_state + (size_t)num_seqs * max_segments * heads * dk * dv;
    }
    const int colblocks = ceil_div(dv, kLaCols);
    cudaStream_t st = as_stream(stream);
    int kr = ceil_div(dk, kLaLanes);
#define TLB_DS_B(KRV, PASS, GZ, BON)                                                                                                                \
    decay_scan_kernel<T, KRV, (KRV > 32 ? 8 : 16), BON><<<dim3(num_seqs, heads * colblocks, GZ), kLaCols * kLaLanes, 0, st>>>(                                           \
        (const T *)q, q_token, q_head, (const T *)k, k_token, k_head, (const T *)v, v_token, v_head, z, z_token, (const T *)z_bias, z ? 1.0f / tau : 0.f, head_decay, \
        rope_cos, rope_sin, rope_dims, rope_interleaved, q_scale, heads, dk, dv, seq_info, state, slot_stride, num_slots, out, PASS, max_segments, seg_state, seg_decay, \
        decay_kind, (const T *)a_log, (const T *)bonus, qk_heads, (const T *)skip)
#define TLB_DS_K(KRV, PASS, GZ) do { if (bonus) TLB_DS_B(KRV, PASS, GZ, true); else TLB_DS_B(KRV, PASS, GZ, false); } while (0)
#define TLB_DS(PASS, GZ) TLB_DISPATCH(dtype, "decay_scan", if (kr <= 8) TLB_DS_K(8, PASS, GZ); else if (kr <= 16) TLB_DS_K(16, PASS, GZ); else if (kr <= 32) TLB_DS_K(32, PASS, GZ); else TLB_DS_K(64, PASS, GZ))
    if (!segmented) {
        TLB_DS(0, 1);
        TL_LAUNCH_CHECK("decay_scan");
        return TL_OK;
    }
    TLB_DS(1, max_segments);
    TL_LAUNCH_CHECK("decay_scan (local states)");
    decay_combine_kernel<<<dim3(num_seqs, heads, ceil_div(dk * dv, 256)), 256, 0, st>>>(seq_info, state, slot_stride, num_slots, heads, dk, dv,
                                                                                           max_segments, seg_state, seg_decay);
    TL_LAUNCH_CHECK("decay_scan (combine)");
    TLB_DS(3, max_segments);
    TL_LAUNCH_CHECK("decay_scan (outputs)");
#undef TLB_DS
#undef TLB_DS_K
#undef TLB_DS_B
    return TL_OK;
}

int tlb_head_norm_gate(const float *o, const void *w, float eps, const void *gate, long long g_token, int act, void *out, int tokens, int heads,
                       int dv, int wide_weight, int gate_first, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!o || !out || heads <= 0 || dv <= 0 || act < 0 || act > 2) return tl::fail(TL_EINVAL, "head_norm_gate: bad argument");
    long long rows = (long long)tokens * heads;
    TLB_DISPATCH(dtype, "head_norm_gate",
                 head_norm_gate_kernel<T><<<(unsigned)((rows + 3) / 4), 128, 0, as_stream(stream)>>>(o, (const T *)w, eps, (const T *)gate, g_token, act,
                                                                                                    (T *)out, rows, heads, dv, wide_weight, gate_first));
    TL_LAUNCH_CHECK("head_norm_gate");
    return TL_OK;
}

}  // extern "C"
