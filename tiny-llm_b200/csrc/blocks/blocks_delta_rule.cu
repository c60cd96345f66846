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
// after the last token.  Single tokens and portions of up to 64 tokens are one walk, whose sums have an order fixed by token
// and channel indices alone.  A longer portion is cut into segments at the multiples of 64 in ABSOLUTE positions, which run
// side by side.  The state after a segment is linear in the state before it, S_end = P S_start + L with P [dk, dk] the
// product of the tokens' transitions (I - beta k k^T) diag(g) and L the end state from zero, and the columns of P come out of
// the same walk started from the identity with zero values.  So: every segment's L and P (pass 1), the segments' start
// states by walking those in order (delta_combine_kernel), then the outputs of every segment from its start state (pass
// 3).  The cuts depend on positions only, so how a prompt was cut into steps changes a result by the rounding of the
// combination at most.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kDrCols = 32;   // state columns per CTA
constexpr int kDrLanes = 4;   // lanes per column

constexpr int kDrSegment = TLB_DELTA_SCAN_SEGMENT;  // positions per segment of a long portion

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// Segment c of a sequence's new tokens [p0, p0 + n), cut at the multiples of kDrSegment in absolute positions; a portion of
// at most one segment's length is never cut.  Returns false when the sequence has no segment c.
__device__ __forceinline__ bool dr_segment(int p0, int n, int c, int &lo, int &hi, int &nseg) {
    const int end = p0 + n, b0 = (p0 / kDrSegment + 1) * kDrSegment;
    nseg = (n <= kDrSegment || end <= b0) ? 1 : 1 + (end - b0 + kDrSegment - 1) / kDrSegment;
    if (c >= nseg) return false;
    lo = c == 0 ? p0 : b0 + (c - 1) * kDrSegment;
    hi = nseg == 1 ? end : min(end, c == 0 ? b0 : lo + kDrSegment);
    return true;
}

// One kernel, three uses (pass):
//   0  the whole portion of a sequence in one CTA per (head, column block): state from the slot (or zero at position 0),
//      outputs, state back to the slot.
//   1  segment c alone, no outputs.  Column blocks below `colblocks` walk the value columns from a ZERO state (L); the
//      blocks after them walk the dk columns of the identity with zero values (P).  Both go to the workspace; the last
//      segment of a sequence is skipped (nobody needs what follows it).
//   3  segment c from the start state that delta_combine_kernel left in the workspace: outputs; the last segment writes
//      the slot.  A sequence of the launch that is short enough for one walk runs here as in pass 0.

template <typename T, int KR /* rows per lane: dk <= 4 * KR */, int kTok /* tokens staged at a time */>
__global__ void __launch_bounds__(kDrCols * kDrLanes)
delta_scan_kernel(const T *__restrict__ q, long long q_token, long long q_head, const T *__restrict__ k, long long k_token, long long k_head,
                  const T *__restrict__ v, long long v_token, long long v_head, const T *__restrict__ beta, long long b_token,
                  const void *__restrict__ a, int a_f32, long long a_token, int per_channel, const T *__restrict__ a_log,
                  const T *__restrict__ dt_bias, float q_scale, float unit_eps, int heads, int group, int dk, int dv,
                  const int32_t *__restrict__ seq_info, float *__restrict__ state, long long slot_stride, int num_slots, float *__restrict__ out,
                  int pass, int max_segments, float *__restrict__ seg_state, float *__restrict__ seg_trans) {
    __shared__ float4 sx[kTok * 4 * KR];  // per token and key channel: (decay, k, q, -)
    __shared__ float sv[kTok * kDrCols];
    __shared__ float sbeta[kTok];
    __shared__ float sinv[kTok * 2];
    const int colblocks = (dv + kDrCols - 1) / kDrCols, kblocks = (dk + kDrCols - 1) / kDrCols;
    const int per_head = pass == 1 ? colblocks + kblocks : colblocks;
    const int s = blockIdx.x, head = blockIdx.y / per_head, block = blockIdx.y % per_head, c = blockIdx.z;
    const bool trans = block >= colblocks;  // pass 1 only: a block of columns of the identity
    const int col0 = (trans ? block - colblocks : block) * kDrCols, width = trans ? dk : dv;
    const int seq_first = seq_info[s * 4 + 0], seq_count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    int lo = start, hi = start + seq_count, nseg = 1;
    if (pass != 0 && !dr_segment(start, seq_count, c, lo, hi, nseg)) return;
    if (pass == 1 && c == nseg - 1) return;
    const bool whole = pass == 0 || (pass == 3 && nseg == 1);  // a short portion in a launch with long ones runs as in pass 0
    const int first = seq_first + (lo - start), count = hi - lo;
    const int cidx = threadIdx.x / kDrLanes, r = threadIdx.x % kDrLanes;
    const int col = col0 + cidx;
    const bool col_ok = col < width;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    const int khead = head / group;
    float *mine = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)head * dk * dv;
    const size_t seg_index = ((size_t)s * max_segments + c) * heads + head;
    float *seg = seg_state ? seg_state + seg_index * dk * dv : nullptr;
    const float rate = expf(to_f(a_log[head]));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    float S[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        int row = r + kDrLanes * i;
        bool ok = col_ok && row < dk;
        if (whole) S[i] = (start > 0 && slot_ok && ok) ? mine[(size_t)row * dv + col] : 0.f;
        else if (pass == 1) S[i] = (trans && ok && row == col) ? 1.f : 0.f;
        else S[i] = ok ? seg[(size_t)row * dv + col] : 0.f;
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
            sv[e] = (!trans && col0 + d < dv) ? to_f(v[(size_t)(first + t0 + j) * v_token + (size_t)head * v_head + col0 + d]) : 0.f;
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
            if (pass != 1) {
                float o = o0 + o1;
                o += __shfl_xor_sync(0xffffffffu, o, 1);
                o += __shfl_xor_sync(0xffffffffu, o, 2);
                if (r == 0 && col_ok) out[((size_t)(first + t0 + j) * heads + head) * dv + col] = o;
            }
        }
    }
    // where the end state goes: the slot (the whole portion, or its last segment), or the workspace (L or P of a segment)
    float *dst = nullptr;
    if (pass == 1) dst = trans ? seg_trans + seg_index * dk * dk : seg;
    else if ((whole || c == nseg - 1) && slot_ok) dst = mine;
    if (dst != nullptr && col_ok) {
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            int row = r + kDrLanes * i;
            if (row < dk) dst[trans ? (size_t)col * dk + row : (size_t)row * dv + col] = S[i];  // P goes out transposed: Pt[j][row]
        }
    }
}

// Between the two passes: walk a sequence's segments in order, S_start[c + 1] = P[c] S_start[c] + L[c], and leave every
// segment's START state where its L was.  One CTA per (sequence, head, 32 state columns): the columns never mix.  The
// CTA keeps its 32 columns of S in shared memory, lanes = columns; pass 1 stored P transposed (Pt[j][row]), so with the
// segment's Pt staged in shared memory (the next segment's arrives by cp.async meanwhile) a warp takes four rows at a time
// from one 16-byte broadcast read per j; every sum runs over j in order.  STAGE = false (dk too large for shared memory)
// reads Pt from global memory instead.
constexpr int kDcThreads = 256;

__device__ __forceinline__ void dr_cp_async16(void *dst, const void *src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// Pt of one segment into shared memory, rows padded to dkp: 16-byte asynchronous copies when nothing has to be padded, else
// plain loads; one commit group per call either way.
__device__ __forceinline__ void dr_stage_pt(float *dst, const float *src, int dk, int dkp) {
    if (dk == dkp) {
        for (int e = threadIdx.x * 4; e < dk * dk; e += kDcThreads * 4) dr_cp_async16(dst + e, src + e);
    } else {
        for (int e = threadIdx.x; e < dk * dkp; e += kDcThreads) {
            int j = e / dkp, row = e - j * dkp;
            dst[e] = row < dk ? src[(size_t)j * dk + row] : 0.f;
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

template <bool STAGE>
__global__ void __launch_bounds__(kDcThreads)
delta_combine_kernel(const int32_t *__restrict__ seq_info, const float *__restrict__ state, long long slot_stride, int num_slots, int heads, int dk,
                     int dv, int max_segments, float *__restrict__ seg_state, const float *__restrict__ seg_trans) {
    extern __shared__ float4 combine_smem[];
    const int dkp = (dk + 3) & ~3;                   // rows padded to whole groups of four
    float *cur = (float *)combine_smem, *nxt = cur + dkp * kDrCols;  // [dkp][32] each
    float *pt = nxt + dkp * kDrCols, *pt_next = pt + dk * dkp;        // STAGE: Pt [dk][dkp] of this segment and of the next
    const int colblocks = (dv + kDrCols - 1) / kDrCols;
    const int s = blockIdx.x, head = blockIdx.y / colblocks, col0 = (blockIdx.y % colblocks) * kDrCols;
    const int count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    int lo, hi, nseg;
    dr_segment(start, count, 0, lo, hi, nseg);
    if (nseg <= 1) return;
    const bool slot_ok = slot >= 0 && slot < num_slots;
    const float *mine = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)head * dk * dv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, col = col0 + lane, warps = kDcThreads / 32;
    const bool col_ok = col < dv;
    const size_t idx0 = (size_t)s * max_segments * heads + head, idx_step = heads;  // workspace index of segment c: idx0 + c * idx_step
    if (STAGE) dr_stage_pt(pt, seg_trans + idx0 * dk * dk, dk, dkp);
    for (int row = warp; row < dkp; row += warps)
        cur[row * kDrCols + lane] = (row < dk && start > 0 && slot_ok && col_ok) ? mine[(size_t)row * dv + col] : 0.f;
    for (int c = 0; c < nseg; ++c) {
        const size_t idx = idx0 + (size_t)c * idx_step;
        float *cell = seg_state + idx * dk * dv;
        const float *gpt = seg_trans + idx * dk * dk;  // Pt[j * dk + row]
        const bool last = c == nseg - 1;
        if (STAGE && !last) {  // the next segment's Pt loads under this segment's products
            if (c + 1 < nseg - 1) {
                dr_stage_pt(pt_next, seg_trans + (idx + idx_step) * dk * dk, dk, dkp);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
        }
        __syncthreads();  // cur (and pt) are complete
        for (int g4 = warp * 4; g4 < dkp; g4 += warps * 4) {
            float local[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = g4 + i;
                const bool ok = row < dk && col_ok;
                local[i] = (!last && ok) ? cell[(size_t)row * dv + col] : 0.f;
                if (ok) cell[(size_t)row * dv + col] = cur[row * kDrCols + lane];  // the segment's start state
            }
            if (last) continue;
#pragma unroll 4
            for (int j = 0; j < dk; ++j) {
                const float x = cur[j * kDrCols + lane];
                if (STAGE) {
                    const float4 p = *reinterpret_cast<const float4 *>(pt + j * dkp + g4);
                    acc[0] = fmaf(p.x, x, acc[0]);
                    acc[1] = fmaf(p.y, x, acc[1]);
                    acc[2] = fmaf(p.z, x, acc[2]);
                    acc[3] = fmaf(p.w, x, acc[3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (g4 + i < dk) acc[i] = fmaf(gpt[(size_t)j * dk + g4 + i], x, acc[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) nxt[(g4 + i) * kDrCols + lane] = acc[i] + local[i];
        }
        __syncthreads();  // everybody is done with cur and pt
        float *t = cur;
        cur = nxt;
        nxt = t;
        t = pt;
        pt = pt_next;
        pt_next = t;
    }
}

// y[t, c] = act(bias[c] + sum_i taps[c, K-1-i] * x[t - i, c] (+ x[t, c], add_input)) along each sequence, act = silu or none, inputs before position 0 being zero and the
// K-1 inputs before this step's first token coming from the sequence's slot (hist [C, K-1] fp32, oldest first).  A thread
// owns V adjacent channels (V = 2: one 4- or 8-byte access per token) for a chunk of tokens and slides the last K inputs
// through registers, so every input is read once (plus the K-1 before the chunk), eight tokens' inputs fetched ahead.  KT = the number of taps when it is one
// of the usual few (the window then lives in registers with no moves), 0 = any number up to kConvMaxTaps.  The CTAs of a
// sequence's first chunk also leave the slot holding the last K-1 inputs for the next step (they are the only ones that
// read the slot, and a thread reads what it needs of its channels before it writes them, so nothing races).
constexpr int kConvMaxTaps = 16;
constexpr int kConvChunk = 64, kConvSmallChunk = 16;  // tokens per CTA; the small one when the launch would leave SMs idle

template <typename T, int V> struct ConvIo;
template <typename T> struct ConvIo<T, 1> {
    static __device__ __forceinline__ void load(const T *p, float *v) { v[0] = to_f(p[0]); }
    static __device__ __forceinline__ void store(T *p, const float *v) { p[0] = from_f<T>(v[0]); }
};
template <> struct ConvIo<float, 2> {
    static __device__ __forceinline__ void load(const float *p, float *v) { float2 t = *reinterpret_cast<const float2 *>(p); v[0] = t.x, v[1] = t.y; }
    static __device__ __forceinline__ void store(float *p, const float *v) { *reinterpret_cast<float2 *>(p) = make_float2(v[0], v[1]); }
};
template <> struct ConvIo<bf16, 2> {
    static __device__ __forceinline__ void load(const bf16 *p, float *v) {
        float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
        v[0] = t.x, v[1] = t.y;
    }
    static __device__ __forceinline__ void store(bf16 *p, const float *v) { *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(v[0], v[1]); }
};

template <typename T, int V, int KT, int CH /* tokens per CTA */>
__global__ void __launch_bounds__(128)
short_conv_kernel(const T *__restrict__ x, long long x_token, const T *__restrict__ taps, const T *__restrict__ bias, int add_input, int channels,
                  int num_taps, int act, const int32_t *__restrict__ seq_info, float *__restrict__ state, long long slot_stride, int num_slots, T *__restrict__ y) {
    constexpr int KM = KT ? KT : kConvMaxTaps;
    const int K = KT ? KT : num_taps;
    const int s = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int first = seq_info[s * 4 + 0], count = seq_info[s * 4 + 1], start = seq_info[s * 4 + 2], slot = seq_info[s * 4 + 3];
    const int lo = blockIdx.z * CH, hi = min(count, lo + CH);
    if (c >= channels || lo >= count) return;
    const bool head_chunk = blockIdx.z == 0, slot_ok = slot >= 0 && slot < num_slots;
    float *hist = state + (size_t)(slot_ok ? slot : 0) * slot_stride + (size_t)c * (K - 1);  // channel c + v: hist + v * (K - 1)
    float b0[V];
#pragma unroll
    for (int v = 0; v < V; ++v) b0[v] = bias ? to_f(bias[c + v]) : 0.f;
    float w[V][KM], win[V][KM], old[V][KM];  // w[i] multiplies the input i tokens back = win[i]; old[i] = the input i + 1 tokens before the step
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
        for (int i = 0; i < KM; ++i) {
            w[v][i] = i < K ? to_f(taps[(size_t)(c + v) * K + (K - 1 - i)]) : 0.f;
            old[v][i] = (head_chunk && i < K - 1 && slot_ok && start - 1 - i >= 0) ? hist[v * (K - 1) + K - 2 - i] : 0.f;
            win[v][i] = 0.f;
        }
    float in[V];
#pragma unroll
    for (int i = 1; i < KM; ++i) {
        if (i < K) {
            if (head_chunk) {
#pragma unroll
                for (int v = 0; v < V; ++v) win[v][i] = old[v][i - 1];
            } else {  // lo >= CH >= K: the inputs before the chunk are this step's
                ConvIo<T, V>::load(x + (size_t)(first + lo - i) * x_token + c, in);
#pragma unroll
                for (int v = 0; v < V; ++v) win[v][i] = in[v];
            }
        }
    }
    constexpr int kAhead = 8;  // inputs fetched before any of them is used: the loads of a thread overlap
    for (int j0 = lo; j0 < hi; j0 += kAhead) {
        float ahead[kAhead][V];
#pragma unroll
        for (int u = 0; u < kAhead; ++u)
            if (j0 + u < hi) ConvIo<T, V>::load(x + (size_t)(first + j0 + u) * x_token + c, ahead[u]);
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            if (j0 + u < hi) {
                float out[V];
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    win[v][0] = ahead[u][v];
                    float acc = b0[v];
#pragma unroll
                    for (int i = 0; i < KM; ++i)
                        if (i < K) acc = fmaf(w[v][i], win[v][i], acc);
                    if (add_input) acc += win[v][0];
                    out[v] = act == 1 ? acc / (1.0f + expf(-acc)) : acc;
#pragma unroll
                    for (int i = KM - 1; i > 0; --i) win[v][i] = win[v][i - 1];
                }
                ConvIo<T, V>::store(y + (size_t)(first + j0 + u) * channels + c, out);
            }
        }
    }
    if (head_chunk && slot_ok) {
        // hist[K-2-i] <- the input i tokens before the step's last one, i = 0 .. K-2: of this step, or (a step shorter than
        // K-1 tokens) what the slot held, i - count places further back
#pragma unroll
        for (int i = 0; i < KM - 1; ++i) {
            if (i < K - 1) {
                const int jj = count - 1 - i;
                if (jj >= 0) {
                    ConvIo<T, V>::load(x + (size_t)(first + jj) * x_token + c, in);
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        in[v] = 0.f;
#pragma unroll
                        for (int m = 0; m < KM - 1; ++m)
                            if (m == -jj - 1) in[v] = old[v][m];
                    }
                }
#pragma unroll
                for (int v = 0; v < V; ++v) hist[v * (K - 1) + K - 2 - i] = in[v];
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

size_t tlb_delta_scan_workspace(int num_seqs, int max_tokens_per_seq, int heads, int dk, int dv) {
    if (max_tokens_per_seq <= kDrSegment) return 0;
    size_t segs = (size_t)num_seqs * (2 + (max_tokens_per_seq - 1) / kDrSegment);
    return segs * heads * ((size_t)dk * dv + (size_t)dk * dk) * sizeof(float);
}

int tlb_delta_scan(const void *q, long long q_token, long long q_head, const void *k, long long k_token, long long k_head, const void *v,
                   long long v_token, long long v_head, const void *beta, long long b_token, const void *a, int a_is_f32, long long a_token,
                   int per_channel, const void *a_log, const void *dt_bias, float q_scale, float unit_eps, int heads, int key_heads, int dk, int dv,
                   const int32_t *seq_info, int num_seqs, int max_tokens_per_seq, float *state, long long slot_stride, int num_slots, float *out,
                   void *workspace, size_t workspace_bytes, int dtype, void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (!q || !k || !v || !beta || !a || !a_log || !dt_bias || !seq_info || !state || !out || heads <= 0 || key_heads <= 0 || heads % key_heads ||
        dk <= 0 || dv <= 0 || num_slots <= 0 || max_tokens_per_seq <= 0)
        return tl::fail(TL_EINVAL, "delta_scan: bad argument");
    if (dk > 256) return tl::fail(TL_EINVAL, "delta_scan: key size %d > 256", dk);
    // portions longer than a segment are cut at absolute multiples of the segment length and run in three passes
    const bool segmented = max_tokens_per_seq > kDrSegment;
    const int max_segments = segmented ? 2 + (max_tokens_per_seq - 1) / kDrSegment : 1;
    float *seg_state = nullptr, *seg_trans = nullptr;
    if (segmented) {
        if (!workspace || workspace_bytes < tlb_delta_scan_workspace(num_seqs, max_tokens_per_seq, heads, dk, dv))
            return tl::fail(TL_EWORKSPACE, "delta_scan: workspace missing or too small");
        seg_state = (float *)workspace;
        seg_trans = seg_state + (size_t)num_seqs * max_segments * heads * dk * dv;
    }
    const int colblocks = ceil_div(dv, kDrCols), kblocks = ceil_div(dk, kDrCols), group = heads / key_heads;
    cudaStream_t st = as_stream(stream);
    const int kr = ceil_div(dk, kDrLanes);
#define TLB_DR_K(KRV, PASS, GY, GZ)                                                                                                                 \
    delta_scan_kernel<T, KRV, (KRV > 32 ? 8 : 16)><<<dim3(num_seqs, heads * (GY), GZ), kDrCols * kDrLanes, 0, st>>>(                                \
        (const T *)q, q_token, q_head, (const T *)k, k_token, k_head, (const T *)v, v_token, v_head, (const T *)beta, b_token, a, a_is_f32, a_token, \
        per_channel, (const T *)a_log, (const T *)dt_bias, q_scale, unit_eps, heads, group, dk, dv, seq_info, state, slot_stride, num_slots, out,    \
        PASS, max_segments, seg_state, seg_trans)
#define TLB_DR(PASS, GY, GZ)                                                                                                                       \
    TLB_DISPATCH(dtype, "delta_scan", if (kr <= 8) TLB_DR_K(8, PASS, GY, GZ); else if (kr <= 16) TLB_DR_K(16, PASS, GY, GZ);                        \
                 else if (kr <= 32) TLB_DR_K(32, PASS, GY, GZ); else TLB_DR_K(64, PASS, GY, GZ))
    if (!segmented) {
        TLB_DR(0, colblocks, 1);
        TL_LAUNCH_CHECK("delta_scan");
        return TL_OK;
    }
    TLB_DR(1, colblocks + kblocks, max_segments);
    TL_LAUNCH_CHECK("delta_scan (local states and transitions)");
    const int dkp = (dk + 3) & ~3;
    const size_t states = (size_t)2 * dkp * kDrCols * sizeof(float), staged = states + (size_t)2 * dk * dkp * sizeof(float);
    const bool stage = staged <= 200 * 1024;
    const size_t smem = stage ? staged : states;
    auto combine = stage ? delta_combine_kernel<true> : delta_combine_kernel<false>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(combine, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return tl::fail(TL_ECUDA, "delta_scan: %s", cudaGetErrorString(e));
    }
    combine<<<dim3(num_seqs, heads * colblocks), kDcThreads, smem, st>>>(seq_info, state, slot_stride, num_slots, heads, dk, dv, max_segments, seg_state,
                                                                       seg_trans);
    TL_LAUNCH_CHECK("delta_scan (combine)");
    TLB_DR(3, colblocks, max_segments);
    TL_LAUNCH_CHECK("delta_scan (outputs)");
#undef TLB_DR
#undef TLB_DR_K
    return TL_OK;
}

int tlb_short_conv(const void *x, long long x_token, const void *taps, const void *bias, int add_input, int channels, int num_taps, int act,
                   const int32_t *seq_info, int num_seqs,
                   int max_tokens_per_seq, float *state, long long slot_stride, int num_slots, void *y, int dtype, void *stream) {
    if (num_seqs <= 0) return TL_OK;
    if (!x || !taps || !seq_info || !y || channels <= 0 || num_taps <= 0 || max_tokens_per_seq <= 0 || (num_taps > 1 && (!state || num_slots <= 0)) ||
        act < 0 || act > 1)
        return tl::fail(TL_EINVAL, "short_conv: bad argument");
    if (num_taps > kConvMaxTaps) return tl::fail(TL_EINVAL, "short_conv: %d taps > %d", num_taps, kConvMaxTaps);
    static_assert(kConvSmallChunk >= kConvMaxTaps, "a chunk after the first finds its K-1 earlier inputs in this step");
    const size_t esize = dtype == TL_F32 ? 4 : 2;
    // two channels per thread when every pair sits on a 2-element boundary
    const bool pairs = channels % 2 == 0 && x_token % 2 == 0 && (uintptr_t)x % (2 * esize) == 0 && (uintptr_t)y % (2 * esize) == 0;
    const int per = pairs ? 2 : 1;
    const int cblocks = ceil_div(ceil_div(channels, per), 128);
    const int chunk = (long long)num_seqs * cblocks * ceil_div(max_tokens_per_seq, kConvChunk) < 148 * 8 ? kConvSmallChunk : kConvChunk;
    dim3 grid(num_seqs, cblocks, ceil_div(max_tokens_per_seq, chunk));
    cudaStream_t st = as_stream(stream);
#define TLB_SC_C(V, KT, CH)                                                                                                              \
    short_conv_kernel<T, V, KT, CH><<<grid, 128, 0, st>>>((const T *)x, x_token, (const T *)taps, (const T *)bias, add_input, channels, num_taps, act, seq_info, state, \
                                                          slot_stride, num_slots, (T *)y)
#define TLB_SC(V, KT)                                                                                                                    \
    if (chunk == kConvChunk) TLB_SC_C(V, KT, kConvChunk); else TLB_SC_C(V, KT, kConvSmallChunk)
#define TLB_SC_K(V)                                                                                                                      \
    switch (num_taps) {                                                                                                                  \
        case 2: TLB_SC(V, 2); break;                                                                                                     \
        case 3: TLB_SC(V, 3); break;                                                                                                     \
        case 4: TLB_SC(V, 4); break;                                                                                                     \
        default: TLB_SC(V, 0);                                                                                                           \
    }
    TLB_DISPATCH(dtype, "short_conv", if (pairs) { TLB_SC_K(2) } else { TLB_SC_K(1) });
#undef TLB_SC_K
#undef TLB_SC
#undef TLB_SC_C
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
