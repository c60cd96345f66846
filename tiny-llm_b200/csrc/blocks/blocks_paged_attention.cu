// Grouped-query softmax attention over a paged key/value cache, ragged batches, and the kernel that fills the cache.
//
// A cache row holds one token of one layer: the keys of all key/value heads, then their values
// ([kv_heads * dk | kv_heads * dv]).  Query head h reads key/value head h / (heads / kv_heads).  A CTA takes a run of
// consecutive tokens of one sequence x up to 4 query heads of ONE key/value head (16 query rows) and streams each
// 32-key tile of that head through shared memory once for all of them.  What a position may see is a parameter:
//   mask 0  every earlier position (causal)
//   mask 1  itself and the size-1 positions before it (sliding window)
//   mask 2  the earlier positions of its own block of `size` positions, blocks counted from position 0 (chunks)
// and so are a tanh soft cap on the scaled scores, a sink (one more term in the softmax's denominator that carries no
// value: exp(0), or exp(head_bias[h]) with a learned number per head) and a per-head output gate (the output of head h
// times sigmoid(gate[t, h])).  weights 1 replaces the softmax: a visible key weighs sigmoid(score + head_bias[h]) and
// nothing is normalised over the keys.
// Scores, the running maximum / sum and the accumulators are fp32; cache rows are converted as they are staged, so the
// same kernel serves the bf16 and the fp32 cache.  Key tiles are 32-aligned in absolute positions and taken in
// ascending order, so a row's sum does not depend on where a prompt was cut or on what shares the launch.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kPaRows = 16;   // query rows per CTA
constexpr int kPaWarps = 8;   // 2 rows per warp
constexpr int kPaKeys = 32;   // keys per staged tile
constexpr int kPaHeads = 4;   // most query heads of one group per CTA

__host__ __device__ inline int pa_heads_per_cta(int group) { return group < kPaHeads ? group : kPaHeads; }

__device__ __forceinline__ bool pa_visible(int p, int key, int mask, int size) {
    if (key > p) return false;
    if (mask == 1) return p - key < size;
    if (mask == 2) return p / size == key / size;
    return true;
}

template <typename T, int VL /* ceil(dv / 32) */>
__global__ void __launch_bounds__(kPaWarps * 32)
paged_attention_kernel(const T *__restrict__ q, long long q_token, long long q_head, const T *__restrict__ slab, int num_pages, int page_size,
                       int row_width, int dk, int dv, int heads, int kv_heads, const int32_t *__restrict__ block_table, int max_pages,
                       const int32_t *__restrict__ tiles, const int32_t *__restrict__ tok_pos, int mask, int mask_size, float scale, float softcap,
                       int sink, const T *__restrict__ gate, long long g_token, T *__restrict__ out, long long o_token, long long o_head,
                       const float *__restrict__ head_bias, int weights) {
    extern __shared__ float smem[];
    const int kstride = dk + 1;            // +1 breaks the bank conflict of lane = key reads
    float *sq = smem;                      // [kPaRows][dk]
    float *sk = sq + kPaRows * dk;         // [kPaKeys][kstride]
    float *sv = sk + kPaKeys * kstride;    // [kPaKeys][dv]

    const int group = heads / kv_heads;
    const int hp = pa_heads_per_cta(group);
    const int parts = (group + hp - 1) / hp;         // CTAs per key/value head
    const int g = blockIdx.y / parts, part = blockIdx.y % parts;
    const int head0 = g * group + part * hp;
    const int nheads = min(hp, group - part * hp);
    const int first = tiles[blockIdx.x * 3 + 0], count = tiles[blockIdx.x * 3 + 1], seq = tiles[blockIdx.x * 3 + 2];
    const int pos0 = tok_pos[first];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int r = warp; r < kPaRows; r += kPaWarps) {
        int tq = r / hp, hh = r % hp;
        bool live = tq < count && hh < nheads;
        const T *src = q + (size_t)(first + tq) * q_token + (size_t)(head0 + hh) * q_head;
        for (int d = lane; d < dk; d += 32) sq[r * dk + d] = live ? to_f(src[d]) * scale : 0.f;
    }

    const int r0 = warp * 2, r1 = warp * 2 + 1;
    const int tq0 = r0 / hp, tq1 = r1 / hp;
    const bool live0 = tq0 < count && (r0 % hp) < nheads, live1 = tq1 < count && (r1 % hp) < nheads;
    const int p0 = pos0 + tq0, p1 = pos0 + tq1;

    // a sink is a key of score 0 (or head_bias[h]) without a value: the running maximum starts there and the sum at 1
    const float hb0 = head_bias && live0 ? head_bias[head0 + r0 % hp] : 0.f, hb1 = head_bias && live1 ? head_bias[head0 + r1 % hp] : 0.f;
    float m0 = sink ? hb0 : -INFINITY, m1 = sink ? hb1 : -INFINITY, l0 = sink ? 1.f : 0.f, l1 = l0;
    if (weights == 1) m0 = m1 = 0.f, l0 = l1 = 1.f;
    float acc0[VL], acc1[VL];
#pragma unroll
    for (int i = 0; i < VL; ++i) acc0[i] = acc1[i] = 0.f;

    const int hi = pos0 + count - 1;  // newest key any row of the tile sees
    int lo = 0;                       // oldest one
    if (mask == 1) lo = max(0, pos0 - mask_size + 1);
    if (mask == 2) lo = pos0 / mask_size * mask_size;
    lo = lo / kPaKeys * kPaKeys;
    const int32_t *table = block_table + (size_t)seq * max_pages;
    const size_t k_off = (size_t)g * dk, v_off = (size_t)kv_heads * dk + (size_t)g * dv;

    for (int k0 = lo; k0 <= hi; k0 += kPaKeys) {
        __syncthreads();
        int page = table[k0 / page_size];
        bool page_ok = page >= 0 && page < num_pages;
        const T *src = slab + ((size_t)(page_ok ? page : 0) * page_size + (k0 % page_size)) * row_width;
        int valid = page_ok ? min(kPaKeys, hi - k0 + 1) : 0;
        for (int e = threadIdx.x; e < kPaKeys * dk; e += blockDim.x) {
            int j = e / dk, d = e - j * dk;
            sk[j * kstride + d] = j < valid ? to_f(src[(size_t)j * row_width + k_off + d]) : 0.f;
        }
        for (int e = threadIdx.x; e < kPaKeys * dv; e += blockDim.x) {
            int j = e / dv, d = e - j * dv;
            sv[j * dv + d] = j < valid ? to_f(src[(size_t)j * row_width + v_off + d]) : 0.f;
        }
        __syncthreads();

        const int key = k0 + lane;
        float s0 = 0.f, s1 = 0.f;
        const float *kr = sk + lane * kstride;
        const float *qa = sq + r0 * dk, *qb = sq + r1 * dk;
        for (int d = 0; d < dk; ++d) {
            float kv = kr[d];
            s0 = fmaf(qa[d], kv, s0);
            s1 = fmaf(qb[d], kv, s1);
        }
        if (softcap > 0.f) s0 = softcap * tanhf(s0 / softcap), s1 = softcap * tanhf(s1 / softcap);
        bool vis0 = live0 && key <= hi && pa_visible(p0, key, mask, mask_size);
        bool vis1 = live1 && key <= hi && pa_visible(p1, key, mask, mask_size);
        float e0, e1;
        if (weights == 1) {
            e0 = vis0 ? 1.0f / (1.0f + expf(-(s0 + hb0))) : 0.f;
            e1 = vis1 ? 1.0f / (1.0f + expf(-(s1 + hb1))) : 0.f;
        } else {
            s0 = vis0 ? s0 : -INFINITY;
            s1 = vis1 ? s1 : -INFINITY;
            float n0 = fmaxf(m0, warp_max(s0)), n1 = fmaxf(m1, warp_max(s1));
            float a0 = n0 == -INFINITY ? 1.f : expf(m0 - n0), a1 = n1 == -INFINITY ? 1.f : expf(m1 - n1);
            e0 = vis0 ? expf(s0 - n0) : 0.f, e1 = vis1 ? expf(s1 - n1) : 0.f;
            l0 = l0 * a0 + warp_sum(e0);
            l1 = l1 * a1 + warp_sum(e1);
            m0 = n0;
            m1 = n1;
#pragma unroll
            for (int i = 0; i < VL; ++i) acc0[i] *= a0, acc1[i] *= a1;
        }
        for (int j = 0; j < kPaKeys; ++j) {
            float w0 = __shfl_sync(0xffffffffu, e0, j), w1 = __shfl_sync(0xffffffffu, e1, j);
            const float *vrow = sv + j * dv;
#pragma unroll
            for (int i = 0; i < VL; ++i) {
                int d = lane + 32 * i;
                float v = d < dv ? vrow[d] : 0.f;
                acc0[i] = fmaf(w0, v, acc0[i]);
                acc1[i] = fmaf(w1, v, acc1[i]);
            }
        }
    }

    auto finish = [&](int r, int tq, float l, const float *acc) {
        int head = head0 + r % hp;
        float inv = 1.0f / l;
        if (gate) inv *= 1.0f / (1.0f + expf(-to_f(gate[(size_t)(first + tq) * g_token + head])));
        T *o = out + (size_t)(first + tq) * o_token + (size_t)head * o_head;
#pragma unroll
        for (int i = 0; i < VL; ++i)
            if (lane + 32 * i < dv) o[lane + 32 * i] = from_f<T>(acc[i] * inv);
    };
    if (live0) finish(r0, tq0, l0, acc0);
    if (live1) finish(r1, tq1, l1, acc1);
}

// One CTA per token: optional per-head RMS norm of the queries (in place) and of the keys, then the token's keys and
// values go to its slot of the cache.  A warp takes a head at a time.
template <typename T>
__global__ void __launch_bounds__(128)
kv_prepare_kernel(T *q, long long q_token, long long q_head, int heads, const T *__restrict__ q_norm, const T *__restrict__ k, long long k_token,
                  long long k_head, const T *__restrict__ v, long long v_token, long long v_head, int kv_heads, int dk, int dv,
                  const T *__restrict__ k_norm, float eps, const int32_t *__restrict__ tok_pos, const int32_t *__restrict__ tok_seq,
                  const int32_t *__restrict__ block_table, int max_pages, int num_pages, int page_size, T *__restrict__ slab) {
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    if (q != nullptr && q_norm != nullptr && heads == 1) {  // one long row (a norm over a whole projection): the CTA shares it
        __shared__ float scratch[33];
        T *row = q + (size_t)t * q_token;
        float ss = 0.f;
        for (int d = threadIdx.x; d < dk; d += blockDim.x) {
            float x = to_f(row[d]);
            ss += x * x;
        }
        ss = block_sum(ss, scratch);
        float inv = 1.0f / sqrtf(ss / (float)dk + eps);
        for (int d = threadIdx.x; d < dk; d += blockDim.x) row[d] = from_f<T>(to_f(row[d]) * inv * to_f(q_norm[d]));
    } else if (q != nullptr && q_norm != nullptr) {
        for (int hd = warp; hd < heads; hd += warps) {
            T *row = q + (size_t)t * q_token + (size_t)hd * q_head;
            float ss = 0.f;
            for (int d = lane; d < dk; d += 32) {
                float x = to_f(row[d]);
                ss += x * x;
            }
            ss = warp_sum(ss);
            float inv = 1.0f / sqrtf(ss / (float)dk + eps);
            for (int d = lane; d < dk; d += 32) row[d] = from_f<T>(to_f(row[d]) * inv * to_f(q_norm[d]));
        }
    }
    if (k == nullptr) return;
    const int pos = tok_pos[t];
    const int page = block_table[(size_t)tok_seq[t] * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) return;  // a bad table entry drops the write instead of corrupting another page
    T *dst = slab + ((size_t)page * page_size + pos % page_size) * ((size_t)kv_heads * (dk + dv));
    for (int hd = warp; hd < kv_heads; hd += warps) {
        const T *row = k + (size_t)t * k_token + (size_t)hd * k_head;
        float inv = 1.f;
        if (k_norm != nullptr) {
            float ss = 0.f;
            for (int d = lane; d < dk; d += 32) {
                float x = to_f(row[d]);
                ss += x * x;
            }
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)dk + eps);
        }
        for (int d = lane; d < dk; d += 32)
            dst[(size_t)hd * dk + d] = k_norm ? from_f<T>(to_f(row[d]) * inv * to_f(k_norm[d])) : row[d];
        const T *vr = v + (size_t)t * v_token + (size_t)hd * v_head;
        for (int d = lane; d < dv; d += 32) dst[(size_t)kv_heads * dk + (size_t)hd * dv + d] = vr[d];
    }
}

// For attention whose queries and keys are RMS-normed over the WHOLE projection (all heads as one row, weights of that size)
// and then rotated: W warps per token (W = 1 for launches with many tokens: no CTA-wide barrier anywhere; W = 8, a whole CTA,
// when a step brings few tokens and a warp alone would be a long chain of loads) read the row once into shared memory as
// fp32, reduce the sum of squares, and apply norm, weight and rotation (the first rot_dims entries of every head by the token's
// position; pairs (2i, 2i+1) or (i, i + rot_dims/2); angles from the step's table, or evaluated in double) on the way out - the
// queries back in place, keys and values to the token's slot of the cache.  Nothing is rounded between the norm and the
// rotation.  The sum of squares is taken in 256 column classes (d mod 256), each class's 32-lane tree, then the eight trees in
// order, in both forms: a token's numbers do not depend on how many tokens share its step.
constexpr int kQkWarps = 8;

template <typename T, int W>
__global__ void __launch_bounds__(256)
qk_whole_prepare_kernel(T *q, long long q_token, int heads, const T *__restrict__ q_norm, const T *__restrict__ k, long long k_token,
                        const T *__restrict__ v, long long v_token, int kv_heads, int dk, int dv, const T *__restrict__ k_norm, float eps, int rot_dims,
                        int interleaved, double log2_base, const int32_t *__restrict__ tok_pos, const int32_t *__restrict__ tok_seq,
                        const int32_t *__restrict__ block_table, int max_pages, int num_pages, int page_size, T *__restrict__ slab,
                        const float *__restrict__ rope_cos, const float *__restrict__ rope_sin /* [T, rot_dims / 2] tabulated, or NULL */, int tokens) {
    extern __shared__ float smem[];  // per token of the CTA: [max(heads, kv_heads) * dk] the row, then [rot_dims] cos | sin
    __shared__ float partial[kQkWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = W == 1 ? warp : 0, me = W == 1 ? lane : (int)threadIdx.x, step = 32 * W;  // this thread's place among its token's threads
    const int t = W == 1 ? blockIdx.x * kQkWarps + warp : blockIdx.x;
    if (t >= tokens) return;  // W == 8: uniform over the CTA
    const int pos = tok_pos[t], half = rot_dims / 2;
    const int longest = max(heads, kv_heads) * dk;
    float *srow = smem + (size_t)group * (longest + rot_dims), *cs = srow + longest, *sn = cs + half;
    auto sync = [&]() {
        if (W == 1) __syncwarp();
        else __syncthreads();
    };
    for (int i = me; i < half; i += step) {
        if (rope_cos) cs[i] = rope_cos[(size_t)t * half + i], sn[i] = rope_sin[(size_t)t * half + i];
        else rope_angle(pos, i, rot_dims, log2_base, cs[i], sn[i]);
    }
    T *dst = nullptr;
    if (k != nullptr) {
        const int page = block_table[(size_t)tok_seq[t] * max_pages + pos / page_size];
        if (page >= 0 && page < num_pages) dst = slab + ((size_t)page * page_size + pos % page_size) * ((size_t)kv_heads * (dk + dv));
    }
    for (int which = 0; which < 2; ++which) {  // 0: queries (in place), 1: keys (to the cache)
        const int nh = which == 0 ? heads : kv_heads;
        const T *src = which == 0 ? q + (size_t)t * q_token : (k ? k + (size_t)t * k_token : nullptr);
        const T *w = which == 0 ? q_norm : k_norm;
        T *out = which == 0 ? q + (size_t)t * q_token : dst;
        if (src == nullptr || out == nullptr) continue;  // uniform over the token's threads
        const int width = nh * dk;
        sync();  // the row of the pass before has been read
        float total;
        if (W == 1) {  // a lane owns eight column classes, lane + 32 j
            float acc[kQkWarps];
#pragma unroll
            for (int j = 0; j < kQkWarps; ++j) acc[j] = 0.f;
            for (int d0 = lane; d0 < width; d0 += 32 * kQkWarps) {
                float x[kQkWarps];
#pragma unroll
                for (int j = 0; j < kQkWarps; ++j) x[j] = d0 + 32 * j < width ? to_f(src[d0 + 32 * j]) : 0.f;
#pragma unroll
                for (int j = 0; j < kQkWarps; ++j) {
                    if (d0 + 32 * j < width) srow[d0 + 32 * j] = x[j];
                    acc[j] = fmaf(x[j], x[j], acc[j]);
                }
            }
            total = 0.f;
#pragma unroll
            for (int j = 0; j < kQkWarps; ++j) total += warp_sum(acc[j]);
        } else {       // a thread owns one column class
            float acc = 0.f;
            for (int d = me; d < width; d += step) {
                float x = to_f(src[d]);
                srow[d] = x;
                acc = fmaf(x, x, acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) partial[warp] = acc;
            __syncthreads();
            total = 0.f;
#pragma unroll
            for (int j = 0; j < kQkWarps; ++j) total += partial[j];
        }
        sync();
        const float inv = w ? 1.0f / sqrtf(total / (float)width + eps) : 1.f;
        for (int d = me; d < width; d += step) {
            const int e = d % dk;
            float x = srow[d] * inv * (w ? to_f(w[d]) : 1.f);
            if (e < rot_dims) {
                const bool low = interleaved ? !(e & 1) : e < half;
                const int i = interleaved ? e >> 1 : (low ? e : e - half);
                const int od = interleaved ? (d ^ 1) : (low ? d + half : d - half);
                const float other = srow[od] * inv * (w ? to_f(w[od]) : 1.f);
                x = low ? x * cs[i] - other * sn[i] : x * cs[i] + other * sn[i];
            }
            out[d] = from_f<T>(x);
        }
    }
    if (dst != nullptr) {
        const T *vr = v + (size_t)t * v_token;
        for (int d = me; d < kv_heads * dv; d += step) dst[(size_t)kv_heads * dk + d] = vr[d];
    }
}

template <typename T, int VL>
static int pa_launch(const void *q, long long q_token, long long q_head, const void *slab, int num_pages, int page_size, int dk, int dv, int heads,
                     int kv_heads, const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles, const int32_t *tok_pos, int mask,
                     int mask_size, float scale, float softcap, int sink, const void *gate, long long g_token, void *out, long long o_token,
                     long long o_head, const float *head_bias, int weights, cudaStream_t st) {
    size_t smem = ((size_t)kPaRows * dk + (size_t)kPaKeys * (dk + 1) + (size_t)kPaKeys * dv) * sizeof(float);
    auto kernel = paged_attention_kernel<T, VL>;
    if (smem > 48 * 1024) {
        if (smem > 227 * 1024) return tl::fail(TL_EINVAL, "paged_attention: head sizes %d + %d do not fit in shared memory", dk, dv);
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return tl::fail(TL_ECUDA, "paged_attention: %s", cudaGetErrorString(e));
    }
    int group = heads / kv_heads;
    dim3 grid(num_tiles, kv_heads * ceil_div(group, pa_heads_per_cta(group)));
    kernel<<<grid, kPaWarps * 32, smem, st>>>((const T *)q, q_token, q_head, (const T *)slab, num_pages, page_size, kv_heads * (dk + dv), dk, dv, heads,
                                              kv_heads, block_table, max_pages, tiles, tok_pos, mask, mask_size, scale, softcap, sink, (const T *)gate,
                                              g_token, (T *)out, o_token, o_head, head_bias, weights);
    return TL_OK;
}

}  // namespace tlb

using namespace tlb;

extern "C" {

int tlb_paged_attention_tile_tokens(int heads, int kv_heads) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    return kPaRows / pa_heads_per_cta(heads / kv_heads);
}

int tlb_paged_attention(const void *q, long long q_token, long long q_head, const void *slab, int num_pages, int page_size, int dk, int dv, int heads,
                        int kv_heads, const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles, const int32_t *tok_pos, int mask,
                        int mask_size, float scale, float softcap, int sink, const void *gate, long long g_token, void *out, long long o_token,
                        long long o_head, const float *head_bias, int weights, int dtype, void *stream) {
    if (num_tiles <= 0) return TL_OK;
    if (weights < 0 || weights > 1 || (weights == 1 && (sink || softcap > 0.f))) return tl::fail(TL_EINVAL, "paged_attention: bad weights mode");
    if (!q || !slab || !block_table || !tiles || !tok_pos || !out || dk <= 0 || dv <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads ||
        max_pages <= 0 || num_pages <= 0)
        return tl::fail(TL_EINVAL, "paged_attention: bad argument");
    if (page_size <= 0 || page_size % kPaKeys != 0) return tl::fail(TL_EINVAL, "paged_attention: page_size must be a multiple of %d", kPaKeys);
    if (mask < 0 || mask > 2 || (mask != 0 && mask_size <= 0)) return tl::fail(TL_EINVAL, "paged_attention: bad mask");
    if (dv > 512) return tl::fail(TL_EINVAL, "paged_attention: value size %d > 512", dv);
    cudaStream_t st = as_stream(stream);
    int vl = ceil_div(dv, 32);
    int rc = TL_OK;
#define TLB_PA(V)                                                                                                                                   \
    rc = pa_launch<T, V>(q, q_token, q_head, slab, num_pages, page_size, dk, dv, heads, kv_heads, block_table, max_pages, tiles, num_tiles, tok_pos, \
                         mask, mask_size, scale, softcap, sink, gate, g_token, out, o_token, o_head, head_bias, weights, st)
    TLB_DISPATCH(dtype, "paged_attention", if (vl <= 1) TLB_PA(1); else if (vl <= 2) TLB_PA(2); else if (vl <= 4) TLB_PA(4); else if (vl <= 8) TLB_PA(8);
                 else TLB_PA(16));
#undef TLB_PA
    if (rc != TL_OK) return rc;
    TL_LAUNCH_CHECK("paged_attention");
    return TL_OK;
}

int tlb_kv_prepare(void *q, long long q_token, long long q_head, int heads, const void *q_norm, const void *k, long long k_token, long long k_head,
                   const void *v, long long v_token, long long v_head, int kv_heads, int dk, int dv, const void *k_norm, float eps,
                   const int32_t *tok_pos, const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages, int page_size, void *slab,
                   int tokens, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (q == nullptr && k == nullptr) return TL_OK;
    if (dk <= 0 || dv <= 0 || (q && heads <= 0)) return tl::fail(TL_EINVAL, "kv_prepare: bad argument");
    if (k && (!v || !slab || !tok_pos || !tok_seq || !block_table || kv_heads <= 0 || page_size <= 0 || max_pages <= 0))
        return tl::fail(TL_EINVAL, "kv_prepare: bad cache argument");
    if (q && !q_norm && !k) return TL_OK;
    TLB_DISPATCH(dtype, "kv_prepare",
                 kv_prepare_kernel<T><<<tokens, 128, 0, as_stream(stream)>>>((T *)q, q_token, q_head, heads, (const T *)q_norm, (const T *)k, k_token, k_head,
                                                                            (const T *)v, v_token, v_head, kv_heads, dk, dv, (const T *)k_norm, eps,
                                                                            tok_pos, tok_seq, block_table, max_pages, num_pages, page_size, (T *)slab));
    TL_LAUNCH_CHECK("kv_prepare");
    return TL_OK;
}

int tlb_qk_whole_prepare(void *q, long long q_token, int heads, const void *q_norm, const void *k, long long k_token, const void *v, long long v_token,
                          int kv_heads, int dk, int dv, const void *k_norm, float eps, int rot_dims, int interleaved, double base, const int32_t *tok_pos,
                          const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages, int page_size, void *slab,
                          const float *rope_cos, const float *rope_sin, int tokens, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if ((rope_cos == nullptr) != (rope_sin == nullptr)) return tl::fail(TL_EINVAL, "qk_whole_prepare: both rotation tables or neither");
    if (!q || !tok_pos || heads <= 0 || dk <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > dk || (rot_dims > 0 && !(base > 0)))
        return tl::fail(TL_EINVAL, "qk_whole_prepare: bad argument");
    if (k && (!v || !slab || !tok_seq || !block_table || kv_heads <= 0 || dv <= 0 || page_size <= 0 || max_pages <= 0))
        return tl::fail(TL_EINVAL, "qk_whole_prepare: bad cache argument");
    if (!k) kv_heads = 0;
    const size_t per_token = ((size_t)(heads > kv_heads ? heads : kv_heads) * dk + rot_dims) * sizeof(float);
    if (per_token > 200 * 1024) return tl::fail(TL_EINVAL, "qk_whole_prepare: a projection of %d entries does not fit in shared memory", heads * dk);
    // a warp per token when there are tokens enough to fill the GPU that way and eight rows fit in shared memory, else a CTA per token
    const bool by_warp = tokens >= 148 * 8 * 2 && per_token * kQkWarps <= 200 * 1024;
    const size_t smem = by_warp ? per_token * kQkWarps : per_token;
    double lb = rot_dims > 0 ? log2(base) : 0.0;
#define TLB_QK_W(WV, GRID)                                                                                                                          \
    do {                                                                                                                                            \
        auto kernel = qk_whole_prepare_kernel<T, WV>;                                                                                               \
        if (smem > 48 * 1024) {                                                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                   \
            if (e != cudaSuccess) return tl::fail(TL_ECUDA, "qk_whole_prepare: %s", cudaGetErrorString(e));                                         \
        }                                                                                                                                           \
        kernel<<<GRID, 32 * kQkWarps, smem, as_stream(stream)>>>((T *)q, q_token, heads, (const T *)q_norm, (const T *)k, k_token, (const T *)v,    \
                                                         v_token, kv_heads, dk, dv, (const T *)k_norm, eps, rot_dims, interleaved, lb, tok_pos,     \
                                                         tok_seq, block_table, max_pages, num_pages, page_size, (T *)slab, rope_cos, rope_sin,      \
                                                         tokens);                                                                                   \
    } while (0)
#define TLB_QK do { if (by_warp) TLB_QK_W(1, ceil_div(tokens, kQkWarps)); else TLB_QK_W(kQkWarps, tokens); } while (0)
    TLB_DISPATCH(dtype, "qk_whole_prepare", TLB_QK);
#undef TLB_QK
#undef TLB_QK_W
    TL_LAUNCH_CHECK("qk_whole_prepare");
    return TL_OK;
}

}  // extern "C"
