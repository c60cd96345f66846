// Grouped-query attention over the paged cache on the tensor cores (bf16 cache, mma.sync m16n8k16, fp32 accumulation and
// softmax): the bf16 serving path of blocks_paged_attention.cu, same arguments and masks.
//
// A CTA takes 32 query rows = a run of consecutive tokens of one sequence x the query heads of ONE key/value head (up to
// 32 of them) and streams every 32-key tile of that head through shared memory once for all of them: keys into one
// buffer, values into another (cp.async, 16 bytes a piece), each twice, so that the next tile loads while this one is
// computed.  Per key tile, with 8 warps:
//   1. scores:  the 32 x 32 block S = Q K^T is 2 x 4 blocks of 16 x 8, one per warp (two accumulator sets alternate over
//               the reduction so that consecutive MMAs do not wait on each other);
//   2. softmax: each warp owns 4 rows, 8 lanes per row, 4 keys per lane: scale, soft cap, mask, running maximum / sum
//               (a sink starts them at 0 / 1), P = exp(S - m) as bf16, rescale factor;
//               what a row sees is a key range worked out once per row, the cap's tanh is the hardware approximation;
//   3. values:  O[32 x dv] += P V, warp = (16-row half, quarter of the value columns).
// A row's arithmetic depends only on its own position (32-aligned key tiles in ascending order): what else is in the
// CTA, the launch or the batch does not change its result, nor does where a prompt was cut.  When a launch alone would
// leave most SMs idle (a few single tokens over long key ranges), the caller may cut every tile's key range over several
// CTAs (flash decoding): partial sums go to a workspace and a second launch merges them; that changes rounding only.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kGRows = 32;        // query rows per CTA
constexpr int kGKeys = 32;        // keys per tile
constexpr int kGSS = kGKeys + 1;  // score row stride (floats)
constexpr int kGSP = kGKeys + 8;  // probability row stride (bf16): (stride / 8) odd
constexpr int kGWarps = 8;

__device__ __forceinline__ void g_ldm_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void g_ldm_x2(uint32_t &r0, uint32_t &r1, const void *p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void g_ldm_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void g_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void g_cp16(void *dst, const void *src) {
    uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// tanh by the hardware approximation (relative error about 2^-11): the probabilities it feeds are rounded to bf16 anyway
__device__ __forceinline__ float g_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// PAIRS = pairs of 8-column value tiles per warp (the warp's quarter of the value columns = 16 * PAIRS columns).
template <int PAIRS>
__global__ void __launch_bounds__(kGWarps * 32)
paged_attention_mma_kernel(const bf16 *__restrict__ q, long long q_token, long long q_head, const bf16 *__restrict__ slab, int num_pages, int page_size,
                           int row_width, int dk, int dv, int heads, int kv_heads, int hp /* query heads per CTA */,
                           const int32_t *__restrict__ block_table, int max_pages, const int32_t *__restrict__ tiles, const int32_t *__restrict__ tok_pos,
                           int mask, int mask_size, float scale, float softcap, int sink, const bf16 *__restrict__ gate, long long g_token,
                           bf16 *__restrict__ out, long long o_token, long long o_head, int k_stride, int v_stride /* shared-memory row strides */,
                           float *__restrict__ partial /* split results, or NULL */, const float *__restrict__ head_bias /* [heads] or NULL */,
                           int weights /* 0 softmax, 1 sigmoid(score + head_bias) without normalisation */) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16 *sq = reinterpret_cast<bf16 *>(smem_raw);              // [32][k_stride]
    bf16 *skv = sq + kGRows * k_stride;                         // [2] x ([32][k_stride] keys | [32][v_stride] values)
    const int buf_elems = kGKeys * (k_stride + v_stride);
    bf16 *sp = skv + 2 * buf_elems;                             // [32][kGSP]
    float *ss = reinterpret_cast<float *>(sp + kGRows * kGSP);  // [32][kGSS]
    float *s_alpha = ss + kGRows * kGSS;                        // [32]
    float *s_l = s_alpha + kGRows;                              // [32]

    const int group = heads / kv_heads;
    const int parts = (group + hp - 1) / hp;
    const int g = blockIdx.y / parts, part = blockIdx.y % parts;
    const int head0 = g * group + part * hp;
    const int nheads = min(hp, group - part * hp);
    const int first = tiles[blockIdx.x * 3 + 0], count = tiles[blockIdx.x * 3 + 1], seq = tiles[blockIdx.x * 3 + 2];
    const int pos0 = tok_pos[first];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_pieces = dk / 8, v_pieces = dv / 8;  // 16-byte pieces of a key / value row

    // zero everything once: padding columns of Q, K and V must read as zero in every product
    for (int i = threadIdx.x; i < (kGRows * k_stride + 2 * buf_elems) / 8; i += blockDim.x)
        reinterpret_cast<uint4 *>(sq)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    for (int r = warp; r < kGRows; r += kGWarps) {  // row = token-in-tile * hp + head-in-group
        int tq = r / hp, hh = r % hp;
        if (tq >= count || hh >= nheads) continue;
        const bf16 *src = q + (size_t)(first + tq) * q_token + (size_t)(head0 + hh) * q_head;
        for (int d = lane; d < dk; d += 32) sq[r * k_stride + d] = src[d];
    }

    const int hi = pos0 + count - 1;
    int lo = 0;
    if (mask == 1) lo = max(0, pos0 - mask_size + 1);
    if (mask == 2) lo = pos0 / mask_size * mask_size;
    lo = lo / kGKeys * kGKeys;
    const int32_t *table = block_table + (size_t)seq * max_pages;
    const int n_tiles = (hi - lo) / kGKeys + 1;
    const size_t k_off = (size_t)g * dk, v_off = (size_t)kv_heads * dk + (size_t)g * dv;

    // which 16-byte piece of which row this thread copies first (the same for every tile); the next ones are 256 pieces on
    const int per_row = k_pieces + v_pieces;
    const int step_rows = (int)blockDim.x / per_row, step_pieces = (int)blockDim.x % per_row;
    auto stage = [&](int tile, int buf) {
        bf16 *sk = skv + buf * buf_elems, *sv = sk + kGKeys * k_stride;
        int k0 = lo + tile * kGKeys;
        int page = table[k0 / page_size];
        bool ok = page >= 0 && page < num_pages;
        int valid = ok ? min(kGKeys, hi - k0 + 1) : 0;
        const bf16 *src = slab + ((size_t)(ok ? page : 0) * page_size + (k0 % page_size)) * row_width;
        int j = (int)threadIdx.x / per_row, piece = (int)threadIdx.x % per_row;
        while (j < kGKeys) {
            bool is_v = piece >= k_pieces;
            int col = (is_v ? piece - k_pieces : piece) * 8;
            bf16 *dst = is_v ? sv + j * v_stride + col : sk + j * k_stride + col;
            if (j < valid) g_cp16(dst, src + (size_t)j * row_width + (is_v ? v_off : k_off) + col);
            else *reinterpret_cast<uint4 *>(dst) = make_uint4(0, 0, 0, 0);
            j += step_rows, piece += step_pieces;
            if (piece >= per_row) piece -= per_row, ++j;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // softmax state of the row this lane works on (a warp owns 4 rows, 8 lanes each; uniform over the 8 lanes)
    const bool sunk = sink && blockIdx.z == 0;  // with the key range split over gridDim.z CTAs the sink's term is counted once
    float m_row = sunk ? 0.f : -INFINITY, l_row = sunk ? 1.f : 0.f;
    float hb = 0.f;  // the row's head's learned number: the sink's score, or the offset inside the sigmoid
    int see_lo = 1, see_hi = 0;  // the keys this row may see (none for a padding row)
    {
        int r = warp * 4 + (lane >> 3), tq = r / hp, hh = r % hp;
        if (tq < count && hh < nheads) {
            if (head_bias) hb = head_bias[head0 + hh];
            if (sunk) m_row = hb;
            if (weights == 1) m_row = 0.f, l_row = blockIdx.z == 0 ? 1.f : 0.f;
            see_hi = pos0 + tq;
            see_lo = mask == 1 ? max(0, see_hi - mask_size + 1) : mask == 2 ? see_hi / mask_size * mask_size : 0;
        }
    }
    const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
    const int mt = warp & 1, nt = warp >> 1;  // score block of this warp; nt is also its quarter of the value columns
    float acc[2 * PAIRS][4];
#pragma unroll
    for (int i = 0; i < 2 * PAIRS; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    const int ksteps = (dk + 15) / 16;
    // with the key range split over gridDim.z CTAs, this one takes a contiguous run of key tiles
    const int per_split = (n_tiles + (int)gridDim.z - 1) / (int)gridDim.z;
    const int tile_begin = (int)blockIdx.z * per_split, tile_end = min(n_tiles, tile_begin + per_split);
    __syncthreads();  // the zero fill is done before the first copies land
    if (tile_begin < tile_end) stage(tile_begin, 0);
    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int buf = (tile - tile_begin) & 1;
        const bf16 *sk = skv + buf * buf_elems, *sv = sk + kGKeys * k_stride;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // this tile has landed, and every warp is done with the previous one: its buffer may be refilled
        if (tile + 1 < tile_end) stage(tile + 1, buf ^ 1);

        // 1. scores: this warp's 16 rows x 8 keys
        {
            float ca0[4] = {}, ca1[4] = {};
            const bf16 *qa = sq + (mt * 16 + (lane & 15)) * k_stride + (lane >> 4) * 8;
            const bf16 *kb = sk + (nt * 8 + (lane & 7)) * k_stride + (lane >> 3) * 8;  // 4 matrices = 32 reduction columns of 8 keys
            int ks = 0;
            for (; ks + 1 < ksteps; ks += 2) {
                uint32_t a0, a1, a2, a3, e0, e1, e2, e3, b0, b1, b2, b3;
                g_ldm_x4(a0, a1, a2, a3, qa + ks * 16);
                g_ldm_x4(e0, e1, e2, e3, qa + ks * 16 + 16);
                g_ldm_x4(b0, b1, b2, b3, kb + ks * 16);
                g_mma(ca0, a0, a1, a2, a3, b0, b1);
                g_mma(ca1, e0, e1, e2, e3, b2, b3);
            }
            if (ks < ksteps) {
                uint32_t a0, a1, a2, a3, b0, b1;
                g_ldm_x4(a0, a1, a2, a3, qa + ks * 16);
                g_ldm_x2(b0, b1, kb + ks * 16);
                g_mma(ca0, a0, a1, a2, a3, b0, b1);
            }
            int gq = lane >> 2, t = lane & 3;
            float *o = ss + (mt * 16 + gq) * kGSS + nt * 8 + 2 * t;
            o[0] = (ca0[0] + ca1[0]) * scale, o[1] = (ca0[1] + ca1[1]) * scale;
            o[8 * kGSS] = (ca0[2] + ca1[2]) * scale, o[8 * kGSS + 1] = (ca0[3] + ca1[3]) * scale;
        }
        __syncthreads();

        // 2. softmax over this tile's keys: a warp owns 4 rows, 8 lanes per row, 4 keys per lane (keys lq + 8 j)
        {
            const int i = lane >> 3, lq = lane & 7, r = warp * 4 + i;
            const int key0 = lo + tile * kGKeys + lq;
            float sv4[kGKeys / 8];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < kGKeys / 8; ++j) {
                int key = key0 + 8 * j;
                bool vis = key >= see_lo && key <= see_hi;
                float s = ss[r * kGSS + lq + 8 * j];
                if (softcap > 0.f) s = softcap * g_tanh(s * inv_cap);
                sv4[j] = vis ? s : -INFINITY;
                mx = fmaxf(mx, sv4[j]);
            }
            if (weights == 1) {  // every visible key by itself: no maximum, no sum, nothing to rescale
#pragma unroll
                for (int j = 0; j < kGKeys / 8; ++j)
                    sp[r * kGSP + lq + 8 * j] = __float2bfloat16_rn(sv4[j] == -INFINITY ? 0.f : 1.0f / (1.0f + expf(-(sv4[j] + hb))));
                if (lq == 0) s_alpha[r] = 1.f;
            } else {
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                float m_new = fmaxf(m_row, mx);
                float alpha = m_new == -INFINITY ? 1.f : expf(m_row - m_new);
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < kGKeys / 8; ++j) {
                    bf16 pb = __float2bfloat16_rn(sv4[j] == -INFINITY ? 0.f : expf(sv4[j] - m_new));
                    sum += __bfloat162float(pb);  // the rounded probability: numerator and denominator see the same weights
                    sp[r * kGSP + lq + 8 * j] = pb;
                }
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                l_row = l_row * alpha + sum;
                m_row = m_new;
                if (lq == 0) s_alpha[r] = alpha;
            }
        }
        __syncthreads();

        // 3. values
        {
            int gq = lane >> 2;
            float a_lo = s_alpha[mt * 16 + gq], a_hi = s_alpha[mt * 16 + gq + 8];
#pragma unroll
            for (int i = 0; i < 2 * PAIRS; ++i) acc[i][0] *= a_lo, acc[i][1] *= a_lo, acc[i][2] *= a_hi, acc[i][3] *= a_hi;
#pragma unroll
            for (int kk = 0; kk < kGKeys / 16; ++kk) {
                uint32_t a0, a1, a2, a3;
                g_ldm_x4(a0, a1, a2, a3, sp + (mt * 16 + (lane & 15)) * kGSP + kk * 16 + (lane >> 4) * 8);
                const bf16 *vb = sv + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * v_stride + nt * (16 * PAIRS) + (lane >> 4) * 8;
#pragma unroll
                for (int pr = 0; pr < PAIRS; ++pr) {
                    uint32_t b0, b1, b2, b3;
                    g_ldm_x4_trans(b0, b1, b2, b3, vb + pr * 16);
                    g_mma(acc[2 * pr], a0, a1, a2, a3, b0, b1);
                    g_mma(acc[2 * pr + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
    }

    __syncthreads();  // the last tile's rescale factors have been read
    if ((lane & 7) == 0) s_l[warp * 4 + (lane >> 3)] = l_row, s_alpha[warp * 4 + (lane >> 3)] = m_row;
    __syncthreads();
    if (partial != nullptr) {
        // split results: [cta (x, y)][split][32 rows][value columns + 2] fp32: un-normalised sums, then the maximum and the sum
        const int cols = 64 * PAIRS + 2;
        float *dst = partial + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * gridDim.z + blockIdx.z) * kGRows * cols;
        int gq = lane >> 2, t = lane & 3;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            int r = mt * 16 + gq + half * 8;
#pragma unroll
            for (int i = 0; i < 2 * PAIRS; ++i) {
                int col = nt * (16 * PAIRS) + i * 8 + 2 * t;
                dst[r * cols + col] = acc[i][half * 2], dst[r * cols + col + 1] = acc[i][half * 2 + 1];
            }
        }
        if (threadIdx.x < kGRows) dst[threadIdx.x * cols + 64 * PAIRS] = s_alpha[threadIdx.x], dst[threadIdx.x * cols + 64 * PAIRS + 1] = s_l[threadIdx.x];
        return;
    }
    {
        int gq = lane >> 2, t = lane & 3;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            int r = mt * 16 + gq + half * 8, tq = r / hp, hh = r % hp;
            if (tq >= count || hh >= nheads) continue;
            int head = head0 + hh;
            float inv = 1.0f / s_l[r];
            if (gate) inv *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)(first + tq) * g_token + head])));
            bf16 *o = out + (size_t)(first + tq) * o_token + (size_t)head * o_head;
#pragma unroll
            for (int i = 0; i < 2 * PAIRS; ++i) {
                int col = nt * (16 * PAIRS) + i * 8 + 2 * t;
                if (col < dv) o[col] = __float2bfloat16_rn(acc[i][half * 2] * inv);
                if (col + 1 < dv) o[col + 1] = __float2bfloat16_rn(acc[i][half * 2 + 1] * inv);
            }
        }
    }
}

// Combine the split results of one query row per CTA: weights exp(m_z - max m), added in split order; then the gate.
__global__ void __launch_bounds__(128)
paged_attention_merge_kernel(const float *__restrict__ part, int splits, int cols, const int32_t *__restrict__ tiles, int heads, int kv_heads, int hp,
                             int dv, const bf16 *__restrict__ gate, long long g_token, bf16 *__restrict__ out, long long o_token, long long o_head) {
    __shared__ float weight[64];
    __shared__ float inv_l;
    const int group = heads / kv_heads, parts = (group + hp - 1) / hp;
    const int g = blockIdx.y / parts, piece = blockIdx.y % parts;
    const int head0 = g * group + piece * hp, nheads = min(hp, group - piece * hp);
    const int first = tiles[blockIdx.x * 3 + 0], count = tiles[blockIdx.x * 3 + 1];
    const int r = blockIdx.z, tq = r / hp, hh = r % hp;
    if (tq >= count || hh >= nheads) return;
    const float *base = part + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * splits * kGRows + r) * cols;
    const size_t step = (size_t)kGRows * cols;  // from one split's row to the next split's
    if (threadIdx.x < 32) {
        float m = -INFINITY;
        for (int z = threadIdx.x; z < splits; z += 32) m = fmaxf(m, base[z * step + cols - 2]);
        m = warp_max(m);
        float l = 0.f;
        for (int z = threadIdx.x; z < splits; z += 32) {
            float mz = base[z * step + cols - 2];
            float w = mz == -INFINITY ? 0.f : expf(mz - m);
            weight[z] = w;
            l += base[z * step + cols - 1] * w;
        }
        l = warp_sum(l);
        if (threadIdx.x == 0) {
            float inv = 1.0f / l;
            if (gate) inv *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)(first + tq) * g_token + head0 + hh])));
            inv_l = inv;
        }
    }
    __syncthreads();
    bf16 *o = out + (size_t)(first + tq) * o_token + (size_t)(head0 + hh) * o_head;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float v = 0.f;
        for (int z = 0; z < splits; ++z) v = fmaf(base[z * step + c], weight[z], v);
        o[c] = __float2bfloat16_rn(v * inv_l);
    }
}

static int g_pairs(int dv) {
    int pairs = ceil_div(ceil_div(dv, 8), 8);  // value tiles (8 columns) -> pairs per quarter
    return pairs <= 1 ? 1 : pairs <= 2 ? 2 : 4;
}

}  // namespace tlb

using namespace tlb;

extern "C" {

// Rows of a CTA: tile_tokens consecutive tokens x hp query heads of one key/value head, hp = min(heads / kv_heads, 32).
int tlb_paged_attention_mma_tile_tokens(int heads, int kv_heads) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    int group = heads / kv_heads;
    return group >= kGRows ? 1 : kGRows / group;
}

int tlb_paged_attention_mma_supported(int dk, int dv, int kv_heads, int page_size) {
    return dk > 0 && dv > 0 && dk % 8 == 0 && dv % 8 == 0 && dk <= 256 && dv <= 256 && kv_heads > 0 && page_size % kGKeys == 0;
}

// Bytes of workspace for `splits` > 1 (0 for one split).
size_t tlb_paged_attention_mma_workspace(int num_tiles, int heads, int kv_heads, int dv, int splits) {
    if (splits <= 1 || heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    int group = heads / kv_heads, hp = group >= kGRows ? kGRows : group;
    return (size_t)num_tiles * kv_heads * ceil_div(group, hp) * splits * kGRows * (64 * g_pairs(dv) + 2) * sizeof(float);
}

int tlb_paged_attention_mma(const void *q, long long q_token, long long q_head, const void *slab, int num_pages, int page_size, int dk, int dv, int heads,
                            int kv_heads, const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles, const int32_t *tok_pos,
                            int mask, int mask_size, float scale, float softcap, int sink, const void *gate, long long g_token, void *out,
                            long long o_token, long long o_head, int splits, void *workspace, size_t workspace_bytes, const float *head_bias,
                            int weights, void *stream) {
    if (num_tiles <= 0) return TL_OK;
    if (weights < 0 || weights > 1 || (weights == 1 && (sink || softcap > 0.f))) return tl::fail(TL_EINVAL, "paged_attention_mma: bad weights mode");
    if (!q || !slab || !block_table || !tiles || !tok_pos || !out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || max_pages <= 0 || num_pages <= 0)
        return tl::fail(TL_EINVAL, "paged_attention_mma: bad argument");
    if (!tlb_paged_attention_mma_supported(dk, dv, kv_heads, page_size))
        return tl::fail(TL_EINVAL, "paged_attention_mma: dk, dv multiples of 8 up to 256 and page_size %% 32 == 0 are required");
    if (mask < 0 || mask > 2 || (mask != 0 && mask_size <= 0)) return tl::fail(TL_EINVAL, "paged_attention_mma: bad mask");
    if (!tl::aligned16(slab)) return tl::fail(TL_EINVAL, "paged_attention_mma: the cache must be 16-byte aligned");
    int group = heads / kv_heads;
    int hp = group >= kGRows ? kGRows : group;
    int pairs = g_pairs(dv);
    if (splits < 1) splits = 1;
    if (splits > 64) splits = 64;
    if (splits > 1 && (!workspace || workspace_bytes < tlb_paged_attention_mma_workspace(num_tiles, heads, kv_heads, dv, splits)))
        return tl::fail(TL_EWORKSPACE, "paged_attention_mma: workspace missing or too small for %d splits", splits);
    float *part = splits > 1 ? (float *)workspace : nullptr;
    int k_stride = ceil_div(dk, 16) * 16 + 8;  // (stride / 8) odd: conflict-free ldmatrix rows
    int v_stride = 64 * pairs + 8;
    size_t smem = (size_t)((kGRows + 2 * kGKeys) * k_stride + 2 * kGKeys * v_stride) * 2 + kGRows * kGSP * 2 + (size_t)kGRows * kGSS * 4 + 2 * kGRows * 4;
    dim3 grid(num_tiles, kv_heads * ceil_div(group, hp), splits);
    cudaStream_t st = as_stream(stream);
#define TLB_PAM(P)                                                                                                                               \
    do {                                                                                                                                         \
        auto kernel = paged_attention_mma_kernel<P>;                                                                                             \
        if (smem > 48 * 1024) {                                                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                \
            if (e != cudaSuccess) return tl::fail(TL_ECUDA, "paged_attention_mma: %s", cudaGetErrorString(e));                                   \
        }                                                                                                                                        \
        kernel<<<grid, kGWarps * 32, smem, st>>>((const bf16 *)q, q_token, q_head, (const bf16 *)slab, num_pages, page_size, kv_heads * (dk + dv), dk, dv, \
                                                 heads, kv_heads, hp, block_table, max_pages, tiles, tok_pos, mask, mask_size, scale, softcap, sink,    \
                                                 (const bf16 *)gate, g_token, (bf16 *)out, o_token, o_head, k_stride, v_stride, part, head_bias, weights); \
    } while (0)
    if (pairs == 1) TLB_PAM(1);
    else if (pairs == 2) TLB_PAM(2);
    else TLB_PAM(4);
#undef TLB_PAM
    TL_LAUNCH_CHECK("paged_attention_mma");
    if (splits > 1) {
        paged_attention_merge_kernel<<<dim3(num_tiles, kv_heads * ceil_div(group, hp), kGRows), 128, 0, st>>>(
            part, splits, 64 * pairs + 2, tiles, heads, kv_heads, hp, dv, (const bf16 *)gate, g_token, (bf16 *)out, o_token, o_head);
        TL_LAUNCH_CHECK("paged_attention_merge");
    }
    return TL_OK;
}

}  // extern "C"
