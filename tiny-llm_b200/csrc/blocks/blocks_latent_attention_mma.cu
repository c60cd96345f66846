// Latent attention on the tensor cores (bf16 cache, mma.sync m16n8k16, fp32 accumulation and softmax).
//
// All heads of a token attend the same keys (cache row j = [latent | rotated shared key part]) and mix the same values
// (the latent part of the row), so a CTA takes 32 query rows = a run of consecutive tokens of one sequence x a group of
// heads and streams every 32-key tile of the paged cache through shared memory ONCE for all of them (cp.async into one
// buffer: at the widest cache row, 576 entries, a CTA holds 82 KB, so two CTAs share an SM and one computes while the
// other loads).  Per key tile, with 8 warps:
//   1. scores:  the 32 x 32 block S = Q K^T is 2 x 4 blocks of 16 x 8, one per warp (two accumulator sets alternate
//               over the reduction so that consecutive MMAs do not wait on each other);
//   2. softmax: each warp owns 4 rows, 8 lanes per row, 4 keys per lane: mask, running maximum / sum, P = exp(S - m) as bf16, rescale factor;
//   3. values:  O[32 x rank] += P V, warp = (16-row half, quarter of the value columns); V is the key tile itself.
// A row's arithmetic depends only on its own position (32-aligned key tiles in ascending order): what else is in the
// CTA, the launch or the batch does not change its result.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kMRows = 32;   // query rows per CTA
constexpr int kMKeys = 32;   // keys per tile
constexpr int kSS = kMKeys + 1;  // score row stride (floats)
constexpr int kSP = kMKeys + 8;  // probability row stride (bf16): (stride / 8) odd
constexpr int kMWarps = 8;

__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t &r0, uint32_t &r1, const void *p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// PAIRS = pairs of 8-column value tiles per warp (the warp's quarter of the value columns = 16 * PAIRS columns).
template <int PAIRS>
__global__ void __launch_bounds__(kMWarps * 32)
latent_attention_mma_kernel(const bf16 *__restrict__ q_lat, long long ql_token, long long ql_head, const bf16 *__restrict__ q_rot, long long qr_token,
                            long long qr_head, const bf16 *__restrict__ slab, int num_pages, int page_size, int rank, int rot,
                            const int32_t *__restrict__ block_table, int max_pages, const int32_t *__restrict__ tiles,
                            const int32_t *__restrict__ tok_pos, int heads, int head_group, int window, float scale, bf16 *__restrict__ out,
                            long long o_token, long long o_head, int row_stride /* shared-memory row stride in elements */,
                            float *__restrict__ part /* split results, or NULL */, const float *__restrict__ sink /* [heads] or NULL */) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int width = rank + rot;
    bf16 *sq = reinterpret_cast<bf16 *>(smem_raw);                  // [32][row_stride]
    bf16 *sk0 = sq + kMRows * row_stride;                           // [32][row_stride], one buffer: two CTAs share an SM and cover each other's loads
    bf16 *sp = sk0 + kMKeys * row_stride;                       // [32][kSP]
    float *ss = reinterpret_cast<float *>(sp + kMRows * kSP);       // [32][kSS]
    float *s_alpha = ss + kMRows * kSS;                             // [32]
    float *s_l = s_alpha + kMRows;                                  // [32]

    const int first = tiles[blockIdx.x * 3 + 0], count = tiles[blockIdx.x * 3 + 1], seq = tiles[blockIdx.x * 3 + 2];
    const int head0 = blockIdx.y * head_group;
    const int nheads = min(head_group, heads - head0);
    const int pos0 = tok_pos[first];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = width / 8;  // 16-byte pieces of a cache row

    // zero everything once: padding columns of Q and K must read as zero in every product
    for (int i = threadIdx.x; i < ((kMRows + kMKeys) * row_stride) / 8; i += blockDim.x) reinterpret_cast<uint4 *>(sq)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    // queries: row = token-in-tile * head_group + head-in-group
    for (int r = warp; r < kMRows; r += kMWarps) {
        int tq = r / head_group, hh = r % head_group;
        if (tq >= count || hh >= nheads) continue;
        const bf16 *ql = q_lat + (size_t)(first + tq) * ql_token + (size_t)(head0 + hh) * ql_head;
        const bf16 *qr = q_rot + (size_t)(first + tq) * qr_token + (size_t)(head0 + hh) * qr_head;
        for (int d = lane; d < width; d += 32) sq[r * row_stride + d] = d < rank ? ql[d] : qr[d - rank];
    }

    const int hi = pos0 + count - 1;
    int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    lo = lo / kMKeys * kMKeys;
    const int32_t *table = block_table + (size_t)seq * max_pages;
    const int n_tiles = (hi - lo) / kMKeys + 1;

    auto stage = [&](int tile, bf16 *dst) {
        int k0 = lo + tile * kMKeys;
        int page = table[k0 / page_size];
        bool ok = page >= 0 && page < num_pages;
        int valid = ok ? min(kMKeys, hi - k0 + 1) : 0;
        const bf16 *src = slab + ((size_t)(ok ? page : 0) * page_size + (k0 % page_size)) * width;
        for (int j = warp; j < kMKeys; j += kMWarps) {  // a warp copies whole rows: no index arithmetic beyond an add
            bf16 *d = dst + j * row_stride;
            const bf16 *g = src + (size_t)j * width;
            if (j < valid) {
                for (int piece = lane; piece < chunks; piece += 32) cp_async16(d + piece * 8, g + piece * 8);
            } else {
                for (int piece = lane; piece < chunks; piece += 32) *reinterpret_cast<uint4 *>(d + piece * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };

    // softmax state of the row this lane works on (a warp owns 4 rows, 8 lanes each; uniform over the 8 lanes)
    float m_row = -INFINITY, l_row = 0.f;
    int pos_row;
    bool live_row;
    {
        int r = warp * 4 + (lane >> 3), tq = r / head_group, hh = r % head_group;
        live_row = tq < count && hh < nheads;
        pos_row = pos0 + tq;
        // a sink: a key without a value whose score is the head's learned number (counted once when the key range is split)
        if (sink && live_row && blockIdx.z == 0) m_row = sink[head0 + hh], l_row = 1.f;
    }
    const int mt = warp & 1, nt = warp >> 1;          // score block of this warp; nt is also its quarter of the value columns
    float acc[2 * PAIRS][4];
#pragma unroll
    for (int i = 0; i < 2 * PAIRS; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    // with the key range split over gridDim.z CTAs, this one takes a contiguous run of key tiles
    const int per_split = (n_tiles + (int)gridDim.z - 1) / (int)gridDim.z;
    const int tile_begin = (int)blockIdx.z * per_split, tile_end = min(n_tiles, tile_begin + per_split);
    const int ksteps = (width + 15) / 16;
    for (int tile = tile_begin; tile < tile_end; ++tile) {
        bf16 *sk = sk0;
        __syncthreads();  // every warp is done with the previous tile (and, first time, the zero fill and the queries are in place)
        stage(tile, sk);
        cp_async_wait<0>();
        __syncthreads();  // this tile is in shared memory

        // 1. scores: this warp's 16 rows x 8 keys, two reduction steps per pair of loads
        {
            float ca0[4] = {}, ca1[4] = {};
            const bf16 *qa = sq + (mt * 16 + (lane & 15)) * row_stride + (lane >> 4) * 8;
            const bf16 *kb = sk + (nt * 8 + (lane & 7)) * row_stride + (lane >> 3) * 8;  // 4 matrices = 32 reduction columns of 8 keys
            int ks = 0;
            for (; ks + 1 < ksteps; ks += 2) {
                uint32_t a0, a1, a2, a3, e0, e1, e2, e3, b0, b1, b2, b3;
                ldmatrix_x4(a0, a1, a2, a3, qa + ks * 16);
                ldmatrix_x4(e0, e1, e2, e3, qa + ks * 16 + 16);
                ldmatrix_x4(b0, b1, b2, b3, kb + ks * 16);
                mma_bf16(ca0, a0, a1, a2, a3, b0, b1);
                mma_bf16(ca1, e0, e1, e2, e3, b2, b3);
            }
            if (ks < ksteps) {
                uint32_t a0, a1, a2, a3, b0, b1;
                ldmatrix_x4(a0, a1, a2, a3, qa + ks * 16);
                ldmatrix_x2(b0, b1, kb + ks * 16);
                mma_bf16(ca0, a0, a1, a2, a3, b0, b1);
            }
            int g = lane >> 2, t = lane & 3;
            float *o = ss + (mt * 16 + g) * kSS + nt * 8 + 2 * t;
            o[0] = (ca0[0] + ca1[0]) * scale, o[1] = (ca0[1] + ca1[1]) * scale;
            o[8 * kSS] = (ca0[2] + ca1[2]) * scale, o[8 * kSS + 1] = (ca0[3] + ca1[3]) * scale;
        }
        __syncthreads();

        // 2. softmax over this tile's keys: a warp owns 4 rows, 8 lanes per row, 4 keys per lane (keys lq + 8 j)
        {
            const int i = lane >> 3, lq = lane & 7, r = warp * 4 + i;
            const int key0 = lo + tile * kMKeys + lq;
            const int rp = pos_row;
            const bool live = live_row;
            float sv[kMKeys / 8];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < kMKeys / 8; ++j) {
                int key = key0 + 8 * j;
                bool vis = live && key <= rp && (window <= 0 || rp - key < window);
                sv[j] = vis ? ss[r * kSS + lq + 8 * j] : -INFINITY;
                mx = fmaxf(mx, sv[j]);
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float m_new = fmaxf(m_row, mx);
            float alpha = m_new == -INFINITY ? 1.f : expf(m_row - m_new);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < kMKeys / 8; ++j) {
                bf16 pb = __float2bfloat16_rn(sv[j] == -INFINITY ? 0.f : expf(sv[j] - m_new));
                sum += __bfloat162float(pb);  // the rounded probability: numerator and denominator see the same weights
                sp[r * kSP + lq + 8 * j] = pb;
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            l_row = l_row * alpha + sum;
            m_row = m_new;
            if (lq == 0) s_alpha[r] = alpha;
        }
        __syncthreads();

        // 3. values
        {
            int g = lane >> 2;
            float a_lo = s_alpha[mt * 16 + g], a_hi = s_alpha[mt * 16 + g + 8];
#pragma unroll
            for (int i = 0; i < 2 * PAIRS; ++i) acc[i][0] *= a_lo, acc[i][1] *= a_lo, acc[i][2] *= a_hi, acc[i][3] *= a_hi;
#pragma unroll
            for (int kk = 0; kk < kMKeys / 16; ++kk) {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(a0, a1, a2, a3, sp + (mt * 16 + (lane & 15)) * kSP + kk * 16 + (lane >> 4) * 8);
                const bf16 *vb = sk + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * row_stride + nt * (16 * PAIRS) + (lane >> 4) * 8;
#pragma unroll
                for (int pr = 0; pr < PAIRS; ++pr) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, vb + pr * 16);
                    mma_bf16(acc[2 * pr], a0, a1, a2, a3, b0, b1);
                    mma_bf16(acc[2 * pr + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
    }

    __syncthreads();  // the last tile's rescale factors have been read
    if ((lane & 7) == 0) s_l[warp * 4 + (lane >> 3)] = l_row, s_alpha[warp * 4 + (lane >> 3)] = m_row;
    __syncthreads();
    if (part != nullptr) {
        // split results: [cta (x, y)][split][32 rows][value columns + 2] fp32: un-normalised sums, then the maximum and the sum
        const int cols = 64 * PAIRS + 2;
        float *dst = part + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * gridDim.z + blockIdx.z) * kMRows * cols;
        int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            int r = mt * 16 + g + half * 8;
#pragma unroll
            for (int i = 0; i < 2 * PAIRS; ++i) {
                int col = nt * (16 * PAIRS) + i * 8 + 2 * t;
                dst[r * cols + col] = acc[i][half * 2], dst[r * cols + col + 1] = acc[i][half * 2 + 1];
            }
        }
        if (threadIdx.x < kMRows) dst[threadIdx.x * cols + 64 * PAIRS] = s_alpha[threadIdx.x], dst[threadIdx.x * cols + 64 * PAIRS + 1] = s_l[threadIdx.x];
        return;
    }
    {
        int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            int r = mt * 16 + g + half * 8, tq = r / head_group, hh = r % head_group;
            if (tq >= count || hh >= nheads) continue;
            float inv = 1.0f / s_l[r];
            bf16 *o = out + (size_t)(first + tq) * o_token + (size_t)(head0 + hh) * o_head;
#pragma unroll
            for (int i = 0; i < 2 * PAIRS; ++i) {
                int col = nt * (16 * PAIRS) + i * 8 + 2 * t;
                if (col < rank) o[col] = __float2bfloat16_rn(acc[i][half * 2] * inv);
                if (col + 1 < rank) o[col + 1] = __float2bfloat16_rn(acc[i][half * 2 + 1] * inv);
            }
        }
    }
}

// Combine the split results of one query row per CTA: weights exp(m_z - max m), added in split order.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float *__restrict__ part, int splits, int cols, const int32_t *__restrict__ tiles, int heads, int head_group,
                              int rank, bf16 *__restrict__ out, long long o_token, long long o_head) {
    __shared__ float weight[64];
    __shared__ float inv_l;
    const int first = tiles[blockIdx.x * 3 + 0], count = tiles[blockIdx.x * 3 + 1];
    const int head0 = blockIdx.y * head_group, nheads = min(head_group, heads - head0);
    const int r = blockIdx.z, tq = r / head_group, hh = r % head_group;
    if (tq >= count || hh >= nheads) return;
    const float *base = part + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * splits * kMRows + r) * cols;
    const size_t step = (size_t)kMRows * cols;  // from one split's row to the next split's
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
        if (threadIdx.x == 0) inv_l = 1.0f / l;
    }
    __syncthreads();
    bf16 *o = out + (size_t)(first + tq) * o_token + (size_t)(head0 + hh) * o_head;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float v = 0.f;
        for (int z = 0; z < splits; ++z) v = fmaf(base[z * step + c], weight[z], v);
        o[c] = __float2bfloat16_rn(v * inv_l);
    }
}

}  // namespace tlb

using namespace tlb;

static int mma_pairs(int rank) {
    int pairs = ceil_div(ceil_div(rank, 8), 8);  // value tiles (8 columns) -> pairs per quarter
    return pairs <= 1 ? 1 : pairs <= 2 ? 2 : pairs <= 4 ? 4 : 8;
}

// Bytes of workspace for `splits` > 1 (0 for one split).
extern "C" size_t tlb_latent_attention_mma_workspace(int num_tiles, int heads, int rank, int splits) {
    if (splits <= 1) return 0;
    int head_group = heads >= kMRows ? kMRows : heads;
    return (size_t)num_tiles * ceil_div(heads, head_group) * splits * kMRows * (64 * mma_pairs(rank) + 2) * sizeof(float);
}

// Rows of a CTA: `tile_tokens` consecutive tokens x `head_group` heads, head_group = min(heads, 32), tile_tokens = 32 / head_group.
extern "C" int tlb_latent_attention_mma_tile_tokens(int heads) { return heads >= kMRows ? 1 : kMRows / heads; }

extern "C" int tlb_latent_attention_mma_supported(int rank, int rot, int page_size) {
    return rank > 0 && rank <= 512 && (rank + rot) % 8 == 0 && page_size % kMKeys == 0;
}

extern "C" int tlb_latent_attention_mma(const void *q_lat, long long ql_token, long long ql_head, const void *q_rot, long long qr_token,
                                        long long qr_head, const void *slab, int num_pages, int page_size, int rank, int rot,
                                        const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles, const int32_t *tok_pos,
                                        int heads, int window, float scale, void *out, long long o_token, long long o_head, int splits,
                                        void *workspace, size_t workspace_bytes, const float *sink, void *stream) {
    if (num_tiles <= 0) return TL_OK;
    if (!q_lat || (!q_rot && rot > 0) || !slab || !block_table || !tiles || !tok_pos || !out || heads <= 0 || max_pages <= 0 || num_pages <= 0)
        return tl::fail(TL_EINVAL, "latent_attention_mma: bad argument");
    if (!tlb_latent_attention_mma_supported(rank, rot, page_size))
        return tl::fail(TL_EINVAL, "latent_attention_mma: rank <= 512, (rank + rot) %% 8 == 0 and page_size %% 32 == 0 are required");
    if (!tl::aligned16(slab)) return tl::fail(TL_EINVAL, "latent_attention_mma: the cache must be 16-byte aligned");
    int width = rank + rot;
    int pairs = mma_pairs(rank);
    if (splits < 1) splits = 1;
    if (splits > 64) splits = 64;
    if (splits > 1 && (!workspace || workspace_bytes < tlb_latent_attention_mma_workspace(num_tiles, heads, rank, splits)))
        return tl::fail(TL_EWORKSPACE, "latent_attention_mma: workspace missing or too small for %d splits", splits);
    float *part = splits > 1 ? (float *)workspace : nullptr;
    int span = max(ceil_div(width, 16) * 16, 64 * pairs);  // columns a row must hold: the padded key width, the four value quarters
    int row_stride = span + 8;                              // (stride / 8) odd: conflict-free ldmatrix rows
    size_t smem = (size_t)(kMRows + kMKeys) * row_stride * 2 + kMRows * kSP * 2 + (size_t)kMRows * kSS * 4 + 2 * kMRows * 4;
    int head_group = heads >= kMRows ? kMRows : heads;
    dim3 grid(num_tiles, ceil_div(heads, head_group), splits);
    cudaStream_t st = as_stream(stream);
#define TLB_LAM(P)                                                                                                                          \
    do {                                                                                                                                    \
        auto kernel = latent_attention_mma_kernel<P>;                                                                                       \
        if (smem > 48 * 1024) {                                                                                                             \
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                           \
            if (e != cudaSuccess) return tl::fail(TL_ECUDA, "latent_attention_mma: %s", cudaGetErrorString(e));                             \
        }                                                                                                                                   \
        kernel<<<grid, kMWarps * 32, smem, st>>>((const bf16 *)q_lat, ql_token, ql_head, (const bf16 *)(q_rot ? q_rot : q_lat), qr_token,   \
                                                 qr_head, (const bf16 *)slab, num_pages, page_size, rank, rot, block_table, max_pages, tiles, \
                                                 tok_pos, heads, head_group, window, scale, (bf16 *)out, o_token, o_head, row_stride, part, sink); \
    } while (0)
    if (pairs == 1) TLB_LAM(1);
    else if (pairs == 2) TLB_LAM(2);
    else if (pairs == 4) TLB_LAM(4);
    else TLB_LAM(8);
#undef TLB_LAM
    TL_LAUNCH_CHECK("latent_attention_mma");
    if (splits > 1) {
        latent_attention_merge_kernel<<<dim3(num_tiles, ceil_div(heads, head_group), kMRows), 128, 0, st>>>(part, splits, 64 * pairs + 2, tiles, heads, head_group,
                                                                                                   rank, (bf16 *)out, o_token, o_head);
        TL_LAUNCH_CHECK("latent_attention_merge");
    }
    return TL_OK;
}
