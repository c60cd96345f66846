// Latent (absorbed multi-query) attention over the paged latent cache, ragged batches, optional sliding window.
//
// Every head of a token attends the SAME keys: slab row j = [latent c_j (rank) | rotated shared key part (rot)], and the
// value is c_j itself, so one CTA serves a tile of up to 4 consecutive tokens of one sequence times a group of 4 heads
// (16 query rows) and streams each 32-key tile of the cache through shared memory once for all of them.  Scores, the
// running maximum / sum and the output accumulators are fp32; cache rows are converted to fp32 as they are staged, so
// the same kernel serves the bf16 and the fp32 cache.
//
// Summation order of a query row is fixed by the key index alone (32-aligned key tiles in ascending order, lanes =
// keys), never by what else shares the CTA or the launch: a row's result does not depend on the batch around it.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kTileTokens = TLB_ATTENTION_TILE_TOKENS;
constexpr int kHeadGroup = 4;
constexpr int kRows = kTileTokens * kHeadGroup;  // 16 query rows per CTA
constexpr int kWarps = 8;                        // 2 rows per warp
constexpr int kKeys = 32;                        // keys per staged tile

template <typename T, int RL /* ceil(rank / 32) */>
__global__ void __launch_bounds__(kWarps * 32)
latent_attention_kernel(const T *__restrict__ q_lat, long long ql_token, long long ql_head, const T *__restrict__ q_rot, long long qr_token,
                        long long qr_head, const T *__restrict__ slab, int num_pages, int page_size, int rank, int rot,
                        const int32_t *__restrict__ block_table, int max_pages, const int32_t *__restrict__ tiles,
                        const int32_t *__restrict__ tok_pos, int heads, int window, float scale, T *__restrict__ out, long long o_token,
                        long long o_head, const float *__restrict__ sink /* [heads]: a term exp(sink[h]) more in the denominator, or NULL */) {
    extern __shared__ float smem[];
    const int width = rank + rot;
    const int kstride = width + 1;           // odd or even, +1 breaks the 32-way conflict of lane = key reads when width % 32 == 0
    float *sq = smem;                        // [kRows][width]
    float *sk = smem + kRows * width;        // [kKeys][kstride]

    const int first = tiles[blockIdx.x * 3 + 0], count = tiles[blockIdx.x * 3 + 1], seq = tiles[blockIdx.x * 3 + 2];
    const int head0 = blockIdx.y * kHeadGroup;
    const int nheads = min(kHeadGroup, heads - head0);
    const int pos0 = tok_pos[first];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // stage the queries (scaled once, in fp32)
    for (int r = warp; r < kRows; r += kWarps) {
        int tq = r / kHeadGroup, hh = r % kHeadGroup;
        bool live = tq < count && hh < nheads;
        const T *ql = q_lat + (size_t)(first + tq) * ql_token + (size_t)(head0 + hh) * ql_head;
        const T *qr = q_rot + (size_t)(first + tq) * qr_token + (size_t)(head0 + hh) * qr_head;
        for (int d = lane; d < width; d += 32) sq[r * width + d] = !live ? 0.f : (d < rank ? to_f(ql[d]) : to_f(qr[d - rank])) * scale;
    }

    const int r0 = warp * 2, r1 = warp * 2 + 1;
    const int tq0 = r0 / kHeadGroup, tq1 = r1 / kHeadGroup;
    const bool live0 = tq0 < count && (r0 % kHeadGroup) < nheads, live1 = tq1 < count && (r1 % kHeadGroup) < nheads;
    const int p0 = pos0 + tq0, p1 = pos0 + tq1;  // positions of this warp's two rows

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    if (sink) {  // a key without a value whose score is the head's learned number: the maximum starts there, the sum at 1
        if (live0) m0 = sink[head0 + r0 % kHeadGroup], l0 = 1.f;
        if (live1) m1 = sink[head0 + r1 % kHeadGroup], l1 = 1.f;
    }
    float acc0[RL], acc1[RL];
#pragma unroll
    for (int i = 0; i < RL; ++i) acc0[i] = acc1[i] = 0.f;

    const int hi = pos0 + count - 1;                                   // newest visible key of the tile
    int lo = window > 0 ? max(0, pos0 - window + 1) : 0;               // oldest visible key of the tile
    lo = lo / kKeys * kKeys;
    const int32_t *table = block_table + (size_t)seq * max_pages;

    for (int k0 = lo; k0 <= hi; k0 += kKeys) {
        __syncthreads();  // previous tile consumed (and, first time, queries staged)
        int page = table[k0 / page_size];
        bool page_ok = page >= 0 && page < num_pages;
        const T *src = slab + ((size_t)(page_ok ? page : 0) * page_size + (k0 % page_size)) * width;
        int valid = page_ok ? min(kKeys, hi - k0 + 1) : 0;
        for (int e = threadIdx.x; e < kKeys * width; e += blockDim.x) {
            int j = e / width, d = e - j * width;
            sk[j * kstride + d] = j < valid ? to_f(src[e]) : 0.f;
        }
        __syncthreads();

        // scores: lane = key
        const int key = k0 + lane;
        float s0 = 0.f, s1 = 0.f;
        const float *kr = sk + lane * kstride;
        const float *qa = sq + r0 * width, *qb = sq + r1 * width;
        for (int d = 0; d < width; ++d) {
            float kv = kr[d];
            s0 = fmaf(qa[d], kv, s0);
            s1 = fmaf(qb[d], kv, s1);
        }
        bool vis0 = live0 && key <= p0 && (window <= 0 || p0 - key < window);
        bool vis1 = live1 && key <= p1 && (window <= 0 || p1 - key < window);
        s0 = vis0 ? s0 : -INFINITY;
        s1 = vis1 ? s1 : -INFINITY;
        float n0 = fmaxf(m0, warp_max(s0)), n1 = fmaxf(m1, warp_max(s1));
        float a0 = n0 == -INFINITY ? 1.f : expf(m0 - n0), a1 = n1 == -INFINITY ? 1.f : expf(m1 - n1);
        float e0 = vis0 ? expf(s0 - n0) : 0.f, e1 = vis1 ? expf(s1 - n1) : 0.f;
        l0 = l0 * a0 + warp_sum(e0);
        l1 = l1 * a1 + warp_sum(e1);
        m0 = n0;
        m1 = n1;
#pragma unroll
        for (int i = 0; i < RL; ++i) acc0[i] *= a0, acc1[i] *= a1;
        for (int j = 0; j < kKeys; ++j) {
            float w0 = __shfl_sync(0xffffffffu, e0, j), w1 = __shfl_sync(0xffffffffu, e1, j);
            const float *vrow = sk + j * kstride;
#pragma unroll
            for (int i = 0; i < RL; ++i) {
                int d = lane + 32 * i;
                float v = d < rank ? vrow[d] : 0.f;
                acc0[i] = fmaf(w0, v, acc0[i]);
                acc1[i] = fmaf(w1, v, acc1[i]);
            }
        }
    }

    if (live0) {
        T *o = out + (size_t)(first + tq0) * o_token + (size_t)(head0 + r0 % kHeadGroup) * o_head;
        float inv = 1.0f / l0;
#pragma unroll
        for (int i = 0; i < RL; ++i)
            if (lane + 32 * i < rank) o[lane + 32 * i] = from_f<T>(acc0[i] * inv);
    }
    if (live1) {
        T *o = out + (size_t)(first + tq1) * o_token + (size_t)(head0 + r1 % kHeadGroup) * o_head;
        float inv = 1.0f / l1;
#pragma unroll
        for (int i = 0; i < RL; ++i)
            if (lane + 32 * i < rank) o[lane + 32 * i] = from_f<T>(acc1[i] * inv);
    }
}

template <typename T, int RL>
static int launch(const void *q_lat, long long ql_token, long long ql_head, const void *q_rot, long long qr_token, long long qr_head,
                  const void *slab, int num_pages, int page_size, int rank, int rot, const int32_t *block_table, int max_pages,
                  const int32_t *tiles, int num_tiles, const int32_t *tok_pos, int heads, int window, float scale, void *out, long long o_token,
                  long long o_head, const float *sink, cudaStream_t st) {
    int width = rank + rot;
    size_t smem = ((size_t)kRows * width + (size_t)kKeys * (width + 1)) * sizeof(float);
    auto kernel = latent_attention_kernel<T, RL>;
    if (smem > 48 * 1024) {
        if (smem > 227 * 1024) return tl::fail(TL_EINVAL, "latent_attention: rank + rot = %d does not fit in shared memory", width);
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return tl::fail(TL_ECUDA, "latent_attention: %s", cudaGetErrorString(e));
    }
    dim3 grid(num_tiles, ceil_div(heads, kHeadGroup));
    kernel<<<grid, kWarps * 32, smem, st>>>((const T *)q_lat, ql_token, ql_head, (const T *)q_rot, qr_token, qr_head, (const T *)slab, num_pages,
                                            page_size, rank, rot, block_table, max_pages, tiles, tok_pos, heads, window, scale, (T *)out, o_token,
                                            o_head, sink);
    return TL_OK;
}

}  // namespace tlb

using namespace tlb;

extern "C" int tlb_latent_attention(const void *q_lat, long long ql_token, long long ql_head, const void *q_rot, long long qr_token,
                                    long long qr_head, const void *slab, int num_pages, int page_size, int rank, int rot,
                                    const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles, const int32_t *tok_pos,
                                    int heads, int window, float scale, void *out, long long o_token, long long o_head, const float *sink, int dtype,
                                    void *stream) {
    if (num_tiles <= 0) return TL_OK;
    if (!q_lat || (!q_rot && rot > 0) || !slab || !block_table || !tiles || !tok_pos || !out || rank <= 0 || rot < 0 || heads <= 0 ||
        max_pages <= 0 || num_pages <= 0)
        return tl::fail(TL_EINVAL, "latent_attention: bad argument");
    if (page_size <= 0 || page_size % kKeys != 0) return tl::fail(TL_EINVAL, "latent_attention: page_size must be a multiple of %d", kKeys);
    if (rank > 1024) return tl::fail(TL_EINVAL, "latent_attention: rank %d > 1024", rank);
    cudaStream_t st = as_stream(stream);
    int rl = ceil_div(rank, 32);
    int rc = TL_OK;
#define TLB_LA(RLV)                                                                                                                          \
    rc = launch<T, RLV>(q_lat, ql_token, ql_head, q_rot ? q_rot : q_lat, qr_token, qr_head, slab, num_pages, page_size, rank, rot, block_table, \
                        max_pages, tiles, num_tiles, tok_pos, heads, window, scale, out, o_token, o_head, sink, st)
    TLB_DISPATCH(dtype, "latent_attention", if (rl <= 4) TLB_LA(4); else if (rl <= 8) TLB_LA(8); else if (rl <= 16) TLB_LA(16); else TLB_LA(32));
#undef TLB_LA
    if (rc != TL_OK) return rc;
    TL_LAUNCH_CHECK("latent_attention");
    return TL_OK;
}
