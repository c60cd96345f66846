// Top-k mixture-of-experts feed-forward: router (fp32 logits, top-k, softmax over the chosen), grouping of the
// (token, choice) pairs by expert on the device, the two grouped products and the weighted combination.
//
// The pairs of one expert occupy whole 32-row tiles of a sorted row list, so every CTA of the grouped products reads
// ONE expert's weights; rows are gathered from / scattered to token order through the list.  Each output row is a sum
// over the reduction index in a fixed order and the combination adds a token's choices in choice order, so a token's
// result does not depend on which other tokens are in the batch.
#include "blocks_common.cuh"

namespace tlb {

constexpr int kTileRows = TLB_MOE_TILE_ROWS;

__device__ __forceinline__ float moe_act(float z, int act) {
    if (act == 0) return z / (1.0f + expf(-z));
    if (act == 2) return z > 0.f ? z * z : 0.f;  // squared ReLU
    float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(inner));
}

// Which rows of `a` a tile's rows read: the sorted rows themselves (the second product), the token of the pair, or the pair.
constexpr int kGatherSorted = 0, kGatherToken = 1, kGatherPair = 2;
__device__ __forceinline__ int moe_src_row(int pair, int sorted_row, int top, int gather) {
    if (pair < 0) return -1;
    return gather == kGatherSorted ? sorted_row : gather == kGatherToken ? pair / top : pair;
}

// One CTA per token: the row of h is staged in shared memory as fp32, the warps share the experts (each logit is one
// warp's dot product in a fixed lane order, so it does not depend on the launch), then warp 0 picks the top-k.
template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T *__restrict__ h, const T *__restrict__ w, const T *__restrict__ b, int tokens, int dim, int experts, int top, int scoring,
                 const T *__restrict__ choice_bias, float weight_scale, int32_t *__restrict__ idx, float *__restrict__ gate) {
    extern __shared__ float route_smem[];
    float *x = route_smem;        // [dim]
    float *z = route_smem + dim;  // [experts]: what the choice is made by
    float *p_all = z + experts;   // [experts]: scoring 2, the softmax over all outputs
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) x[d] = to_f(h[(size_t)t * dim + d]);
    __syncthreads();
    for (int e = warp; e < experts; e += warps) {
        const T *row = w + (size_t)e * dim;
        float s = 0.f;
        for (int d = lane; d < dim; d += 32) s = fmaf(x[d], to_f(row[d]), s);
        s = warp_sum(s);
        if (lane == 0) z[e] = s + (b ? to_f(b[e]) : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    if (scoring == 2) {  // scores = softmax over ALL outputs; the choice adds a bias to them, the weights do not
        float m = -INFINITY, sum = 0.f;
        for (int e = lane; e < experts; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        for (int e = lane; e < experts; e += 32) sum += expf(z[e] - m);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) {
            float p = expf(z[e] - m) / sum;
            p_all[e] = p;
            z[e] = p + (choice_bias ? to_f(choice_bias[e]) : 0.f);
        }
        __syncwarp();
    }
    // top-k by repeated arg-max over the warp (lower index wins a tie); weights = softmax over the chosen logits
    float first_v = 0.f, denom = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            float v = z[e];
            if (v > bv || (v == bv && e < bi)) bv = v, bi = e;
        }
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        if (k == 0) first_v = bv;
        // scoring 0: softmax over the chosen logits (the first choice is the largest); 1: each choice's own sigmoid, as it is
        float p = scoring == 1 ? 1.0f / (1.0f + expf(-bv)) : scoring == 2 ? p_all[min(bi, experts - 1)] : expf(bv - first_v);
        denom += p;
        if (lane == 0) {
            idx[(size_t)t * top + k] = bi;
            gate[(size_t)t * top + k] = p;
            if (bi != 0x7fffffff) z[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (scoring == 1) return;
    // scoring 2: the chosen scores renormalised (a guard against an all-zero choice) and scaled
    for (int k = lane; k < top; k += 32)
        gate[(size_t)t * top + k] = scoring == 2 ? gate[(size_t)t * top + k] / (denom + 1e-20f) * weight_scale : gate[(size_t)t * top + k] / denom;
}

// Single CTA: histogram, padded exclusive scan, scatter.
__global__ void moe_sort_kernel(const int32_t *__restrict__ idx, int pairs, int experts, int max_rows, int tile_rows, int32_t *__restrict__ sorted_pair,
                                int32_t *__restrict__ tile_expert, int32_t *__restrict__ counters) {
    extern __shared__ int sm[];
    int *count = sm, *start = sm + experts, *cursor = sm + 2 * experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0, cursor[e] = 0;
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x) sorted_pair[r] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        int e = idx[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = row;
            int tiles = (count[e] + tile_rows - 1) / tile_rows;
            for (int i = 0; i < tiles; ++i) tile_expert[row / tile_rows + i] = e;
            row += tiles * tile_rows;
        }
        counters[0] = row / tile_rows;
        counters[1] = row;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        int e = idx[p];
        if (e >= 0 && e < experts) sorted_pair[start[e] + atomicAdd(&cursor[e], 1)] = p;
    }
}

// C tile [32 rows x 64 columns] of  A[rows, K] . W[e][cols, K]^T, fp32 accumulation in k order.
// 256 threads: thread (ty, tx) owns rows 2 ty .. 2 ty + 1 and columns tx + 16 c, c = 0..3.
constexpr int kBN = 64, kBK = 16;

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T *__restrict__ a, const T *__restrict__ w1, const T *__restrict__ w2, const int32_t *__restrict__ sorted_pair,
                   const int32_t *__restrict__ tile_expert, const int32_t *__restrict__ counters, int top, int K, int N, int act, int gather,
                   T *__restrict__ inter, float *__restrict__ pair_out) {
    if ((int)blockIdx.x >= counters[0]) return;
    __shared__ float sa[kBK][kTileRows + 1];
    __shared__ float sb1[kBK][kBN + 1];
    __shared__ float sb2[GATED ? kBK : 1][kBN + 1];
    __shared__ int src_row[kTileRows];
    const int e = tile_expert[blockIdx.x];
    const int row0 = blockIdx.x * kTileRows, col0 = blockIdx.y * kBN;
    if (threadIdx.x < kTileRows) {
        // the first product gathers rows of h (or of its scaled copy); the second reads the sorted intermediate rows
        src_row[threadIdx.x] = moe_src_row(sorted_pair[row0 + threadIdx.x], row0 + (int)threadIdx.x, top, gather);
    }
    __syncthreads();
    const T *wa = w1 + (size_t)e * N * K;
    const T *wb = GATED ? w2 + (size_t)e * N * K : nullptr;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    float c1[2][4] = {}, c2[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += kBK) {
        for (int i = threadIdx.x; i < kTileRows * kBK; i += 256) {
            int r = i / kBK, k = i % kBK;
            int sr = src_row[r];
            sa[k][r] = (sr >= 0 && k0 + k < K) ? to_f(a[(size_t)sr * K + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < kBN * kBK; i += 256) {
            int n = i / kBK, k = i % kBK;
            bool ok = col0 + n < N && k0 + k < K;
            sb1[k][n] = ok ? to_f(wa[(size_t)(col0 + n) * K + k0 + k]) : 0.f;
            if (GATED) sb2[k][n] = ok ? to_f(wb[(size_t)(col0 + n) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kBK; ++k) {
            float a0 = sa[k][2 * ty], a1 = sa[k][2 * ty + 1];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float b = sb1[k][tx + 16 * c];
                c1[0][c] = fmaf(a0, b, c1[0][c]);
                c1[1][c] = fmaf(a1, b, c1[1][c]);
                if (GATED) {
                    float b2 = sb2[k][tx + 16 * c];
                    c2[0][c] = fmaf(a0, b2, c2[0][c]);
                    c2[1][c] = fmaf(a1, b2, c2[1][c]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        int row = row0 + 2 * ty + r;
        int pair = sorted_pair[row];
        if (pair < 0) continue;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            int col = col0 + tx + 16 * c;
            if (col >= N) continue;
            if (GATED) inter[(size_t)row * N + col] = from_f<T>(moe_act(c1[r][c], act) * c2[r][c]);
            else if (inter) inter[(size_t)row * N + col] = from_f<T>(moe_act(c1[r][c], act));
            else pair_out[(size_t)pair * N + col] = c1[r][c];
        }
    }
}


// ---- the grouped products on the tensor cores (bf16, K % 8 == 0) ------------------------------------------------
// One CTA = one 32- or 64-row expert tile x 128 output columns; 8 warps = 2 row halves x 4 column quarters (4 x 2 for 64 rows), each
// mma.sync m16n8k16 over 32-wide reduction blocks that cp.async brings into a two-stage ring (A rows gathered
// through the sorted pair list).  fp32 accumulators; the reduction order of a row is k ascending in both kernels.
constexpr int kTN = 128, kTK = 32, kTS = kTK + 8;  // row stride 40 elements = 80 B: (80 / 16) odd, conflict-free ldmatrix

__device__ __forceinline__ void moe_ldm_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void moe_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void moe_cp16(void *dst, const void *src, bool ok) {
    uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    int bytes = ok ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <bool GATED, int BM>
__global__ void __launch_bounds__(256)
moe_grouped_mma_kernel(const bf16 *__restrict__ a, const bf16 *__restrict__ w1, const bf16 *__restrict__ w2, const int32_t *__restrict__ sorted_pair,
                       const int32_t *__restrict__ tile_expert, const int32_t *__restrict__ counters, int top, int K, int N, int act, int gather,
                       bf16 *__restrict__ inter, float *__restrict__ pair_out) {
    if ((int)blockIdx.x >= counters[0]) return;
    constexpr int MT = BM / 16;          // 16-row halves/quarters of the tile
    constexpr int NW = 8 / MT;           // warps along the columns
    constexpr int NPW = kTN / NW / 8;    // 8-column blocks per warp
    extern __shared__ __align__(16) unsigned char moe_smem[];
    bf16 (*sa)[BM * kTS] = reinterpret_cast<bf16 (*)[BM * kTS]>(moe_smem);                              // [2]
    bf16 (*sb1)[kTN * kTS] = reinterpret_cast<bf16 (*)[kTN * kTS]>(moe_smem + 2 * BM * kTS * 2);        // [2]
    bf16 (*sb2)[kTN * kTS] = reinterpret_cast<bf16 (*)[kTN * kTS]>(moe_smem + 2 * (BM + kTN) * kTS * 2);  // [2], gated only
    __shared__ int src_row[BM];
    const int e = tile_expert[blockIdx.x];
    const int row0 = blockIdx.x * BM, col0 = blockIdx.y * kTN;
    if (threadIdx.x < BM) {
        src_row[threadIdx.x] = moe_src_row(sorted_pair[row0 + threadIdx.x], row0 + (int)threadIdx.x, top, gather);
    }
    __syncthreads();
    const bf16 *wa = w1 + (size_t)e * N * K;
    const bf16 *wb = GATED ? w2 + (size_t)e * N * K : nullptr;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = warp % MT, nq = warp / MT;

    auto stage = [&](int kb, int buf) {
        int k0 = kb * kTK;
        if (threadIdx.x < BM * 4) {  // A: BM rows x 4 pieces of 8
            int r = threadIdx.x >> 2, piece = threadIdx.x & 3;
            int sr = src_row[r], k = k0 + piece * 8;
            bool ok = sr >= 0 && k < K;
            moe_cp16(&sa[buf][r * kTS + piece * 8], a + (ok ? (size_t)sr * K + k : 0), ok);
        }
        for (int c = threadIdx.x; c < kTN * 4; c += 256) {  // B: 128 rows x 4 pieces
            int n = c >> 2, piece = c & 3;
            int k = k0 + piece * 8;
            bool ok = col0 + n < N && k < K;
            size_t off = ok ? (size_t)(col0 + n) * K + k : 0;
            moe_cp16(&sb1[buf][n * kTS + piece * 8], wa + off, ok);
            if (GATED) moe_cp16(&sb2[buf][n * kTS + piece * 8], wb + off, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float c1[NPW][4] = {}, c2[GATED ? NPW : 1][4] = {};
    const int kblocks = (K + kTK - 1) / kTK;
    stage(0, 0);
    for (int kb = 0; kb < kblocks; ++kb) {
        int buf = kb & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // this block has landed; everybody is done with the other buffer
        if (kb + 1 < kblocks) stage(kb + 1, buf ^ 1);
#pragma unroll
        for (int ks = 0; ks < kTK / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            moe_ldm_x4(a0, a1, a2, a3, &sa[buf][(mt * 16 + (lane & 15)) * kTS + ks * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int np = 0; np < NPW / 2; ++np) {  // two n8 tiles per ldmatrix.x4: rows n..n+7 and n+8..n+15, k halves 0 / 8
                int n = nq * (8 * NPW) + np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
                int kk = ks * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                moe_ldm_x4(b0, b1, b2, b3, &sb1[buf][n * kTS + kk]);
                moe_mma(c1[2 * np], a0, a1, a2, a3, b0, b1);
                moe_mma(c1[2 * np + 1], a0, a1, a2, a3, b2, b3);
                if (GATED) {
                    moe_ldm_x4(b0, b1, b2, b3, &sb2[buf][n * kTS + kk]);
                    moe_mma(c2[2 * np], a0, a1, a2, a3, b0, b1);
                    moe_mma(c2[2 * np + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
    }
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        int row = row0 + mt * 16 + g + half * 8;
        int pair = sorted_pair[row];
        if (pair < 0) continue;
#pragma unroll
        for (int i = 0; i < NPW; ++i) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                int col = col0 + nq * (8 * NPW) + i * 8 + 2 * t + j;
                if (col >= N) continue;
                float v = c1[i][half * 2 + j];
                if (GATED) inter[(size_t)row * N + col] = __float2bfloat16_rn(moe_act(v, act) * c2[i][half * 2 + j]);
                else if (inter) inter[(size_t)row * N + col] = __float2bfloat16_rn(moe_act(v, act));
                else pair_out[(size_t)pair * N + col] = v;
            }
        }
    }
}

// out[pair, :] = gate[pair] * h[pair / top, :] rounded to T: the rows of experts whose weight multiplies their input.
template <typename T>
__global__ void moe_scale_rows_kernel(const T *__restrict__ h, const float *__restrict__ gate, T *__restrict__ out, int top, int dim) {
    const int pair = blockIdx.x;
    const float g = gate[pair];
    const T *src = h + (size_t)(pair / top) * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) out[(size_t)pair * dim + d] = from_f<T>(g * to_f(src[d]));
}

// idx != NULL: a choice whose expert id is >= experts is an identity expert, its output the token's input row h[t, :].
template <typename T>
__global__ void moe_combine_kernel(const float *__restrict__ pair_out, const float *__restrict__ gate, const T *__restrict__ shared,
                                   const int32_t *__restrict__ idx, int experts, const T *__restrict__ h, float *__restrict__ y, int top, int dim) {
    int t = blockIdx.x;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const bool same = idx != nullptr && idx[(size_t)t * top + k] >= experts;
            s = fmaf(gate ? gate[(size_t)t * top + k] : 1.f, same ? to_f(h[(size_t)t * dim + d]) : pair_out[((size_t)t * top + k) * dim + d], s);
        }
        if (shared) s += to_f(shared[(size_t)t * dim + d]);
        y[(size_t)t * dim + d] = s;
    }
}

}  // namespace tlb

using namespace tlb;

template <bool GATED, int BM>
static int launch_grouped_mma(dim3 grid, cudaStream_t st, const bf16 *a, const bf16 *w1, const bf16 *w2, const int32_t *sorted_pair,
                              const int32_t *tile_expert, const int32_t *counters, int top, int K, int N, int act, int gather, bf16 *inter,
                              float *pair_out) {
    size_t smem = (size_t)2 * (BM + kTN * (GATED ? 2 : 1)) * kTS * sizeof(bf16);
    auto kernel = moe_grouped_mma_kernel<GATED, BM>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return tl::fail(TL_ECUDA, "moe_grouped: %s", cudaGetErrorString(e));
    }
    kernel<<<grid, 256, smem, st>>>(a, w1, w2, sorted_pair, tile_expert, counters, top, K, N, act, gather, inter, pair_out);
    return TL_OK;
}

static bool moe_mma_ok(int dtype, int k, const void *a, const void *w1, const void *w2) {
    return dtype == TL_BF16 && k % 8 == 0 && tl::aligned16(a) && tl::aligned16(w1) && (!w2 || tl::aligned16(w2));
}

extern "C" {

int tlb_moe_route(const void *h, const void *w, const void *b, int tokens, int dim, int experts, int top, int scoring, const void *choice_bias,
                  float weight_scale, int32_t *idx, float *gate, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!h || !w || !idx || !gate || dim <= 0 || experts <= 0 || top <= 0 || top > experts || scoring < 0 || scoring > 2)
        return tl::fail(TL_EINVAL, "moe_route: bad argument");
    size_t smem = ((size_t)dim + 2 * (size_t)experts) * sizeof(float);
    if (smem > 48 * 1024) return tl::fail(TL_EINVAL, "moe_route: width %d + %d experts do not fit", dim, experts);
    TLB_DISPATCH(dtype, "moe_route",
                 moe_route_kernel<T><<<tokens, 256, smem, as_stream(stream)>>>((const T *)h, (const T *)w, (const T *)b, tokens, dim, experts, top, scoring,
                                                                             (const T *)choice_bias, weight_scale, idx, gate));
    TL_LAUNCH_CHECK("moe_route");
    return TL_OK;
}

long long tlb_moe_max_rows(int tokens, int top, int experts, int tile_rows) {
    long long pairs = (long long)tokens * top;
    long long groups = pairs < experts ? pairs : experts;  // at most min(pairs, experts) groups carry padding
    long long rows = pairs + groups * (tile_rows - 1);
    return (rows + tile_rows - 1) / tile_rows * tile_rows;
}

int tlb_moe_sort(const int32_t *idx, int tokens, int top, int experts, int tile_rows, int32_t *sorted_pair, int32_t *tile_expert,
                 int32_t *counters, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!idx || !sorted_pair || !tile_expert || !counters || top <= 0 || experts <= 0 || (tile_rows != 32 && tile_rows != 64))
        return tl::fail(TL_EINVAL, "moe_sort: bad argument");
    size_t smem = (size_t)3 * experts * sizeof(int);
    if (smem > 48 * 1024) return tl::fail(TL_EINVAL, "moe_sort: %d experts do not fit", experts);
    moe_sort_kernel<<<1, 1024, smem, as_stream(stream)>>>(idx, tokens * top, experts, (int)tlb_moe_max_rows(tokens, top, experts, tile_rows), tile_rows,
                                                          sorted_pair, tile_expert, counters);
    TL_LAUNCH_CHECK("moe_sort");
    return TL_OK;
}

// The tensor-core kernels take 32- or 64-row expert tiles (64 halves the weight traffic per row when experts get many
// rows); the fp32 kernels 32 only.
int tlb_moe_gate_up(const void *h, const void *wg, const void *wu, const int32_t *sorted_pair, const int32_t *tile_expert, const int32_t *counters,
                    int tokens, int top, int experts, int tile_rows, int dim, int ff, int act, void *inter, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!h || !wg || !wu || !sorted_pair || !tile_expert || !counters || !inter || dim <= 0 || ff <= 0 || top <= 0)
        return tl::fail(TL_EINVAL, "moe_gate_up: bad argument");
    if (moe_mma_ok(dtype, dim, h, wg, wu)) {
        dim3 tc((unsigned)(tlb_moe_max_rows(tokens, top, experts, tile_rows) / tile_rows), ceil_div(ff, kTN));
        int rc = tile_rows == 64 ? launch_grouped_mma<true, 64>(tc, as_stream(stream), (const bf16 *)h, (const bf16 *)wg, (const bf16 *)wu, sorted_pair,
                                                                tile_expert, counters, top, dim, ff, act, kGatherToken, (bf16 *)inter, nullptr)
                                 : launch_grouped_mma<true, 32>(tc, as_stream(stream), (const bf16 *)h, (const bf16 *)wg, (const bf16 *)wu, sorted_pair,
                                                                tile_expert, counters, top, dim, ff, act, kGatherToken, (bf16 *)inter, nullptr);
        if (rc != TL_OK) return rc;
        TL_LAUNCH_CHECK("moe_gate_up");
        return TL_OK;
    }
    if (tile_rows != kTileRows) return tl::fail(TL_EINVAL, "moe_gate_up: %d-row tiles need the tensor-core kernel", tile_rows);
    dim3 grid((unsigned)(tlb_moe_max_rows(tokens, top, experts, kTileRows) / kTileRows), ceil_div(ff, kBN));
    TLB_DISPATCH(dtype, "moe_gate_up",
                 moe_grouped_kernel<T, true><<<grid, 256, 0, as_stream(stream)>>>((const T *)h, (const T *)wg, (const T *)wu, sorted_pair, tile_expert,
                                                                                 counters, top, dim, ff, act, kGatherToken, (T *)inter, nullptr));
    TL_LAUNCH_CHECK("moe_gate_up");
    return TL_OK;
}

// The first product of experts without a gate: inter[row, :] = act(W[e] a[src(row)]), a = token rows (rows_are_pairs = 0) or one row per
// (token, choice) pair (rows_are_pairs = 1: the scaled copies tlb_moe_scale_rows makes).
int tlb_moe_up(const void *a, const void *wu, const int32_t *sorted_pair, const int32_t *tile_expert, const int32_t *counters, int tokens, int top,
               int experts, int tile_rows, int dim, int ff, int act, int rows_are_pairs, void *inter, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!a || !wu || !sorted_pair || !tile_expert || !counters || !inter || dim <= 0 || ff <= 0 || top <= 0 || act < 0 || act > 2)
        return tl::fail(TL_EINVAL, "moe_up: bad argument");
    int gather = rows_are_pairs ? kGatherPair : kGatherToken;
    if (moe_mma_ok(dtype, dim, a, wu, nullptr)) {
        dim3 tc((unsigned)(tlb_moe_max_rows(tokens, top, experts, tile_rows) / tile_rows), ceil_div(ff, kTN));
        int rc = tile_rows == 64 ? launch_grouped_mma<false, 64>(tc, as_stream(stream), (const bf16 *)a, (const bf16 *)wu, nullptr, sorted_pair, tile_expert,
                                                                 counters, top, dim, ff, act, gather, (bf16 *)inter, nullptr)
                                 : launch_grouped_mma<false, 32>(tc, as_stream(stream), (const bf16 *)a, (const bf16 *)wu, nullptr, sorted_pair, tile_expert,
                                                                 counters, top, dim, ff, act, gather, (bf16 *)inter, nullptr);
        if (rc != TL_OK) return rc;
        TL_LAUNCH_CHECK("moe_up");
        return TL_OK;
    }
    if (tile_rows != kTileRows) return tl::fail(TL_EINVAL, "moe_up: %d-row tiles need the tensor-core kernel", tile_rows);
    dim3 grid((unsigned)(tlb_moe_max_rows(tokens, top, experts, kTileRows) / kTileRows), ceil_div(ff, kBN));
    TLB_DISPATCH(dtype, "moe_up",
                 moe_grouped_kernel<T, false><<<grid, 256, 0, as_stream(stream)>>>((const T *)a, (const T *)wu, nullptr, sorted_pair, tile_expert, counters,
                                                                                  top, dim, ff, act, gather, (T *)inter, nullptr));
    TL_LAUNCH_CHECK("moe_up");
    return TL_OK;
}

int tlb_moe_scale_rows(const void *h, const float *gate, void *out, int tokens, int top, int dim, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!h || !gate || !out || top <= 0 || dim <= 0) return tl::fail(TL_EINVAL, "moe_scale_rows: bad argument");
    TLB_DISPATCH(dtype, "moe_scale_rows",
                 moe_scale_rows_kernel<T><<<tokens * top, 128, 0, as_stream(stream)>>>((const T *)h, gate, (T *)out, top, dim));
    TL_LAUNCH_CHECK("moe_scale_rows");
    return TL_OK;
}

int tlb_moe_down(const void *inter, const void *wd, const int32_t *sorted_pair, const int32_t *tile_expert, const int32_t *counters, int tokens,
                 int top, int experts, int tile_rows, int dim, int ff, float *pair_out, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!inter || !wd || !sorted_pair || !tile_expert || !counters || !pair_out || dim <= 0 || ff <= 0 || top <= 0)
        return tl::fail(TL_EINVAL, "moe_down: bad argument");
    if (moe_mma_ok(dtype, ff, inter, wd, nullptr)) {
        dim3 tc((unsigned)(tlb_moe_max_rows(tokens, top, experts, tile_rows) / tile_rows), ceil_div(dim, kTN));
        int rc = tile_rows == 64 ? launch_grouped_mma<false, 64>(tc, as_stream(stream), (const bf16 *)inter, (const bf16 *)wd, nullptr, sorted_pair,
                                                                 tile_expert, counters, top, ff, dim, 0, kGatherSorted, nullptr, pair_out)
                                 : launch_grouped_mma<false, 32>(tc, as_stream(stream), (const bf16 *)inter, (const bf16 *)wd, nullptr, sorted_pair,
                                                                 tile_expert, counters, top, ff, dim, 0, kGatherSorted, nullptr, pair_out);
        if (rc != TL_OK) return rc;
        TL_LAUNCH_CHECK("moe_down");
        return TL_OK;
    }
    if (tile_rows != kTileRows) return tl::fail(TL_EINVAL, "moe_down: %d-row tiles need the tensor-core kernel", tile_rows);
    dim3 grid((unsigned)(tlb_moe_max_rows(tokens, top, experts, kTileRows) / kTileRows), ceil_div(dim, kBN));
    TLB_DISPATCH(dtype, "moe_down",
                 moe_grouped_kernel<T, false><<<grid, 256, 0, as_stream(stream)>>>((const T *)inter, (const T *)wd, nullptr, sorted_pair, tile_expert,
                                                                                  counters, top, ff, dim, 0, kGatherSorted, nullptr, pair_out));
    TL_LAUNCH_CHECK("moe_down");
    return TL_OK;
}

int tlb_moe_combine(const float *pair_out, const float *gate, const void *shared, const int32_t *idx, int experts, const void *h, float *y, int tokens,
                    int top, int dim, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!pair_out || !y || top <= 0 || dim <= 0 || (idx && !h)) return tl::fail(TL_EINVAL, "moe_combine: bad argument");
    TLB_DISPATCH(dtype, "moe_combine",
                 moe_combine_kernel<T><<<tokens, 256, 0, as_stream(stream)>>>(pair_out, gate, (const T *)shared, idx, experts, (const T *)h, y, top, dim));
    TL_LAUNCH_CHECK("moe_combine");
    return TL_OK;
}

}  // extern "C"
