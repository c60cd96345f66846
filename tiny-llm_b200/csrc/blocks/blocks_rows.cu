// Row-wise kernels of the blocks library: embedding rows, RMS norm + layer scale + fp32 residual, rotary
// positions, latent cache append, gated activations, arg-max; and the library's error / launch bookkeeping.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "blocks_common.cuh"

namespace tl {
// The helpers common.cuh declares; this library is linked on its own.
static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};
int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}
int check_launch(const char *what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e == cudaSuccess) return TL_OK;
    cudaGetLastError();
    return fail(TL_ECUDA, "%s: kernel launch failed: %s", what, cudaGetErrorString(e));
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
bool use_pdl() { return false; }
}  // namespace tl

namespace tlb {

template <typename T>
__global__ void embed_rows_kernel(const int32_t *__restrict__ ids, const T *__restrict__ table, float *__restrict__ x32, T *__restrict__ h,
                                  int vocab, int dim) {
    int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    const T *row = table + (size_t)id * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        T v = row[d];
        x32[(size_t)t * dim + d] = to_f(v);
        if (h) h[(size_t)t * dim + d] = v;
    }
}

// 4 consecutive elements of a row as floats (one 8- or 16-byte access)
__device__ __forceinline__ float4 load4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 load4(const bf16 *p) {
    uint2 u = *reinterpret_cast<const uint2 *>(p);
    float2 a = tl::unpack2<bf16>(u.x), b = tl::unpack2<bf16>(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(bf16 *p, float4 v) {
    *reinterpret_cast<uint2 *>(p) = make_uint2(tl::pack2<bf16>(v.x, v.y), tl::pack2<bf16>(v.z, v.w));
}

// VEC: rows are read and written 4 elements at a time (dim % 4 == 0, 16-byte aligned bases); the row's values stay in
// registers between the two passes when it has at most 4 * KEEP * blockDim elements.
template <typename T, typename TY, bool VEC>
__global__ void norm_residual_kernel(const TY *__restrict__ y, const T *__restrict__ w, float weight_offset, const T *__restrict__ scale,
                                     float eps, float *__restrict__ residual, T *__restrict__ h, int dim) {
    __shared__ float scratch[33];
    size_t base = (size_t)blockIdx.x * dim;
    float ss = 0.f;
    if constexpr (VEC) {
        constexpr int KEEP = 4;
        float4 kept[KEEP];
        const int quads = dim / 4;
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            int q = threadIdx.x + i * blockDim.x;
            kept[i] = q < quads ? load4(y + base + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += kept[i].x * kept[i].x + kept[i].y * kept[i].y + kept[i].z * kept[i].z + kept[i].w * kept[i].w;
        }
        for (int q = threadIdx.x + KEEP * blockDim.x; q < quads; q += blockDim.x) {
            float4 v = load4(y + base + 4 * q);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        auto finish = [&](int q, float4 v) {
            float4 g = load4(w + 4 * q);
            float4 n = make_float4(v.x * inv * (g.x + weight_offset), v.y * inv * (g.y + weight_offset), v.z * inv * (g.z + weight_offset),
                                   v.w * inv * (g.w + weight_offset));
            if (scale) {
                float4 sc = load4(scale + 4 * q);
                n.x *= sc.x, n.y *= sc.y, n.z *= sc.z, n.w *= sc.w;
            }
            if (residual) {
                float4 r = load4(residual + base + 4 * q);
                n.x += r.x, n.y += r.y, n.z += r.z, n.w += r.w;
                store4(residual + base + 4 * q, n);
            }
            if (h) store4(h + base + 4 * q, n);
        };
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            int q = threadIdx.x + i * blockDim.x;
            if (q < quads) finish(q, kept[i]);
        }
        for (int q = threadIdx.x + KEEP * blockDim.x; q < quads; q += blockDim.x) finish(q, load4(y + base + 4 * q));
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float v = to_f(y[base + d]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float n = to_f(y[base + d]) * inv * (to_f(w[d]) + weight_offset);
            if (scale) n *= to_f(scale[d]);
            if (residual) {
                n += residual[base + d];
                residual[base + d] = n;
            }
            if (h) h[base + d] = from_f<T>(n);
        }
    }
}


// residual += a (+ b) in fp32, then (w != NULL) h = residual / rms(residual) * w rounded to T: the end of a sublayer (or of
// a layer whose sublayers both read one norm of the stream), fused with the norm that reads the stream next.  a_row: `a`
// is ONE row [dim] added to every row (a learned offset).
template <typename T>
__global__ void add_norm_kernel(float *__restrict__ residual, const float *__restrict__ a, int a_row, const float *__restrict__ b,
                                const T *__restrict__ w, float eps, T *__restrict__ h, int dim) {
    __shared__ float scratch[33];
    size_t base = (size_t)blockIdx.x * dim, abase = a_row ? 0 : base;
    float ss = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float x = residual[base + d] + (b ? a[abase + d] + b[base + d] : a[abase + d]);
        residual[base + d] = x;
        ss += x * x;
    }
    if (w == nullptr || h == nullptr) return;
    ss = block_sum(ss, scratch);
    float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) h[base + d] = from_f<T>(residual[base + d] * inv * to_f(w[d]));
}

// y = coef * (a / rms(a) * wa + b / rms(b) * wb), fp32 in and out: two mixers side by side, each normed before they meet.
template <typename T>
__global__ void norm_mix2_kernel(const float *__restrict__ a, const T *__restrict__ wa, const float *__restrict__ b, const T *__restrict__ wb,
                                 float coef, float eps, float *__restrict__ y, int dim) {
    __shared__ float scratch[33];
    size_t base = (size_t)blockIdx.x * dim;
    float sa = 0.f, sb = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float u = a[base + d], v = b[base + d];
        sa += u * u;
        sb += v * v;
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    float ia = 1.0f / sqrtf(sa / (float)dim + eps), ib = 1.0f / sqrtf(sb / (float)dim + eps);
    for (int d = threadIdx.x; d < dim; d += blockDim.x)
        y[base + d] = coef * (a[base + d] * ia * to_f(wa[d]) + b[base + d] * ib * to_f(wb[d]));
}

template <typename T>
__global__ void rope_rows_kernel(T *x, long long row_stride, long long head_stride, int first, int heads, int dims, int interleaved,
                                 double log2_base, double inv_factor, const int32_t *__restrict__ tok_pos) {
    int row = blockIdx.x;
    int pos = tok_pos[row];
    int half = dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float c, s;
        if (inv_factor == 1.0) rope_angle(pos, i, dims, log2_base, c, s);
        else {  // linear scaling: every frequency divided by the factor
            double sn, cs;
            sincos((double)pos * exp2(-2.0 * (double)i / (double)dims * log2_base) * inv_factor, &sn, &cs);
            c = (float)cs, s = (float)sn;
        }
        int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        for (int hd = 0; hd < heads; ++hd) {
            T *p = x + (size_t)row * row_stride + (size_t)hd * head_stride + first;
            float u = to_f(p[a]), v = to_f(p[b]);
            p[a] = from_f<T>(u * c - v * s);
            p[b] = from_f<T>(v * c + u * s);
        }
    }
}

template <typename T>
__global__ void latent_append_kernel(const T *__restrict__ down, const T *__restrict__ norm_w, float eps, int rank, int rot, int rot_dims,
                                     int interleaved, double log2_base, const int32_t *__restrict__ tok_pos, const int32_t *__restrict__ tok_seq,
                                     const int32_t *__restrict__ block_table, int max_pages, int num_pages, int page_size, T *__restrict__ slab,
                                     long long down_stride, T *q, long long q_stride, int q_heads, int q_head_stride, int q_first) {
    __shared__ float scratch[33];
    int t = blockIdx.x;
    int pos = tok_pos[t];
    int width = rank + rot;
    const T *src = down + (size_t)t * down_stride;
    if (q != nullptr) {  // the same launch rotates the token's query heads in place (same angles as the shared key part)
        int half = rot_dims / 2;
        for (int i = threadIdx.x; i < half * q_heads; i += blockDim.x) {
            int hd = i / half, k = i - hd * half;
            float c, s;
            rope_angle(pos, k, rot_dims, log2_base, c, s);
            int a = interleaved ? 2 * k : k, b = interleaved ? 2 * k + 1 : k + half;
            T *p = q + (size_t)t * q_stride + (size_t)hd * q_head_stride + q_first;
            float u = to_f(p[a]), v = to_f(p[b]);
            p[a] = from_f<T>(u * c - v * s);
            p[b] = from_f<T>(v * c + u * s);
        }
    }
    int page = block_table[(size_t)tok_seq[t] * max_pages + pos / page_size];
    bool ok = page >= 0 && page < num_pages;  // a bad table entry drops the write instead of corrupting another page
    T *dst = slab + ((size_t)(ok ? page : 0) * page_size + pos % page_size) * width;
    float ss = 0.f;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float v = to_f(src[d]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    if (!ok) return;
    float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = from_f<T>(to_f(src[d]) * inv * to_f(norm_w[d]));
    int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float c, s;
        rope_angle(pos, i, rot_dims, log2_base, c, s);
        int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        float u = to_f(src[rank + a]), v = to_f(src[rank + b]);
        dst[rank + a] = from_f<T>(u * c - v * s);
        dst[rank + b] = from_f<T>(v * c + u * s);
    }
    for (int d = rot_dims + threadIdx.x; d < rot; d += blockDim.x) dst[rank + d] = src[rank + d];  // entries past the rotated ones pass
}

__device__ __forceinline__ float act_apply(float z, int act) {
    if (act == 0) return z / (1.0f + expf(-z));
    float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(inner));
}

// out = act(x) elementwise; act 0 = silu, 1 = gelu (tanh form), 2 = squared relu, 4 = tanh.
template <typename T>
__global__ void act_rows_kernel(const T *__restrict__ x, T *__restrict__ out, long long total, int act) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float z = to_f(x[i]);
    out[i] = from_f<T>(act == 2 ? (z > 0.f ? z * z : 0.f) : act == 4 ? tanhf(z) : act_apply(z, act));
}

// x <- cap * tanh(x / cap), fp32 in place.
__global__ void softcap_rows_kernel(float *__restrict__ x, long long total, float cap) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] / cap);
}

// dst[r, :] = src[r, :] rounded to T; dst rows dst_stride elements apart (a column block of a wider matrix).
template <typename T>
__global__ void cast_rows_kernel(const float *__restrict__ src, T *__restrict__ dst, long long dst_stride, int dim) {
    const float *s = src + (size_t)blockIdx.x * dim;
    T *d = dst + (size_t)blockIdx.x * dst_stride;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) d[i] = from_f<T>(s[i]);
}

__device__ __forceinline__ float gated_pair(float g, float u, int act, float limit, float slope) {
    if (act == 3) {  // clamped: the gate from above, the other half on both sides; g sigmoid(slope g) (u + 1)
        g = fminf(g, limit), u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
    }
    return act_apply(g, act) * u;
}

template <typename T>
__global__ void gated_act_kernel(const T *__restrict__ gu, T *__restrict__ out, long long total, int width, int act, float limit, float slope) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    long long row = i / width;
    int j = (int)(i - row * width);
    out[i] = from_f<T>(gated_pair(to_f(gu[row * 2 * width + j]), to_f(gu[row * 2 * width + width + j]), act, limit, slope));
}

// Eight adjacent columns per thread, 16-byte accesses (bf16, width % 8 == 0).
__global__ void gated_act_wide_kernel(const bf16 *__restrict__ gu, bf16 *__restrict__ out, long long total8, int width, int act, float limit, float slope) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const int per_row = width / 8;
    long long row = i / per_row;
    int j = (int)(i - row * per_row) * 8;
    uint4 g4 = *reinterpret_cast<const uint4 *>(gu + row * 2 * width + j), u4 = *reinterpret_cast<const uint4 *>(gu + row * 2 * width + width + j), o4;
    const __nv_bfloat162 *gp = reinterpret_cast<const __nv_bfloat162 *>(&g4), *up = reinterpret_cast<const __nv_bfloat162 *>(&u4);
    __nv_bfloat162 *op = reinterpret_cast<__nv_bfloat162 *>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float2 g = __bfloat1622float2(gp[e]), u = __bfloat1622float2(up[e]);
        op[e] = __floats2bfloat162_rn(gated_pair(g.x, u.x, act, limit, slope), gated_pair(g.y, u.y, act, limit, slope));
    }
    *reinterpret_cast<uint4 *>(out + row * width + j) = o4;
}

__global__ void argmax_rows_kernel(const float *__restrict__ logits, int32_t *__restrict__ out, int vocab) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float *row = logits + (size_t)blockIdx.x * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        float v = row[j];
        if (v > bv || (v == bv && j < bi)) bv = v, bi = j;
    }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
    }
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) best_v[warp] = bv, best_i[warp] = bi;
    __syncthreads();
    if (warp == 0) {
        int n = blockDim.x >> 5;
        bv = lane < n ? best_v[lane] : -INFINITY;
        bi = lane < n ? best_i[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

}  // namespace tlb

using namespace tlb;

extern "C" {

int tlb_abi_version(void) { return 5; }
const char *tlb_last_error(void) { return tl::g_error; }
long long tlb_launch_count(void) { return tl::g_launches.load(std::memory_order_relaxed); }

int tlb_embed_rows(const int32_t *ids, const void *table, float *x32, void *h, int tokens, int vocab, int dim, int dtype, void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!ids || !table || !x32 || vocab <= 0 || dim <= 0) return tl::fail(TL_EINVAL, "embed_rows: bad argument");
    TLB_DISPATCH(dtype, "embed_rows",
                 embed_rows_kernel<T><<<tokens, 256, 0, as_stream(stream)>>>(ids, (const T *)table, x32, (T *)h, vocab, dim));
    TL_LAUNCH_CHECK("embed_rows");
    return TL_OK;
}

int tlb_norm_residual(const void *y, int y_is_f32, const void *w, float weight_offset, const void *scale, float eps, float *residual, void *h,
                      int rows, int dim, int dtype, void *stream) {
    if (rows <= 0) return TL_OK;
    if (!y || !w || dim <= 0 || (!residual && !h)) return tl::fail(TL_EINVAL, "norm_residual: bad argument");
    bool vec = dim % 4 == 0 && tl::aligned16(y) && tl::aligned16(w) && (!scale || tl::aligned16(scale)) && (!residual || tl::aligned16(residual)) &&
               (!h || tl::aligned16(h));
    int threads = dim >= 2048 ? 256 : 128;
    cudaStream_t st = as_stream(stream);
#define TLB_NORM(TY, V)                                                                                                                        \
    norm_residual_kernel<T, TY, V><<<rows, threads, 0, st>>>((const TY *)y, (const T *)w, weight_offset, (const T *)scale, eps, residual, (T *)h, dim)
    TLB_DISPATCH(dtype, "norm_residual",
                 if (y_is_f32) { if (vec) TLB_NORM(float, true); else TLB_NORM(float, false); }
                 else { if (vec) TLB_NORM(T, true); else TLB_NORM(T, false); });
#undef TLB_NORM
    TL_LAUNCH_CHECK("norm_residual");
    return TL_OK;
}

int tlb_add_norm(float *residual, const float *a, int a_row, const float *b, const void *w, float eps, void *h, int rows, int dim, int dtype,
                 void *stream) {
    if (rows <= 0) return TL_OK;
    if (!residual || !a || dim <= 0 || ((w == nullptr) != (h == nullptr))) return tl::fail(TL_EINVAL, "add_norm: bad argument");
    int threads = dim >= 2048 ? 256 : 128;
    TLB_DISPATCH(dtype, "add_norm", add_norm_kernel<T><<<rows, threads, 0, as_stream(stream)>>>(residual, a, a_row, b, (const T *)w, eps, (T *)h, dim));
    TL_LAUNCH_CHECK("add_norm");
    return TL_OK;
}

int tlb_norm_mix2(const float *a, const void *wa, const float *b, const void *wb, float coef, float eps, float *y, int rows, int dim, int dtype,
                  void *stream) {
    if (rows <= 0) return TL_OK;
    if (!a || !wa || !b || !wb || !y || dim <= 0) return tl::fail(TL_EINVAL, "norm_mix2: bad argument");
    int threads = dim >= 2048 ? 256 : 128;
    TLB_DISPATCH(dtype, "norm_mix2",
                 norm_mix2_kernel<T><<<rows, threads, 0, as_stream(stream)>>>(a, (const T *)wa, b, (const T *)wb, coef, eps, y, dim));
    TL_LAUNCH_CHECK("norm_mix2");
    return TL_OK;
}

int tlb_rope_rows(void *x, long long row_stride, long long head_stride, int first, int heads, int dims, int interleaved, double base,
                  double factor, const int32_t *tok_pos, int rows, int dtype, void *stream) {
    if (rows <= 0 || dims <= 0) return TL_OK;
    if (!x || !tok_pos || heads <= 0 || (dims & 1) || base <= 0 || !(factor > 0)) return tl::fail(TL_EINVAL, "rope_rows: bad argument");
    double lb = log2(base);
    TLB_DISPATCH(dtype, "rope_rows",
                 rope_rows_kernel<T><<<rows, 64, 0, as_stream(stream)>>>((T *)x, row_stride, head_stride, first, heads, dims, interleaved, lb, 1.0 / factor, tok_pos));
    TL_LAUNCH_CHECK("rope_rows");
    return TL_OK;
}

int tlb_latent_append(const void *down, const void *norm_w, float eps, int rank, int rot, int rot_dims, int interleaved, double base,
                      const int32_t *tok_pos, const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages, int page_size,
                      void *slab, int tokens, int dtype, void *stream) {
    return tlb_latent_prepare(down, rank + rot, norm_w, eps, rank, rot, rot_dims, interleaved, base, tok_pos, tok_seq, block_table, max_pages, num_pages,
                              page_size, slab, nullptr, 0, 0, 0, 0, tokens, dtype, stream);
}

int tlb_latent_prepare(const void *down, long long down_stride, const void *norm_w, float eps, int rank, int rot, int rot_dims, int interleaved,
                       double base, const int32_t *tok_pos, const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages,
                       int page_size, void *slab, void *q, long long q_stride, int q_heads, int q_head_stride, int q_first, int tokens, int dtype,
                       void *stream) {
    if (tokens <= 0) return TL_OK;
    if (!down || !norm_w || !tok_pos || !tok_seq || !block_table || !slab || rank <= 0 || rot < 0 || rot_dims > rot || (rot_dims & 1) ||
        page_size <= 0 || max_pages <= 0 || base <= 0)
        return tl::fail(TL_EINVAL, "latent_append: bad argument");
    if (q && (q_heads <= 0 || q_first < 0 || q_first + rot_dims > q_head_stride)) return tl::fail(TL_EINVAL, "latent_prepare: bad query layout");
    double lb = log2(base);
    TLB_DISPATCH(dtype, "latent_append",
                 latent_append_kernel<T><<<tokens, 128, 0, as_stream(stream)>>>((const T *)down, (const T *)norm_w, eps, rank, rot, rot_dims, interleaved,
                                                                               lb, tok_pos, tok_seq, block_table, max_pages, num_pages, page_size,
                                                                               (T *)slab, down_stride, (T *)q, q_stride, q_heads, q_head_stride,
                                                                               q_first));
    TL_LAUNCH_CHECK("latent_append");
    return TL_OK;
}

int tlb_gated_act(const void *gu, void *out, int rows, int width, int act, float limit, float slope, int dtype, void *stream) {
    if (rows <= 0 || width <= 0) return TL_OK;
    if (!gu || !out || (act != 0 && act != 1 && act != 3) || (act == 3 && !(limit > 0.f))) return tl::fail(TL_EINVAL, "gated_act: bad argument");
    long long total = (long long)rows * width;
    if (dtype == TL_BF16 && width % 8 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0) {
        long long total8 = total / 8;
        gated_act_wide_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, as_stream(stream)>>>((const bf16 *)gu, (bf16 *)out, total8, width, act, limit, slope);
    } else
        TLB_DISPATCH(dtype, "gated_act",
                     gated_act_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>((const T *)gu, (T *)out, total, width, act, limit, slope));
    TL_LAUNCH_CHECK("gated_act");
    return TL_OK;
}

int tlb_act_rows(const void *x, void *out, int rows, int width, int act, int dtype, void *stream) {
    if (rows <= 0 || width <= 0) return TL_OK;
    if (!x || !out || act < 0 || act > 4 || act == 3) return tl::fail(TL_EINVAL, "act_rows: bad argument");
    long long total = (long long)rows * width;
    TLB_DISPATCH(dtype, "act_rows", act_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>((const T *)x, (T *)out, total, act));
    TL_LAUNCH_CHECK("act_rows");
    return TL_OK;
}

int tlb_softcap_rows(float *x, int rows, int width, float cap, void *stream) {
    if (rows <= 0 || width <= 0) return TL_OK;
    if (!x || !(cap > 0.f)) return tl::fail(TL_EINVAL, "softcap_rows: bad argument");
    long long total = (long long)rows * width;
    softcap_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(x, total, cap);
    TL_LAUNCH_CHECK("softcap_rows");
    return TL_OK;
}

int tlb_cast_rows(const float *src, void *dst, long long dst_stride, int rows, int dim, int dtype, void *stream) {
    if (rows <= 0 || dim <= 0) return TL_OK;
    if (!src || !dst || dst_stride < dim) return tl::fail(TL_EINVAL, "cast_rows: bad argument");
    TLB_DISPATCH(dtype, "cast_rows", cast_rows_kernel<T><<<rows, 128, 0, as_stream(stream)>>>(src, (T *)dst, dst_stride, dim));
    TL_LAUNCH_CHECK("cast_rows");
    return TL_OK;
}

int tlb_argmax_rows(const float *logits, int32_t *out, int rows, int vocab, void *stream) {
    if (rows <= 0) return TL_OK;
    if (!logits || !out || vocab <= 0) return tl::fail(TL_EINVAL, "argmax_rows: bad argument");
    argmax_rows_kernel<<<rows, 256, 0, as_stream(stream)>>>(logits, out, vocab);
    TL_LAUNCH_CHECK("argmax_rows");
    return TL_OK;
}

}  // extern "C"
