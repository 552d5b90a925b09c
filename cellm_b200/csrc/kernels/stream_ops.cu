// Small kernels around the 32-bit residual stream for layers whose two sublayers read the same stream through
// norms of their own and whose sum joins the stream times a constant:
//
//   norm_pair        y1 = x / rms(x) * w1,  y2 = x / rms(x) * w2      (the stream is read once for both norms)
//   scaled_add2      x += m * (a + b)
//   pair_norm_mean   out = (a / rms(a) * wa + b / rms(b) * wb) / 2     (two mixers side by side, each normed; a, b 32-bit)
//
// Sums of squares, the factors and the stream are 32-bit; a block's sum has a fixed order. Rows whose width is a multiple
// of four, in buffers that start on 16 bytes, move in pieces of four values (`vec`, decided by the launcher from the sizes
// and addresses, so a model always takes the same path).
#include "common.cuh"

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&a);
    u.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
static bool fits4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
norm_pair_kernel(TA* __restrict__ y1, TA* __restrict__ y2, const float* __restrict__ x, const TW* __restrict__ w1,
                 const TW* __restrict__ w2, int H, float eps, int vec) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const float* row = x + (size_t)blockIdx.x * H;
    float ss = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = load4(row + i);
            ss = fmaf(v.x, v.x, ss), ss = fmaf(v.y, v.y, ss), ss = fmaf(v.z, v.z, ss), ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.f / sqrtf(ss / (float)H + eps);
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = load4(row + i), a = load4(w1 + i);
            store4(y1 + (size_t)blockIdx.x * H + i, make_float4(v.x * inv * a.x, v.y * inv * a.y, v.z * inv * a.z, v.w * inv * a.w));
            if (y2) {
                const float4 b = load4(w2 + i);
                store4(y2 + (size_t)blockIdx.x * H + i, make_float4(v.x * inv * b.x, v.y * inv * b.y, v.z * inv * b.z, v.w * inv * b.w));
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float r = row[i] * inv;
        y1[(size_t)blockIdx.x * H + i] = from_float<TA>(r * to_float(w1[i]));
        if (y2) y2[(size_t)blockIdx.x * H + i] = from_float<TA>(r * to_float(w2[i]));
    }
}

CELLM_API int cellm_norm_pair(void* y1, void* y2, const float* x, const void* w1, const void* w2, int w_dtype, int T, int H,
                              float eps, int dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (H <= 0) return CELLM_ERR_SIZE;
    if (!y1 || !w1 || (y2 && !w2)) return CELLM_ERR_ARG;
    const int vec = H % 4 == 0 && fits4(x) && fits4(y1) && fits4(y2) && fits4(w1) && fits4(w2);
#define NP_RUN(TA, TW) CELLM_RUN((norm_pair_kernel<TA, TW>), T, 256, 0, stream, (TA*)y1, (TA*)y2, x, (const TW*)w1, (const TW*)w2, H, eps, vec)
    if (dtype == CELLM_F32 && w_dtype == CELLM_F32) NP_RUN(float, float);
    else if (dtype == CELLM_BF16 && w_dtype == CELLM_BF16) NP_RUN(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == CELLM_BF16 && w_dtype == CELLM_F32) NP_RUN(__nv_bfloat16, float);
    else if (dtype == CELLM_F32 && w_dtype == CELLM_BF16) NP_RUN(float, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef NP_RUN
    return CELLM_OK;
}

template <typename TA>
__global__ void __launch_bounds__(256)
scaled_add2_kernel(float* __restrict__ x, const TA* __restrict__ a, const TA* __restrict__ b, float m, size_t n, int vec) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        i *= 4;
        if (i >= n) return;
        float4 s = load4(a + i);
        if (b) {
            const float4 t = load4(b + i);
            s.x += t.x, s.y += t.y, s.z += t.z, s.w += t.w;
        }
        const float4 v = load4(x + i);
        store4(x + i, make_float4(fmaf(m, s.x, v.x), fmaf(m, s.y, v.y), fmaf(m, s.z, v.z), fmaf(m, s.w, v.w)));
        return;
    }
    if (i >= n) return;
    float s = to_float(a[i]);
    if (b) s += to_float(b[i]);
    x[i] = fmaf(m, s, x[i]);
}

CELLM_API int cellm_scaled_add2(float* x, const void* a, const void* b, float m, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return CELLM_OK;
    if (!a) return CELLM_ERR_ARG;
    const int vec = n % 4 == 0 && fits4(x) && fits4(a) && fits4(b);
    const unsigned blocks = (unsigned)(((vec ? n / 4 : n) + 255) / 256);
    if (dtype == CELLM_F32) CELLM_RUN(scaled_add2_kernel<float>, blocks, 256, 0, stream, x, (const float*)a, (const float*)b, m, (size_t)n, vec);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(scaled_add2_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, m, (size_t)n, vec);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

template <typename TA>
__global__ void __launch_bounds__(256)
pair_norm_mean_kernel(TA* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                      const float* __restrict__ wb, int H, float eps, int vec) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const float* ra = a + (size_t)blockIdx.x * H;
    const float* rb = b + (size_t)blockIdx.x * H;
    float sa = 0.f, sb = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 u = load4(ra + i), v = load4(rb + i);
            sa = fmaf(u.x, u.x, sa), sa = fmaf(u.y, u.y, sa), sa = fmaf(u.z, u.z, sa), sa = fmaf(u.w, u.w, sa);
            sb = fmaf(v.x, v.x, sb), sb = fmaf(v.y, v.y, sb), sb = fmaf(v.z, v.z, sb), sb = fmaf(v.w, v.w, sb);
        }
        sa = block_sum(sa, scratch);
        sb = block_sum(sb, scratch);
        const float ia = 1.f / sqrtf(sa / (float)H + eps), ib = 1.f / sqrtf(sb / (float)H + eps);
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 u = load4(ra + i), v = load4(rb + i), p = load4(wa + i), q = load4(wb + i);
            store4(out + (size_t)blockIdx.x * H + i,
                   make_float4(0.5f * (u.x * ia * p.x + v.x * ib * q.x), 0.5f * (u.y * ia * p.y + v.y * ib * q.y),
                               0.5f * (u.z * ia * p.z + v.z * ib * q.z), 0.5f * (u.w * ia * p.w + v.w * ib * q.w)));
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float u = ra[i], v = rb[i];
        sa = fmaf(u, u, sa);
        sb = fmaf(v, v, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = 1.f / sqrtf(sa / (float)H + eps), ib = 1.f / sqrtf(sb / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t)blockIdx.x * H + i] = from_float<TA>(0.5f * (ra[i] * ia * wa[i] + rb[i] * ib * wb[i]));
}

// a, b [T, H] 32-bit (the two mixers' last products keep their 32-bit sums); out in the activations' element type.
CELLM_API int cellm_pair_norm_mean(void* out, const float* a, const float* b, const float* wa, const float* wb, int T, int H, float eps,
                                   int dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (H <= 0) return CELLM_ERR_SIZE;
    const int vec = H % 4 == 0 && fits4(out) && fits4(a) && fits4(b) && fits4(wa) && fits4(wb);
    if (dtype == CELLM_F32)
        CELLM_RUN(pair_norm_mean_kernel<float>, T, 256, 0, stream, (float*)out, a, b, wa, wb, H, eps, vec);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(pair_norm_mean_kernel<__nv_bfloat16>, T, 256, 0, stream, (__nv_bfloat16*)out, a, b, wa, wb, H, eps, vec);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
