// Kernels around the 32-bit residual stream for layers that run their sublayers one after the other, add each result
// times a constant, and norm with a mean as well as a variance:
//
//   add_scaled_norm   x += ma * a + mb * b;  y = norm(x)      norm: layer norm (x - mean) / sqrt(var + eps) * w + bias,
//                                                             RMS norm x / sqrt(mean(x^2) + eps) * w, or none (y = x in
//                                                             the activations' type); with `rows`, y holds the given rows
//                                                             only and the stream stays as it was
//   stream_add_rows   x[t] += scale * table[ids[t]] + vec     (the embedding row once more and a learned vector: the
//                                                             start of another pass over the same layers)
//   token_gate_mul    out[t] = act(g[t]) * table[ids[t]][col0 .. col0 + n]     (a token's own row gated by the stream)
//   scaled_rms_add    x[t] += m * y[t] / sqrt(mean(y[t]^2) + eps) * w
//   weighted_sum2     out = ca * a + cb * b
//
// Means, variances, factors and the stream are 32-bit. The variance is the mean of the squared deviations from the mean
// (two passes over a row held in shared memory). A block's sums have a fixed order that depends on the width alone.
#include "common.cuh"

// Rows whose width is a multiple of four, in buffers that start on 16 bytes, move in pieces of four values (`vec`, decided
// by the launcher from the sizes and addresses, so a model always takes the same path).
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&a);
    u.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
static bool on16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename TA, typename TD>
__global__ void __launch_bounds__(256)
add_scaled_norm_kernel(TA* __restrict__ y, float* __restrict__ x, const TD* __restrict__ a, float ma, const TD* __restrict__ b, float mb,
                       const float* __restrict__ w, const float* __restrict__ bias, const int* __restrict__ rows, int H, float eps,
                       int kind, int vec) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const size_t t = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + t * H;
    TA* yr = y ? y + (size_t)blockIdx.x * H : nullptr;
    const bool write_x = (a || b) && !rows;
    float s = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 v = ld4(xr + i);
            if (a) { const float4 u = ld4(a + t * H + i); v.x = fmaf(ma, u.x, v.x), v.y = fmaf(ma, u.y, v.y), v.z = fmaf(ma, u.z, v.z), v.w = fmaf(ma, u.w, v.w); }
            if (b) { const float4 u = ld4(b + t * H + i); v.x = fmaf(mb, u.x, v.x), v.y = fmaf(mb, u.y, v.y), v.z = fmaf(mb, u.z, v.z), v.w = fmaf(mb, u.w, v.w); }
            if (write_x) st4(xr + i, v);
            if (kind == 2) { if (yr) st4(yr + i, v); }
            else st4(row_s + i, v);
            s += (v.x + v.y) + (v.z + v.w);
        }
        if (!y || kind == 2) return;
        float mean = 0.f;
        if (kind == 1) mean = block_sum(s, scratch) / (float)H;
        float ss = 0.f;
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = ld4(row_s + i);
            const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
            ss = fmaf(d0, d0, ss), ss = fmaf(d1, d1, ss), ss = fmaf(d2, d2, ss), ss = fmaf(d3, d3, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.f / sqrtf(ss / (float)H + eps);
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = ld4(row_s + i), g = ld4(w + i);
            float4 o = make_float4((v.x - mean) * inv * g.x, (v.y - mean) * inv * g.y, (v.z - mean) * inv * g.z, (v.w - mean) * inv * g.w);
            if (bias) { const float4 c = ld4(bias + i); o.x += c.x, o.y += c.y, o.z += c.z, o.w += c.w; }
            st4(yr + i, o);
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (a) v = fmaf(ma, to_float(a[t * H + i]), v);
        if (b) v = fmaf(mb, to_float(b[t * H + i]), v);
        if (write_x) xr[i] = v;
        row_s[i] = v;
        s += v;
    }
    if (!y) return;
    if (kind == 2) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_float<TA>(row_s[i]);
        return;
    }
    float mean = 0.f;
    if (kind == 1) mean = block_sum(s, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row_s[i] - mean;
        ss = fmaf(d, d, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = (row_s[i] - mean) * inv * w[i];
        if (bias) v += bias[i];
        yr[i] = from_float<TA>(v);
    }
}

// x [T, H] 32-bit, updated in place unless `rows` is given; a, b [T, H] of element type add_dtype (null: none);
// w, bias [H] 32-bit (bias null: none); y [T or n_rows, H] of element type dtype (null: the sum only); kind 0 RMS norm,
// 1 layer norm, 2 none.
CELLM_API int cellm_add_scaled_norm(void* y, float* x, const void* a, float ma, const void* b, float mb, int add_dtype,
                                    const float* w, const float* bias, const int* rows, int n_rows, int T, int H, float eps,
                                    int kind, int dtype, cudaStream_t stream) {
    const int n = rows ? n_rows : T;
    if (n <= 0) return CELLM_OK;
    if (H <= 0 || kind < 0 || kind > 2) return CELLM_ERR_SIZE;
    if ((y && kind != 2 && !w) || (!y && !a && !b)) return CELLM_ERR_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return CELLM_ERR_SIZE;
    const int vec = H % 4 == 0 && on16(x) && on16(y) && on16(a) && on16(b) && on16(w) && on16(bias);
    const int threads = H >= 1024 ? 256 : 128;
#define ASN_RUN(TA, TD)                                                                                                         \
    do {                                                                                                                        \
        if (smem > 48 * 1024) {                                                                                                 \
            cudaError_t e = cudaFuncSetAttribute(add_scaled_norm_kernel<TA, TD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                                \
        }                                                                                                                       \
        CELLM_RUN((add_scaled_norm_kernel<TA, TD>), n, threads, smem, stream, (TA*)y, x, (const TD*)a, ma, (const TD*)b, mb, w, bias, rows, H, eps, kind, vec); \
    } while (0)
    if (dtype == CELLM_F32 && add_dtype == CELLM_F32) ASN_RUN(float, float);
    else if (dtype == CELLM_BF16 && add_dtype == CELLM_F32) ASN_RUN(__nv_bfloat16, float);
    else if (dtype == CELLM_BF16 && add_dtype == CELLM_BF16) ASN_RUN(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == CELLM_F32 && add_dtype == CELLM_BF16) ASN_RUN(float, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef ASN_RUN
    return CELLM_OK;
}

template <typename TW>
__global__ void __launch_bounds__(256)
stream_add_rows_kernel(float* __restrict__ x, const TW* __restrict__ table, const int* __restrict__ ids, int V, float scale,
                       const float* __restrict__ vec, int H, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    const TW* row = nullptr;
    if (table) {
        int id = ids[t];
        if (id < 0 || id >= V) { if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_TOKEN); id = 0; }
        row = table + (size_t)id * H;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[t * H + i];
        if (row) v += to_float(row[i]) * scale;
        if (vec) v += vec[i];
        x[t * H + i] = v;
    }
}

// x [T, H] 32-bit += scale * table[ids[t]] (table [V, H] of element type w_dtype; null: none) + vec [H] (32-bit; null: none).
// The row times the scale is formed as the embedding forms it (the product rounded to 32-bit, then added).
CELLM_API int cellm_stream_add_rows(float* x, const void* table, int w_dtype, const int* ids, int V, float scale, const float* vec,
                                    int T, int H, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (H <= 0 || (table && (!ids || V <= 0))) return CELLM_ERR_ARG;
    if (w_dtype == CELLM_F32) CELLM_RUN(stream_add_rows_kernel<float>, T, 256, 0, stream, x, (const float*)table, ids, V, scale, vec, H, err);
    else if (w_dtype == CELLM_BF16)
        CELLM_RUN(stream_add_rows_kernel<__nv_bfloat16>, T, 256, 0, stream, x, (const __nv_bfloat16*)table, ids, V, scale, vec, H, err);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
token_gate_mul_kernel(TA* __restrict__ out, const float* __restrict__ g, long long ld_g, const TW* __restrict__ table, long long ld_t,
                      int col0, const int* __restrict__ ids, int V, int n, int act, size_t total, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / n;
    const int i = (int)(idx % n);
    int id = ids[t];
    if (id < 0 || id >= V) { atomicOr(err, CELLM_DEV_BAD_TOKEN); id = 0; }
    out[idx] = from_float<TA>(cellm_activate(g[t * ld_g + i], act) * to_float(table[(size_t)id * ld_t + col0 + i]));
}

// out [T, n] (element type dtype) = act(g [T, n] 32-bit, rows ld_g apart) * table[ids[t]][col0 .. col0 + n] (table
// [V, ld_t] of element type w_dtype).
CELLM_API int cellm_token_gate_mul(void* out, const float* g, long long ld_g, const void* table, long long ld_t, int col0, int w_dtype,
                                   const int* ids, int V, int T, int n, int act, int dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (n <= 0 || V <= 0 || col0 < 0 || col0 + n > ld_t) return CELLM_ERR_SIZE;
    const size_t total = (size_t)T * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
#define TGM_RUN(TA, TW) CELLM_RUN((token_gate_mul_kernel<TA, TW>), blocks, 256, 0, stream, (TA*)out, g, ld_g, (const TW*)table, ld_t, col0, ids, V, n, act, total, err)
    if (dtype == CELLM_F32 && w_dtype == CELLM_F32) TGM_RUN(float, float);
    else if (dtype == CELLM_BF16 && w_dtype == CELLM_BF16) TGM_RUN(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == CELLM_BF16 && w_dtype == CELLM_F32) TGM_RUN(__nv_bfloat16, float);
    else if (dtype == CELLM_F32 && w_dtype == CELLM_BF16) TGM_RUN(float, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef TGM_RUN
    return CELLM_OK;
}

__global__ void __launch_bounds__(256)
scaled_rms_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, float m, int H, float eps, int vec) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    const float* yr = y + t * H;
    float ss = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = ld4(yr + i);
            ss = fmaf(v.x, v.x, ss), ss = fmaf(v.y, v.y, ss), ss = fmaf(v.z, v.z, ss), ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = m / sqrtf(ss / (float)H + eps);
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = ld4(yr + i), g = ld4(w + i), o = ld4(x + t * H + i);
            st4(x + t * H + i, make_float4(fmaf(v.x * inv, g.x, o.x), fmaf(v.y * inv, g.y, o.y), fmaf(v.z * inv, g.z, o.z), fmaf(v.w * inv, g.w, o.w)));
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = m / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) x[t * H + i] = fmaf(yr[i] * inv, w[i], x[t * H + i]);
}

// x [T, H] += m * y / sqrt(mean(y^2) + eps) * w, all 32-bit.
CELLM_API int cellm_scaled_rms_add(float* x, const float* y, const float* w, float m, int T, int H, float eps, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (H <= 0) return CELLM_ERR_SIZE;
    const int vec = H % 4 == 0 && on16(x) && on16(y) && on16(w);
    CELLM_RUN(scaled_rms_add_kernel, T, H >= 1024 ? 256 : 128, 0, stream, x, y, w, m, H, eps, vec);
    return CELLM_OK;
}

template <typename TD>
__global__ void __launch_bounds__(256)
weighted_sum2_kernel(float* __restrict__ out, const TD* __restrict__ a, float ca, const TD* __restrict__ b, float cb, size_t n, int vec) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        i *= 4;
        if (i >= n) return;
        const float4 u = ld4(a + i), v = ld4(b + i);
        st4(out + i, make_float4(ca * u.x + cb * v.x, ca * u.y + cb * v.y, ca * u.z + cb * v.z, ca * u.w + cb * v.w));
        return;
    }
    if (i < n) out[i] = ca * to_float(a[i]) + cb * to_float(b[i]);
}

// out (32-bit) = ca * a + cb * b; a, b of element type dtype.
CELLM_API int cellm_weighted_sum2(float* out, const void* a, float ca, const void* b, float cb, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return CELLM_OK;
    const int vec = n % 4 == 0 && on16(out) && on16(a) && on16(b);
    const unsigned blocks = (unsigned)(((vec ? n / 4 : n) + 255) / 256);
    if (dtype == CELLM_F32) CELLM_RUN(weighted_sum2_kernel<float>, blocks, 256, 0, stream, out, (const float*)a, ca, (const float*)b, cb, (size_t)n, vec);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(weighted_sum2_kernel<__nv_bfloat16>, blocks, 256, 0, stream, out, (const __nv_bfloat16*)a, ca, (const __nv_bfloat16*)b, cb, (size_t)n, vec);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// xIELU with two learned numbers p, q (read on the device): z > 0: softplus(p) z^2 + z / 2; otherwise
// (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2. A block a run of 1,024 columns of one row.
template <typename TA>
__global__ void __launch_bounds__(256)
xielu_kernel(TA* __restrict__ out, const float* __restrict__ u, long long ld, int n, const float* __restrict__ pq) {
    pdl_trigger();
    const float ap = cellm_softplus(pq[0]), aq = 0.5f + cellm_softplus(pq[1]);
    pdl_wait();
    const float* row = u + (size_t)blockIdx.y * ld;
    TA* dst = out + (size_t)blockIdx.y * n;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = blockIdx.x * 1024 + k * 256 + threadIdx.x;
        if (i < n) dst[i] = from_float<TA>(cellm_xielu(row[i], ap, aq));
    }
}

// out [T, n] (element type dtype) = xielu(u [T, n] 32-bit, rows ld apart) with pq = (p, q), 32-bit on the device.
CELLM_API int cellm_xielu(void* out, const float* u, long long ld, int T, int n, const float* pq, int dtype, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return CELLM_OK;
    if (!pq) return CELLM_ERR_ARG;
    for (int t0 = 0; t0 < T; t0 += 65535) {          // a grid's second extent holds 65,535 rows
        const int rows = T - t0 < 65535 ? T - t0 : 65535;
        const dim3 grid((unsigned)((n + 1023) / 1024), (unsigned)rows);
        const float* src = u + (size_t)t0 * ld;
        if (dtype == CELLM_F32) CELLM_RUN(xielu_kernel<float>, grid, 256, 0, stream, (float*)out + (size_t)t0 * n, src, ld, n, pq);
        else if (dtype == CELLM_BF16) CELLM_RUN(xielu_kernel<__nv_bfloat16>, grid, 256, 0, stream, (__nv_bfloat16*)out + (size_t)t0 * n, src, ld, n, pq);
        else return CELLM_ERR_DTYPE;
    }
    return CELLM_OK;
}

template <typename TA>
__global__ void __launch_bounds__(256)
head_gate_mul_kernel(TA* __restrict__ o, const float* __restrict__ gate, long long gate_ld, int heads, int vd, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / ((size_t)heads * vd);
    const int h = (int)((idx / vd) % heads);
    o[idx] = from_float<TA>(to_float(o[idx]) / (1.f + expf(-gate[t * gate_ld + h])));
}

// o [T, heads * vd] (element type dtype), in place: head h of token t times sigmoid(gate[t * gate_ld + h]) (32-bit).
CELLM_API int cellm_head_gate_mul(void* o, const float* gate, long long gate_ld, int T, int heads, int vd, int dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (heads <= 0 || vd <= 0) return CELLM_ERR_SIZE;
    const size_t total = (size_t)T * heads * vd;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == CELLM_F32) CELLM_RUN(head_gate_mul_kernel<float>, blocks, 256, 0, stream, (float*)o, gate, gate_ld, heads, vd, total);
    else if (dtype == CELLM_BF16) CELLM_RUN(head_gate_mul_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)o, gate, gate_ld, heads, vd, total);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
