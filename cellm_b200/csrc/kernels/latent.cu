// Latent attention: what lies between the products of a mixer that keeps one compressed row per token instead of
// keys and values per head.
//
// Per token the down projection gives a latent c (kv_rank values, RMS-normed with a weight) and one rotated key part
// (rot_dim values) that all heads share; only these kv_rank + rot_dim values are cached. A head's unrotated key is
// K_h c and its value V_h c with per-head matrices K_h [dim, kv_rank], V_h [vdim, kv_rank]. Because q.(K_h c) =
// (K_h^T q).c, the attention runs over the cached rows themselves: the query of head h becomes [K_h^T q_h | rotated
// part] (kv_rank + rot_dim values), every head reads the same rows, the weighted sum of the rows' first kv_rank
// values is formed, and V_h turns that sum into the head's output.
//
//   latent_prep     norm of c, rotation of the shared key part, cache write; the queries' unrotated parts gathered
//                   head by head, their rotated parts turned and put behind the place of K_h^T q_h
//   head_product    out[t, h, :] = W[h] in[t, h, :] for per-head matrices W[h] [N, K] (K_h^T and V_h above)
//
// Norm, angles and rotation are 32-bit. Cache layout of one layer: [page][slot in page][kv_rank + rot_dim].
#include "common.cuh"

// cos and sin of pos * inv_freq, the frequency given as a float and the remainder the float dropped: the product's
// rounding error enters through the addition formulas, so the rotation carries no error that grows with the position.
__device__ __forceinline__ void split_angle(int pos, float hi, float lo, float* c_out, float* s_out) {
    const float fp = (float)pos;
    const float a = fp * hi;
    const float e = fmaf(fp, hi, -a) + fp * lo;
    float s, c, se, ce;
    sincosf(a, &s, &c);
    sincosf(e, &se, &ce);
    *c_out = c * ce - s * se;
    *s_out = s * ce + c * se;
}

template <typename TP, typename TA, typename TW>
__global__ void __launch_bounds__(128)
latent_prep_kernel(TA* __restrict__ q_plain, TA* __restrict__ q_full, const TP* __restrict__ proj, long long ld,
                   const TW* __restrict__ c_norm_w, float eps, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
                   TA* __restrict__ pool, int num_pages, int page_size, int heads, int dim, int rot_dim, int rank,
                   int rot, int interleaved, const float* __restrict__ inv_freq, int* __restrict__ err) {
    extern __shared__ float smem[];
    float* cs = smem;                // [rot/2]
    float* sn = smem + rot / 2;      // [rot/2]
    __shared__ float scratch[32];
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int p = threadIdx.x; p < rot / 2; p += blockDim.x) split_angle(pos, inv_freq[2 * p], inv_freq[2 * p + 1], &cs[p], &sn[p]);
    TA* cache_row = nullptr;
    if (pool) {
        const int b = seq_of_token[t];
        const int page = block_table[(size_t)b * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_PAGE);
        } else {
            cache_row = pool + ((size_t)page * page_size + pos % page_size) * (rank + rot_dim);
        }
    }
    __syncthreads();
    pdl_wait();
    const TP* row = proj + (size_t)t * ld;
    const int qw = dim + rot_dim, kw = rank + rot_dim;
    // blockIdx.y = 0: the latent and the shared key part; 1..: a run of query heads each, so that a token's work is
    // spread over several blocks when the tokens are few
    if (blockIdx.y > 0) {
    const int per = (heads + gridDim.y - 2) / (gridDim.y - 1);
    const int h_lo = min(heads, ((int)blockIdx.y - 1) * per), h_hi = min(heads, h_lo + per);
    // queries: the unrotated part head by head; the rotated part turned, behind the kv_rank places of its head
    for (int i = h_lo * dim + threadIdx.x; i < h_hi * dim; i += blockDim.x) {
        const int h = i / dim, d = i - h * dim;
        q_plain[(size_t)t * heads * dim + i] = from_float<TA>(to_float(row[h * qw + d]));
    }
    for (int i = h_lo * rot_dim + threadIdx.x; i < h_hi * rot_dim; i += blockDim.x) {
        const int h = i / rot_dim, d = i - h * rot_dim;
        const TP* src = row + h * qw + dim;
        float v = to_float(src[d]);
        if (d < rot) {
            // pairs (2p, 2p + 1) when interleaved, (p, p + rot/2) otherwise; the pair's first entry is u cos - v sin
            const int half = rot >> 1;
            const int p = interleaved ? d >> 1 : (d < half ? d : d - half);
            const bool second = interleaved ? (d & 1) : d >= half;
            const float other = to_float(src[interleaved ? d ^ 1 : (second ? d - half : d + half)]);
            v = second ? v * cs[p] + other * sn[p] : v * cs[p] - other * sn[p];
        }
        q_full[((size_t)t * heads + h) * kw + rank + d] = from_float<TA>(v);
    }
    return;
    }
    // the latent: divided by its root mean square, times its weight; the shared key part turned; both to the cache
    const TP* down = row + (size_t)heads * qw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(down[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    if (cache_row) {
        for (int i = threadIdx.x; i < rank; i += blockDim.x)
            cache_row[i] = from_float<TA>(to_float(down[i]) * inv * to_float(c_norm_w[i]));
        for (int d = threadIdx.x; d < rot_dim; d += blockDim.x) {
            float v = to_float(down[rank + d]);
            if (d < rot) {
                const int half = rot >> 1;
                const int p = interleaved ? d >> 1 : (d < half ? d : d - half);
                const bool second = interleaved ? (d & 1) : d >= half;
                const float other = to_float(down[rank + (interleaved ? d ^ 1 : (second ? d - half : d + half))]);
                v = second ? v * cs[p] + other * sn[p] : v * cs[p] - other * sn[p];
            }
            cache_row[rank + d] = from_float<TA>(v);
        }
    }
}

// proj: [T, ld] = [heads * (dim + rot_dim) queries | kv_rank latent | rot_dim shared key part] (32-bit, or the
// activations' type); q_plain: [T, heads * dim]; q_full: [T, heads, kv_rank + rot_dim] (only the last rot_dim of each
// head are written); pool: one layer's rows or null (the item reads another's cache). rot: how many of the rot_dim
// values turn (even), in pairs (2p, 2p + 1) if `interleaved`, else (p, p + rot / 2); inv_freq: [rot / 2] pairs of floats
// (frequency, remainder).
CELLM_API int cellm_latent_prep(void* q_plain, void* q_full, const void* proj, long long ld, int proj_dtype, const void* c_norm_w,
                                int w_dtype, float eps, const int* positions, const int* seq_of_token, const int* block_table,
                                int bt_stride, void* pool, int num_pages, int page_size, int T, int heads, int dim, int rot_dim,
                                int rank, int rot, int interleaved, const float* inv_freq, int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (heads <= 0 || dim < 0 || rot_dim < 0 || rank <= 0 || rot < 0 || rot > rot_dim || (rot & 1)) return CELLM_ERR_SIZE;
    if (ld < (long long)heads * (dim + rot_dim) + rank + rot_dim) return CELLM_ERR_SIZE;
    if (rot > 0 && !inv_freq) return CELLM_ERR_ARG;
    if (pool && (!block_table || page_size <= 0)) return CELLM_ERR_ARG;
    const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
    // few tokens: a token's query heads in up to 8 blocks beside the block of its latent
    const int qblocks = T >= 256 ? 1 : (heads < 8 ? heads : 8);
    const dim3 grid((unsigned)T, (unsigned)(1 + qblocks));
#define LAUNCH(TP, TA, TW)                                                                                              \
    CELLM_RUN((latent_prep_kernel<TP, TA, TW>), grid, 128, smem, stream, (TA*)q_plain, (TA*)q_full, (const TP*)proj, ld,    \
              (const TW*)c_norm_w, eps, positions, seq_of_token, block_table, bt_stride, (TA*)pool, num_pages, page_size, \
              heads, dim, rot_dim, rank, rot, interleaved, inv_freq, err)
    if (act_dtype == CELLM_F32 && proj_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float, float);
    else if (act_dtype == CELLM_F32 && proj_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, __nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}

// ---- per-head products ------------------------------------------------------------------------------------------
// out[t, h * out_hs + n] = sum_k in[t, h * in_hs + k] * w[h][n][k]; tiles of 32 tokens by 32 outputs, K in runs of 32
// summed in order, 32-bit accumulation.
#define HP_TILE 32
template <typename TA>
__global__ void __launch_bounds__(HP_TILE * 8)
head_product_kernel(TA* __restrict__ out, long long ldo, long long out_hs, const TA* __restrict__ in, long long ldi,
                    long long in_hs, const TA* __restrict__ w, int T, int N, int K) {
    __shared__ float as[HP_TILE][HP_TILE + 1];
    __shared__ float ws[HP_TILE][HP_TILE + 1];
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.z;
    const int t0 = blockIdx.y * HP_TILE, n0 = blockIdx.x * HP_TILE;
    const int tx = threadIdx.x, ty = threadIdx.y;            // 32 x 8
    const TA* wh = w + (size_t)h * N * K;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += HP_TILE) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int rr = ty + r * 8;
            const int t = t0 + rr, n = n0 + rr, k = k0 + tx;
            as[rr][tx] = (t < T && k < K) ? to_float(in[(size_t)t * ldi + h * in_hs + k]) : 0.f;
            ws[rr][tx] = (n < N && k < K) ? to_float(wh[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HP_TILE; ++kk) {
            const float b = ws[tx][kk];
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[r] = fmaf(as[ty + r * 8][kk], b, acc[r]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int t = t0 + ty + r * 8, n = n0 + tx;
        if (t < T && n < N) out[(size_t)t * ldo + h * out_hs + n] = from_float<TA>(acc[r]);
    }
}

// A few tokens (decoding, bfloat16): the matrices are what has to be read, once. A block takes 16 output rows of one
// head; the tokens' inputs wait in shared memory; eight neighbouring threads share a row and take neighbouring 16-byte
// pieces of it by turns (so a row's loads are whole 128-byte lines and the inputs' reads fall into different banks),
// and add their sums by three shuffles. K (a multiple of 64) is summed in the same order for every token count up to
// HP_SMALL_T.
#define HP_SMALL_T 16
__global__ void __launch_bounds__(128)
head_product_small_kernel(__nv_bfloat16* __restrict__ out, long long ldo, long long out_hs, const __nv_bfloat16* __restrict__ in,
                          long long ldi, long long in_hs, const __nv_bfloat16* __restrict__ w, int T, int N, int K, int vec_in) {
    extern __shared__ __align__(16) __nv_bfloat16 xin[];       // [T][K]
    pdl_trigger();
    const int h = blockIdx.y;
    const int n = blockIdx.x * 16 + (threadIdx.x >> 3), kq = threadIdx.x & 7;
    const bool on = n < N;
    const __nv_bfloat16* wr = w + ((size_t)h * N + (on ? n : 0)) * K;
    pdl_wait();
    if (vec_in) {                        // the inputs' rows start on 16-byte borders: eight values a load
        const int K8 = K / 8;
        for (int i = threadIdx.x; i < T * K8; i += blockDim.x) {
            const int t = i / K8, k = (i - t * K8) * 8;
            *reinterpret_cast<uint4*>(xin + t * K + k) = *reinterpret_cast<const uint4*>(in + (size_t)t * ldi + h * in_hs + k);
        }
    } else {
        for (int i = threadIdx.x; i < T * K; i += blockDim.x) {
            const int t = i / K, k = i - t * K;
            xin[i] = in[(size_t)t * ldi + h * in_hs + k];
        }
    }
    __syncthreads();
    float acc[HP_SMALL_T];
#pragma unroll
    for (int t = 0; t < HP_SMALL_T; ++t) acc[t] = 0.f;
#pragma unroll 2
    for (int k0 = kq * 8; k0 < K; k0 += 64) {
        const uint4 wq = *reinterpret_cast<const uint4*>(wr + k0);
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wq);
        float wv[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(wp[j]); wv[2 * j] = f.x; wv[2 * j + 1] = f.y; }
#pragma unroll
        for (int t = 0; t < HP_SMALL_T; ++t) {
            if (t < T) {
                const uint4 xq = *reinterpret_cast<const uint4*>(xin + t * K + k0);
                const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xq);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(xp[j]);
                    acc[t] = fmaf(f.x, wv[2 * j], acc[t]);
                    acc[t] = fmaf(f.y, wv[2 * j + 1], acc[t]);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < HP_SMALL_T; ++t) {
        if (t < T) {
            float v = acc[t];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if (kq == 0 && on) out[(size_t)t * ldo + h * out_hs + n] = __float2bfloat16_rn(v);
        }
    }
}

// in: [T, ldi] with head h at columns h * in_hs; w: [heads, N, K]; out: [T, ldo] with head h at columns h * out_hs.
CELLM_API int cellm_head_product(void* out, long long ldo, long long out_hs, const void* in, long long ldi, long long in_hs,
                                 const void* w, int T, int heads, int N, int K, int dtype, cudaStream_t stream) {
    if (T <= 0 || heads <= 0 || N <= 0) return CELLM_OK;
    if (K <= 0) return CELLM_ERR_SIZE;
    // (32-bit activations always take the tiles below: one order of the sums whatever the number of tokens)
    if (dtype == CELLM_BF16 && T <= HP_SMALL_T && (size_t)T * K * 2 <= 48 * 1024 && (K & 63) == 0 &&
        ((uintptr_t)w & 15) == 0) {
        const dim3 sgrid((unsigned)((N + 15) / 16), (unsigned)heads);
        const size_t smem = (size_t)T * K * 2;
        CELLM_RUN(head_product_small_kernel, sgrid, 128, smem, stream, (__nv_bfloat16*)out, ldo, out_hs,
                  (const __nv_bfloat16*)in, ldi, in_hs, (const __nv_bfloat16*)w, T, N, K,
                  (int)((((uintptr_t)in & 15) == 0) && (ldi & 7) == 0 && (in_hs & 7) == 0));
        return CELLM_OK;
    }
    const dim3 grid((unsigned)((N + HP_TILE - 1) / HP_TILE), (unsigned)((T + HP_TILE - 1) / HP_TILE), (unsigned)heads);
    const dim3 block(HP_TILE, 8);
    if (dtype == CELLM_F32)
        CELLM_RUN(head_product_kernel<float>, grid, block, 0, stream, (float*)out, ldo, out_hs, (const float*)in, ldi, in_hs,
                  (const float*)w, T, N, K);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(head_product_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)out, ldo, out_hs,
                  (const __nv_bfloat16*)in, ldi, in_hs, (const __nv_bfloat16*)w, T, N, K);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
