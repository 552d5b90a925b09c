// Attention over a latent cache on the tensor cores (mma.sync m16n8k16, bfloat16): every head of a token reads the
// same cached rows of `kw` values (one key/value "head"), and a value is a row's first `dv` values, so keys and
// values are one tile in shared memory. Serves prompt portions and decoded tokens alike.
//
// A CTA takes 64 consecutive (token, head) rows of one request's portion (the queries lie [T, heads, kw], so these are
// 64 consecutive rows of kw values) and walks the keys in blocks of BN through the block table (cp.async, two stages;
// a block's keys are worked on in runs of SUB, which is what the score registers hold).
// Its warps are 4 groups of 16 rows times NC groups of DVW value columns: a warp forms S = Q K^T for its 16 rows and
// the block's keys (the NC warps of a row group each form the same S: the scores cost kw/dv of the values' work, and
// nothing has to pass between warps), keeps the running maximum and sum of flash attention in registers, and adds
// P V for its own DVW columns. The keys may be cut into `nsplit` pieces (blockIdx.y): each piece leaves its maximum,
// sum and unnormalised output in a workspace and a second kernel merges the pieces in their order.
//
// Softmax is 32-bit (scores stay raw; scale * log2(e) enters with the subtraction of the maximum; ex2.approx).
// Cache layout of one layer: [page][slot in page][kw].
#include "mma_tiles.cuh"

namespace {

constexpr int LA_BM = 64;

template <int DVW, int BN, int SUB, int MAXT>
__global__ void __launch_bounds__(MAXT)
latent_flash_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens, const int* __restrict__ block_table,
                    int bt_stride, int B, int T, int num_pages, int page_size, int nh, int kw, int dv, float scale_log2e,
                    int nsplit, int window, const float* __restrict__ sinks, int* __restrict__ err) {
    constexpr int NT = DVW / 8;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int stride = kw + 8;                                   // elements per row in shared memory (16 bytes of padding)
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* k_s = q_s + LA_BM * stride;                   // two stages of BN rows
    const int threads = blockDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rw = warp & 3, cg = warp >> 2;
    const int CH = kw / 8;                                       // 16-byte chunks per row
    pdl_trigger();
    // which request and which of its tiles (the step's index arrays are not the work of the kernel before this one)
    int tile = blockIdx.x, b = 0, rows = 0;
    for (; b < B; ++b) {
        rows = (cu_seqlens[b + 1] - cu_seqlens[b]) * nh;
        const int n = (rows + LA_BM - 1) / LA_BM;
        if (tile < n) break;
        tile -= n;
    }
    if (b >= B) return;
    const int split = blockIdx.y;
    const int t_base = cu_seqlens[b], ctx = ctx_lens[b];
    const int r0 = tile * LA_BM;
    const int t_hi = min(r0 + LA_BM - 1, rows - 1) / nh;
    const int key_end = ctx + t_hi + 1;
    // with a window a row reads its last `window` rows only: the tile's first key is its first row's
    const int key_begin = window > 0 ? max(0, ctx + r0 / nh - window + 1) : 0;
    const int kb_begin = key_begin / BN, kb_end = (key_end + BN - 1) / BN;
    const int per = (kb_end - kb_begin + nsplit - 1) / nsplit;
    const int my_begin = kb_begin + split * per, my_end = min(kb_end, my_begin + per);
    const int* bt = block_table + (size_t)b * bt_stride;
    pdl_wait();

    for (int i = threadIdx.x; i < LA_BM * CH; i += threads) {
        const int row = i / CH, chunk = i - row * CH, r = r0 + row;
        const bool ok = r < rows;
        const __nv_bfloat16* src = q + ((size_t)t_base * nh + (ok ? r : 0)) * kw + chunk * 8;
        cp_async16(q_s + row * stride + chunk * 8, src, ok ? 16 : 0);
    }
    // The rows of a block's keys are looked up first, all at once (one thread a key), so that the copies that follow do
    // not each wait for a load of the block table.
    __shared__ long long row_at[2][BN];
    auto load_k = [&](int kb, int stage) {
        if (threadIdx.x < BN) {
            const int j = kb * BN + threadIdx.x;
            long long at = -1;
            if (j >= key_begin && j < key_end) {
                const int page = bt[j / page_size];
                if (page < 0 || page >= num_pages) atomicOr(err, CELLM_DEV_BAD_PAGE);
                else at = ((long long)page * page_size + j % page_size) * kw;
            }
            row_at[stage][threadIdx.x] = at;
        }
        __syncthreads();
        __nv_bfloat16* ks = k_s + stage * BN * stride;
        for (int i = threadIdx.x; i < BN * CH; i += threads) {
            const int row = i / CH, chunk = i - row * CH;
            const long long at = row_at[stage][row];
            cp_async16(ks + row * stride + chunk * 8, pool + (at >= 0 ? at + chunk * 8 : 0), at >= 0 ? 16 : 0);
        }
    };
    if (my_begin < my_end) load_k(my_begin, 0);
    cp_async_commit();

    const int row_a = r0 + rw * 16 + (lane >> 2), row_b = row_a + 8;
    const int pos_a = row_a < rows ? ctx + row_a / nh : -1, pos_b = row_b < rows ? ctx + row_b / nh : -1;
    const int lo_a = window > 0 ? pos_a - window + 1 : 0, lo_b = window > 0 ? pos_b - window + 1 : 0;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    for (int kb = my_begin, it = 0; kb < my_end; ++kb, ++it) {
        const int stage = it & 1;
        if (kb + 1 < my_end) load_k(kb + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (r0 + rw * 16 < rows) {           // (a decoded token's heads fill one or two of the four row groups)
        // the block's keys in runs of SUB: scores, softmax and values of one run after the other (a block is what is
        // fetched and waited for at once; a run is what the score registers hold)
#pragma unroll 1
        for (int sub = 0; sub < BN / SUB; ++sub) {
        if ((kb * BN + sub * SUB) >= key_end) break;
        if (kb * BN + sub * SUB + SUB <= key_begin) continue;
        const __nv_bfloat16* ks_ = k_s + (stage * BN + sub * SUB) * stride;
        float s[SUB / 8][4];
#pragma unroll
        for (int n = 0; n < SUB / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const __nv_bfloat16* q_row = q_s + (rw * 16 + (lane & 15)) * stride + (lane >> 4) * 8;
        const __nv_bfloat16* k_row = ks_ + ((lane & 7) + ((lane >> 4) << 3)) * stride + ((lane >> 3) & 1) * 8;
#pragma unroll 4
        for (int k0 = 0; k0 < kw; k0 += 16) {
            uint32_t qf[4];
            ldmatrix_x4(qf, q_row + k0);
#pragma unroll
            for (int n2 = 0; n2 < SUB / 16; ++n2) {
                uint32_t kf[4];
                ldmatrix_x4(kf, k_row + n2 * 16 * stride + k0);
                mma_bf16(s[2 * n2], qf, kf[0], kf[1]);
                mma_bf16(s[2 * n2 + 1], qf, kf[2], kf[3]);
            }
        }
        // mask (a key after the row's own position), running maximum and sum
        const int j0 = kb * BN + sub * SUB + (lane & 3) * 2;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < SUB / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j0 + n * 8 + e;
                const float va = (j <= pos_a && j >= lo_a) ? s[n][e] : -INFINITY;
                const float vb = (j <= pos_b && j >= lo_b) ? s[n][2 + e] : -INFINITY;
                s[n][e] = va;
                s[n][2 + e] = vb;
                mx_a = fmaxf(mx_a, va);
                mx_b = fmaxf(mx_b, vb);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a * scale_log2e), mn_b = fmaxf(m_b, mx_b * scale_log2e);
        const float use_a = mn_a == -INFINITY ? 0.f : mn_a, use_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float corr_a = fast_exp2(m_a - use_a), corr_b = fast_exp2(m_b - use_b);
        m_a = mn_a;
        m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pf[SUB / 16][4];
#pragma unroll
        for (int n = 0; n < SUB / 8; ++n) {
            const float p0 = fast_exp2(fmaf(s[n][0], scale_log2e, -use_a)), p1 = fast_exp2(fmaf(s[n][1], scale_log2e, -use_a));
            const float p2 = fast_exp2(fmaf(s[n][2], scale_log2e, -use_b)), p3 = fast_exp2(fmaf(s[n][3], scale_log2e, -use_b));
            sum_a += p0 + p1;
            sum_b += p2 + p3;
            pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_a = l_a * corr_a + sum_a;
        l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int n = 0; n < NT; ++n) { o[n][0] *= corr_a; o[n][1] *= corr_a; o[n][2] *= corr_b; o[n][3] *= corr_b; }
        // O += P V over this warp's DVW columns of the rows' first dv values
        const __nv_bfloat16* v_row = ks_ + ((lane & 7) + (((lane >> 3) & 1) << 3)) * stride + cg * DVW + (lane >> 4) * 8;
#pragma unroll
        for (int kk = 0; kk < SUB / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, v_row + kk * 16 * stride + n2 * 16);
                mma_bf16(o[2 * n2], pf[kk], vf[0], vf[1]);
                mma_bf16(o[2 * n2 + 1], pf[kk], vf[2], vf[3]);
            }
        }
        }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const int col = cg * DVW + (lane & 3) * 2;
    const size_t base_row = (size_t)t_base * nh;
    if (nsplit == 1) {
        if (sinks) {
            // a sink: one more term exp(sink_h) in the row's denominator, with no key and no value
            if (row_a < rows) l_a += exp2f(sinks[row_a % nh] * 1.4426950408889634f - (m_a == -INFINITY ? 0.f : m_a));
            if (row_b < rows) l_b += exp2f(sinks[row_b % nh] * 1.4426950408889634f - (m_b == -INFINITY ? 0.f : m_b));
        }
        const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
        if (row_a < rows) {
            __nv_bfloat16* dst = out + (base_row + row_a) * dv + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][0] * inv_a, o[n][1] * inv_a);
        }
        if (row_b < rows) {
            __nv_bfloat16* dst = out + (base_row + row_b) * dv + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][2] * inv_b, o[n][3] * inv_b);
        }
    } else {
        const size_t n_rows = (size_t)T * nh;
        if (row_a < rows) {
            const size_t gr = (size_t)split * n_rows + base_row + row_a;
            float* dst = part_o + gr * dv + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][0], o[n][1]);
            if (cg == 0 && (lane & 3) == 0) { part_ml[gr * 2] = m_a; part_ml[gr * 2 + 1] = l_a; }
        }
        if (row_b < rows) {
            const size_t gr = (size_t)split * n_rows + base_row + row_b;
            float* dst = part_o + gr * dv + col;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2], o[n][3]);
            if (cg == 0 && (lane & 3) == 0) { part_ml[gr * 2] = m_b; part_ml[gr * 2 + 1] = l_b; }
        }
    }
}

// The pieces of a row merged in their order: out = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s.
__global__ void latent_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, size_t n_rows, int dv, int nsplit,
                                    const float* __restrict__ sinks, int nh) {
    extern __shared__ float ml[];        // [nsplit][2]: maximum and sum of each piece, then its weight in [s][0]
    pdl_trigger();
    pdl_wait();
    const size_t r = blockIdx.x;
    for (int s = threadIdx.x; s < nsplit; s += blockDim.x) {
        const float2 v = *reinterpret_cast<const float2*>(part_ml + ((size_t)s * n_rows + r) * 2);
        ml[2 * s] = v.x;
        ml[2 * s + 1] = v.y;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ml[2 * s]);
    float L = 0.f;
    for (int s = 0; s < nsplit; ++s) L += ml[2 * s] == -INFINITY ? 0.f : fast_exp2(ml[2 * s] - M) * ml[2 * s + 1];   // in the pieces' order
    if (sinks) L += exp2f(sinks[r % nh] * 1.4426950408889634f - (M == -INFINITY ? 0.f : M));          // the sink counts once
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < nsplit; ++s) {
            const float wgt = ml[2 * s] == -INFINITY ? 0.f : fast_exp2(ml[2 * s] - M) * inv;
            acc = fmaf(wgt, part_o[((size_t)s * n_rows + r) * dv + d], acc);
        }
        out[r * dv + d] = __float2bfloat16_rn(acc);
    }
}

// value columns per warp for a value width, or 0 if no form of the kernel takes it
int value_columns(int dv) {
    if (dv % 256 == 0 && dv / 256 <= 2) return 256;     // 8 warps with 128 accumulator registers each: the scores are formed twice, not four times
    if (dv % 128 == 0 && dv / 128 <= 4) return 128;
    if (dv % 64 == 0 && dv / 64 <= 4) return 64;
    if (dv % 32 == 0 && dv / 32 <= 8) return 32;
    if (dv % 16 == 0 && dv / 16 <= 8) return 16;
    return 0;
}
// keys fetched and waited for at once (256 value columns a warp: 64 where two such stages fit beside the queries)
int keys_per_block(int dvw, int kw) {
    if (dvw == 256) return (size_t)(LA_BM + 128) * (kw + 8) * 2 + 2048 <= 227 * 1024 ? 64 : 32;
    return dvw == 64 ? 64 : 32;
}

// Per-head products on the tensor cores: out[t, h, n] = sum_k in[t, h, k] * w[h][n][k]. A CTA forms 64 tokens by 64
// outputs of one head: both operands' tiles wait whole in shared memory (K at most 512), each of the four warps forms
// 16 tokens by 64 outputs as the attention forms its scores (rows of `in` against rows of `w`).
__global__ void __launch_bounds__(128)
head_product_mma_kernel(__nv_bfloat16* __restrict__ out, long long ldo, long long out_hs, const __nv_bfloat16* __restrict__ in,
                        long long ldi, long long in_hs, const __nv_bfloat16* __restrict__ w, int T, int N, int K) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int stride = K + 8;
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* w_s = a_s + 64 * stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.z, t0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int CH = K / 8;
    pdl_trigger();
    const __nv_bfloat16* wh = w + (size_t)h * N * K;
    for (int i = threadIdx.x; i < 64 * CH; i += 128) {          // the matrices are not the work of the kernel before this one
        const int row = i / CH, chunk = i - row * CH, n = n0 + row;
        cp_async16(w_s + row * stride + chunk * 8, wh + (size_t)(n < N ? n : 0) * K + chunk * 8, n < N ? 16 : 0);
    }
    pdl_wait();
    for (int i = threadIdx.x; i < 64 * CH; i += 128) {
        const int row = i / CH, chunk = i - row * CH, t = t0 + row;
        cp_async16(a_s + row * stride + chunk * 8, in + (size_t)(t < T ? t : 0) * ldi + h * in_hs + chunk * 8, t < T ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    float c[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
    const __nv_bfloat16* a_row = a_s + (warp * 16 + (lane & 15)) * stride + (lane >> 4) * 8;
    const __nv_bfloat16* w_row = w_s + ((lane & 7) + ((lane >> 4) << 3)) * stride + ((lane >> 3) & 1) * 8;
#pragma unroll 2
    for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t af[4];
        ldmatrix_x4(af, a_row + k0);
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
            uint32_t wf[4];
            ldmatrix_x4(wf, w_row + n2 * 16 * stride + k0);
            mma_bf16(c[2 * n2], af, wf[0], wf[1]);
            mma_bf16(c[2 * n2 + 1], af, wf[2], wf[3]);
        }
    }
    const int ta = t0 + warp * 16 + (lane >> 2), tb = ta + 8;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const int col = n0 + n * 8 + (lane & 3) * 2;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (col + e < N) {
                if (ta < T) out[(size_t)ta * ldo + h * out_hs + col + e] = __float2bfloat16_rn(c[n][e]);
                if (tb < T) out[(size_t)tb * ldo + h * out_hs + col + e] = __float2bfloat16_rn(c[n][2 + e]);
            }
        }
    }
}

}  // namespace

// 1 if the kernel takes rows of kw values whose first dv are the value (else the plain kernel serves them)
CELLM_API int cellm_attention_latent_supports(int kw, int dv) {
    if (kw <= 0 || dv <= 0 || dv > kw || (kw & 15) || (dv & 15)) return 0;
    const int dvw = value_columns(dv);
    if (!dvw) return 0;
    const size_t smem = (size_t)(LA_BM + 2 * keys_per_block(dvw, kw)) * (kw + 8) * 2 + 2048;
    return smem <= 227 * 1024 ? 1 : 0;
}

// q: [T, nh, kw] (a head's query against the cached rows); out: [T, nh, dv]; pool: one layer's rows. part_o
// [nsplit, T * nh, dv] and part_ml [nsplit, T * nh, 2] floats are needed when nsplit > 1. n_tiles: the sum over the
// requests of ceil(tokens * nh / 64). window: 0, or how many of its last rows a token reads (itself included). sinks [nh]
// 32-bit: one more term exp(sink_h) in a head's denominator (null: none).
CELLM_API int cellm_attention_latent(void* out, float* part_o, float* part_ml, const void* q, const void* pool,
                                     const int* cu_seqlens, const int* ctx_lens, const int* block_table, int bt_stride, int B,
                                     int T, int n_tiles, int num_pages, int page_size, int nh, int kw, int dv, float scale,
                                     int nsplit, int window, const float* sinks, int* err, cudaStream_t stream) {
    if (T <= 0 || B <= 0 || n_tiles <= 0) return CELLM_OK;
    if (!cellm_attention_latent_supports(kw, dv) || nh <= 0 || page_size <= 0 || nsplit < 1 || !(scale > 0.f) || window < 0) return CELLM_ERR_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)pool & 15) || ((uintptr_t)out & 3)) return CELLM_ERR_ALIGN;
    if (nsplit > 1 && (!part_o || !part_ml)) return CELLM_ERR_ARG;
    const int dvw = value_columns(dv), bn = keys_per_block(dvw, kw);
    const int threads = 128 * (dv / dvw);
    const size_t smem = (size_t)(LA_BM + 2 * bn) * (kw + 8) * 2;
    const float scale_log2e = scale * 1.4426950408889634f;
    const dim3 grid((unsigned)n_tiles, (unsigned)nsplit);
#define LAUNCH(DVW, BN, SUB, MAXT)                                                                                       \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(latent_flash_kernel<DVW, BN, SUB, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        CELLM_RUN((latent_flash_kernel<DVW, BN, SUB, MAXT>), grid, threads, smem, stream, (__nv_bfloat16*)out, part_o, part_ml,  \
                  (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, cu_seqlens, ctx_lens, block_table, bt_stride, B, T,  \
                  num_pages, page_size, nh, kw, dv, scale_log2e, nsplit, window, sinks, err);                               \
    } while (0)
    if (dvw == 256 && bn == 64) LAUNCH(256, 64, 32, 256);
    else if (dvw == 256) LAUNCH(256, 32, 32, 256);
    else if (dvw == 128) LAUNCH(128, 32, 32, 512);
    else if (dvw == 64) LAUNCH(64, 64, 64, 512);
    else if (dvw == 32) LAUNCH(32, 32, 32, 1024);
    else LAUNCH(16, 32, 32, 1024);
#undef LAUNCH
    if (nsplit > 1)
        CELLM_RUN(latent_merge_kernel, (unsigned)((size_t)T * nh), dv >= 256 ? 256 : (dv >= 128 ? 128 : 64), (size_t)nsplit * 2 * sizeof(float), stream, (__nv_bfloat16*)out, part_o,
                  part_ml, (size_t)T * nh, dv, nsplit, sinks, nh);
    return CELLM_OK;
}

// Per-head products of many tokens: in [T, ldi] with head h at columns h * in_hs (K values, 16-byte aligned), w [heads, N,
// K], out [T, ldo] with head h at columns h * out_hs. K a multiple of 16 and at most 512.
CELLM_API int cellm_head_product_mma(void* out, long long ldo, long long out_hs, const void* in, long long ldi, long long in_hs,
                                     const void* w, int T, int heads, int N, int K, cudaStream_t stream) {
    if (T <= 0 || heads <= 0 || N <= 0) return CELLM_OK;
    if (K <= 0 || (K & 15) || K > 512) return CELLM_ERR_SIZE;
    if (((uintptr_t)in & 15) || ((uintptr_t)w & 15) || (ldi & 7) || (in_hs & 7)) return CELLM_ERR_ALIGN;
    const size_t smem = (size_t)2 * 64 * (K + 8) * 2;
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_product_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const dim3 grid((unsigned)((N + 63) / 64), (unsigned)((T + 63) / 64), (unsigned)heads);
    CELLM_RUN(head_product_mma_kernel, grid, 128, smem, stream, (__nv_bfloat16*)out, ldo, out_hs, (const __nv_bfloat16*)in, ldi,
              in_hs, (const __nv_bfloat16*)w, T, N, K);
    return CELLM_OK;
}
