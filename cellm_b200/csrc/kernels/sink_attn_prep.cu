// What lies between the q, k, v projection and the attention itself for an attention whose projections pass a
// short causal convolution, are normed over the whole projection, and whose values are rotated as well as its
// queries and keys. One block a token:
//
//   1. projected value + bias, then the convolution over time (conv_taps.cuh) for every channel of q, k and v;
//   2. RMS norm of q over all its heads at once, and of k, with plain weights;
//   3. rotation of the first `rot` entries of every q and k head by pos * f_i (f from a table that may be scaled);
//   4. rotation of every value head over all its entries by pos * g_m (a table of its own);
//   5. q into the step's buffer, k and v into the token's page.
//
// All arithmetic is 32-bit; angles are pos * (hi + lo) in split arithmetic from tables made in 64-bit.
#include "conv_taps.cuh"

template <typename TA>
__global__ void __launch_bounds__(1024)
sink_attn_prep_kernel(TA* __restrict__ q_out, TA* __restrict__ k_pool, TA* __restrict__ v_pool, ConvTaps cv,
                      const float* __restrict__ state_base, long long slot_stride, int n_slots,
                      const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
                      const float* __restrict__ qk_freq, int rot, const float* __restrict__ v_freq, int interleaved,
                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                      const int* __restrict__ block_table, int bt_stride, int num_pages, int page_size,
                      int nh, int nkv, int hd, int vd, const float* __restrict__ q_mult, int* __restrict__ err) {
    extern __shared__ float sm[];
    const int Cq = nh * hd, Ck = nkv * hd, Cv = nkv * vd, C = Cq + Ck + Cv;
    float* buf = sm;                       // [C]
    float* cq = buf + C;                   // [rot/2] cos, then [rot/2] sin
    float* sq = cq + rot / 2;
    float* cvv = sq + rot / 2;             // [vd/2] cos, then [vd/2] sin (values; only where v_freq is given)
    float* svv = cvv + vd / 2;
    __shared__ float scratch[32];
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t], b = seq_of_token[t], start = cu_seqlens[b];
    for (int p = threadIdx.x; p < rot / 2; p += blockDim.x)
        split_sincos((float)pos, qk_freq[2 * p], qk_freq[2 * p + 1], &cq[p], &sq[p]);
    if (v_freq)
        for (int p = threadIdx.x; p < vd / 2; p += blockDim.x)
            split_sincos((float)pos, v_freq[2 * p], v_freq[2 * p + 1], &cvv[p], &svv[p]);
    int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); slot = 0; }
    cv.state = state_base + (size_t)slot * slot_stride;
    const int page = block_table[(size_t)b * bt_stride + pos / page_size];
    const bool page_ok = page >= 0 && page < num_pages;
    if (!page_ok && threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_PAGE);
    pdl_wait();
    for (int c = threadIdx.x; c < C; c += blockDim.x) buf[c] = conv_taps_at(cv, t, start, c);
    __syncthreads();
    if (q_norm_w) {
        float s1 = 0.f, s2 = 0.f;
        for (int c = threadIdx.x; c < Cq; c += blockDim.x) s1 = fmaf(buf[c], buf[c], s1);
        for (int c = threadIdx.x; c < Ck; c += blockDim.x) s2 = fmaf(buf[Cq + c], buf[Cq + c], s2);
        s1 = block_sum(s1, scratch);
        s2 = block_sum(s2, scratch);
        const float rq = 1.f / sqrtf(s1 / (float)Cq + eps), rk = 1.f / sqrtf(s2 / (float)Ck + eps);
        for (int c = threadIdx.x; c < Cq; c += blockDim.x) buf[c] *= rq * q_norm_w[c];
        for (int c = threadIdx.x; c < Ck; c += blockDim.x) buf[Cq + c] *= rk * k_norm_w[c];
        __syncthreads();
    }
    const int half = rot / 2;
    for (int idx = threadIdx.x; idx < (nh + nkv) * half; idx += blockDim.x) {
        const int head = idx / half, i = idx % half;
        float* x = buf + head * hd;        // q heads, then k heads, all hd wide
        const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
        const float u = x[i0], v = x[i1];
        x[i0] = u * cq[i] - v * sq[i];
        x[i1] = v * cq[i] + u * sq[i];
    }
    if (v_freq) {
        const int vhalf = vd / 2;
        for (int idx = threadIdx.x; idx < nkv * vhalf; idx += blockDim.x) {
            const int head = idx / vhalf, m = idx % vhalf;
            float* x = buf + Cq + Ck + head * vd;
            const int i0 = interleaved ? 2 * m : m, i1 = interleaved ? 2 * m + 1 : m + vhalf;
            const float u = x[i0], v = x[i1];
            x[i0] = u * cvv[m] - v * svv[m];
            x[i1] = v * cvv[m] + u * svv[m];
        }
    }
    __syncthreads();
    // q_mult: one factor per query head (a learned temperature of the head's scores), applied in 32-bit
    for (int c = threadIdx.x; c < Cq; c += blockDim.x) q_out[(size_t)t * Cq + c] = from_float<TA>(q_mult ? buf[c] * q_mult[c / hd] : buf[c]);
    if (page_ok) {
        const int in_page = pos % page_size;
        for (int c = threadIdx.x; c < Ck; c += blockDim.x) {
            const int head = c / hd, i = c % hd;
            k_pool[(((size_t)page * nkv + head) * page_size + in_page) * hd + i] = from_float<TA>(buf[Cq + c]);
        }
        for (int c = threadIdx.x; c < Cv; c += blockDim.x) {
            const int head = c / vd, i = c % vd;
            v_pool[(((size_t)page * nkv + head) * page_size + in_page) * vd + i] = from_float<TA>(buf[Cq + Ck + c]);
        }
    }
}

// proj [T, ld] 32-bit: q (nh x hd), k (nkv x hd), v (nkv x vd) from col0 on; bias, taps [C, n_taps] and the state
// [slots][n_taps - 1][C] follow the same order of channels. q_norm_w / k_norm_w: null for no norm. qk_freq [rot/2][2],
// v_freq [vd/2][2] (null: values are not rotated). q_mult [nh]: a factor per query head (null: none). q_out [T, nh * hd]; pools [page][kv head][slot in page][hd | vd].
CELLM_API int cellm_sink_attn_prep(void* q_out, void* k_pool, void* v_pool, const float* proj, long long ld, int col0,
                                   const float* bias, const float* taps, int n_taps, const float* state, long long slot_stride,
                                   int n_slots, const float* q_norm_w, const float* k_norm_w, float eps, const float* qk_freq,
                                   int rot, const float* v_freq, int interleaved, const int* positions, const int* seq_of_token,
                                   const int* cu_seqlens, const int* slot_ids, const int* block_table, int bt_stride,
                                   int num_pages, int page_size, int T, int nh, int nkv, int hd, int vd, const float* q_mult,
                                   int dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || vd <= 0 || rot < 0 || rot > hd || rot % 2 || (v_freq && vd % 2) ||
        n_taps > CONV_TAPS_MAX || page_size <= 0)
        return CELLM_ERR_SIZE;
    if ((n_taps > 1 && !state) || (rot > 0 && !qk_freq) || (!q_norm_w != !k_norm_w)) return CELLM_ERR_ARG;
    ConvTaps cv;
    cv.proj = proj; cv.ld = ld; cv.col0 = col0; cv.bias = bias; cv.taps = taps; cv.state = nullptr; cv.n_taps = n_taps;
    cv.C = nh * hd + nkv * hd + nkv * vd;
    const size_t smem = (size_t)(cv.C + rot + vd) * sizeof(float);
    if (smem > 200 * 1024) return CELLM_ERR_SIZE;
    // few tokens: a thread about four channels, since a step of single tokens is too few blocks to hide a thread's chain
    // of loads behind other blocks (the sums of squares are then added in another order: a rounding apart)
    const int threads = T >= 512 ? 256 : cv.C >= 4096 ? 1024 : cv.C >= 2048 ? 512 : 256;
#define PREP_RUN(TA)                                                                                                          \
    do {                                                                                                                      \
        if (smem > 48 * 1024) {                                                                                               \
            cudaError_t e = cudaFuncSetAttribute(sink_attn_prep_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                              \
        }                                                                                                                     \
        CELLM_RUN(sink_attn_prep_kernel<TA>, T, threads, smem, stream, (TA*)q_out, (TA*)k_pool, (TA*)v_pool, cv, state, slot_stride, \
                  n_slots, q_norm_w, k_norm_w, eps, qk_freq, rot, v_freq, interleaved, positions, seq_of_token, cu_seqlens, \
                  slot_ids, block_table, bt_stride, num_pages, page_size, nh, nkv, hd, vd, q_mult, err);                             \
    } while (0)
    if (dtype == CELLM_F32) PREP_RUN(float);
    else if (dtype == CELLM_BF16) PREP_RUN(__nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef PREP_RUN
    return CELLM_OK;
}
