// Plain attention over the paged cache: one block per (token, head), every
// earlier key of the request (or the last `window` of them) read through the
// block table. It serves the 32-bit path and is the reference for the faster
// attention kernels.
//
// For head h the key/value head is h / (nh / nkv); scores are q.k * scale;
// softmax takes the maximum off first; all of it in 32-bit
// (crates/cellm-cache/src/kvcache.rs:753-787, :1206-1227). Keys are walked in
// chunks that start at multiples of the chunk size counted from key 0, so the
// order of every sum depends only on the token's position, never on how the
// sequence was cut into steps or what else is in the batch.
//
// Cache layout of one layer: [page][kv_head][slot in page][head_dim].
#include "common.cuh"

#define ATTN_PLAIN_THREADS 128
#define ATTN_PLAIN_MAX_HD 2048

template <typename TA>
__global__ void __launch_bounds__(ATTN_PLAIN_THREADS)
attention_plain_kernel(TA* __restrict__ out, const TA* __restrict__ q, const TA* __restrict__ k_pool,
                       const TA* __restrict__ v_pool, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                       int bt_stride, int num_pages, int page_size, int nh, int nkv, int hd, int hdv, int v_row, float scale,
                       int window, const float* __restrict__ sinks, const float* __restrict__ unrot, int interleaved,
                       int keep_first, float fixed_sink, int has_fixed_sink, const float* __restrict__ gate, long long gate_ld,
                       int* __restrict__ err) {
    constexpr int CH = ATTN_PLAIN_THREADS;
    extern __shared__ float smem[];
    float* qs = smem;             // [hd]
    float* sc = smem + hd;        // [CH]
    int* pg = (int*)(sc + CH);    // [CH] page of each key in the chunk
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x / nh, h = blockIdx.x % nh;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int b = seq_of_token[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < hd; i += CH) qs[i] = to_float(q[(size_t)t * nh * hd + (size_t)h * hd + i]) * scale;
    float m = -INFINITY, l = 0.f;
    float acc[ATTN_PLAIN_MAX_HD / CH];
#pragma unroll
    for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) acc[r] = 0.f;
    const size_t page_elems = (size_t)nkv * page_size * hd, v_page_elems = (size_t)nkv * page_size * v_row;
    // with `keep_first` the first keys of the sequence stay visible behind the window: chunks are walked from key 0
    // and those that hold neither a kept key nor a key of the window are passed over
    for (int c0 = keep_first > 0 ? 0 : (lo / CH) * CH; c0 <= pos; c0 += CH) {
        if (c0 >= keep_first && c0 + CH <= lo) continue;
        __syncthreads();
        {   // page of key c0 + tid
            const int j = c0 + threadIdx.x;
            int p = -1;
            if ((j >= lo || j < keep_first) && j <= pos) {
                p = block_table[(size_t)b * bt_stride + j / page_size];
                if (p < 0 || p >= num_pages) { atomicOr(err, CELLM_DEV_BAD_PAGE); p = -1; }
            }
            pg[threadIdx.x] = p;
        }
        __syncthreads();
        for (int jj = warp; jj < CH; jj += CH / 32) {
            const int p = pg[jj];
            float s = -INFINITY;
            if (p >= 0) {
                const int j = c0 + jj;
                const TA* kr = k_pool + (size_t)p * page_elems + ((size_t)kvh * page_size + j % page_size) * hd;
                float d = 0.f;
                for (int i = lane; i < hd; i += 32) d += qs[i] * to_float(kr[i]);
                s = warp_sum(d);
            }
            if (lane == 0) sc[jj] = s;
        }
        __syncthreads();
        const float cmax = block_max(sc[threadIdx.x], scratch);
        const float m_new = fmaxf(m, cmax);
        const float s = sc[threadIdx.x];
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float psum = block_sum(p, scratch);
        __syncthreads();
        sc[threadIdx.x] = p;
        __syncthreads();
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + psum;
        m = m_new;
#pragma unroll
        for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) {
            const int d = threadIdx.x + r * CH;
            if (d < hdv) {
                float a = acc[r] * corr;
                for (int jj = 0; jj < CH; ++jj) {
                    const int pgj = pg[jj];
                    if (pgj < 0) continue;
                    const int j = c0 + jj;
                    a += sc[jj] * to_float(v_pool[(size_t)pgj * v_page_elems + ((size_t)kvh * page_size + j % page_size) * v_row + d]);
                }
                acc[r] = a;
            }
        }
    }
    if (sinks || has_fixed_sink) {
        // a sink: one more term exp(sink_h) in the denominator, with no key and no value (learned per head, or one
        // fixed score for all heads)
        const float sk = sinks ? sinks[h] : fixed_sink;
        const float m_new = fmaxf(m, sk);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) acc[r] *= corr;
    }
    // an output gate: the head's sum times sigmoid of one number per (token, head)
    const float inv = (gate ? 1.f / (1.f + expf(-gate[(size_t)t * gate_ld + h])) : 1.f) / l;
    if (unrot) {
        // values were cached rotated by their own positions: the sum is turned back by the token's position
        // (pair m by -pos * f_m; f as [hdv/2][2] floats, high part and remainder)
        float* ov = smem;                   // the queries are not needed any more
        __syncthreads();
#pragma unroll
        for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) {
            const int d = threadIdx.x + r * CH;
            if (d < hdv) ov[d] = acc[r] * inv;
        }
        __syncthreads();
        const int half = hdv / 2;
        for (int mm = threadIdx.x; mm < half; mm += CH) {
            const float hi = unrot[2 * mm], lo = unrot[2 * mm + 1], fp = (float)pos;
            const float a = fp * hi;
            const float e = fmaf(fp, hi, -a) + fp * lo;
            float sn, cs, se, ce;
            sincosf(a, &sn, &cs);
            sincosf(e, &se, &ce);
            const float c = cs * ce - sn * se, s = sn * ce + cs * se;
            const int i0 = interleaved ? 2 * mm : mm, i1 = interleaved ? 2 * mm + 1 : mm + half;
            const float u = ov[i0], v = ov[i1];
            out[(size_t)t * nh * hdv + (size_t)h * hdv + i0] = from_float<TA>(u * c + v * s);
            out[(size_t)t * nh * hdv + (size_t)h * hdv + i1] = from_float<TA>(v * c - u * s);
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < ATTN_PLAIN_MAX_HD / CH; ++r) {
        const int d = threadIdx.x + r * CH;
        if (d < hdv) out[(size_t)t * nh * hdv + (size_t)h * hdv + d] = from_float<TA>(acc[r] * inv);
    }
}

// q: [T, nh*hd]; out: [T, nh*hdv]; pools: one layer's keys and values; positions[t] is the
// token's place in its request (keys 0..positions[t] are read; the token's own
// key must already be in the cache). Value rows are v_row wide and a value is a row's first hdv entries.
static int attention_plain_impl(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const int* positions, const int* seq_of_token, const int* block_table,
                                int bt_stride, int num_pages, int page_size, int T, int nh, int nkv,
                                int hd, int hdv, int v_row, float scale, int window, int dtype, int* err,
                                cudaStream_t stream, const float* sinks = nullptr, const float* unrot = nullptr,
                                int interleaved = 0, int keep_first = 0, float fixed_sink = 0.f, int has_fixed_sink = 0,
                                const float* gate = nullptr, long long gate_ld = 0) {
    if (T <= 0) return CELLM_OK;
    if (unrot && hdv % 2) return CELLM_ERR_SIZE;
    if (keep_first < 0) return CELLM_ERR_SIZE;
    if (hd > ATTN_PLAIN_MAX_HD || hd <= 0 || hdv <= 0 || hdv > v_row || hdv > ATTN_PLAIN_MAX_HD || nkv <= 0 || nh % nkv) return CELLM_ERR_SIZE;
    // the first hd floats hold the query; the output is turned back in the same place (hdv floats)
    const size_t smem = (size_t)((hd > hdv ? hd : hdv) + 2 * ATTN_PLAIN_THREADS) * sizeof(float);
    const unsigned grid = (unsigned)T * (unsigned)nh;
    if (dtype == CELLM_F32)
        CELLM_RUN(attention_plain_kernel<float>, grid, ATTN_PLAIN_THREADS, smem, stream,
            (float*)out, (const float*)q, (const float*)k_pool, (const float*)v_pool, positions, seq_of_token,
            block_table, bt_stride, num_pages, page_size, nh, nkv, hd, hdv, v_row, scale, window, sinks, unrot, interleaved, keep_first, fixed_sink, has_fixed_sink, gate, gate_ld, err);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(attention_plain_kernel<__nv_bfloat16>, grid, ATTN_PLAIN_THREADS, smem, stream,
            (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, positions, seq_of_token, block_table, bt_stride, num_pages,
            page_size, nh, nkv, hd, hdv, v_row, scale, window, sinks, unrot, interleaved, keep_first, fixed_sink, has_fixed_sink, gate, gate_ld, err);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// Values in rows as wide as the keys' (hdv = hd for ordinary attention; hdv < hd with v_pool = k_pool for a cache
// whose rows serve as keys and, in their first part, as values).
CELLM_API int cellm_attention_plain(void* out, const void* q, const void* k_pool, const void* v_pool,
                                    const int* positions, const int* seq_of_token, const int* block_table,
                                    int bt_stride, int num_pages, int page_size, int T, int nh, int nkv,
                                    int hd, int hdv, float scale, int window, int dtype, int* err,
                                    cudaStream_t stream) {
    if (hdv > hd) return CELLM_ERR_SIZE;
    return attention_plain_impl(out, q, k_pool, v_pool, positions, seq_of_token, block_table, bt_stride, num_pages, page_size, T, nh, nkv,
                                hd, hdv, hd, scale, window, dtype, err, stream);
}

// Values of a width of their own: a pool of values [page][kv_head][slot][hdv] beside the keys' [..][hd].
CELLM_API int cellm_attention_plain_wide(void* out, const void* q, const void* k_pool, const void* v_pool,
                                         const int* positions, const int* seq_of_token, const int* block_table,
                                         int bt_stride, int num_pages, int page_size, int T, int nh, int nkv,
                                         int hd, int hdv, float scale, int window, int dtype, int* err,
                                         cudaStream_t stream) {
    return attention_plain_impl(out, q, k_pool, v_pool, positions, seq_of_token, block_table, bt_stride, num_pages, page_size, T, nh, nkv,
                                hd, hdv, hdv, scale, window, dtype, err, stream);
}

// The same with a learned sink per head in the softmax's denominator (`sinks` [nh], 32-bit; null: none) and with the
// output turned back by the token's position (`unrot` [hdv/2][2]: the values' frequencies; null: values were
// not rotated). Values have rows of their own width hdv.
CELLM_API int cellm_attention_plain_sink(void* out, const void* q, const void* k_pool, const void* v_pool,
                                         const int* positions, const int* seq_of_token, const int* block_table,
                                         int bt_stride, int num_pages, int page_size, int T, int nh, int nkv,
                                         int hd, int hdv, float scale, int window, const float* sinks, const float* unrot,
                                         int interleaved, int dtype, int* err, cudaStream_t stream) {
    return attention_plain_impl(out, q, k_pool, v_pool, positions, seq_of_token, block_table, bt_stride, num_pages, page_size, T, nh, nkv,
                                hd, hdv, hdv, scale, window, dtype, err, stream, sinks, unrot, interleaved);
}

// The general form: a window that keeps the sequence's first `keep_first` keys visible (from position i a key j <= i is visible when
// i - j < window or j < keep_first; window 0: every earlier key), a learned sink per head (`sinks`) or one fixed sink
// score for all heads (`has_fixed_sink`), an output gate (`gate` [T, gate_ld] 32-bit pre-activations, one per head: the
// head's output is multiplied by its sigmoid; null: none), and value rows `v_row` wide of which the first hdv entries are
// the value (v_pool may be k_pool for a cache whose rows serve as both).
CELLM_API int cellm_attention_plain_masked(void* out, const void* q, const void* k_pool, const void* v_pool,
                                           const int* positions, const int* seq_of_token, const int* block_table,
                                           int bt_stride, int num_pages, int page_size, int T, int nh, int nkv,
                                           int hd, int hdv, int v_row, float scale, int window, int keep_first,
                                           const float* sinks, float fixed_sink, int has_fixed_sink, const float* gate,
                                           long long gate_ld, int dtype, int* err, cudaStream_t stream) {
    return attention_plain_impl(out, q, k_pool, v_pool, positions, seq_of_token, block_table, bt_stride, num_pages, page_size, T, nh, nkv,
                                hd, hdv, v_row, scale, window, dtype, err, stream, sinks, nullptr, 0, keep_first, fixed_sink, has_fixed_sink,
                                gate, gate_ld);
}
