// Embedding: out[t, :] = float(table[ids[t], :]) * scale into the 32-bit residual stream
// (scale = 1 for a plain look-up; some designs multiply the row by a constant).
// The reference gathers one row per token and refuses an id beyond the
// vocabulary (crates/cellm-model/src/lfm.rs:817-890). Here a bad id sets a bit
// in the device error word and its row is written as zeros.
#include "common.cuh"

// With a table of learned position vectors, out[t, :] += float(pos_table[positions[t], :]) (not scaled); a
// position beyond the table sets the same error bit and adds nothing.
template <typename T>
__global__ void embed_pos_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                 const T* __restrict__ pos_table, const int* __restrict__ positions, int max_pos, int H, int V,
                                 float scale, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t], pos = positions[t];
    const bool ok = id >= 0 && id < V, pos_ok = pos >= 0 && pos < max_pos;
    if ((!ok || !pos_ok) && threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_TOKEN);
    const T* row = table + (size_t)(ok ? id : 0) * H;
    const T* prow = pos_table + (size_t)(pos_ok ? pos : 0) * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = (ok ? to_float(row[i]) * scale : 0.f) + (pos_ok ? to_float(prow[i]) : 0.f);
}

template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int H, int V, float scale, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_TOKEN);
    const T* row = table + (size_t)(ok ? id : 0) * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? to_float(row[i]) * scale : 0.f;
}

// The step's index arrays go up in one asynchronous copy from pinned host memory (a plain call of the runtime,
// here so that the step function pays one short foreign call for it instead of a tensor operation).
CELLM_API int cellm_upload(void* dst, const void* pinned_src, long long bytes, cudaStream_t stream) {
    if (bytes <= 0) return CELLM_OK;
    const cudaError_t e = cudaMemcpyAsync(dst, pinned_src, (size_t)bytes, cudaMemcpyHostToDevice, stream);
    return e == cudaSuccess ? CELLM_OK : (int)e;
}

// The embedding is the first kernel of a forward pass: it is launched without the attribute that lets a kernel
// start under its predecessor (see common.cuh), so that no kernel of this pass overlaps the pass before it.
CELLM_API int cellm_embed(float* out, const void* table, int table_dtype, const int* ids, int T, int H,
                          int V, float scale, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == CELLM_F32)
        CELLM_RUN_SERIAL(embed_kernel<float>, T, threads, 0, stream, out, (const float*)table, ids, H, V, scale, err);
    else if (table_dtype == CELLM_BF16)
        CELLM_RUN_SERIAL(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, out, (const __nv_bfloat16*)table, ids, H, V, scale, err);
    else
        return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// The same with learned position vectors added: pos_table [max_pos, H] of the table's element type.
CELLM_API int cellm_embed_pos(float* out, const void* table, int table_dtype, const int* ids, const void* pos_table,
                              const int* positions, int max_pos, int T, int H, int V, float scale, int* err,
                              cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (!pos_table || !positions || max_pos < 1) return CELLM_ERR_ARG;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == CELLM_F32)
        CELLM_RUN_SERIAL(embed_pos_kernel<float>, T, threads, 0, stream, out, (const float*)table, ids, (const float*)pos_table,
                         positions, max_pos, H, V, scale, err);
    else if (table_dtype == CELLM_BF16)
        CELLM_RUN_SERIAL(embed_pos_kernel<__nv_bfloat16>, T, threads, 0, stream, out, (const __nv_bfloat16*)table, ids,
                         (const __nv_bfloat16*)pos_table, positions, max_pos, H, V, scale, err);
    else
        return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// With a hashed table of token pairs: out[t, :] += float(pair_table[row, :]) (not scaled), where row =
// (previous token * mul_prev + token * mul_cur) mod buckets, and the table's last row (number `buckets`) for a
// sequence's first token. The previous token of a portion's first token is the request's state (one int32 a slot),
// which the block of that token reads and then sets to the portion's last token.
template <typename T>
__global__ void embed_pairs_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                   const T* __restrict__ pair_table, long long buckets, long long mul_prev, long long mul_cur,
                                   int* __restrict__ prev_state, long long slot_stride, int n_slots,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, int H, int V,
                                   float scale, int* __restrict__ err) {
    __shared__ int prev_s;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t], pos = positions[t], b = seq_of_token[t], start = cu_seqlens[b];
    if (threadIdx.x == 0) {
        int prev = -1;
        if (t > start) prev = ids[t - 1];
        else {
            const int slot = slot_ids[b];
            if (slot < 0 || slot >= n_slots) atomicOr(err, CELLM_DEV_BAD_SLOT);
            else {
                int* st = prev_state + (size_t)slot * slot_stride;
                prev = st[0];
                st[0] = ids[cu_seqlens[b + 1] - 1];
            }
        }
        prev_s = prev;
    }
    __syncthreads();
    const int prev = prev_s;
    const bool ok = id >= 0 && id < V && (pos == 0 || (prev >= 0 && prev < V));
    if (!ok && threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_TOKEN);
    const long long prow = pos == 0 ? buckets : ((long long)(ok ? prev : 0) * mul_prev + (long long)(ok ? id : 0) * mul_cur) % buckets;
    const T* row = table + (size_t)(ok ? id : 0) * H;
    const T* pr = pair_table + (size_t)prow * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? fmaf(to_float(row[i]), scale, to_float(pr[i])) : 0.f;
}

// pair_table [buckets + 1, H] of the table's element type; prev_state: one int32 a slot (slot_stride in elements).
CELLM_API int cellm_embed_pairs(float* out, const void* table, int table_dtype, const int* ids, const void* pair_table,
                                long long buckets, long long mul_prev, long long mul_cur, int* prev_state, long long slot_stride,
                                int n_slots, const int* positions, const int* seq_of_token, const int* cu_seqlens,
                                const int* slot_ids, int T, int H, int V, float scale, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (!pair_table || !prev_state || buckets < 1 || mul_prev < 0 || mul_cur < 0) return CELLM_ERR_ARG;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == CELLM_F32)
        CELLM_RUN_SERIAL(embed_pairs_kernel<float>, T, threads, 0, stream, out, (const float*)table, ids, (const float*)pair_table,
                         buckets, mul_prev, mul_cur, prev_state, slot_stride, n_slots, positions, seq_of_token, cu_seqlens, slot_ids,
                         H, V, scale, err);
    else if (table_dtype == CELLM_BF16)
        CELLM_RUN_SERIAL(embed_pairs_kernel<__nv_bfloat16>, T, threads, 0, stream, out, (const __nv_bfloat16*)table, ids,
                         (const __nv_bfloat16*)pair_table, buckets, mul_prev, mul_cur, prev_state, slot_stride, n_slots, positions,
                         seq_of_token, cu_seqlens, slot_ids, H, V, scale, err);
    else
        return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
