// Recurrent mixers whose state is a matrix per head, S [dim, vdim] in 32-bit floats in the request's state slot:
//
//   HGRN2            S <- diag(f) S + (1 - f) v^T                      o = S^T q
//   gated delta rule S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//
// In both, column j of S needs only v_j (and the token's vectors over the rows), so a thread owns a column and a
// warp 32 neighbouring columns of one (request, head); it walks the request's tokens of the step in order, from the
// state the step before left. The walk is the same however the sequence was cut, so the state after a token is
// bit-identical. Everything that enters the recurrence is 32-bit: the projections come as 32-bit sums.
//
// Also here: the update of a short convolution's state (conv_taps.cuh), the preparation of the delta rule's
// inputs (convolution + silu, unit vectors, beta, decays), and the norm over a head's output with an optional gate.
#include "conv_taps.cuh"

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

// ------------------------------------------------------------------------------------------------ conv state
// New state of request b: the last taps - 1 rows of (old state ‖ the portion's projected values). One thread a
// channel: it reads what it needs before it writes.
__global__ void conv_state_update_kernel(float* __restrict__ state, long long slot_stride, int n_slots,
                                         const int* __restrict__ slot_ids, const int* __restrict__ cu_seqlens,
                                         const float* __restrict__ proj, long long ld, int col0,
                                         const float* __restrict__ bias, int n_taps, int C, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { atomicOr(err, CELLM_DEV_BAD_SLOT); return; }
    const int start = cu_seqlens[b], L = cu_seqlens[b + 1] - start, n = n_taps - 1;
    float* st = state + (size_t)slot * slot_stride;
    const float bc = bias ? bias[c] : 0.f;
    float vals[CONV_TAPS_MAX];
    for (int s = 0; s < n; ++s) {
        const int tp = L - n + s;
        vals[s] = tp >= 0 ? proj[(size_t)(start + tp) * ld + col0 + c] + bc : st[(size_t)(s + L) * C + c];
    }
    for (int s = 0; s < n; ++s) st[(size_t)s * C + c] = vals[s];
}

CELLM_API int cellm_conv_state_update(float* state, long long slot_stride, int n_slots, const int* slot_ids,
                                      const int* cu_seqlens, const float* proj, long long ld, int col0, const float* bias,
                                      int n_taps, int C, int B, int* err, cudaStream_t stream) {
    if (B <= 0 || C <= 0 || n_taps <= 1) return CELLM_OK;
    if (n_taps > CONV_TAPS_MAX) return CELLM_ERR_SIZE;
    CELLM_RUN(conv_state_update_kernel, dim3(B, (C + 127) / 128), 128, 0, stream, state, slot_stride, n_slots, slot_ids,
              cu_seqlens, proj, ld, col0, bias, n_taps, C, err);
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ HGRN2
// proj row: q at col_q (heads x dim), forget gate at col_f (heads x dim), v at col_v (heads x vdim).
// q = silu(.), f = lower + (1 - lower) sigmoid(. + f_bias). o_out [T, heads * vdim] gets S^T q (not normed).
template <int DIM>
__global__ void __launch_bounds__(32)
hgrn2_scan_kernel(float* __restrict__ o_out, float* __restrict__ state, long long slot_stride, int n_slots,
                  const float* __restrict__ proj, long long ld, int col_q, int col_f, int col_v,
                  const float* __restrict__ f_bias, const float* __restrict__ lower,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, int heads, int dim, int vd,
                  int* __restrict__ err) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dim]
    float* fs = sm + dim;           // [dim]
    float* Ssh = sm + 2 * dim;      // [dim][32] when the column does not live in registers
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x, j = blockIdx.z * 32 + lane;
    float Sreg[DIM > 0 ? DIM : 1];
    auto S = [&](int i) -> float& {
        if constexpr (DIM > 0) return Sreg[i];
        else return Ssh[i * 32 + lane];
    };
    const int n_rows = DIM > 0 ? DIM : dim;
    pdl_trigger();
    pdl_wait();
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { if (lane == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); return; }
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    float* st = state + (size_t)slot * slot_stride + (size_t)h * dim * vd;
    const bool live = j < vd;
#pragma unroll
    for (int i = 0; i < n_rows; ++i) S(i) = live ? st[(size_t)i * vd + j] : 0.f;
    for (int t = start; t < end; ++t) {
        const float* row = proj + (size_t)t * ld;
        for (int i = lane; i < dim; i += 32) {
            const float xq = row[col_q + h * dim + i];
            qs[i] = xq * sigmoidf_(xq);
            const float l = lower[h * dim + i];
            fs[i] = l + (1.f - l) * sigmoidf_(row[col_f + h * dim + i] + f_bias[h * dim + i]);
        }
        const float v = live ? row[col_v + h * vd + j] : 0.f;
        __syncwarp();
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < n_rows; ++i) {
            const float f = fs[i];
            const float s = fmaf(f, S(i), (1.f - f) * v);
            S(i) = s;
            o = fmaf(s, qs[i], o);
        }
        if (live) o_out[(size_t)t * heads * vd + (size_t)h * vd + j] = o;
        __syncwarp();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < n_rows; ++i) st[(size_t)i * vd + j] = S(i);
    }
}

#define RECURRENT_MAX_DIM 512

CELLM_API int cellm_hgrn2_scan(float* o_out, float* state, long long slot_stride, int n_slots, const float* proj, long long ld,
                               int col_q, int col_f, int col_v, const float* f_bias, const float* lower,
                               const int* cu_seqlens, const int* slot_ids, int B, int heads, int dim, int vd, int* err,
                               cudaStream_t stream) {
    if (B <= 0) return CELLM_OK;
    if (heads <= 0 || dim <= 0 || vd <= 0 || dim > RECURRENT_MAX_DIM) return CELLM_ERR_SIZE;
    const dim3 grid(B, heads, (vd + 31) / 32);
#define HGRN2_RUN(D, smem)                                                                                         \
    CELLM_RUN(hgrn2_scan_kernel<D>, grid, 32, smem, stream, o_out, state, slot_stride, n_slots, proj, ld, col_q, col_f, col_v, \
              f_bias, lower, cu_seqlens, slot_ids, heads, dim, vd, err)
    const size_t small = (size_t)2 * dim * sizeof(float);
    if (dim == 16) HGRN2_RUN(16, small);
    else if (dim == 32) HGRN2_RUN(32, small);
    else if (dim == 64) HGRN2_RUN(64, small);
    else if (dim == 128) HGRN2_RUN(128, small);
    else {
        const size_t big = (size_t)(2 + 32) * dim * sizeof(float);
        if (big > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(hgrn2_scan_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big);
            if (e != cudaSuccess) return (int)e;
        }
        HGRN2_RUN(0, big);
    }
#undef HGRN2_RUN
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ delta rule: inputs
// One block a token. proj row: q (kvh x dim), k (kvh x dim), v (heads x vdim) from col0 on, side by side (the
// convolution's channels in this order), beta's pre-activation at col_b (heads). a2 [T, heads * dim]: the decay's
// pre-activation without its bias. Writes qk [T, 2 * kvh * dim] (unit q times dim^-1/2, then unit k), v [T, heads * vdim],
// beta [T, heads], decay [T, heads * dim] = exp(-exp(A_log_h) * softplus(a2 + dt_bias)).
__global__ void __launch_bounds__(256)
delta_prep_kernel(float* __restrict__ qk, float* __restrict__ v_out, float* __restrict__ beta, float* __restrict__ decay,
                  ConvTaps cv, long long slot_stride, int n_slots, const float* __restrict__ state_base, int col_b,
                  const float* __restrict__ a2, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                  const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                  int heads, int kvh, int dim, int vd, float l2_eps, int* __restrict__ err) {
    extern __shared__ float buf[];      // [2 * kvh * dim + heads * vd]
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, b = seq_of_token[t], start = cu_seqlens[b];
    int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); slot = 0; }
    cv.state = state_base + (size_t)slot * slot_stride;
    const int Cqk = 2 * kvh * dim, C = cv.C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float y = conv_taps_at(cv, t, start, c);
        buf[c] = y * sigmoidf_(y);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const float q_scale = rsqrtf((float)dim);
    for (int hh = warp; hh < 2 * kvh; hh += nwarps) {
        const float* x = buf + hh * dim;
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float r = (1.f / sqrtf(ss + l2_eps)) * (hh < kvh ? q_scale : 1.f);
        for (int i = lane; i < dim; i += 32) qk[(size_t)t * Cqk + hh * dim + i] = x[i] * r;
    }
    const int Cv = heads * vd;
    for (int c = threadIdx.x; c < Cv; c += blockDim.x) v_out[(size_t)t * Cv + c] = buf[Cqk + c];
    for (int h = threadIdx.x; h < heads; h += blockDim.x)
        beta[(size_t)t * heads + h] = sigmoidf_(cv.proj[(size_t)t * cv.ld + col_b + h]);
    for (int idx = threadIdx.x; idx < heads * dim; idx += blockDim.x) {
        const float x = a2[(size_t)t * heads * dim + idx] + dt_bias[idx];
        const float sp = x > 20.f ? x : log1pf(expf(x));
        decay[(size_t)t * heads * dim + idx] = expf(-expf(A_log[idx / dim]) * sp);
    }
}

CELLM_API int cellm_delta_prep(float* qk, float* v_out, float* beta, float* decay, const float* proj, long long ld, int col0,
                               int col_b, const float* taps, int n_taps, const float* state, long long slot_stride, int n_slots,
                               const float* a2, const float* dt_bias, const float* A_log, const int* seq_of_token,
                               const int* cu_seqlens, const int* slot_ids, int T, int heads, int kvh, int dim, int vd,
                               float l2_eps, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (heads <= 0 || kvh <= 0 || heads % kvh || dim <= 0 || vd <= 0 || n_taps > CONV_TAPS_MAX) return CELLM_ERR_SIZE;
    if (n_taps > 1 && !state) return CELLM_ERR_ARG;
    ConvTaps cv;
    cv.proj = proj; cv.ld = ld; cv.col0 = col0; cv.bias = nullptr; cv.taps = taps; cv.state = nullptr; cv.n_taps = n_taps;
    cv.C = 2 * kvh * dim + heads * vd;
    const size_t smem = (size_t)cv.C * sizeof(float);
    if (smem > 200 * 1024) return CELLM_ERR_SIZE;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    CELLM_RUN(delta_prep_kernel, T, 256, smem, stream, qk, v_out, beta, decay, cv, slot_stride, n_slots, state, col_b, a2, dt_bias,
              A_log, seq_of_token, cu_seqlens, slot_ids, heads, kvh, dim, vd, l2_eps, err);
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ delta rule: the walk
// qk [T, 2 * kvh * dim], v [T, heads * vd], beta [T, heads], decay [T, heads * dim] as delta_prep left them.
template <int DIM>
__global__ void __launch_bounds__(32)
delta_scan_kernel(float* __restrict__ o_out, float* __restrict__ state, long long slot_stride, int n_slots,
                  const float* __restrict__ qk, const float* __restrict__ v_in, const float* __restrict__ beta,
                  const float* __restrict__ decay, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                  int heads, int kvh, int dim, int vd, int* __restrict__ err) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dim]
    float* ks = sm + dim;           // [dim]
    float* gs = sm + 2 * dim;       // [dim]
    float* Ssh = sm + 3 * dim;      // [dim][32] when the column does not live in registers
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x, j = blockIdx.z * 32 + lane;
    const int g = h / (heads / kvh);
    float Sreg[DIM > 0 ? DIM : 1];
    auto S = [&](int i) -> float& {
        if constexpr (DIM > 0) return Sreg[i];
        else return Ssh[i * 32 + lane];
    };
    const int n_rows = DIM > 0 ? DIM : dim;
    pdl_trigger();
    pdl_wait();
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { if (lane == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); return; }
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    float* st = state + (size_t)slot * slot_stride + (size_t)h * dim * vd;
    const bool live = j < vd;
#pragma unroll
    for (int i = 0; i < n_rows; ++i) S(i) = live ? st[(size_t)i * vd + j] : 0.f;
    const int Cqk = 2 * kvh * dim;
    for (int t = start; t < end; ++t) {
        for (int i = lane; i < dim; i += 32) {
            qs[i] = qk[(size_t)t * Cqk + g * dim + i];
            ks[i] = qk[(size_t)t * Cqk + (kvh + g) * dim + i];
            gs[i] = decay[(size_t)t * heads * dim + h * dim + i];
        }
        const float v = live ? v_in[(size_t)t * heads * vd + h * vd + j] : 0.f;
        const float bt = beta[(size_t)t * heads + h];
        __syncwarp();
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < n_rows; ++i) {
            const float s = S(i) * gs[i];
            S(i) = s;
            acc = fmaf(s, ks[i], acc);
        }
        const float u = bt * (v - acc);
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < n_rows; ++i) {
            const float s = fmaf(ks[i], u, S(i));
            S(i) = s;
            o = fmaf(s, qs[i], o);
        }
        if (live) o_out[(size_t)t * heads * vd + (size_t)h * vd + j] = o;
        __syncwarp();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < n_rows; ++i) st[(size_t)i * vd + j] = S(i);
    }
}

CELLM_API int cellm_delta_scan(float* o_out, float* state, long long slot_stride, int n_slots, const float* qk, const float* v_in,
                               const float* beta, const float* decay, const int* cu_seqlens, const int* slot_ids, int B,
                               int heads, int kvh, int dim, int vd, int* err, cudaStream_t stream) {
    if (B <= 0) return CELLM_OK;
    if (heads <= 0 || kvh <= 0 || heads % kvh || dim <= 0 || vd <= 0 || dim > RECURRENT_MAX_DIM) return CELLM_ERR_SIZE;
    const dim3 grid(B, heads, (vd + 31) / 32);
#define DELTA_RUN(D, smem)                                                                                           \
    CELLM_RUN(delta_scan_kernel<D>, grid, 32, smem, stream, o_out, state, slot_stride, n_slots, qk, v_in, beta, decay, cu_seqlens, \
              slot_ids, heads, kvh, dim, vd, err)
    const size_t small = (size_t)3 * dim * sizeof(float);
    if (dim == 16) DELTA_RUN(16, small);
    else if (dim == 32) DELTA_RUN(32, small);
    else if (dim == 64) DELTA_RUN(64, small);
    else if (dim == 128) DELTA_RUN(128, small);
    else {
        const size_t big = (size_t)(3 + 32) * dim * sizeof(float);
        if (big > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big);
            if (e != cudaSuccess) return (int)e;
        }
        DELTA_RUN(0, big);
    }
#undef DELTA_RUN
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ norm over a head's output
// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w[:] (* sigmoid(gate[t, h, :])): a warp a (token, head).
template <typename TA>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(TA* __restrict__ out, const float* __restrict__ o, const float* __restrict__ w,
                      const float* __restrict__ gate, long long gate_ld, int n_rows, int heads, int vd, float eps) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const float* x = o + (size_t)r * vd;
    float ss = 0.f;
    for (int j = lane; j < vd; j += 32) ss = fmaf(x[j], x[j], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)vd + eps);
    const int t = r / heads, h = r % heads;
    for (int j = lane; j < vd; j += 32) {
        float y = x[j] * inv * w[j];
        if (gate) y *= sigmoidf_(gate[(size_t)t * gate_ld + (size_t)h * vd + j]);
        out[(size_t)r * vd + j] = from_float<TA>(y);
    }
}

CELLM_API int cellm_head_norm_gate(void* out, const float* o, const float* w, const float* gate, long long gate_ld, int T,
                                   int heads, int vd, float eps, int dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (heads <= 0 || vd <= 0) return CELLM_ERR_SIZE;
    const int n_rows = T * heads;
    const unsigned blocks = (unsigned)((n_rows + 7) / 8);
    if (dtype == CELLM_F32)
        CELLM_RUN(head_norm_gate_kernel<float>, blocks, 256, 0, stream, (float*)out, o, w, gate, gate_ld, n_rows, heads, vd, eps);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(head_norm_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, o, w, gate, gate_ld, n_rows, heads, vd, eps);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
