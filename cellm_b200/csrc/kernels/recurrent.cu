// Recurrent mixers whose state is a matrix per head, S [dim, vdim] in 32-bit floats in the request's state slot:
//
//   HGRN2            S <- diag(f) S + (1 - f) v^T                      o = S^T q
//   gated delta rule S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   generalized delta rule   S <- diag(d) S - (a * u)(u^T S) + k v^T (the old S on the right)   o = S^T r
//
// In both, column j of S needs only v_j (and the token's vectors over the rows), so the columns are independent: a
// block walks some neighbouring columns of one (request, head) through the request's tokens of the step in order,
// from the state the step before left. The walk and the order of every sum depend on the head's sizes alone, not on
// how the sequence was cut, so the state after a token is bit-identical. Everything that enters the recurrence is
// 32-bit: the projections come as 32-bit sums. Heads of more than 128 rows keep a warp's 32 columns in shared memory
// (`*_scan_kernel`); the others live in registers (`state_walk_kernel`).
//
// Also here: the update of a short convolution's state (conv_taps.cuh), the preparation of the delta rule's
// inputs (convolution + silu, unit vectors, beta, decays), and the norm over a head's output with an optional gate.
#include <algorithm>

#include "conv_taps.cuh"

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

// ------------------------------------------------------------------------------------------------ the walk
// Heads of up to 128 rows. The walk is a chain of dependent steps, token after token, and a head's state is small: one
// request's walk is bound by the chain's latency, many requests' walks by the instructions issued. A column of S is
// shared by DIM / ROWS neighbouring lanes, each holding ROWS of its rows in registers (the delta rule: eight for heads
// of 64 and 128 rows, since every token's u waits for a sum over the lanes; HGRN2, whose state waits for no sum: four;
// measured), in groups of four dealt round robin to the lanes, so that the lanes' 16-byte reads of the token's vectors
// in shared memory are neighbours. A block of eight warps walks 256 / (DIM / ROWS) neighbouring columns of one (request, head).
// The tokens' vectors over the rows, the block's entries of v and beta come in chunks of eight tokens through
// asynchronous copies into three stages of shared memory, two chunks ahead of the one in use: a chunk costs one
// barrier and no wait for memory, and within a chunk the warps run free. Sums over a column's rows are added lane by
// lane (shuffles) in a fixed order; the read-outs of a whole chunk's tokens wait as the lanes' shares and are summed
// together, step by step, so that a shuffle's latency is paid once a chunk (the same sums in the same order as token
// by token). The block's tile of S goes through shared memory on its way in and out, in rows of whole sectors.
// DIM is the next of 16, 32, 64, 128 above the head's rows; the rows beyond are zeros that nothing reads back.
template <int DIM, int ROWS> struct WalkShape {
    static constexpr int RG = DIM / ROWS;          // lanes a column
    static constexpr int CPW = 32 / RG;            // columns a warp
    static constexpr int CPB = 8 * CPW;            // columns a block
};
#define WALK_THREADS 256
#define WALK_CHUNK 8
#define WALK_STAGES 3

template <int RG> __device__ __forceinline__ float sum_over_rows(float x) {
#pragma unroll
    for (int d = 1; d < RG; d <<= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
    return x;
}

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Where the vectors over a head's rows lie: array a of token t and head h starts at p[a] + t * ld[a] + (h / heads_per[a]) * dim.
// Delta rule: q, k, decay. HGRN2: q, f. Generalized delta rule: r, k, decay, unit key, removal rate times unit key.
struct WalkVectors {
    const float* p[5];
    long long ld[5];
    int heads_per[5];
    int vec16;          // every start is a multiple of 16 bytes: copies of four values
};

// MODE 0: HGRN2; 1: the gated delta rule; 2: the generalized delta rule (five vectors a token: chunks of four tokens for
// heads of 128 rows, so that three stages stay within the static shared memory).
template <int DIM, int ROWS, int MODE>
__global__ void __launch_bounds__(WALK_THREADS)
state_walk_kernel(float* __restrict__ o_out, float* __restrict__ state, long long slot_stride, int n_slots, const WalkVectors vec,
                  const float* __restrict__ v_in, long long ld_v, const float* __restrict__ beta,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, int heads, int dim, int vd,
                  int* __restrict__ err) {
    using W = WalkShape<DIM, ROWS>;
    constexpr bool DELTA = MODE == 1;
    constexpr int RG = W::RG, CPB = W::CPB, NV = MODE == 2 ? 5 : (DELTA ? 3 : 2), NG = ROWS / 4;
    constexpr int CHUNK = (MODE == 2 && DIM > 64) ? 4 : WALK_CHUNK;
    constexpr int TOK = NV * DIM + CPB + 4;          // a token in a stage: its vectors | the block's entries of v | beta
    __shared__ __align__(16) float buf[WALK_STAGES][CHUNK * TOK];
    __shared__ float tile[DIM][CPB + 1];             // the block's columns of S on their way in and out
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane % RG, cl = warp * W::CPW + lane / RG, col0 = blockIdx.z * CPB, j = col0 + cl;
    pdl_trigger();
    pdl_wait();
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { if (tid == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); return; }
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    if (end <= start) return;
    float* st = state + (size_t)slot * slot_stride + (size_t)h * dim * vd;
    const bool live = j < vd;
    if (dim < DIM) {            // the rows beyond the head's own stay zero in every stage
        for (int i = tid; i < WALK_STAGES * CHUNK * TOK; i += WALK_THREADS) (&buf[0][0])[i] = 0.f;
        __syncthreads();
    }
    const int n_chunks = (end - start + CHUNK - 1) / CHUNK;
    auto issue = [&](int c) {
        float* dst = buf[c % WALK_STAGES];
        const int t0 = start + c * CHUNK, nt = min(CHUNK, end - t0);
#pragma unroll
        for (int a = 0; a < NV; ++a) {
            const float* src = vec.p[a] + (size_t)t0 * vec.ld[a] + (h / vec.heads_per[a]) * dim;
            if (vec.vec16) {
                for (int idx = tid; idx < nt * (DIM / 4); idx += WALK_THREADS) {
                    const int i = (idx % (DIM / 4)) * 4, tt = idx / (DIM / 4);
                    if (i < dim) copy_async16(dst + tt * TOK + a * DIM + i, src + (size_t)tt * vec.ld[a] + i);
                }
            } else {
                for (int idx = tid; idx < nt * DIM; idx += WALK_THREADS) {
                    const int i = idx % DIM, tt = idx / DIM;
                    if (i < dim) copy_async4(dst + tt * TOK + a * DIM + i, src + (size_t)tt * vec.ld[a] + i);
                }
            }
        }
        for (int idx = tid; idx < nt * CPB; idx += WALK_THREADS) {
            const int c_ = idx % CPB, tt = idx / CPB;
            if (col0 + c_ < vd) copy_async4(dst + tt * TOK + NV * DIM + c_, v_in + (size_t)(t0 + tt) * ld_v + h * vd + col0 + c_);
        }
        if (DELTA && tid < nt) copy_async4(dst + tid * TOK + NV * DIM + CPB, beta + (size_t)(t0 + tid) * heads + h);
    };
#pragma unroll
    for (int c = 0; c < WALK_STAGES - 1; ++c) {
        if (c < n_chunks) issue(c);
        copy_async_commit();
    }
    for (int idx = tid; idx < DIM * CPB; idx += WALK_THREADS) {
        const int row = idx / CPB, c_ = idx % CPB;
        tile[row][c_] = (row < dim && col0 + c_ < vd) ? st[(size_t)row * vd + col0 + c_] : 0.f;
    }
    __syncthreads();
    // the lane's rows: groups of four, group g at rows (g * RG + r) * 4 ..
    float S[ROWS];
#pragma unroll
    for (int ii = 0; ii < ROWS; ++ii) S[ii] = tile[((ii >> 2) * RG + r) * 4 + (ii & 3)][cl];
    // one token: the lane's rows of the column move on; returns the lane's share of the column's read-out
    auto token = [&](const float* tok) -> float {
        const float4* q4 = reinterpret_cast<const float4*>(tok);
        const float v = tok[NV * DIM + cl];
        float o0 = 0.f, o1 = 0.f;
        if constexpr (MODE == 2) {
            // S <- diag(d) S - (a u)(u^T S) + k v^T, both terms over the old S: the sum u^T S over the column's rows first
            const float4* k4 = reinterpret_cast<const float4*>(tok + DIM);
            const float4* d4 = reinterpret_cast<const float4*>(tok + 2 * DIM);
            const float4* u4 = reinterpret_cast<const float4*>(tok + 3 * DIM);
            const float4* a4 = reinterpret_cast<const float4*>(tok + 4 * DIM);
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const float4 u = u4[g * RG + r];
                a0 = fmaf(S[4 * g + 0], u.x, a0), a1 = fmaf(S[4 * g + 1], u.y, a1);
                a0 = fmaf(S[4 * g + 2], u.z, a0), a1 = fmaf(S[4 * g + 3], u.w, a1);
            }
            const float dot = -sum_over_rows<RG>(a0 + a1);
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const float4 q = q4[g * RG + r], k = k4[g * RG + r], d = d4[g * RG + r], au = a4[g * RG + r];
                S[4 * g + 0] = fmaf(k.x, v, fmaf(d.x, S[4 * g + 0], au.x * dot)), S[4 * g + 1] = fmaf(k.y, v, fmaf(d.y, S[4 * g + 1], au.y * dot));
                S[4 * g + 2] = fmaf(k.z, v, fmaf(d.z, S[4 * g + 2], au.z * dot)), S[4 * g + 3] = fmaf(k.w, v, fmaf(d.w, S[4 * g + 3], au.w * dot));
                o0 = fmaf(S[4 * g + 0], q.x, o0), o1 = fmaf(S[4 * g + 1], q.y, o1);
                o0 = fmaf(S[4 * g + 2], q.z, o0), o1 = fmaf(S[4 * g + 3], q.w, o1);
            }
        } else if constexpr (DELTA) {
            const float4* k4 = reinterpret_cast<const float4*>(tok + DIM);
            const float4* g4 = reinterpret_cast<const float4*>(tok + 2 * DIM);
            const float bt = tok[NV * DIM + CPB];
            float4 kk[NG];
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const float4 k = k4[g * RG + r], gd = g4[g * RG + r];
                kk[g] = k;
                S[4 * g + 0] *= gd.x, S[4 * g + 1] *= gd.y, S[4 * g + 2] *= gd.z, S[4 * g + 3] *= gd.w;
                a0 = fmaf(S[4 * g + 0], k.x, a0), a1 = fmaf(S[4 * g + 1], k.y, a1);
                a0 = fmaf(S[4 * g + 2], k.z, a0), a1 = fmaf(S[4 * g + 3], k.w, a1);
            }
            const float u = bt * (v - sum_over_rows<RG>(a0 + a1));
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const float4 q = q4[g * RG + r];
                S[4 * g + 0] = fmaf(kk[g].x, u, S[4 * g + 0]), S[4 * g + 1] = fmaf(kk[g].y, u, S[4 * g + 1]);
                S[4 * g + 2] = fmaf(kk[g].z, u, S[4 * g + 2]), S[4 * g + 3] = fmaf(kk[g].w, u, S[4 * g + 3]);
                o0 = fmaf(S[4 * g + 0], q.x, o0), o1 = fmaf(S[4 * g + 1], q.y, o1);
                o0 = fmaf(S[4 * g + 2], q.z, o0), o1 = fmaf(S[4 * g + 3], q.w, o1);
            }
        } else {
            const float4* f4 = reinterpret_cast<const float4*>(tok + DIM);
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const float4 q = q4[g * RG + r], f = f4[g * RG + r];
                S[4 * g + 0] = fmaf(f.x, S[4 * g + 0], (1.f - f.x) * v), S[4 * g + 1] = fmaf(f.y, S[4 * g + 1], (1.f - f.y) * v);
                S[4 * g + 2] = fmaf(f.z, S[4 * g + 2], (1.f - f.z) * v), S[4 * g + 3] = fmaf(f.w, S[4 * g + 3], (1.f - f.w) * v);
                o0 = fmaf(S[4 * g + 0], q.x, o0), o1 = fmaf(S[4 * g + 1], q.y, o1);
                o0 = fmaf(S[4 * g + 2], q.z, o0), o1 = fmaf(S[4 * g + 3], q.w, o1);
            }
        }
        return o0 + o1;
    };
    float* o_col = o_out + (size_t)h * vd + j;
    const size_t o_ld = (size_t)heads * vd;
    for (int c = 0; c < n_chunks; ++c) {
        copy_async_wait<WALK_STAGES - 2>();
        __syncthreads();        // chunk c has arrived for every thread, and every thread has left chunk c - 1
        if (c + WALK_STAGES - 1 < n_chunks) issue(c + WALK_STAGES - 1);
        copy_async_commit();
        const float* stage = buf[c % WALK_STAGES];
        const int t0 = start + c * CHUNK, nt = min(CHUNK, end - t0);
        if (nt == CHUNK) {
            // a whole chunk: the tokens' read-outs wait as the lanes' shares and are summed over the lanes together, step
            // by step, so that a shuffle's latency is paid once a chunk and not once a token (the same sums in the same order)
            float share[CHUNK];
#pragma unroll
            for (int tt = 0; tt < CHUNK; ++tt) share[tt] = token(stage + tt * TOK);
#pragma unroll
            for (int d = 1; d < RG; d <<= 1) {
                float other[CHUNK];
#pragma unroll
                for (int tt = 0; tt < CHUNK; ++tt) other[tt] = __shfl_xor_sync(0xffffffffu, share[tt], d);
#pragma unroll
                for (int tt = 0; tt < CHUNK; ++tt) share[tt] += other[tt];
            }
            if (live && r == 0) {
#pragma unroll
                for (int tt = 0; tt < CHUNK; ++tt) o_col[(size_t)(t0 + tt) * o_ld] = share[tt];
            }
        } else {
            for (int tt = 0; tt < nt; ++tt) {
                const float o = sum_over_rows<RG>(token(stage + tt * TOK));
                if (live && r == 0) o_col[(size_t)(t0 + tt) * o_ld] = o;
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int ii = 0; ii < ROWS; ++ii) tile[((ii >> 2) * RG + r) * 4 + (ii & 3)][cl] = S[ii];
    __syncthreads();
    for (int idx = tid; idx < DIM * CPB; idx += WALK_THREADS) {
        const int row = idx / CPB, c_ = idx % CPB;
        if (row < dim && col0 + c_ < vd) st[(size_t)row * vd + col0 + c_] = tile[row][c_];
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

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
// First, in place and for all tokens at once: q = silu(.), f = lower + (1 - lower) sigmoid(. + f_bias). Then the walk;
// o_out [T, heads * vdim] gets S^T q (not normed).
__global__ void __launch_bounds__(256)
hgrn2_gates_kernel(float* __restrict__ proj, long long ld, int col_q, int col_f, const float* __restrict__ f_bias,
                   const float* __restrict__ lower, int T, int n) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)T * 2 * n;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % (2 * n));
        float* row = proj + (idx / (2 * n)) * ld;
        if (c < n) {
            const float x = row[col_q + c];
            row[col_q + c] = x * sigmoidf_(x);
        } else {
            const int i = c - n;
            const float l = lower[i];
            row[col_f + i] = l + (1.f - l) * sigmoidf_(row[col_f + i] + f_bias[i]);
        }
    }
}

__global__ void __launch_bounds__(32)
hgrn2_scan_kernel(float* __restrict__ o_out, float* __restrict__ state, long long slot_stride, int n_slots,
                  const float* __restrict__ proj, long long ld, int col_q, int col_f, int col_v,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, int heads, int dim, int vd,
                  int* __restrict__ err) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dim]
    float* fs = sm + dim;           // [dim]
    float* Ssh = sm + 2 * dim;      // [dim][32]: the warp's columns of S
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x, j = blockIdx.z * 32 + lane;
    auto S = [&](int i) -> float& { return Ssh[i * 32 + lane]; };
    const int n_rows = dim;
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
            qs[i] = row[col_q + h * dim + i];
            fs[i] = row[col_f + h * dim + i];
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

CELLM_API int cellm_hgrn2_scan(float* o_out, float* state, long long slot_stride, int n_slots, float* proj, long long ld,
                               int col_q, int col_f, int col_v, const float* f_bias, const float* lower,
                               const int* cu_seqlens, const int* slot_ids, int B, int T, int heads, int dim, int vd, int* err,
                               cudaStream_t stream) {
    if (B <= 0 || T <= 0) return CELLM_OK;
    if (heads <= 0 || dim <= 0 || vd <= 0 || dim > RECURRENT_MAX_DIM) return CELLM_ERR_SIZE;
    const size_t total = (size_t)T * 2 * heads * dim;
    CELLM_RUN(hgrn2_gates_kernel, (unsigned)std::min<size_t>((total + 255) / 256, 148 * 16), 256, 0, stream, proj, ld, col_q, col_f, f_bias,
              lower, T, heads * dim);
    WalkVectors vec;
    for (int a = 0; a < 5; ++a) vec.p[a] = nullptr, vec.ld[a] = ld, vec.heads_per[a] = 1;
    vec.p[0] = proj + col_q, vec.p[1] = proj + col_f;
    vec.vec16 = dim % 4 == 0 && ld % 4 == 0 && aligned16(vec.p[0]) && aligned16(vec.p[1]);
#define HGRN2_WALK(D, R)                                                                                           \
    CELLM_RUN((state_walk_kernel<D, R, 0>), dim3(B, heads, (vd + WalkShape<D, R>::CPB - 1) / WalkShape<D, R>::CPB), WALK_THREADS, 0, stream, \
              o_out, state, slot_stride, n_slots, vec, (const float*)(proj + col_v), ld, (const float*)nullptr, cu_seqlens, slot_ids,  \
              heads, dim, vd, err)
    if (dim <= 16) HGRN2_WALK(16, 4);
    else if (dim <= 32) HGRN2_WALK(32, 4);
    else if (dim <= 64) HGRN2_WALK(64, 4);
    else if (dim <= 128) HGRN2_WALK(128, 4);
    else {
        const size_t big = (size_t)(2 + 32) * dim * sizeof(float);
        if (big > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(hgrn2_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big);
            if (e != cudaSuccess) return (int)e;
        }
        CELLM_RUN(hgrn2_scan_kernel, dim3(B, heads, (vd + 31) / 32), 32, big, stream, o_out, state, slot_stride, n_slots,
                  (const float*)proj, ld, col_q, col_f, col_v, cu_seqlens, slot_ids, heads, dim, vd, err);
    }
#undef HGRN2_WALK
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ delta rule: inputs
// A few blocks a token. proj row: q (kvh x dim), k (kvh x dim), v (heads x vdim) from col0 on, side by side (the
// convolution's channels in this order), beta's pre-activation at col_b (heads). a2 [T, heads * dim]: the decay's
// pre-activation without its bias (rows ld_a2 apart). Writes qk [T, 2 * kvh * dim] (unit q times dim^-1/2, then unit k), v [T, heads * vdim],
// beta [T, heads], decay [T, heads * dim] = exp(-exp(A_log_h) * softplus(a2 + dt_bias)).
__global__ void __launch_bounds__(256)
delta_prep_kernel(float* __restrict__ qk, float* __restrict__ v_out, float* __restrict__ beta, float* __restrict__ decay,
                  ConvTaps cv, long long slot_stride, int n_slots, const float* __restrict__ state_base, int col_b,
                  const float* __restrict__ a2, long long ld_a2, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                  const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                  int heads, int kvh, int dim, int vd, float l2_eps, int* __restrict__ err) {
    extern __shared__ float buf[];      // [warps][dim]: a q or k head of the token
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, b = seq_of_token[t], start = cu_seqlens[b];
    int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); slot = 0; }
    cv.state = state_base + (size_t)slot * slot_stride;
    const int Cqk = 2 * kvh * dim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int part = blockIdx.y, parts = gridDim.y, thread = part * blockDim.x + threadIdx.x, threads = parts * blockDim.x;
    // q and k: a warp a head (convolution + silu, then the unit vector); the token's parts share the heads
    const float q_scale = rsqrtf((float)dim);
    float* x = buf + warp * dim;
    for (int hh = part * nwarps + warp; hh < 2 * kvh; hh += parts * nwarps) {
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) {
            const float y = conv_taps_at(cv, t, start, hh * dim + i);
            const float a = y * sigmoidf_(y);
            x[i] = a;
            ss = fmaf(a, a, ss);
        }
        ss = warp_sum(ss);
        const float r = (1.f / sqrtf(ss + l2_eps)) * (hh < kvh ? q_scale : 1.f);
        for (int i = lane; i < dim; i += 32) qk[(size_t)t * Cqk + hh * dim + i] = x[i] * r;     // a lane reads back its own entries
    }
    const int Cv = heads * vd;
    for (int c = thread; c < Cv; c += threads) {
        const float y = conv_taps_at(cv, t, start, Cqk + c);
        v_out[(size_t)t * Cv + c] = y * sigmoidf_(y);
    }
    if (part == 0)
        for (int h = threadIdx.x; h < heads; h += blockDim.x)
            beta[(size_t)t * heads + h] = sigmoidf_(cv.proj[(size_t)t * cv.ld + col_b + h]);
    for (int idx = thread; idx < heads * dim; idx += threads) {
        const float xa = a2[(size_t)t * ld_a2 + idx] + dt_bias[idx];
        const float sp = xa > 20.f ? xa : log1pf(expf(xa));
        decay[(size_t)t * heads * dim + idx] = expf(-expf(A_log[idx / dim]) * sp);
    }
}

CELLM_API int cellm_delta_prep(float* qk, float* v_out, float* beta, float* decay, const float* proj, long long ld, int col0,
                               int col_b, const float* taps, int n_taps, const float* state, long long slot_stride, int n_slots,
                               const float* a2, long long ld_a2, const float* dt_bias, const float* A_log, const int* seq_of_token,
                               const int* cu_seqlens, const int* slot_ids, int T, int heads, int kvh, int dim, int vd,
                               float l2_eps, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (heads <= 0 || kvh <= 0 || heads % kvh || dim <= 0 || vd <= 0 || n_taps > CONV_TAPS_MAX) return CELLM_ERR_SIZE;
    if (n_taps > 1 && !state) return CELLM_ERR_ARG;
    ConvTaps cv;
    cv.proj = proj; cv.ld = ld; cv.col0 = col0; cv.bias = nullptr; cv.taps = taps; cv.state = nullptr; cv.n_taps = n_taps;
    cv.C = 2 * kvh * dim + heads * vd;
    if (dim > RECURRENT_MAX_DIM) return CELLM_ERR_SIZE;
    // few tokens: a token's channels over as many blocks as leave a thread about four of them (no sum crosses blocks)
    const int widest = std::max(cv.C, heads * dim), parts = T >= 512 ? 1 : std::max(1, std::min((widest + 1023) / 1024, 64));
    CELLM_RUN(delta_prep_kernel, dim3(T, parts), 256, (size_t)8 * dim * sizeof(float), stream, qk, v_out, beta, decay, cv, slot_stride,
              n_slots, state, col_b, a2, ld_a2, dt_bias, A_log, seq_of_token, cu_seqlens, slot_ids, heads, kvh, dim, vd, l2_eps, err);
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ delta rule: the walk
// qk [T, 2 * kvh * dim], v [T, heads * vd], beta [T, heads], decay [T, heads * dim] as delta_prep left them.
__global__ void __launch_bounds__(32)
delta_scan_kernel(float* __restrict__ o_out, float* __restrict__ state, long long slot_stride, int n_slots,
                  const float* __restrict__ qk, const float* __restrict__ v_in, const float* __restrict__ beta,
                  const float* __restrict__ decay, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                  int heads, int kvh, int dim, int vd, int* __restrict__ err) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dim]
    float* ks = sm + dim;           // [dim]
    float* gs = sm + 2 * dim;       // [dim]
    float* Ssh = sm + 3 * dim;      // [dim][32]: the warp's columns of S
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x, j = blockIdx.z * 32 + lane;
    const int g = h / (heads / kvh);
    auto S = [&](int i) -> float& { return Ssh[i * 32 + lane]; };
    const int n_rows = dim;
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
    WalkVectors vec;
    for (int a = 0; a < 5; ++a) vec.p[a] = nullptr, vec.ld[a] = 0, vec.heads_per[a] = 1;
    vec.p[0] = qk, vec.p[1] = qk + (size_t)kvh * dim, vec.p[2] = decay;
    vec.ld[0] = vec.ld[1] = 2LL * kvh * dim, vec.ld[2] = (long long)heads * dim;
    vec.heads_per[0] = vec.heads_per[1] = heads / kvh, vec.heads_per[2] = 1;
    vec.vec16 = dim % 4 == 0 && aligned16(qk) && aligned16(decay);
#define DELTA_WALK(D, R)                                                                                           \
    CELLM_RUN((state_walk_kernel<D, R, 1>), dim3(B, heads, (vd + WalkShape<D, R>::CPB - 1) / WalkShape<D, R>::CPB), WALK_THREADS, 0, stream, \
              o_out, state, slot_stride, n_slots, vec, v_in, (long long)heads * vd, beta, cu_seqlens, slot_ids, heads, dim, vd, err)
    if (dim <= 16) DELTA_WALK(16, 4);
    else if (dim <= 32) DELTA_WALK(32, 4);
    else if (dim <= 64) DELTA_WALK(64, 8);
    else if (dim <= 128) DELTA_WALK(128, 8);
    else {
        const size_t big = (size_t)(3 + 32) * dim * sizeof(float);
        if (big > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big);
            if (e != cudaSuccess) return (int)e;
        }
        CELLM_RUN(delta_scan_kernel, dim3(B, heads, (vd + 31) / 32), 32, big, stream, o_out, state, slot_stride, n_slots, qk, v_in, beta,
                  decay, cu_seqlens, slot_ids, heads, kvh, dim, vd, err);
    }
#undef DELTA_WALK
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ generalized delta rule
// S <- diag(d) S - (a * u)(u^T S) + k v^T, where both the decay and the removal read the old S; o = S^T r.
//   d = exp(-c * sigmoid(w_pre + w0))   a decay per head and key channel, c a constant of the design
//   a = sigmoid(a_pre + a_bias)         a removal rate per head and key channel
//   u = k / sqrt(sum(k^2) + unit_eps)   the unit key of each head
// The inputs' kernel forms d, u and a * u for every token (a warp a head); the walk reads r, k, v from the projection.
__global__ void __launch_bounds__(256)
gdelta_prep_kernel(float* __restrict__ vecs, const float* __restrict__ proj, long long ld, int col_k, int col_a,
                   const float* __restrict__ w_pre, long long ld_w, const float* __restrict__ w0, const float* __restrict__ a_bias,
                   float c, float unit_eps, int heads, int dim) {
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5, HD = heads * dim;
    const float* row = proj + t * ld;
    float* out = vecs + t * 3 * HD;
    for (int h = warp; h < heads; h += nwarps) {
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) {
            const float k = row[col_k + h * dim + i];
            ss = fmaf(k, k, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss + unit_eps);
        for (int i = lane; i < dim; i += 32) {
            const int ch = h * dim + i;
            const float u = row[col_k + ch] * inv;
            const float a = sigmoidf_(row[col_a + ch] + a_bias[ch]);
            out[ch] = expf(-c * sigmoidf_(w_pre[t * ld_w + ch] + w0[ch]));
            out[HD + ch] = u;
            out[2 * HD + ch] = a * u;
        }
    }
}

// vecs [T, 3, heads * dim] 32-bit: decay | unit key | removal rate times unit key.
CELLM_API int cellm_gdelta_prep(float* vecs, const float* proj, long long ld, int col_k, int col_a, const float* w_pre, long long ld_w,
                                const float* w0, const float* a_bias, float c, float unit_eps, int T, int heads, int dim,
                                cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (heads <= 0 || dim <= 0) return CELLM_ERR_SIZE;
    CELLM_RUN(gdelta_prep_kernel, T, 256, 0, stream, vecs, proj, ld, col_k, col_a, w_pre, ld_w, w0, a_bias, c, unit_eps, heads, dim);
    return CELLM_OK;
}

// The walk, a warp a (request, head, 32 columns of S): the columns in shared memory, one lane a column. Every sum
// runs over the head's rows in order, so the state after a token does not depend on how the sequence was cut.
__global__ void __launch_bounds__(32)
gdelta_scan_kernel(float* __restrict__ o_out, float* __restrict__ state, long long slot_stride, int n_slots,
                   const float* __restrict__ proj, long long ld, int col_r, int col_k, int col_v, const float* __restrict__ vecs,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, int heads, int dim, int vd,
                   int* __restrict__ err) {
    extern __shared__ float sm[];
    float* rs = sm;                 // [dim] each: r, k, decay, u, a * u
    float* ks = sm + dim;
    float* ds = sm + 2 * dim;
    float* us = sm + 3 * dim;
    float* as = sm + 4 * dim;
    float* Ssh = sm + 5 * dim;      // [dim][32]: the warp's columns of S
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x, j = blockIdx.z * 32 + lane;
    auto S = [&](int i) -> float& { return Ssh[i * 32 + lane]; };
    pdl_trigger();
    pdl_wait();
    const int slot = slot_ids[b];
    if (slot < 0 || slot >= n_slots) { if (lane == 0) atomicOr(err, CELLM_DEV_BAD_SLOT); return; }
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1], HD = heads * dim;
    float* st = state + (size_t)slot * slot_stride + (size_t)h * dim * vd;
    const bool live = j < vd;
    for (int i = 0; i < dim; ++i) S(i) = live ? st[(size_t)i * vd + j] : 0.f;
    for (int t = start; t < end; ++t) {
        const float* row = proj + (size_t)t * ld;
        const float* vt = vecs + (size_t)t * 3 * HD + h * dim;
        for (int i = lane; i < dim; i += 32) {
            rs[i] = row[col_r + h * dim + i];
            ks[i] = row[col_k + h * dim + i];
            ds[i] = vt[i];
            us[i] = vt[HD + i];
            as[i] = vt[2 * HD + i];
        }
        const float v = live ? row[col_v + h * vd + j] : 0.f;
        __syncwarp();
        float dot = 0.f;
        for (int i = 0; i < dim; ++i) dot = fmaf(us[i], S(i), dot);
        float o = 0.f;
        for (int i = 0; i < dim; ++i) {
            const float s_new = fmaf(ks[i], v, fmaf(ds[i], S(i), as[i] * -dot));
            S(i) = s_new;
            o = fmaf(s_new, rs[i], o);
        }
        if (live) o_out[(size_t)t * heads * vd + (size_t)h * vd + j] = o;
        __syncwarp();
    }
    if (live)
        for (int i = 0; i < dim; ++i) st[(size_t)i * vd + j] = S(i);
}

// proj [T, ld] 32-bit holds r (heads x dim) at col_r, k at col_k, v (heads x vd) at col_v; vecs as gdelta_prep left them;
// state [slots][heads][dim][vd] is moved on; o_out [T, heads * vd] gets S^T r (not normed).
CELLM_API int cellm_gdelta_scan(float* o_out, float* state, long long slot_stride, int n_slots, const float* proj, long long ld,
                                int col_r, int col_k, int col_v, const float* vecs, const int* cu_seqlens, const int* slot_ids,
                                int B, int heads, int dim, int vd, int* err, cudaStream_t stream) {
    if (B <= 0) return CELLM_OK;
    if (heads <= 0 || dim <= 0 || vd <= 0 || dim > RECURRENT_MAX_DIM) return CELLM_ERR_SIZE;
    if (dim <= 128) {       // the head's columns in registers (state_walk_kernel)
        const long long HD = (long long)heads * dim;
        WalkVectors vec;
        vec.p[0] = proj + col_r, vec.p[1] = proj + col_k, vec.p[2] = vecs, vec.p[3] = vecs + HD, vec.p[4] = vecs + 2 * HD;
        vec.ld[0] = vec.ld[1] = ld, vec.ld[2] = vec.ld[3] = vec.ld[4] = 3 * HD;
        for (int a = 0; a < 5; ++a) vec.heads_per[a] = 1;
        vec.vec16 = dim % 4 == 0 && ld % 4 == 0 && aligned16(vec.p[0]) && aligned16(vec.p[1]) && aligned16(vecs);
#define GDELTA_WALK(D, R)                                                                                          \
    CELLM_RUN((state_walk_kernel<D, R, 2>), dim3(B, heads, (vd + WalkShape<D, R>::CPB - 1) / WalkShape<D, R>::CPB), WALK_THREADS, 0, stream, \
              o_out, state, slot_stride, n_slots, vec, (const float*)(proj + col_v), ld, (const float*)nullptr, cu_seqlens, slot_ids,  \
              heads, dim, vd, err)
        if (dim <= 16) GDELTA_WALK(16, 4);
        else if (dim <= 32) GDELTA_WALK(32, 4);
        else if (dim <= 64) GDELTA_WALK(64, 8);
        else GDELTA_WALK(128, 8);
#undef GDELTA_WALK
        return CELLM_OK;
    }
    const size_t smem = (size_t)(5 + 32) * dim * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(gdelta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    CELLM_RUN(gdelta_scan_kernel, dim3(B, heads, (vd + 31) / 32), 32, smem, stream, o_out, state, slot_stride, n_slots, proj, ld, col_r,
              col_k, col_v, vecs, cu_seqlens, slot_ids, heads, dim, vd, err);
    return CELLM_OK;
}

// ------------------------------------------------------------------------------------------------ norm over a head's output
// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w[:] (* sigmoid(gate[t, h, :])): a warp a (token, head). w is one row
// of vd values for all heads, or (w_per_head) a row for every head.
template <typename TA>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(TA* __restrict__ out, const float* __restrict__ o, const float* __restrict__ w,
                      const float* __restrict__ gate, long long gate_ld, int n_rows, int heads, int vd, float eps, int w_per_head) {
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
    const float* wr = w + (w_per_head ? (size_t)h * vd : 0);
    for (int j = lane; j < vd; j += 32) {
        float y = x[j] * inv * wr[j];
        if (gate) y *= sigmoidf_(gate[(size_t)t * gate_ld + (size_t)h * vd + j]);
        out[(size_t)r * vd + j] = from_float<TA>(y);
    }
}

CELLM_API int cellm_head_norm_gate(void* out, const float* o, const float* w, const float* gate, long long gate_ld, int T,
                                   int heads, int vd, float eps, int w_per_head, int dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (heads <= 0 || vd <= 0) return CELLM_ERR_SIZE;
    const int n_rows = T * heads;
    const unsigned blocks = (unsigned)((n_rows + 7) / 8);
    if (dtype == CELLM_F32)
        CELLM_RUN(head_norm_gate_kernel<float>, blocks, 256, 0, stream, (float*)out, o, w, gate, gate_ld, n_rows, heads, vd, eps, w_per_head);
    else if (dtype == CELLM_BF16)
        CELLM_RUN(head_norm_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, o, w, gate, gate_ld, n_rows, heads, vd, eps, w_per_head);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
