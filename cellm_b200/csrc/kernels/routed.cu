// Routed feed-forward ("mixture of experts"): the choice of experts from the router's sums (which a product forms),
// the experts' two products in the form that serves few tokens and the 32-bit path (a token's chosen experts, and the
// shared expert, walked row by row), and for many tokens the sort of the (token, choice) slots by expert, the gather
// of their rows and the weighted sum of the results around the grouped tensor-core products (gemm_tcgen05.cu).
//
//   z = R h (32-bit sums);  s = sigmoid(z);  c = s + correction          (c chooses, s weighs)
//   experts lie in `n_groups` equal runs of neighbours; a run's score is the sum of its two largest c (its
//   only c for runs of one); only experts of the `keep` best runs can be chosen (the others count as -inf)
//   the `top` experts with the largest c are chosen; their weights are s / (sum of the chosen s + 1e-20) * scale
//   out = sum_k weight_k * D_k act(U_k h)  [+ sigmoid(g . h) * shared(h)]
//
// Ties go to the lower index. The chosen experts are listed by descending c, and every sum runs in an order
// that depends on the sizes alone, so a token's result does not depend on what else is in the batch.
#include "common.cuh"


// Whether rows of n values (pitch ld) can be read in pieces of 16 bytes.
template <typename TW> __device__ __forceinline__ bool rows_vectorise(const TW* base, long long ld, int n) {
    constexpr int per = 16 / (int)sizeof(TW);
    return (n % per) == 0 && (ld % per) == 0 && (((uintptr_t)base) & 15) == 0;
}

// A lane's share of the dot products of up to four weight rows (row j at w + j * stride; rows >= nrows count as zeros)
// with a vector held as floats, in pieces of 16 bytes where the rows allow it (`vec`), else element by element:
// a[j] += f * (row j . v). The rows' loads are issued together, so a lane has four of them in flight.
template <typename TW>
__device__ __forceinline__ void lane_dot4(float (&a)[4], float f, const TW* __restrict__ w, size_t stride, int nrows, const float* __restrict__ v,
                                          int n, int lane, bool vec) {
    constexpr int PER = 16 / (int)sizeof(TW);
    float p[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec) {
#pragma unroll 2
        for (int i = lane * PER; i < n; i += 32 * PER) {
            uint4 x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = j < nrows ? *reinterpret_cast<const uint4*>(w + j * stride + i) : make_uint4(0, 0, 0, 0);
            float y[PER];
#pragma unroll
            for (int k = 0; k < PER; k += 4) {
                const float4 t = *reinterpret_cast<const float4*>(v + i + k);
                y[k] = t.x; y[k + 1] = t.y; y[k + 2] = t.z; y[k + 3] = t.w;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const TW* xp = reinterpret_cast<const TW*>(&x[j]);
#pragma unroll
                for (int k = 0; k < PER; ++k) p[j] += to_float(xp[k]) * y[k];
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            const float y = v[i];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < nrows) p[j] += to_float(w[j * stride + i]) * y;
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) a[j] += f * p[j];
}

// One output row of up to four experts at once (expert j: row w[j] against its own vector v[j], factor f[j]): the sum of
// f[j] * (w[j] . v[j]) in the order of j, a lane's share. The experts' loads are issued together.
template <typename TW>
__device__ __forceinline__ float lane_dot_experts(const TW* const (&w)[4], const float* const (&v)[4], const float (&f)[4], int count, int n, int lane,
                                                  bool vec) {
    constexpr int PER = 16 / (int)sizeof(TW);
    float p[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec) {
#pragma unroll 2
        for (int i = lane * PER; i < n; i += 32 * PER) {
            uint4 x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = j < count ? *reinterpret_cast<const uint4*>(w[j] + i) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (j < count) {
                    const TW* xp = reinterpret_cast<const TW*>(&x[j]);
#pragma unroll
                    for (int k = 0; k < PER; k += 4) {
                        const float4 t = *reinterpret_cast<const float4*>(v[j] + i + k);
                        p[j] += to_float(xp[k]) * t.x;
                        p[j] += to_float(xp[k + 1]) * t.y;
                        p[j] += to_float(xp[k + 2]) * t.z;
                        p[j] += to_float(xp[k + 3]) * t.w;
                    }
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < count) p[j] += to_float(w[j][i]) * v[j][i];
    }
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (j < count) a += f[j] * p[j];
    return a;
}

// ---- the router ----------------------------------------------------------------------------------------------------
// The choice from the router's 32-bit sums z [T, E (+1)] (a product's output; column E is the shared expert's gate): a
// warp a token, its scores in shared memory.
#define ROUTE_THREADS 128

template <typename TC>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_kernel(int* __restrict__ idx, float* __restrict__ wts, float* __restrict__ gate_out, const float* __restrict__ z_all, long long ldz,
             const TC* __restrict__ correction, int T, int E, int top, int n_groups, int keep, float scale, int has_gate) {
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = ROUTE_THREADS / 32;
    const int per = 2 * E + 2 * n_groups + top;
    float* z = smem + (size_t)warp * per;       // [E]: s
    float* c = z + E;                           // [E]: choice scores
    float* g = c + E;                           // [n_groups]: scores of the runs
    float* k = g + n_groups;                    // [n_groups]: 1 = the run is kept
    float* chosen = k + n_groups;               // [top]: s of the chosen, by rank
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x * nwarps + warp;
    if (t >= T) return;
    const float* zr = z_all + (size_t)t * ldz;
    const int gsz = E / n_groups;
    for (int e = lane; e < E; e += 32) {
        const float s = 1.f / (1.f + expf(-zr[e]));
        z[e] = s;
        c[e] = s + to_float(correction[e]);
    }
    if (has_gate && lane == 0) gate_out[t] = 1.f / (1.f + expf(-zr[E]));
    __syncwarp();
    if (n_groups > 1) {
        for (int gi = lane; gi < n_groups; gi += 32) {
            float m1 = -INFINITY, m2 = -INFINITY;
            for (int e = gi * gsz; e < (gi + 1) * gsz; ++e) {
                const float v = c[e];
                if (v > m1) { m2 = m1; m1 = v; }
                else if (v > m2) m2 = v;
            }
            g[gi] = gsz >= 2 ? m1 + m2 : m1;
        }
        __syncwarp();
        for (int gi = lane; gi < n_groups; gi += 32) {
            int rank = 0;
            const float mine = g[gi];
            for (int gj = 0; gj < n_groups; ++gj) rank += (g[gj] > mine || (g[gj] == mine && gj < gi)) ? 1 : 0;
            k[gi] = rank < keep ? 1.f : 0.f;
        }
        __syncwarp();
        for (int e = lane; e < E; e += 32)
            if (k[e / gsz] == 0.f) c[e] = -INFINITY;
        __syncwarp();
    }
    for (int e = lane; e < E; e += 32) {
        int rank = 0;
        const float mine = c[e];
        for (int f = 0; f < E; ++f) rank += (c[f] > mine || (c[f] == mine && f < e)) ? 1 : 0;
        if (rank < top) {
            idx[(size_t)t * top + rank] = e;
            chosen[rank] = z[e];
        }
    }
    __syncwarp();
    float sum = 0.f;
    for (int r = 0; r < top; ++r) sum += chosen[r];
    for (int r = lane; r < top; r += 32) wts[(size_t)t * top + r] = chosen[r] / (sum + 1e-20f) * scale;
}

// z: [T, E (+1)] float (row pitch ldz), column E the shared expert's gate when has_gate; correction: [E].
// idx: [T, top] int, wts: [T, top] float, gate_out: [T] float (sigmoid of the gate column).
CELLM_API int cellm_route(int* idx, float* wts, float* gate_out, const float* z, long long ldz, const void* correction, int c_dtype, int T,
                          int E, int top, int n_groups, int keep, float scale, int has_gate, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (E < 1 || top < 1 || top > E || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups) return CELLM_ERR_SIZE;
    if (has_gate && !gate_out) return CELLM_ERR_ARG;
    const size_t smem = (size_t)(ROUTE_THREADS / 32) * (2 * E + 2 * n_groups + top) * sizeof(float);
    if (smem > 48 * 1024) return CELLM_ERR_SIZE;
    const unsigned blocks = (unsigned)((T + ROUTE_THREADS / 32 - 1) / (ROUTE_THREADS / 32));
    if (c_dtype == CELLM_F32)
        CELLM_RUN(route_kernel<float>, blocks, ROUTE_THREADS, smem, stream, idx, wts, gate_out, z, ldz, (const float*)correction, T, E, top,
                  n_groups, keep, scale, has_gate);
    else if (c_dtype == CELLM_BF16)
        CELLM_RUN(route_kernel<__nv_bfloat16>, blocks, ROUTE_THREADS, smem, stream, idx, wts, gate_out, z, ldz, (const __nv_bfloat16*)correction,
                  T, E, top, n_groups, keep, scale, has_gate);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// ---- the experts, row by row ----------------------------------------------------------------------------------------
#define EXPERT_THREADS 128
#define EXPERT_WARPS 4           // a warp forms `rpw` (1, 2 or 4) output rows at once; a block of the first kernel 4 * rpw
#define EXPERT_DOWN_WARPS 8      // the second kernel's blocks hold a token's middles in shared memory: more warps share them

// mid[t * top + k, :] = act(U_e y[t]) for e = idx[t, k]; up: [E * ff, H]. Blocks with blockIdx.x >= T * top take the shared
// expert: smid[t, :] = act(U_s y[t]), U_s: [sff, H].
template <typename TA>
__global__ void __launch_bounds__(EXPERT_THREADS)
expert_up_kernel(TA* __restrict__ mid, TA* __restrict__ smid, const TA* __restrict__ y, long long ldy, const TA* __restrict__ up,
                 const TA* __restrict__ sup, const int* __restrict__ idx, int T, int H, int ff, int sff, int top, int E, int act, int rpw) {
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool is_shared = (int)blockIdx.x >= T * top;
    const int slot = is_shared ? (int)blockIdx.x - T * top : (int)blockIdx.x;
    const int t = is_shared ? slot : slot / top;
    const int rows = is_shared ? sff : ff;
    if ((int)blockIdx.y * EXPERT_WARPS * rpw >= rows) return;
    const bool vec = rows_vectorise(is_shared ? sup : up, H, H);
    pdl_trigger();
    pdl_wait();
    {   // the token's input into shared memory as floats, in 16-byte pieces where its row allows it
        constexpr int PER = 16 / (int)sizeof(TA);
        const TA* src = y + (size_t)t * ldy;
        if (H % PER == 0 && (((uintptr_t)src) & 15) == 0) {
            for (int i = threadIdx.x * PER; i < H; i += EXPERT_THREADS * PER) {
                const uint4 x = *reinterpret_cast<const uint4*>(src + i);
                const TA* xp = reinterpret_cast<const TA*>(&x);
#pragma unroll
                for (int k = 0; k < PER; ++k) smem[i + k] = to_float(xp[k]);
            }
        } else {
            for (int i = threadIdx.x; i < H; i += EXPERT_THREADS) smem[i] = to_float(src[i]);
        }
    }
    const TA* base = sup;
    if (!is_shared) base = up + (size_t)min(max(idx[slot], 0), E - 1) * ff * H;
    __syncthreads();
    const int r0 = (blockIdx.y * EXPERT_WARPS + warp) * rpw, nr = min(rpw, rows - r0);
    if (nr <= 0) return;
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    lane_dot4<TA>(d, 1.f, base + (size_t)r0 * H, (size_t)H, nr, smem, H, lane, vec);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float v = warp_sum(d[j]);
        if (lane == 0 && j < nr) (is_shared ? smid : mid)[(size_t)slot * rows + r0 + j] = from_float<TA>(cellm_activate(v, act));
    }
}

// out[t, r] = sum_k wts[t, k] * (D_e mid[t * top + k])[r] (+ gate[t] * (D_s smid[t])[r]); down: [E * H, ff], D_s: [H, sff]
template <typename TA>
__global__ void __launch_bounds__(EXPERT_DOWN_WARPS * 32)
expert_down_kernel(TA* __restrict__ out, const TA* __restrict__ mid, const TA* __restrict__ smid, const TA* __restrict__ down,
                   const TA* __restrict__ sdown, const int* __restrict__ idx, const float* __restrict__ wts, const float* __restrict__ gate,
                   int H, int ff, int sff, int top, int E, int rpw) {
    extern __shared__ __align__(16) float smem[];   // [top * ff] the token's middles, [sff] the shared expert's, then [top] weights and experts
    float* ms = smem;
    float* ss = smem + (size_t)top * ff;
    float* wk = ss + sff;
    int* ek = (int*)(wk + top);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const bool vec = rows_vectorise(down, ff, ff) && (ff & 3) == 0, svec = sdown && rows_vectorise(sdown, sff, sff) && ((top * ff) & 3) == 0;
    pdl_trigger();
    pdl_wait();
    {   // the token's middles into shared memory as floats, in 16-byte pieces where their rows allow it
        constexpr int PER = 16 / (int)sizeof(TA);
        const TA* src = mid + (size_t)t * top * ff;
        const int n = top * ff;
        if (n % PER == 0 && (((uintptr_t)src) & 15) == 0) {
            for (int i = threadIdx.x * PER; i < n; i += EXPERT_DOWN_WARPS * 32 * PER) {
                const uint4 x = *reinterpret_cast<const uint4*>(src + i);
                const TA* xp = reinterpret_cast<const TA*>(&x);
#pragma unroll
                for (int k = 0; k < PER; ++k) ms[i + k] = to_float(xp[k]);
            }
        } else {
            for (int i = threadIdx.x; i < n; i += EXPERT_DOWN_WARPS * 32) ms[i] = to_float(src[i]);
        }
        if (sdown) {
            const TA* ssrc = smid + (size_t)t * sff;
            if (sff % PER == 0 && (((uintptr_t)ssrc) & 15) == 0) {
                for (int i = threadIdx.x * PER; i < sff; i += EXPERT_DOWN_WARPS * 32 * PER) {
                    const uint4 x = *reinterpret_cast<const uint4*>(ssrc + i);
                    const TA* xp = reinterpret_cast<const TA*>(&x);
#pragma unroll
                    for (int k = 0; k < PER; ++k) ss[i + k] = to_float(xp[k]);
                }
            } else {
                for (int i = threadIdx.x; i < sff; i += EXPERT_DOWN_WARPS * 32) ss[i] = to_float(ssrc[i]);
            }
        }
    }
    for (int k = threadIdx.x; k < top; k += EXPERT_DOWN_WARPS * 32) {
        wk[k] = wts[(size_t)t * top + k];
        ek[k] = min(max(idx[(size_t)t * top + k], 0), E - 1);
    }
    __syncthreads();
    const int r0 = (blockIdx.y * EXPERT_DOWN_WARPS + warp) * rpw, nr = min(rpw, H - r0);
    if (nr <= 0) return;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    if (rpw == 1) {     // few tokens: one row a warp, four experts' rows in flight at once
        for (int k0 = 0; k0 < top; k0 += 4) {
            const TA* w[4];
            const float* v[4];
            float f[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = min(k0 + j, top - 1);
                w[j] = down + ((size_t)ek[k] * H + r0) * ff;
                v[j] = ms + (size_t)k * ff;
                f[j] = wk[k];
            }
            a[0] += lane_dot_experts<TA>(w, v, f, min(4, top - k0), ff, lane, vec);
        }
    } else {
        for (int k = 0; k < top; ++k)
            lane_dot4<TA>(a, wk[k], down + ((size_t)ek[k] * H + r0) * ff, (size_t)ff, nr, ms + (size_t)k * ff, ff, lane, vec);
    }
    if (sdown) lane_dot4<TA>(a, gate ? gate[t] : 1.f, sdown + (size_t)r0 * sff, (size_t)sff, nr, ss, sff, lane, svec);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float v = warp_sum(a[j]);
        if (lane == 0 && j < nr) out[(size_t)t * H + r0 + j] = from_float<TA>(v);
    }
}

// The chosen experts of every token, and the shared expert (sup null: none), walked row by row. mid: [T * top, ff] and
// smid: [T, sff], scratch of the activations' type. gate: [T] (null: the shared expert's result as it is).
CELLM_API int cellm_experts_rowwise(void* out, void* mid, void* smid, const void* y, long long ldy, const void* up, const void* down,
                                    const void* sup, const void* sdown, const int* idx, const float* wts, const float* gate, int T, int H,
                                    int ff, int sff, int top, int E, int act, int dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (H < 1 || ff < 1 || top < 1 || E < 1 || sff < 0) return CELLM_ERR_SIZE;
    if ((sup == nullptr) != (sdown == nullptr) || (sup && (sff < 1 || !smid))) return CELLM_ERR_ARG;
    if (!sup) sff = 0;
    const size_t smem_up = (size_t)H * sizeof(float), smem_down = ((size_t)top * ff + sff + 2 * top) * sizeof(float);
    if (smem_up > 200 * 1024 || smem_down > 200 * 1024) return CELLM_ERR_SIZE;
    const int up_rows = ff > sff ? ff : sff;
    // rows a warp: four where that still leaves some 600 blocks (four an SM) at work, else two, else one
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
    }
    auto rows_a_warp = [&](long long rows_in_all) {
        for (int r = 4; r > 1; r /= 2)
            if (rows_in_all / (EXPERT_WARPS * r) >= 4LL * sms) return r;
        return 1;
    };
    const int rpw_up = rows_a_warp((long long)T * top * ff + (sup ? (long long)T * sff : 0));
    int rpw_down = 1;
    for (int r = 4; r > 1; r /= 2)
        if ((long long)T * H / (EXPERT_DOWN_WARPS * r) >= 2LL * sms) { rpw_down = r; break; }
    const dim3 grid_up((unsigned)(T * top + (sup ? T : 0)), (unsigned)((up_rows + EXPERT_WARPS * rpw_up - 1) / (EXPERT_WARPS * rpw_up)));
    const dim3 grid_down((unsigned)T, (unsigned)((H + EXPERT_DOWN_WARPS * rpw_down - 1) / (EXPERT_DOWN_WARPS * rpw_down)));
    if (grid_up.y > 65535 || grid_down.y > 65535) return CELLM_ERR_SIZE;
#define GO(TA)                                                                                                                    \
    do {                                                                                                                          \
        static bool configured = false;                                                                                           \
        if (!configured && (smem_up > 48 * 1024 || smem_down > 48 * 1024)) {                                                      \
            cudaError_t e = cudaFuncSetAttribute(expert_up_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);  \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(expert_down_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e;                                                                                  \
            configured = true;                                                                                                    \
        }                                                                                                                         \
        CELLM_RUN(expert_up_kernel<TA>, grid_up, EXPERT_THREADS, smem_up, stream, (TA*)mid, (TA*)smid, (const TA*)y, ldy, (const TA*)up,  \
                  (const TA*)sup, idx, T, H, ff, sff, top, E, act, rpw_up);                                                               \
        CELLM_RUN(expert_down_kernel<TA>, grid_down, EXPERT_DOWN_WARPS * 32, smem_down, stream, (TA*)out, (const TA*)mid, (const TA*)smid, \
                  (const TA*)down, (const TA*)sdown, idx, wts, gate, H, ff, sff, top, E, rpw_down);                                         \
    } while (0)
    if (dtype == CELLM_F32) GO(float);
    else if (dtype == CELLM_BF16) GO(__nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef GO
    return CELLM_OK;
}

// ---- a plain activation: h = act(u) for 32-bit sums u [T, n] (row pitch ld) ----------------------------------------------
template <typename T>
__global__ void activation_kernel(T* __restrict__ h, const float* __restrict__ u, long long ld, int n, int act, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / n, c = i - t * n;
    h[i] = from_float<T>(cellm_activate(u[t * ld + c], act));
}

CELLM_API int cellm_activation(void* h, const float* u, long long ld, int T, int n, int act, int dtype, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return CELLM_OK;
    if (act < 0 || act > 5) return CELLM_ERR_ARG;
    const size_t total = (size_t)T * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == CELLM_F32) CELLM_RUN(activation_kernel<float>, blocks, 256, 0, stream, (float*)h, u, ld, n, act, total);
    else if (dtype == CELLM_BF16) CELLM_RUN(activation_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)h, u, ld, n, act, total);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// ---- many tokens: the (token, choice) slots sorted by expert ------------------------------------------------------------
// For the grouped tensor-core product every expert's slots form one run of rows, padded to whole tiles of 128 rows, in
// the order of the slots themselves (so a row's place depends on the step's tokens alone, never on timing).
#define MOE_TILE 128
#define MOE_SORT_THREADS 256

// One block an expert: it counts the slots of every expert (a histogram in shared memory), finds where its own run
// begins, names its tiles, and places its slots in their order. row_slot[row] = slot or -1 (padding); slot_row[slot] = row;
// tile_group[tile] = expert or -1 (behind the last run).
__global__ void __launch_bounds__(MOE_SORT_THREADS)
moe_sort_kernel(int* __restrict__ row_slot, int* __restrict__ slot_row, int* __restrict__ tile_group, const int* __restrict__ idx, int S,
                int E, int max_tiles) {
    extern __shared__ int sh[];
    int* hist = sh;             // [E]
    int* wsum = sh + E;         // [warps]
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = MOE_SORT_THREADS / 32;
    pdl_trigger();
    pdl_wait();
    for (int i = tid; i < E; i += MOE_SORT_THREADS) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < S; i += MOE_SORT_THREADS) {
        const int x = idx[i];
        if (x >= 0 && x < E) atomicAdd(&hist[x], 1);
    }
    __syncthreads();
    int start = 0;
    for (int f = 0; f < e; ++f) start += (hist[f] + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
    const int count = hist[e], padded = (count + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
    for (int i = tid; i < padded / MOE_TILE; i += MOE_SORT_THREADS) tile_group[start / MOE_TILE + i] = e;
    if (e == E - 1)
        for (int i = (start + padded) / MOE_TILE + tid; i < max_tiles; i += MOE_SORT_THREADS) tile_group[i] = -1;
    for (int i = count + tid; i < padded; i += MOE_SORT_THREADS) row_slot[start + i] = -1;
    int base = 0;
    for (int c0 = 0; c0 < S; c0 += MOE_SORT_THREADS) {
        const int i = c0 + tid;
        const bool mine = i < S && idx[i] == e;
        const unsigned b = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) wsum[warp] = __popc(b);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < nwarps; ++w) {
            if (w < warp) before += wsum[w];
            total += wsum[w];
        }
        if (mine) {
            const int r = start + base + before + __popc(b & ((1u << lane) - 1u));
            row_slot[r] = i;
            slot_row[i] = r;
        }
        base += total;
        __syncthreads();
    }
}

CELLM_API int cellm_moe_sort(int* row_slot, int* slot_row, int* tile_group, const int* idx, int S, int E, int max_tiles, cudaStream_t stream) {
    if (S <= 0) return CELLM_OK;
    if (E < 1 || max_tiles < 1 || E > 8192) return CELLM_ERR_SIZE;
    CELLM_RUN(moe_sort_kernel, E, MOE_SORT_THREADS, (size_t)(E + 32) * sizeof(int), stream, row_slot, slot_row, tile_group, idx, S, E, max_tiles);
    return CELLM_OK;
}

// xs[row, :] = y[row_slot[row] / top, :] for the rows of the named tiles (zeros in padding rows); 16-byte pieces.
__global__ void moe_gather_kernel(uint4* __restrict__ xs, const uint4* __restrict__ y, long long ldy16, const int* __restrict__ row_slot,
                                  const int* __restrict__ tile_group, int top, int H16) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    if (tile_group[row / MOE_TILE] < 0) return;
    const int slot = row_slot[row];
    uint4* dst = xs + (size_t)row * H16;
    if (slot < 0) {
        for (int i = threadIdx.x; i < H16; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* src = y + (size_t)(slot / top) * ldy16;
    for (int i = threadIdx.x; i < H16; i += blockDim.x) dst[i] = src[i];
}

// rows: the sorted buffer's rows (a multiple of 128); y: [T, H] bfloat16 with H a multiple of 8.
CELLM_API int cellm_moe_gather(void* xs, const void* y, long long ldy, const int* row_slot, const int* tile_group, int rows, int top, int H,
                               cudaStream_t stream) {
    if (rows <= 0) return CELLM_OK;
    if ((H & 7) || (ldy & 7) || (rows % MOE_TILE) || top < 1) return CELLM_ERR_SIZE;
    if (((uintptr_t)xs | (uintptr_t)y) & 15) return CELLM_ERR_ALIGN;
    CELLM_RUN(moe_gather_kernel, rows, 128, 0, stream, (uint4*)xs, (const uint4*)y, ldy / 8, row_slot, tile_group, top, H / 8);
    return CELLM_OK;
}

// out[t, :] = sum_k wts[t, k] * Y[slot_row[t * top + k], :] (+ gate[t] * shared[t, :]), the sum in the order of k, 32-bit.
__global__ void moe_combine_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ Y, const int* __restrict__ slot_row,
                                   const float* __restrict__ wts, const float* __restrict__ shared, const float* __restrict__ gate, int H,
                                   int top) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float g = shared ? (gate ? gate[t] : 1.f) : 0.f;
    for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
        float a0 = 0.f, a1 = 0.f;
        for (int k = 0; k < top; ++k) {
            const float w = wts[(size_t)t * top + k];
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Y + (size_t)slot_row[(size_t)t * top + k] * H + c));
            a0 += w * v.x;
            a1 += w * v.y;
        }
        if (shared) {
            a0 += g * shared[(size_t)t * H + c];
            a1 += g * shared[(size_t)t * H + c + 1];
        }
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * H + c) = __floats2bfloat162_rn(a0, a1);
    }
}

CELLM_API int cellm_moe_combine(void* out, const void* Y, const int* slot_row, const float* wts, const float* shared, const float* gate, int T,
                                int H, int top, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if ((H & 1) || top < 1) return CELLM_ERR_SIZE;
    CELLM_RUN(moe_combine_kernel, T, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)Y, slot_row, wts, shared, gate, H, top);
    return CELLM_OK;
}
