// A short causal convolution over time on the channels of a projection, for kernels that apply it while they read
// the projection: y_t[c] = sum_j w[c][j] * u_(t - taps + 1 + j)[c], where u is the projected value (plus its bias).
// Rows before the portion's first token come from the request's state, which holds the last taps - 1 projected
// values of the request (zeros at its start), so a sequence cut anywhere gives the same sums in the same order.
#pragma once
#include "common.cuh"

#define CONV_TAPS_MAX 16

struct ConvTaps {
    const float* proj;      // [T, ld]: the step's projections, 32-bit
    long long ld;
    int col0;               // column of channel 0 in a row of proj
    const float* bias;      // [C] or null
    const float* taps;      // [C, n_taps]
    const float* state;     // this request's [n_taps - 1, C]
    int n_taps;             // 0: no convolution (the projected value itself)
    int C;
};

// Channel c of token t (an index into the step's rows); `start` is the first row of the token's portion.
__device__ __forceinline__ float conv_taps_at(const ConvTaps& s, int t, int start, int c) {
    const float b = s.bias ? s.bias[c] : 0.f;
    if (s.n_taps <= 0) return s.proj[(size_t)t * s.ld + s.col0 + c] + b;
    float y = 0.f;
    for (int j = 0; j < s.n_taps; ++j) {
        const int tt = t - (s.n_taps - 1) + j;
        const float u = tt >= start ? s.proj[(size_t)tt * s.ld + s.col0 + c] + b
                                    : s.state[(size_t)(tt - start + s.n_taps - 1) * s.C + c];
        y = fmaf(s.taps[(size_t)c * s.n_taps + j], u, y);
    }
    return y;
}
