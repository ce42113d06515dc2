// Kernels of mixers that carry a state per sequence instead of keys and values: a short causal convolution over time
// whose last inputs a sequence keeps, the preparation and the output stage of a state-space mixer (whose recurrence runs
// in the delta rule's kernel, in its form without a correction term), and a gated linear recurrent unit with
// block-diagonal gates.  Everything here is float32; the one rounding is at the store of a result that a product reads.
//
// Rows of a sequence are consecutive and in order; row_slot says whose a row is.  A sequence's kept inputs live in
// state[slot][conv_off ...] as [taps - 1, C], oldest first, zero at its start (so tokens before the start count as zero).
#include "api.h"
#include "common.cuh"

namespace citlali {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The convolved value of channel c at `row`: sum_j w[c, j] u(t - taps + 1 + j) (+ bias[c]), where u of a row of this step
// is in[row, c] + in_bias[c] and u of an earlier token is what the sequence kept.
__device__ __forceinline__ float convolve(const float* __restrict__ in, int in_stride, const float* __restrict__ in_bias,
                                          const float* __restrict__ taps_w, int taps, const float* __restrict__ bias,
                                          const float* __restrict__ kept, int C, int row, int in_step, int c) {
    float acc = bias ? bias[c] : 0.0f;
    const float ib = in_bias ? in_bias[c] : 0.0f;
    for (int back = taps - 1; back >= 0; --back) {            // `back` tokens back; oldest first
        float u;
        if (back <= in_step) u = in[(size_t)(row - back) * in_stride + c] + ib;
        else u = kept[(size_t)(taps - 1 - back + in_step) * C + c];
        acc = fmaf(taps_w[(size_t)c * taps + (taps - 1 - back)], u, acc);
    }
    return acc;
}

__device__ __forceinline__ int rows_before_in_step(const int32_t* __restrict__ row_slot, int row, int slot, int taps) {
    int in_step = 0;
    while (in_step < taps - 1 && row - in_step - 1 >= 0 && row_slot[row - in_step - 1] == slot) ++in_step;
    return in_step;
}

// out[row, c] = act(conv(in)[row, c]); act 0: none, 1: SiLU.  One thread a (row, channel).
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* __restrict__ in, int in_stride, const float* __restrict__ in_bias,
                   const float* __restrict__ taps_w, int taps, const float* __restrict__ bias, int act,
                   const float* __restrict__ state, size_t state_stride, size_t conv_off,
                   const int32_t* __restrict__ row_slot, float* __restrict__ out, int out_stride, int C) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const int slot = row_slot[row];
    const int in_step = rows_before_in_step(row_slot, row, slot, taps);
    const float* kept = state + (size_t)slot * state_stride + conv_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float v = convolve(in, in_stride, in_bias, taps_w, taps, bias, kept, C, row, in_step, c);
        out[(size_t)row * out_stride + c] = act == 1 ? silu_f(v) : v;
    }
}

// After a step's rows were convolved: every sequence keeps its last taps - 1 inputs (with in_bias added, as the
// convolution saw them).  One thread a (sequence, channel).
__global__ void conv_keep_kernel(const float* __restrict__ in, int in_stride, const float* __restrict__ in_bias, int taps,
                                 float* __restrict__ state, size_t state_stride, size_t conv_off,
                                 const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot, int C) {
    dependents_may_launch();
    wait_for_predecessor();
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r0 = seq_start[seq], n = seq_start[seq + 1] - r0, keep = taps - 1;
    const float ib = in_bias ? in_bias[c] : 0.0f;
    float* kept = state + (size_t)seq_slot[seq] * state_stride + conv_off;
    if (n >= keep) {
        for (int i = 0; i < keep; ++i) kept[(size_t)i * C + c] = in[(size_t)(r0 + n - keep + i) * in_stride + c] + ib;
    } else {
        for (int i = 0; i < keep - n; ++i) kept[(size_t)i * C + c] = kept[(size_t)(i + n) * C + c];
        for (int i = 0; i < n; ++i) kept[(size_t)(keep - n + i) * C + c] = in[(size_t)(r0 + i) * in_stride + c] + ib;
    }
}

// ---- the state-space mixer ---------------------------------------------------------------------------------------
// proj [rows, proj_stride] = z (H P) | x (H P) | B (G N) | C (G N) | dt (H).  x, B, C pass the convolution (with bias) and
// SiLU; dt <- softplus(dt + dt_bias).  prep [rows, 2 G N + H P + 2 H] receives, in the layout the recurrence kernel reads
// (query | key | value | write strength | decay):  C | B | x | dt | exp(-exp(A_log) dt).
__global__ void __launch_bounds__(256)
ssm_prepare_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ taps_w, int taps,
                   const float* __restrict__ conv_bias, const float* __restrict__ state, size_t state_stride, size_t conv_off,
                   const int32_t* __restrict__ row_slot, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                   float* __restrict__ prep, int H, int P, int G, int N) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const int inner = H * P, GN = G * N, Cc = inner + 2 * GN;
    const int slot = row_slot[row];
    const int in_step = rows_before_in_step(row_slot, row, slot, taps);
    const float* kept = state + (size_t)slot * state_stride + conv_off;
    float* dst = prep + (size_t)row * (Cc + 2 * H);
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < Cc + H; c += gridDim.y * blockDim.x) {
        if (c < Cc) {
            const float v = silu_f(convolve(proj + inner, proj_stride, nullptr, taps_w, taps, conv_bias, kept, Cc, row, in_step, c));
            // x -> the values, B -> the keys, C -> the queries
            const int at = c < inner ? 2 * GN + c : (c < inner + GN ? GN + (c - inner) : c - inner - GN);
            dst[at] = v;
        } else {
            const int h = c - Cc;
            const float dt = softplus_f(proj[(size_t)row * proj_stride + inner + Cc + h] + dt_bias[h]);
            dst[Cc + h] = dt;
            dst[Cc + H + h] = expf(-expf(a_log[h]) * dt);
        }
    }
}

// y = (o + D_h x) * silu(z), then divided by the root mean square of its norm group (`groups` equal parts of the row),
// times the weight; rounded once.  One block a (row, group).
template <typename TO>
__global__ void __launch_bounds__(1024)
ssm_output_kernel(const float* __restrict__ o, const float* __restrict__ prep, int prep_stride, int x_col,
                  const float* __restrict__ proj, int proj_stride, const float* __restrict__ skip,
                  const float* __restrict__ weight, TO* __restrict__ y, int H, int P, int groups, float eps) {
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, grp = blockIdx.y;
    const int inner = H * P, n = inner / groups, c0 = grp * n;
    auto gated = [&](int c) {
        const float x = prep[(size_t)row * prep_stride + x_col + c];
        const float v = fmaf(skip[c / P], x, o[(size_t)row * inner + c]);
        return v * silu_f(proj[(size_t)row * proj_stride + c]);
    };
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = gated(c0 + i);
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        stf(y, (size_t)row * inner + c0 + i, gated(c0 + i) * inv * weight[c0 + i]);
}

// ---- the gated linear recurrent unit ------------------------------------------------------------------------------
// u [rows, width] is cut into `blocks` equal parts of bw; in part b:  r = sigmoid(Wa_b u_b + ba_b), i = sigmoid(Wi_b u_b +
// bi_b), with the matrices given transposed [blocks, in, out] so that neighbouring threads read neighbouring words.
//   log a = -8 r softplus(lam);  a = exp(log a);  coef = sqrt(1 - a^2) i u   (1 - a^2 = -expm1(2 log a)).
// A block of the grid takes one part, 32 of its output channels and kGateRows rows; its four warps split the part's inputs
// into quarters (lane = output channel), and the four partial sums of an output meet in shared memory and are added in
// quarter order: the order of a row's sums depends on the part's size alone.
constexpr int kGateRows = 8;

__global__ void __launch_bounds__(128)
lru_gates_kernel(const float* __restrict__ u, const float* __restrict__ wa_t, const float* __restrict__ ba,
                 const float* __restrict__ wi_t, const float* __restrict__ bi, const float* __restrict__ lam,
                 float* __restrict__ a_out, float* __restrict__ coef_out, int rows, int width, int bw) {
    extern __shared__ float us[];                             // [kGateRows][bw]
    __shared__ float part_a[4][kGateRows][32], part_i[4][kGateRows][32];
    dependents_may_launch();
    wait_for_predecessor();
    const int b = blockIdx.y, r0 = blockIdx.x * kGateRows;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int o = blockIdx.z * 32 + lane;
    const int nr = min(kGateRows, rows - r0);
    for (int i = threadIdx.x; i < kGateRows * bw; i += blockDim.x) {
        const int r = i / bw, k = i % bw;
        us[i] = r < nr ? u[(size_t)(r0 + r) * width + b * bw + k] : 0.0f;
    }
    __syncthreads();
    const float* wa = wa_t + (size_t)b * bw * bw;
    const float* wi = wi_t + (size_t)b * bw * bw;
    const int quarter = (bw + 3) / 4;
    const int k0 = warp * quarter, k1 = min(bw, k0 + quarter);
    float ra[kGateRows], ri[kGateRows];
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) { ra[r] = 0.0f; ri[r] = 0.0f; }
    if (o < bw) {
#pragma unroll 4
        for (int k = k0; k < k1; ++k) {
            const float a = wa[(size_t)k * bw + o], c = wi[(size_t)k * bw + o];
#pragma unroll
            for (int r = 0; r < kGateRows; ++r) {
                const float x = us[r * bw + k];
                ra[r] = fmaf(a, x, ra[r]);
                ri[r] = fmaf(c, x, ri[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) { part_a[warp][r][lane] = ra[r]; part_i[warp][r][lane] = ri[r]; }
    __syncthreads();
    if (o >= bw) return;
    const float sp = softplus_f(lam[b * bw + o]);
    for (int r = warp; r < nr; r += 4) {                      // a warp finishes every fourth row
        const float za = ((part_a[0][r][lane] + part_a[1][r][lane]) + part_a[2][r][lane]) + part_a[3][r][lane] + ba[b * bw + o];
        const float zi = ((part_i[0][r][lane] + part_i[1][r][lane]) + part_i[2][r][lane]) + part_i[3][r][lane] + bi[b * bw + o];
        const float log_a = -8.0f * sigmoid_f(za) * sp;
        const size_t at = (size_t)(r0 + r) * width + b * bw + o;
        a_out[at] = expf(log_a);
        coef_out[at] = sqrtf(-expm1f(2.0f * log_a)) * sigmoid_f(zi) * us[r * bw + o];
    }
}

// S_t = a_t S_(t-1) + coef_t per channel, from and into state[slot][state_off + c]; out[row, c] = S_t *
// gelu_tanh(side[row, c] + side_bias[c]), rounded once.  One thread a (sequence, channel), tokens in order.
template <typename TO>
__global__ void __launch_bounds__(32)
gated_scan_kernel(const float* __restrict__ a, const float* __restrict__ coef, const float* __restrict__ side, int side_stride,
                  const float* __restrict__ side_bias, float* __restrict__ state, size_t state_stride, size_t state_off,
                  const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot, TO* __restrict__ out, int width) {
    dependents_may_launch();
    wait_for_predecessor();
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int r0 = seq_start[seq], r1 = seq_start[seq + 1];
    float* sp = state + (size_t)seq_slot[seq] * state_stride + state_off + c;
    float S = *sp;
    const float sb = side_bias ? side_bias[c] : 0.0f;
    // eight tokens' inputs are fetched before the eight dependent steps that use them: a thread is alone with the latency
    constexpr int AHEAD = 8;
    int row = r0;
    for (; row + AHEAD <= r1; row += AHEAD) {
        float av[AHEAD], cv[AHEAD], sv[AHEAD];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            const size_t at = (size_t)(row + j) * width + c;
            av[j] = a[at];
            cv[j] = coef[at];
            sv[j] = side[(size_t)(row + j) * side_stride + c];
        }
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            S = fmaf(av[j], S, cv[j]);
            stf(out, (size_t)(row + j) * width + c, S * gelu_tanh_f(sv[j] + sb));
        }
    }
    for (; row < r1; ++row) {
        const size_t at = (size_t)row * width + c;
        S = fmaf(a[at], S, coef[at]);
        stf(out, at, S * gelu_tanh_f(side[(size_t)row * side_stride + c] + sb));
    }
    *sp = S;
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_causal_conv(const float* in, int in_stride, const float* in_bias, const float* taps_w, int taps,
                                   const float* bias, int act, float* state, size_t state_stride, size_t conv_off,
                                   const int32_t* row_slot, const int32_t* seq_start, const int32_t* seq_slot, int sequences,
                                   float* out, int out_stride, int rows, int C, int keep, cudaStream_t stream) {
    if (rows <= 0 || C <= 0) return 0;
    if (taps < 1 || (act != 0 && act != 1)) {
        set_last_error("causal_conv: %d taps, activation %d", taps, act);
        return kBadShape;
    }
    const int by = (C + 255) / 256;
    dim3 grid(rows, by < 65535 ? by : 65535);
    launch_kernel(causal_conv_kernel, grid, 256, 0, stream, in, in_stride, in_bias, taps_w, taps, bias, act, (const float*)state,
                  state_stride, conv_off, row_slot, out, out_stride, C);
    int code = CITLALI_LAUNCH_CHECK();
    if (code != 0 || taps == 1 || !keep) return code;
    return citlali_conv_keep(in, in_stride, in_bias, taps, state, state_stride, conv_off, seq_start, seq_slot, sequences, C, stream);
}

extern "C" int citlali_conv_keep(const float* in, int in_stride, const float* in_bias, int taps, float* state,
                                 size_t state_stride, size_t conv_off, const int32_t* seq_start, const int32_t* seq_slot,
                                 int sequences, int C, cudaStream_t stream) {
    if (sequences <= 0 || C <= 0 || taps <= 1) return 0;
    if ((C + 127) / 128 > 65535) {
        set_last_error("conv_keep: %d channels are too many", C);
        return kTooLarge;
    }
    dim3 grid(sequences, (C + 127) / 128);
    launch_kernel(conv_keep_kernel, grid, 128, 0, stream, in, in_stride, in_bias, taps, state, state_stride, conv_off, seq_start,
                  seq_slot, C);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_ssm_prepare(const float* proj, int proj_stride, const float* taps_w, int taps, const float* conv_bias,
                                   float* state, size_t state_stride, size_t conv_off, const int32_t* row_slot,
                                   const int32_t* seq_start, const int32_t* seq_slot, int sequences, const float* a_log,
                                   const float* dt_bias, float* prep, int rows, int H, int P, int G, int N, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || P <= 0 || G <= 0 || N <= 0 || H % G != 0 || taps < 1) {
        set_last_error("ssm_prepare: %d heads of %d over %d groups with a state of %d, %d taps", H, P, G, N, taps);
        return kBadShape;
    }
    const int Cc = H * P + 2 * G * N;
    const int by = (Cc + H + 255) / 256;
    dim3 grid(rows, by < 65535 ? by : 65535);
    launch_kernel(ssm_prepare_kernel, grid, 256, 0, stream, proj, proj_stride, taps_w, taps, conv_bias, (const float*)state,
                  state_stride, conv_off, row_slot, a_log, dt_bias, prep, H, P, G, N);
    int code = CITLALI_LAUNCH_CHECK();
    if (code != 0 || taps == 1) return code;
    return citlali_conv_keep(proj + H * P, proj_stride, nullptr, taps, state, state_stride, conv_off, seq_start, seq_slot,
                             sequences, Cc, stream);
}

extern "C" int citlali_ssm_output(const float* o, const float* prep, int prep_stride, int x_col, const float* proj,
                                  int proj_stride, const float* skip, const float* weight, void* y, int y_dtype, int rows,
                                  int H, int P, int groups, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (groups <= 0 || (H * P) % groups != 0 || groups > 65535) {
        set_last_error("ssm_output: %d channels do not split into %d norm groups", H * P, groups);
        return kBadShape;
    }
    return CITLALI_DISPATCH_FLOAT(y_dtype, TO, [&] {
        dim3 grid(rows, groups);
        const int threads = (H * P) / groups >= 4096 ? 1024 : 256;       // by the group's size alone: one order of sums
        launch_kernel(ssm_output_kernel<TO>, grid, threads, 0, stream, o, prep, prep_stride, x_col, proj, proj_stride, skip, weight,
                      (TO*)y, H, P, groups, eps);
        return CITLALI_LAUNCH_CHECK();
    });
}

extern "C" int citlali_lru_gates(const float* u, const float* wa_t, const float* ba, const float* wi_t, const float* bi,
                                 const float* lam, float* a_out, float* coef_out, int rows, int width, int blocks,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (blocks <= 0 || width % blocks != 0 || blocks > 65535) {
        set_last_error("lru_gates: a width of %d does not split into %d blocks", width, blocks);
        return kBadShape;
    }
    const int bw = width / blocks;
    const size_t smem = (size_t)kGateRows * bw * sizeof(float);
    if (smem > 48 * 1024) {
        set_last_error("lru_gates: gate blocks of %d channels exceed the kernel's 1536", bw);
        return kTooLarge;
    }
    dim3 grid((rows + kGateRows - 1) / kGateRows, blocks, (bw + 31) / 32);
    launch_kernel(lru_gates_kernel, grid, 128, smem, stream, u, wa_t, ba, wi_t, bi, lam, a_out, coef_out, rows, width, bw);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_gated_scan(const float* a, const float* coef, const float* side, int side_stride, const float* side_bias,
                                  float* state, size_t state_stride, size_t state_off, const int32_t* seq_start,
                                  const int32_t* seq_slot, int sequences, void* out, int out_dtype, int width,
                                  cudaStream_t stream) {
    if (sequences <= 0 || width <= 0) return 0;
    if ((width + 31) / 32 > 65535) {
        set_last_error("gated_scan: a width of %d is too large", width);
        return kTooLarge;
    }
    return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
        dim3 grid(sequences, (width + 31) / 32);          // a warp a block: a sequence's channels spread over many SMs
        launch_kernel(gated_scan_kernel<TO>, grid, 32, 0, stream, a, coef, side, side_stride, side_bias, state, state_stride,
                      state_off, seq_start, seq_slot, (TO*)out, width);
        return CITLALI_LAUNCH_CHECK();
    });
}
