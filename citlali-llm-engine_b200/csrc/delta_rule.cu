// The gated delta rule: a recurrent mixer whose state per head is a matrix S [D, V] in float32.
//
// For every token, with unit vectors q and k (q also times D^-1/2), a value v, a write strength beta in (0, 1) and a
// decay g in (0, 1):   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
// The columns of S do not meet: column j only ever needs v[j], so four lanes own one column in registers and walk
// their sequence's tokens in order.  One order of operations serves prompts, parts of prompts and single tokens, so the
// state and the outputs do not depend on how a sequence was cut into steps.
//
// Three kernels:
//   delta_prepare   one warp a (row, q head / k head / head's values): the short causal convolution over time of the q, k, v channels (earlier tokens
//                   from the step's rows or, before its first row, from the sequence's kept inputs), SiLU, unit length
//                   for q and k heads, beta = sigmoid(.), g = exp(-exp(A_log) softplus(. + dt_bias)).  All float32.
//                   A second launch then moves the sequence's last taps-1 inputs into its state.
//   delta_rule      one warp a (sequence, head, 8 columns), four lanes a column: the recurrence.
//   delta_output    one warp a (row, head): each head's output divided by its root mean square, times a weight, times
//                   SiLU(gate); rounded once to the compute dtype.
#include "api.h"
#include "common.cuh"

namespace citlali {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Head h's write strength beta_h = sigmoid(row[beta_col + h]) and its decays, by the `threads` threads (this one is number
// `tid` of them) that own the head's values.  One decay a head: g_h = exp(-exp(a_log[h]) softplus(pre[h] + dt_bias[h])),
// pre = row[decay_col ...] or, if given, decay_row.  One a key channel (GD = D): g_(h,i) = exp(-exp(a_log[h])
// softplus(decay_row[h D + i] + dt_bias[h D + i])).  dst receives beta [H] | g [H GD].
__device__ __forceinline__ void write_strength_and_decay(const float* __restrict__ row, int beta_col, int decay_col,
                                                         const float* __restrict__ decay_row, const float* __restrict__ a_log,
                                                         const float* __restrict__ dt_bias, float* __restrict__ dst, int H, int GD,
                                                         int h, int tid, int threads) {
    if (tid == 0) dst[h] = sigmoidf_(row[beta_col + h]);
    const float rate = expf(a_log[h]);
    for (int j = tid; j < GD; j += threads) {
        const int i = h * GD + j;
        const float pre = decay_row ? decay_row[i] : row[decay_col + i];
        dst[H + i] = expf(-rate * softplusf_(pre + dt_bias[i]));
    }
}

// proj [rows, proj_stride] float32 holds, per row: q (KH*D) | k (KH*D) | v (H*V) | gate (H*V) | b (H) | a (H).
// prep [rows, C + 2H] receives q^ | k^ | v | beta | g, C = 2 KH D + H V.
// conv_state [slot] is [taps-1, C]: the inputs at the sequence's last taps-1 positions, oldest first.
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ taps_w, int taps,
                     const float* __restrict__ state, size_t state_stride, size_t conv_off,
                     const int32_t* __restrict__ row_slot, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, float* __restrict__ prep, int H, int KH, int D, int V, float unit_eps,
                     int beta_col, int decay_col, const float* __restrict__ decay_in, int decay_stride, int channel_decay) {
    dependents_may_launch();
    wait_for_predecessor();
    // A warp: one row and one segment of its channels (a q head, a k head, or a head's values); eight segments a block.
    const int row = blockIdx.x, lane = threadIdx.x & 31;
    const int seg = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int C = 2 * KH * D + H * V;
    const int GD = channel_decay ? D : 1;                          // decays a head: one, or one a key channel
    float* dst = prep + (size_t)row * (C + H + H * GD);
    if (seg >= 2 * KH && seg < 2 * KH + H)
        write_strength_and_decay(proj + (size_t)row * proj_stride, beta_col, decay_col,
                                 decay_in ? decay_in + (size_t)row * decay_stride : nullptr, a_log, dt_bias, dst + C, H, GD,
                                 seg - 2 * KH, lane, 32);
    if (seg >= 2 * KH + H) return;
    const bool unit = seg < 2 * KH;                           // q and k heads are made unit vectors
    const int c0 = unit ? seg * D : 2 * KH * D + (seg - 2 * KH) * V, n = unit ? D : V;
    const int slot = row_slot[row];
    int in_step = 0;                        // how many of the tokens before this one are rows of this step
    while (in_step < taps - 1 && row - in_step - 1 >= 0 && row_slot[row - in_step - 1] == slot) ++in_step;
    const float* kept = state + (size_t)slot * state_stride + conv_off;
    auto convolved = [&](int i) {
        const int c = c0 + i;
        float acc = 0.0f;
        for (int back = taps - 1; back >= 0; --back) {        // `back` tokens back; oldest first
            float x;
            if (back <= in_step) x = proj[(size_t)(row - back) * proj_stride + c];
            else x = kept[(size_t)(taps - 1 - back + in_step) * C + c];
            acc = fmaf(taps_w[(size_t)c * taps + (taps - 1 - back)], x, acc);
        }
        return siluf_(acc);
    };
    // a lane's channels are lane, lane + 32, ...: the first eight stay in registers between the two passes, a longer
    // segment parks the rest in the output row
    float keep[8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = lane + 32 * j;
        keep[j] = i < n ? convolved(i) : 0.0f;
        ss = fmaf(keep[j], keep[j], ss);
    }
    for (int i = lane + 256; i < n; i += 32) {
        const float v = convolved(i);
        dst[c0 + i] = v;
        ss = fmaf(v, v, ss);
    }
    float f = 1.0f;
    if (unit) {
        ss = warp_sum(ss);
        f = 1.0f / sqrtf(ss + unit_eps);
        if (seg < KH) f /= sqrtf((float)D);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = lane + 32 * j;
        if (i < n) dst[c0 + i] = keep[j] * f;
    }
    for (int i = lane + 256; i < n; i += 32) dst[c0 + i] *= f;
}

// The same with a block of 128 threads a segment, a thread a channel: for steps of few rows, where a row's segments
// are all the parallelism there is.  (It sums a head's squares in another order than the kernel above.)
__global__ void __launch_bounds__(128)
delta_prepare_block_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ taps_w, int taps,
                     const float* __restrict__ state, size_t state_stride, size_t conv_off,
                     const int32_t* __restrict__ row_slot, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, float* __restrict__ prep, int H, int KH, int D, int V, float unit_eps,
                     int beta_col, int decay_col, const float* __restrict__ decay_in, int decay_stride, int channel_decay) {
    extern __shared__ float act[];          // max(D, V) floats
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    // A block: one row and one segment of its channels: a q head, a k head, or a head's values.
    const int row = blockIdx.x, seg = blockIdx.y;
    const int C = 2 * KH * D + H * V;
    const bool unit = seg < 2 * KH;                           // q and k heads are made unit vectors
    const int c0 = unit ? seg * D : 2 * KH * D + (seg - 2 * KH) * V, n = unit ? D : V;
    const int slot = row_slot[row];
    int in_step = 0;                        // how many of the tokens before this one are rows of this step
    while (in_step < taps - 1 && row - in_step - 1 >= 0 && row_slot[row - in_step - 1] == slot) ++in_step;
    const float* kept = state + (size_t)slot * state_stride + conv_off;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int c = c0 + i;
        float acc = 0.0f;
        for (int j = taps - 1; j >= 0; --j) {                 // j tokens back; oldest first
            float x;
            if (j <= in_step) x = proj[(size_t)(row - j) * proj_stride + c];
            else x = kept[(size_t)(taps - 1 - j + in_step) * C + c];
            acc = fmaf(taps_w[(size_t)c * taps + (taps - 1 - j)], x, acc);
        }
        const float v = siluf_(acc);
        act[i] = v;
        ss = fmaf(v, v, ss);
    }
    float f = 1.0f;
    if (unit) {
        ss = block_sum(ss, scratch);
        f = 1.0f / sqrtf(ss + unit_eps);
        if (seg < KH) f /= sqrtf((float)D);
    }
    const int GD = channel_decay ? D : 1;
    float* dst = prep + (size_t)row * (C + H + H * GD);
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[c0 + i] = act[i] * f;      // a thread reads back what it wrote
    if (seg >= 2 * KH)
        write_strength_and_decay(proj + (size_t)row * proj_stride, beta_col, decay_col,
                                 decay_in ? decay_in + (size_t)row * decay_stride : nullptr, a_log, dt_bias, dst + C, H, GD,
                                 seg - 2 * KH, threadIdx.x, blockDim.x);
}

// After the step's rows were convolved: the sequence keeps its last taps-1 inputs.  One thread a channel.
__global__ void delta_conv_state_kernel(const float* __restrict__ proj, int proj_stride, int taps, float* __restrict__ state,
                                        size_t state_stride, size_t conv_off, const int32_t* __restrict__ seq_start,
                                        const int32_t* __restrict__ seq_slot, int C) {
    dependents_may_launch();
    wait_for_predecessor();
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r0 = seq_start[seq], n = seq_start[seq + 1] - r0, keep = taps - 1;
    float* kept = state + (size_t)seq_slot[seq] * state_stride + conv_off;
    if (n >= keep) {
        for (int i = 0; i < keep; ++i) kept[(size_t)i * C + c] = proj[(size_t)(r0 + n - keep + i) * proj_stride + c];
    } else {
        for (int i = 0; i < keep - n; ++i) kept[(size_t)i * C + c] = kept[(size_t)(i + n) * C + c];
        for (int i = 0; i < n; ++i) kept[(size_t)(keep - n + i) * C + c] = proj[(size_t)(r0 + i) * proj_stride + c];
    }
}

// One warp a (sequence, head, 8 columns of S); four lanes share a column and hold a quarter of its rows each (the
// 16-byte groups of rows g with g mod 4 = the lane's part, so that the four parts read neighbouring words of shared
// memory; eight lanes a column were measured slower: a token's fixed work then weighs more than its sums).  DP: the head size rounded up to a multiple of 32; rows of S beyond D stay zero.  The two dot products of a
// token are summed over a lane's rows first and over the four lanes after, in one fixed order.  The inputs of the next
// tokens (seven, or three for heads over 128) are on their way into a ring in shared memory (cp.async) while the current token is computed.
// MODE 0: one decay a head.  MODE 1: a decay a key channel (row i of S is multiplied by g_i; the token's D decays follow
// its query in the ring).  MODE 2: no correction term, u = beta v (a state-space recurrence S <- g S + beta k v^T,
// o = S^T q, with the step size as beta).
template <int DP, int MODE>
__global__ void __launch_bounds__(128)
delta_rule_kernel(const float* __restrict__ prep, int prep_stride, float* __restrict__ state, size_t state_stride,
                  const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot, int sequences,
                  int H, int KH, int D, int V, float* __restrict__ out, int pairs) {
    // tokens in flight from global memory (a warp is alone with their latency); fewer where a token takes more of the 48 KB
    constexpr int STAGES = MODE == 1 ? (DP <= 96 ? 8 : (DP <= 192 ? 4 : 3)) : (DP <= 128 ? 8 : 4);
    constexpr int VOFF = MODE == 1 ? 3 * DP : 2 * DP;   // where a token's scalars start in its place of the ring
    constexpr int STRIDE = VOFF + 16;            // floats a token takes in the ring: k | q | (decays) | v of 8 columns | beta | g
    __shared__ __align__(16) float ring[4][STAGES][STRIDE];
    dependents_may_launch();
    wait_for_predecessor();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = lane & 3;
    const int chunks = (V + 7) / 8;
    const long unit = (long)blockIdx.x * 4 + warp;
    if (unit >= (long)sequences * H * chunks) return;
    const int chunk = (int)(unit % chunks);
    const int head = (int)((unit / chunks) % H);
    const int seq = (int)(unit / ((long)chunks * H));
    const int col = chunk * 8 + (lane >> 2);
    const bool live = col < V;
    const int kv_head = head / (H / KH);
    const int C = 2 * KH * D + H * V;
    const int r0 = seq_start[seq], r1 = seq_start[seq + 1];
    float* S_g = state + (size_t)seq_slot[seq] * state_stride + (size_t)head * D * V + col;
    constexpr int GROUPS = DP / 16;              // 16-byte groups of rows a lane holds
    float S[GROUPS][4];
#pragma unroll
    for (int j = 0; j < GROUPS; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = (4 * j + part) * 4 + e;
            S[j][e] = (live && i < D) ? S_g[(size_t)i * V] : 0.0f;
        }
    constexpr int PER = DP / 32;
    for (int i = lane; i < STAGES * STRIDE; i += 32) (&ring[warp][0][0])[i] = 0.0f;     // rows beyond D and dead columns stay zero
    __syncwarp();
    auto issue = [&](int row) {                  // the row's inputs into its place in the ring, asynchronously
        if (row < r1) {
            const float* p = prep + (size_t)row * prep_stride;
            float* dst = ring[warp][(row - r0) % STAGES];
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int i = j * 32 + lane;
                if (i < D) {
                    cp_async4(dst + i, p + (KH + kv_head) * D + i);
                    cp_async4(dst + DP + i, p + kv_head * D + i);
                    if (MODE == 1) cp_async4(dst + 2 * DP + i, p + C + H + head * D + i);
                }
            }
            if (lane < 8 && chunk * 8 + lane < V) cp_async4(dst + VOFF + lane, p + 2 * KH * D + head * V + chunk * 8 + lane);
            if (lane == 8) cp_async4(dst + VOFF + 8, p + C + head);
            if (MODE != 1 && lane == 9) cp_async4(dst + VOFF + 9, p + C + H + head);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int s = 0; s < STAGES - 1; ++s) issue(r0 + s);
    int row = r0;
    if (MODE == 0 && pairs) {
        // Two tokens at a time.  With S the state before both, every sum over the rows of S is taken against S itself,
        //   a1 = S^T k1, a2 = S^T k2, b1 = S^T q1, b2 = S^T q2   (four independent chains over the lane's rows),
        // and the rest are scalars of the head (k1.k2, q1.k1, q2.k1, q2.k2) and of the column:
        //   u1 = beta1 (v1 - g1 a1);            o1 = g1 b1 + u1 (q1.k1)
        //   u2 = beta2 (v2 - g2 (g1 a2 + u1 (k1.k2)));   o2 = g2 (g1 b2 + u1 (q2.k1)) + u2 (q2.k2)
        //   S <- g2 g1 S + k1 (g2 u1) + k2 u2.
        // The same numbers as two single steps up to rounding; half the dependent steps a token.
        for (; row + 1 < r1; row += 2) {
            asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 3) : "memory");
            __syncwarp();
            issue(row + STAGES - 1);                      // into the place of the row before this pair
            const float* c1 = ring[warp][(row - r0) % STAGES];
            const float* c2 = ring[warp][(row + 1 - r0) % STAGES];
            float kk = 0.0f, q1k1 = 0.0f, q2k1 = 0.0f, q2k2 = 0.0f;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int i = j * 32 + lane;
                const float a = c1[i], b = c2[i], c = c1[DP + i], d = c2[DP + i];
                kk = fmaf(a, b, kk); q1k1 = fmaf(c, a, q1k1); q2k1 = fmaf(d, a, q2k1); q2k2 = fmaf(d, b, q2k2);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                kk += __shfl_xor_sync(0xffffffffu, kk, o);
                q1k1 += __shfl_xor_sync(0xffffffffu, q1k1, o);
                q2k1 += __shfl_xor_sync(0xffffffffu, q2k1, o);
                q2k2 += __shfl_xor_sync(0xffffffffu, q2k2, o);
            }
            const float v1 = c1[2 * DP + (lane >> 2)], beta1 = c1[2 * DP + 8], g1 = c1[2 * DP + 9];
            const float v2 = c2[2 * DP + (lane >> 2)], beta2 = c2[2 * DP + 8], g2 = c2[2 * DP + 9];
            float a1x = 0.f, a1y = 0.f, a2x = 0.f, a2y = 0.f, b1x = 0.f, b1y = 0.f, b2x = 0.f, b2y = 0.f;
            float4 k1r[GROUPS], k2r[GROUPS];
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                const int at = (4 * j + part) * 4;
                k1r[j] = *reinterpret_cast<const float4*>(c1 + at);
                k2r[j] = *reinterpret_cast<const float4*>(c2 + at);
                const float4 q1 = *reinterpret_cast<const float4*>(c1 + DP + at);
                const float4 q2 = *reinterpret_cast<const float4*>(c2 + DP + at);
                a1x = fmaf(S[j][0], k1r[j].x, a1x); a1y = fmaf(S[j][1], k1r[j].y, a1y);
                a1x = fmaf(S[j][2], k1r[j].z, a1x); a1y = fmaf(S[j][3], k1r[j].w, a1y);
                a2x = fmaf(S[j][0], k2r[j].x, a2x); a2y = fmaf(S[j][1], k2r[j].y, a2y);
                a2x = fmaf(S[j][2], k2r[j].z, a2x); a2y = fmaf(S[j][3], k2r[j].w, a2y);
                b1x = fmaf(S[j][0], q1.x, b1x); b1y = fmaf(S[j][1], q1.y, b1y);
                b1x = fmaf(S[j][2], q1.z, b1x); b1y = fmaf(S[j][3], q1.w, b1y);
                b2x = fmaf(S[j][0], q2.x, b2x); b2y = fmaf(S[j][1], q2.y, b2y);
                b2x = fmaf(S[j][2], q2.z, b2x); b2y = fmaf(S[j][3], q2.w, b2y);
            }
            float a1 = a1x + a1y, a2 = a2x + a2y, b1 = b1x + b1y, b2 = b2x + b2y;
#pragma unroll
            for (int o = 1; o <= 2; o <<= 1) {
                a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                a2 += __shfl_xor_sync(0xffffffffu, a2, o);
                b1 += __shfl_xor_sync(0xffffffffu, b1, o);
                b2 += __shfl_xor_sync(0xffffffffu, b2, o);
            }
            const float u1 = beta1 * (v1 - g1 * a1);
            const float o1 = fmaf(u1, q1k1, g1 * b1);
            const float u2 = beta2 * (v2 - g2 * fmaf(u1, kk, g1 * a2));
            const float o2 = fmaf(u2, q2k2, g2 * fmaf(u1, q2k1, g1 * b2));
            const float gg = g1 * g2, w1 = g2 * u1;
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                S[j][0] = fmaf(k2r[j].x, u2, fmaf(k1r[j].x, w1, gg * S[j][0]));
                S[j][1] = fmaf(k2r[j].y, u2, fmaf(k1r[j].y, w1, gg * S[j][1]));
                S[j][2] = fmaf(k2r[j].z, u2, fmaf(k1r[j].z, w1, gg * S[j][2]));
                S[j][3] = fmaf(k2r[j].w, u2, fmaf(k1r[j].w, w1, gg * S[j][3]));
            }
            if (live && part == 0) {
                out[(size_t)row * H * V + head * V + col] = o1;
                out[(size_t)(row + 1) * H * V + head * V + col] = o2;
            }
            __syncwarp();                                 // both rows' places are read for the last time
            issue(row + STAGES);
        }
    }
    for (; row < r1; ++row) {
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncwarp();                            // this row's inputs are visible; the row before is no longer read
        issue(row + STAGES - 1);
        const float* cur = ring[warp][(row - r0) % STAGES];
        const float* ks = cur;
        const float* qs = cur + DP;
        const float v = cur[VOFF + (lane >> 2)], beta = cur[VOFF + 8];
        const float g = MODE == 1 ? 1.0f : cur[VOFF + 9];
        if (MODE == 1) {                         // every row of S decays by its own factor before it is read
            const float* gs = cur + 2 * DP;
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                const float4 g4 = *reinterpret_cast<const float4*>(gs + (4 * j + part) * 4);
                S[j][0] *= g4.x; S[j][1] *= g4.y; S[j][2] *= g4.z; S[j][3] *= g4.w;
            }
        }
        float u;
        if (MODE == 2) {
            u = beta * v;
        } else {
            float sk0 = 0.0f, sk1 = 0.0f, sk2 = 0.0f, sk3 = 0.0f;
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + (4 * j + part) * 4);
                sk0 = fmaf(S[j][0], k4.x, sk0); sk1 = fmaf(S[j][1], k4.y, sk1);
                sk2 = fmaf(S[j][2], k4.z, sk2); sk3 = fmaf(S[j][3], k4.w, sk3);
            }
            float sk = (sk0 + sk1) + (sk2 + sk3);
            sk += __shfl_xor_sync(0xffffffffu, sk, 1);
            sk += __shfl_xor_sync(0xffffffffu, sk, 2);
            u = beta * (v - g * sk);
        }
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int j = 0; j < GROUPS; ++j) {
            const float4 k4 = *reinterpret_cast<const float4*>(ks + (4 * j + part) * 4);
            const float4 q4 = *reinterpret_cast<const float4*>(qs + (4 * j + part) * 4);
            S[j][0] = fmaf(k4.x, u, g * S[j][0]); o0 = fmaf(S[j][0], q4.x, o0);
            S[j][1] = fmaf(k4.y, u, g * S[j][1]); o1 = fmaf(S[j][1], q4.y, o1);
            S[j][2] = fmaf(k4.z, u, g * S[j][2]); o2 = fmaf(S[j][2], q4.z, o2);
            S[j][3] = fmaf(k4.w, u, g * S[j][3]); o3 = fmaf(S[j][3], q4.w, o3);
        }
        float o = (o0 + o1) + (o2 + o3);
        o += __shfl_xor_sync(0xffffffffu, o, 1);
        o += __shfl_xor_sync(0xffffffffu, o, 2);
        if (live && part == 0) out[(size_t)row * H * V + head * V + col] = o;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (live) {
#pragma unroll
        for (int j = 0; j < GROUPS; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = (4 * j + part) * 4 + e;
                if (i < D) S_g[(size_t)i * V] = S[j][e];
            }
    }
}

// y[row, h, :] = o[row, h, :] / sqrt(mean(o^2) + eps) * weight * act(gate[row, h, :]), act = SiLU (gate_act 0) or the
// sigmoid (1).  One warp a head.
template <typename TO>
__global__ void __launch_bounds__(256)
delta_output_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride,
                    const float* __restrict__ weight, TO* __restrict__ y, int H, int V, float eps, int gate_act) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int h = blockIdx.y * warps + warp; h < H; h += gridDim.y * warps) {
        const float* src = o + ((size_t)row * H + h) * V;
        float ss = 0.0f;
        for (int i = lane; i < V; i += 32) ss = fmaf(src[i], src[i], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)V + eps);
        const float* gt = gate + (size_t)row * gate_stride + h * V;
        for (int i = lane; i < V; i += 32)
            stf(y, ((size_t)row * H + h) * V + i, src[i] * inv * weight[i] * (gate_act == 1 ? sigmoidf_(gt[i]) : siluf_(gt[i])));
    }
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_delta_prepare(const float* proj, int proj_stride, const float* taps_w, int taps, float* state,
                                     size_t state_stride, size_t conv_off, const int32_t* row_slot,
                                     const int32_t* seq_start, const int32_t* seq_slot, int sequences,
                                     const float* a_log, const float* dt_bias, float* prep, int rows, int H, int KH,
                                     int D, int V, float unit_eps, int block_a_segment, int beta_col, int decay_col,
                                     const float* decay_in, int decay_stride, int channel_decay, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || KH <= 0 || H % KH != 0 || D <= 0 || V <= 0 || taps < 1 || (channel_decay && !decay_in)) {
        set_last_error("delta_prepare: %d heads over %d key heads of %d, values of %d, %d taps (a decay per channel comes in a buffer of its own)", H, KH, D, V, taps);
        return kBadShape;
    }
    const int C = 2 * KH * D + H * V;
    const int segments = 2 * KH + H;
    if ((segments + 7) / 8 > 65535) {
        set_last_error("delta_prepare: %d segments a row are too many", segments);
        return kTooLarge;
    }
    if (block_a_segment) {
        const size_t smem = (size_t)(D > V ? D : V) * sizeof(float);
        if (smem > 48 * 1024 || segments > 65535) {
            set_last_error("delta_prepare: heads of %d and values of %d, or %d segments a row, are too many", D, V, segments);
            return kTooLarge;
        }
        dim3 prepare_grid(rows, segments);
        launch_kernel(delta_prepare_block_kernel, prepare_grid, 128, smem, stream, proj, proj_stride, taps_w, taps,
                      (const float*)state, state_stride, conv_off, row_slot, a_log, dt_bias, prep, H, KH, D, V, unit_eps,
                      beta_col, decay_col, decay_in, decay_stride, channel_decay);
    } else {
        dim3 prepare_grid(rows, (segments + 7) / 8);
        launch_kernel(delta_prepare_kernel, prepare_grid, 256, 0, stream, proj, proj_stride, taps_w, taps, (const float*)state,
                      state_stride, conv_off, row_slot, a_log, dt_bias, prep, H, KH, D, V, unit_eps, beta_col, decay_col,
                      decay_in, decay_stride, channel_decay);
    }
    int code = CITLALI_LAUNCH_CHECK();
    if (code != 0 || taps == 1) return code;
    dim3 grid(sequences, (C + 127) / 128);
    launch_kernel(delta_conv_state_kernel, grid, 128, 0, stream, proj, proj_stride, taps, state, state_stride, conv_off,
                  seq_start, seq_slot, C);
    return CITLALI_LAUNCH_CHECK();
}

template <int MODE>
static int launch_delta_rule(const float* prep, int prep_stride, float* state, size_t state_stride, const int32_t* seq_start,
                             const int32_t* seq_slot, int sequences, int H, int KH, int D, int V, float* out, int pairs,
                             cudaStream_t stream) {
    const long units = (long)sequences * H * ((V + 7) / 8);
    const int blocks = (int)((units + 3) / 4);
#define CITLALI_DELTA(DP)                                                                                         \
    launch_kernel(delta_rule_kernel<DP, MODE>, blocks, 128, 0, stream, prep, prep_stride, state, state_stride, seq_start, \
                  seq_slot, sequences, H, KH, D, V, out, pairs)
    switch ((D + 31) / 32) {
        case 1: CITLALI_DELTA(32); break;
        case 2: CITLALI_DELTA(64); break;
        case 3: CITLALI_DELTA(96); break;
        case 4: CITLALI_DELTA(128); break;
        case 5: CITLALI_DELTA(160); break;
        case 6: CITLALI_DELTA(192); break;
        case 7: CITLALI_DELTA(224); break;
        default: CITLALI_DELTA(256); break;
    }
#undef CITLALI_DELTA
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_delta_rule(const float* prep, int prep_stride, float* state, size_t state_stride,
                                  const int32_t* seq_start, const int32_t* seq_slot, int sequences, int H, int KH, int D,
                                  int V, float* out, int pairs, int mode, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if (D > 256) {
        set_last_error("delta_rule: a head size of %d exceeds 256", D);
        return kTooLarge;
    }
    if (mode < 0 || mode > 2 || H <= 0 || KH <= 0 || H % KH != 0) {
        set_last_error("delta_rule: form %d, %d heads over %d key heads", mode, H, KH);
        return kBadShape;
    }
    if (mode == 1) return launch_delta_rule<1>(prep, prep_stride, state, state_stride, seq_start, seq_slot, sequences, H, KH, D, V, out, 0, stream);
    if (mode == 2) return launch_delta_rule<2>(prep, prep_stride, state, state_stride, seq_start, seq_slot, sequences, H, KH, D, V, out, 0, stream);
    return launch_delta_rule<0>(prep, prep_stride, state, state_stride, seq_start, seq_slot, sequences, H, KH, D, V, out, pairs, stream);
}

extern "C" int citlali_delta_output(const float* o, const float* gate, int gate_stride, const float* weight, void* y,
                                    int y_dtype, int rows, int H, int V, float eps, int gate_act, cudaStream_t stream) {
    if (rows <= 0) return 0;
    return CITLALI_DISPATCH_FLOAT(y_dtype, TO, [&] {
        dim3 grid(rows, (H + 7) / 8 < 64 ? (H + 7) / 8 : 64);             // a warp a head, eight heads a block
        launch_kernel(delta_output_kernel<TO>, grid, 256, 0, stream, o, gate, gate_stride, weight, (TO*)y, H, V, eps, gate_act);
        return CITLALI_LAUNCH_CHECK();
    });
}
