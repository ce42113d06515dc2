// The walk over a latent cache on the tensor cores (bfloat16 cache; see latent_attention.cu for the mechanism).
//
// All heads of a token look at the same cached vectors [c | r], so sixteen heads of one token are the sixteen rows of
// an m16n8k16 MMA tile: scores S [16 heads, 64 keys] = Q [16, E] . K^T and, with P = softmax weights in bfloat16,
// O [16, R] += P [16, 64] . K[:, :R].  A block of four warps owns one (token, sixteen heads) unit and walks the keys
// lo..pos in tiles of 64: the tile's rows are gathered from the pages into shared memory once (rows past pos are
// zeros), warp w computes the scores of keys 16 w .. 16 w + 15, the row maxima and sums meet in shared memory, and
// warp w accumulates the output columns R/4 w .. R/4 (w + 1).  Softmax is float32 (online, base 2); the sink joins
// the denominator at the end.  In steps of few rows (decoding) a unit's tiles are dealt to several blocks in runs, whose
// unnormalised sums, maxima and denominators a second kernel merges in run order; the number of runs follows the
// number of rows in the step alone, so what else is in the step changes a row by rounding at most.  Needs E a multiple of 16 and R a multiple of 64.
#include "api.h"
#include "common.cuh"
#include "mma_common.cuh"

namespace citlali {

constexpr int kTileKeys = 64;
constexpr int kPStride = kTileKeys + 8;

template <int NTMAX>
__global__ void __launch_bounds__(128, 2)
latent_attention_mma_kernel(const float* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                            const int32_t* __restrict__ page_table, int table_stride,
                            const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                            const float* __restrict__ sink, float* __restrict__ out, int rows, int H, int R, int E,
                            int page_size, int window, float scale, int splits, float* __restrict__ partial) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int ES = E + 8;                                   // row stride in elements: rows start 16 bytes apart in banks
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* Ks = Qs + 16 * ES;
    __nv_bfloat16* Ps = Ks + kTileKeys * ES;
    float* red = reinterpret_cast<float*>(Ps + 16 * kPStride);       // [2][4][16]: the warps' row maxima, row sums
    dependents_may_launch();
    wait_for_predecessor();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int groups = (H + 15) / 16;
    const int unit = blockIdx.x / splits, split = blockIdx.x % splits;
    const int row = unit / groups, h0 = (unit % groups) * 16;
    const int pos = row_pos[row];
    const int32_t* table = page_table + (size_t)row_slot[row] * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    {   // the queries of the sixteen heads, rounded to bfloat16: 16-byte loads, four elements a thread and turn
        const int quads = E / 4;
        for (int hh = 0; hh < 16; ++hh) {
            const bool real = h0 + hh < H;
            const float4* src = reinterpret_cast<const float4*>(q + ((size_t)row * H + h0 + hh) * E);
            for (int i = tid; i < quads; i += 128) {
                const float4 v = real ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<uint2*>(Qs + hh * ES + i * 4) = make_uint2(fa::pack_bf16(v.x, v.y), fa::pack_bf16(v.z, v.w));
            }
        }
    }
    const float sl2 = scale * 1.4426950408889634f;          // scores in units of log 2
    const int NT = R / 32;                                   // tiles of 8 output columns a warp owns
    const int col0 = warp * (R / 4);
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    float O[NTMAX][4];
#pragma unroll
    for (int n = 0; n < NTMAX; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.0f;
    const int chunks = E / 8;                                // 16-byte pieces of a cached vector
    const uint32_t Qs_a = (uint32_t)__cvta_generic_to_shared(Qs), Ks_a = (uint32_t)__cvta_generic_to_shared(Ks),
                   Ps_a = (uint32_t)__cvta_generic_to_shared(Ps);
    // with several blocks a unit, this block walks a run of the unit's tiles; the runs are merged in their order
    const int tiles = (pos - lo) / kTileKeys + 1, per = (tiles + splits - 1) / splits;
    const int first = lo + split * per * kTileKeys;
    const int last = min(pos, first + per * kTileKeys - 1);
    for (int t0 = first; t0 <= last; t0 += kTileKeys) {
        __syncthreads();                                     // the tile before is no longer read; Q is in place
        for (int kr = tid >> 3; kr < kTileKeys; kr += 16) {      // eight threads a cached vector, sixteen vectors a pass
            const int key = t0 + kr;
            __nv_bfloat16* dst = Ks + kr * ES;
            if (key <= pos) {
                const __nv_bfloat16* src = pool + ((size_t)table[key / page_size] * page_size + key % page_size) * E;
                for (int ch = tid & 7; ch < chunks; ch += 8) fa::cp_async16((uint32_t)__cvta_generic_to_shared(dst + ch * 8), src + ch * 8);
            } else {
                for (int ch = tid & 7; ch < chunks; ch += 8) *reinterpret_cast<uint4*>(dst + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        fa::cp_async_commit();
        fa::cp_async_wait<0>();
        __syncthreads();
        // scores of this warp's 16 keys
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const uint32_t a_row = Qs_a + (uint32_t)(((lane & 15) * ES + (lane >> 4) * 8) * 2);
        const uint32_t b_row = Ks_a + (uint32_t)((((warp * 16) + ((lane >> 4) << 3) + (lane & 7)) * ES + ((lane >> 3) & 1) * 8) * 2);
        for (int kk = 0; kk < E; kk += 16) {
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
            fa::ldmatrix_x4(a_row + kk * 2, a0, a1, a2, a3);
            fa::ldmatrix_x4(b_row + kk * 2, b0, b1, b2, b3);
            fa::mma_16816(s[0], a0, a1, a2, a3, b0, b1);
            fa::mma_16816(s[1], a0, a1, a2, a3, b2, b3);
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = t0 + warp * 16 + j * 8 + t * 2 + (c & 1);
                s[j][c] = key <= pos ? s[j][c] * sl2 : -INFINITY;
                if (c < 2) mx0 = fmaxf(mx0, s[j][c]); else mx1 = fmaxf(mx1, s[j][c]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (t == 0) { red[warp * 16 + g] = mx0; red[warp * 16 + g + 8] = mx1; }
        __syncthreads();
        float n0 = m0, n1 = m1;
#pragma unroll
        for (int w = 0; w < 4; ++w) { n0 = fmaxf(n0, red[w * 16 + g]); n1 = fmaxf(n1, red[w * 16 + g + 8]); }
        // the tile's first key is at most pos, so every row has a finite maximum from the first tile on
        const float corr0 = fa::fast_exp2(m0 - n0), corr1 = fa::fast_exp2(m1 - n1);
        m0 = n0; m1 = n1;
        float ps0 = 0.0f, ps1 = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float p0 = fa::fast_exp2(s[j][0] - m0), p1 = fa::fast_exp2(s[j][1] - m0);
            const float p2 = fa::fast_exp2(s[j][2] - m1), p3 = fa::fast_exp2(s[j][3] - m1);
            ps0 += p0 + p1; ps1 += p2 + p3;
            const int kc = warp * 16 + j * 8 + t * 2;
            *reinterpret_cast<uint32_t*>(Ps + g * kPStride + kc) = fa::pack_bf16(p0, p1);
            *reinterpret_cast<uint32_t*>(Ps + (g + 8) * kPStride + kc) = fa::pack_bf16(p2, p3);
        }
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1); ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1); ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
        if (t == 0) { red[64 + warp * 16 + g] = ps0; red[64 + warp * 16 + g + 8] = ps1; }
        __syncthreads();
        l0 *= corr0; l1 *= corr1;
#pragma unroll
        for (int w = 0; w < 4; ++w) { l0 += red[64 + w * 16 + g]; l1 += red[64 + w * 16 + g + 8]; }
#pragma unroll
        for (int n = 0; n < NTMAX; ++n) { O[n][0] *= corr0; O[n][1] *= corr0; O[n][2] *= corr1; O[n][3] *= corr1; }
        // O += P . K[:, this warp's columns]
        const uint32_t p_row = Ps_a + (uint32_t)(((lane & 15) * kPStride + (lane >> 4) * 8) * 2);
        const uint32_t v_row = Ks_a + (uint32_t)(((((lane >> 3) & 1) * 8 + (lane & 7)) * ES + col0 + (lane >> 4) * 8) * 2);
#pragma unroll
        for (int k2 = 0; k2 < kTileKeys; k2 += 16) {
            uint32_t a0, a1, a2, a3;
            fa::ldmatrix_x4(p_row + k2 * 2, a0, a1, a2, a3);
#pragma unroll
            for (int n = 0; n < NTMAX; n += 2) {
                if (n < NT) {
                    uint32_t b0, b1, b2, b3;
                    fa::ldmatrix_x4_trans(v_row + (uint32_t)((k2 * ES + n * 8) * 2), b0, b1, b2, b3);
                    fa::mma_16816(O[n], a0, a1, a2, a3, b0, b1);
                    fa::mma_16816(O[n + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
    }
    if (splits > 1) {
        // unnormalised sums, the running maximum and the denominator of this run: [unit][split][16][R + 2]
        float* dst = partial + ((size_t)unit * splits + split) * 16 * (R + 2);
#pragma unroll
        for (int n = 0; n < NTMAX; ++n) {
            if (n < NT) {
                const int col = col0 + n * 8 + t * 2;
                *reinterpret_cast<float2*>(dst + g * (R + 2) + col) = make_float2(O[n][0], O[n][1]);
                *reinterpret_cast<float2*>(dst + (g + 8) * (R + 2) + col) = make_float2(O[n][2], O[n][3]);
            }
        }
        if (warp == 0 && t == 0) {
            dst[g * (R + 2) + R] = m0; dst[g * (R + 2) + R + 1] = l0;
            dst[(g + 8) * (R + 2) + R] = m1; dst[(g + 8) * (R + 2) + R + 1] = l1;
        }
        return;
    }
    if (sink) {
        const float s0 = h0 + g < H ? sink[h0 + g] * 1.4426950408889634f : -INFINITY;
        const float s1 = h0 + g + 8 < H ? sink[h0 + g + 8] * 1.4426950408889634f : -INFINITY;
        const float n0 = fmaxf(m0, s0), n1 = fmaxf(m1, s1);
        const float c0 = fa::fast_exp2(m0 - n0), c1 = fa::fast_exp2(m1 - n1);
        l0 = l0 * c0 + fa::fast_exp2(s0 - n0);
        l1 = l1 * c1 + fa::fast_exp2(s1 - n1);
#pragma unroll
        for (int n = 0; n < NTMAX; ++n) { O[n][0] *= c0; O[n][1] *= c0; O[n][2] *= c1; O[n][3] *= c1; }
    }
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
#pragma unroll
    for (int n = 0; n < NTMAX; ++n) {
        if (n < NT) {
            const int col = col0 + n * 8 + t * 2;
            if (h0 + g < H)
                *reinterpret_cast<float2*>(out + ((size_t)row * H + h0 + g) * R + col) = make_float2(O[n][0] * inv0, O[n][1] * inv0);
            if (h0 + g + 8 < H)
                *reinterpret_cast<float2*>(out + ((size_t)row * H + h0 + g + 8) * R + col) = make_float2(O[n][2] * inv1, O[n][3] * inv1);
        }
    }
}

// The runs of a unit put together in run order: one block a (row, head), a thread a column at a time.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sink, float* __restrict__ out,
                              int H, int R, int splits) {
    __shared__ float weight[64];
    dependents_may_launch();
    wait_for_predecessor();
    const int groups = (H + 15) / 16, row = blockIdx.x / H, h = blockIdx.x % H;
    const int unit = row * groups + h / 16, hh = h % 16;
    const float* src = partial + (size_t)unit * splits * 16 * (R + 2) + (size_t)hh * (R + 2);
    const size_t run = (size_t)16 * (R + 2);
    float top = sink ? sink[h] * 1.4426950408889634f : -INFINITY;
    const float sk = top;
    for (int s = 0; s < splits; ++s) top = fmaxf(top, src[s * run + R]);
    float denom = sink ? fa::fast_exp2(sk - top) : 0.0f;
    for (int s = 0; s < splits; ++s) denom += src[s * run + R + 1] * fa::fast_exp2(src[s * run + R] - top);   // an empty run: maximum -inf, counts nothing
    if (threadIdx.x < splits) weight[threadIdx.x] = fa::fast_exp2(src[threadIdx.x * run + R] - top) / denom;
    __syncthreads();
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < splits; ++s) acc = fmaf(src[s * run + i], weight[s], acc);
        out[((size_t)row * H + h) * R + i] = acc;
    }
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_latent_attention_mma_supports(int R, int E) {
    return (E % 16 == 0 && R % 64 == 0 && R <= 512 && R <= E && E <= 1024) ? 1 : 0;
}

extern "C" int citlali_latent_attention_mma(const float* q, const void* pool, const int32_t* page_table, int table_stride,
                                            const int32_t* row_slot, const int32_t* row_pos, const float* sink, float* out,
                                            int rows, int H, int R, int E, int page_size, int window, float scale,
                                            int splits, float* partial, size_t partial_floats, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!citlali_latent_attention_mma_supports(R, E)) {
        set_last_error("latent_attention_mma: a latent of %d in a cached vector of %d (multiples of 64 and 16, at most 512 and 1024)", R, E);
        return kBadShape;
    }
    const size_t smem = (size_t)(16 + kTileKeys) * (E + 8) * 2 + 16 * kPStride * 2 + 2 * 4 * 16 * sizeof(float);
    const long units = (long)rows * ((H + 15) / 16);
    if (splits < 1) splits = 1;
    if (splits > 64) splits = 64;
    if (splits > 1 && (size_t)units * splits * 16 * (R + 2) > partial_floats) {
        set_last_error("latent_attention_mma: %d runs a unit need %zu floats of scratch, %zu were given", splits,
                       (size_t)units * splits * 16 * (R + 2), partial_floats);
        return kBadShape;
    }
    const long blocks = units * splits;
    if (blocks > 0x7fffffffL) {
        set_last_error("latent_attention_mma: %d rows of %d heads exceed the grid", rows, H);
        return kTooLarge;
    }
#define CITLALI_LATENT_MMA(NTMAX)                                                                                          \
    do {                                                                                                                 \
        cudaFuncSetAttribute(latent_attention_mma_kernel<NTMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(latent_attention_mma_kernel<NTMAX>, (int)blocks, 128, smem, stream, q, (const __nv_bfloat16*)pool,  \
                      page_table, table_stride, row_slot, row_pos, sink, out, rows, H, R, E, page_size, window, scale,    \
                      splits, partial);                                                                                  \
    } while (0)
    const int nt = R / 32;
    if (nt <= 4) CITLALI_LATENT_MMA(4);
    else if (nt <= 8) CITLALI_LATENT_MMA(8);
    else CITLALI_LATENT_MMA(16);
#undef CITLALI_LATENT_MMA
    int code = CITLALI_LAUNCH_CHECK();
    if (code != 0 || splits == 1) return code;
    launch_kernel(latent_attention_merge_kernel, rows * H, 128, 0, stream, (const float*)partial, sink, out, H, R, splits);
    return CITLALI_LAUNCH_CHECK();
}
