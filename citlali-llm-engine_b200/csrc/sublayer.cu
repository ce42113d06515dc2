// Kernels of a layer whose norm sits on the sub-layer's OUTPUT:  x <- x + layer_norm(sublayer(x)).
//
//   layer_norm_add   x[r] += (y[r] - mean) / sqrt(var + eps) * w  (var = mean of squared deviations, no bias), all
//                    32-bit; optionally the updated row is also left in the compute dtype for the sub-layer that reads
//                    it next, so that the residual is read once.
//   layer_norm_rows  out[i] = layer_norm(x[index[i]]) * w, rounded once (the model's last norm).
//   cast_rows        float32 -> the compute dtype.
//   scaled_sum       out = a * l + b * r (two mixers side by side).
// One block a row; the row waits in shared memory between the passes (mean, then deviations, then the store), so every
// row is read from global memory once.
#include "api.h"
#include "common.cuh"

namespace citlali {

template <typename TG, typename TE>
__global__ void __launch_bounds__(256)
layer_norm_add_kernel(const float* __restrict__ y, const TG* __restrict__ gain, float* __restrict__ x, TE* __restrict__ emit,
                      int hidden, float eps) {
    extern __shared__ float row_s[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = y + (size_t)row * hidden;
    float s = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i];
        row_s[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_s[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    float* dst = x + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = dst[i] + (row_s[i] - mean) * inv * ldf(gain, i);
        dst[i] = v;
        if (emit) stf(emit, (size_t)row * hidden + i, v);
    }
}

template <typename TG, typename TO>
__global__ void __launch_bounds__(256)
layer_norm_rows_kernel(const float* __restrict__ x, const TG* __restrict__ gain, const int32_t* __restrict__ row_index,
                       TO* __restrict__ out, int hidden, float eps) {
    extern __shared__ float row_s[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[row] : row) * hidden;
    float s = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i];
        row_s[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_s[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        stf(out, (size_t)row * hidden + i, (row_s[i] - mean) * inv * ldf(gain, i));
}

template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, size_t n) {
    dependents_may_launch();
    wait_for_predecessor();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) stf(out, i, x[i]);
}

__global__ void scaled_sum_kernel(float a, const float* __restrict__ l, float b, const float* __restrict__ r,
                                  float* __restrict__ out, size_t n) {
    dependents_may_launch();
    wait_for_predecessor();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = a * l[i] + b * r[i];
}

static int grid_for(size_t n) {
    const size_t blocks = (n + 255) / 256;
    return (int)(blocks < 8192 ? (blocks ? blocks : 1) : 8192);
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_layer_norm_add(const float* y, const void* gain, int gain_dtype, float* x, void* emit, int emit_dtype,
                                      int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (hidden <= 0 || smem > 200 * 1024) {
        set_last_error("layer_norm_add: rows of %d elements do not fit a block's shared memory", hidden);
        return kTooLarge;
    }
    return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
        return CITLALI_DISPATCH_FLOAT(emit_dtype, TE, [&] {
            auto kernel = layer_norm_add_kernel<TG, TE>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            launch_kernel(kernel, rows, 256, smem, stream, y, (const TG*)gain, x, (TE*)emit, hidden, eps);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_layer_norm_rows(const float* x, const void* gain, int gain_dtype, const int32_t* row_index, void* out,
                                       int out_dtype, int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (hidden <= 0 || smem > 200 * 1024) {
        set_last_error("layer_norm_rows: rows of %d elements do not fit a block's shared memory", hidden);
        return kTooLarge;
    }
    return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
        return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
            auto kernel = layer_norm_rows_kernel<TG, TO>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            launch_kernel(kernel, rows, 256, smem, stream, x, (const TG*)gain, row_index, (TO*)out, hidden, eps);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_cast_rows(const float* x, void* out, int out_dtype, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
        launch_kernel(cast_rows_kernel<TO>, grid_for(n), 256, 0, stream, x, (TO*)out, n);
        return CITLALI_LAUNCH_CHECK();
    });
}

extern "C" int citlali_scaled_sum(float a, const float* l, float b, const float* r, float* out, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    launch_kernel(scaled_sum_kernel, grid_for(n), 256, 0, stream, a, l, b, r, out, n);
    return CITLALI_LAUNCH_CHECK();
}
