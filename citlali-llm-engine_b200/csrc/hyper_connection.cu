// Hyper-connections: the residual is kept as S parallel streams X [S, rows, W] in float32.  A sub-layer reads one
// mixture of them, u = sum_s in[s] X_s, and its output y goes back into all of them at once,
// X_t <- sum_s mix[s, t] X_s + out[t] y.  With S = 1, in = out = mix = 1 this is the plain residual sum.
//
//   hyper_read_norm   one block a row: u, then u / sqrt(mean(u^2) + eps) * gain, rounded once to the compute dtype.
//   hyper_write       one thread an element of a row: the S old values are read, the S new ones written in place.
//   hyper_write_read_norm   both for one row in one pass: a sub-layer's write-back and the next sub-layer's read.
//   stream_sum        out[i] = sum_s X[s, index[i]]: what the model's last norm reads.
// Also here: the squared ReLU of a feed-forward without a gate.
#include "api.h"
#include "common.cuh"

namespace citlali {

constexpr int kMaxStreams = 8;

template <typename TO>
__global__ void __launch_bounds__(1024)
hyper_read_norm_kernel(const float* __restrict__ X, size_t stream_stride, int S, const float* __restrict__ w_in,
                       const float* __restrict__ gain, TO* __restrict__ out, int W, float eps) {
    extern __shared__ __align__(16) float u[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    float ss = 0.0f;
    if (W % 4 == 0 && stream_stride % 4 == 0) {               // four features a thread and turn, 16-byte loads
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < S; ++s) {
                const float4 xv = *reinterpret_cast<const float4*>(X + s * stream_stride + (size_t)row * W + i);
                const float w = w_in[s];
                v.x = fmaf(w, xv.x, v.x); v.y = fmaf(w, xv.y, v.y); v.z = fmaf(w, xv.z, v.z); v.w = fmaf(w, xv.w, v.w);
            }
            *reinterpret_cast<float4*>(u + i) = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            float v = 0.0f;
            for (int s = 0; s < S; ++s) v = fmaf(w_in[s], X[s * stream_stride + (size_t)row * W + i], v);
            u[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) stf(out, (size_t)row * W + i, u[i] * inv * gain[i]);
}

__global__ void hyper_write_kernel(float* __restrict__ X, size_t stream_stride, int S, const float* __restrict__ y,
                                   const float* __restrict__ w_mix, const float* __restrict__ w_out, size_t n) {
    dependents_may_launch();
    wait_for_predecessor();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        float old[kMaxStreams];
        for (int s = 0; s < S; ++s) old[s] = X[s * stream_stride + e];
        const float yv = y[e];
        for (int t = 0; t < S; ++t) {
            float v = 0.0f;
            for (int s = 0; s < S; ++s) v = fmaf(w_mix[s * S + t], old[s], v);
            X[t * stream_stride + e] = fmaf(w_out[t], yv, v);
        }
    }
}

// hyper_write for one row and, on the new values, the next sub-layer's hyper_read_norm: the streams are read once.
template <typename TO>
__global__ void __launch_bounds__(1024)
hyper_write_read_norm_kernel(float* __restrict__ X, size_t stream_stride, int S, const float* __restrict__ y,
                             const float* __restrict__ w_mix, const float* __restrict__ w_out,
                             const float* __restrict__ w_in, const float* __restrict__ gain, TO* __restrict__ out, int W,
                             float eps) {
    extern __shared__ __align__(16) float u[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    float ss = 0.0f;
    if (W % 4 == 0 && stream_stride % 4 == 0) {               // four features a thread and turn, 16-byte loads and stores
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
            const size_t e = (size_t)row * W + i;
            float4 old[kMaxStreams];
            for (int s = 0; s < S; ++s) old[s] = *reinterpret_cast<const float4*>(X + s * stream_stride + e);
            const float4 yv = *reinterpret_cast<const float4*>(y + e);
            float4 mixed = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int t = 0; t < S; ++t) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int s = 0; s < S; ++s) {
                    const float m = w_mix[s * S + t];
                    v.x = fmaf(m, old[s].x, v.x); v.y = fmaf(m, old[s].y, v.y); v.z = fmaf(m, old[s].z, v.z); v.w = fmaf(m, old[s].w, v.w);
                }
                const float o = w_out[t], wi = w_in[t];
                v.x = fmaf(o, yv.x, v.x); v.y = fmaf(o, yv.y, v.y); v.z = fmaf(o, yv.z, v.z); v.w = fmaf(o, yv.w, v.w);
                *reinterpret_cast<float4*>(X + t * stream_stride + e) = v;
                mixed.x = fmaf(wi, v.x, mixed.x); mixed.y = fmaf(wi, v.y, mixed.y);
                mixed.z = fmaf(wi, v.z, mixed.z); mixed.w = fmaf(wi, v.w, mixed.w);
            }
            *reinterpret_cast<float4*>(u + i) = mixed;
            ss = fmaf(mixed.x, mixed.x, ss); ss = fmaf(mixed.y, mixed.y, ss);
            ss = fmaf(mixed.z, mixed.z, ss); ss = fmaf(mixed.w, mixed.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            const size_t e = (size_t)row * W + i;
            float old[kMaxStreams];
            for (int s = 0; s < S; ++s) old[s] = X[s * stream_stride + e];
            const float yv = y[e];
            float mixed = 0.0f;
            for (int t = 0; t < S; ++t) {
                float v = 0.0f;
                for (int s = 0; s < S; ++s) v = fmaf(w_mix[s * S + t], old[s], v);
                v = fmaf(w_out[t], yv, v);
                X[t * stream_stride + e] = v;
                mixed = fmaf(w_in[t], v, mixed);
            }
            u[i] = mixed;
            ss = fmaf(mixed, mixed, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) stf(out, (size_t)row * W + i, u[i] * inv * gain[i]);
}

__global__ void stream_sum_kernel(const float* __restrict__ X, size_t stream_stride, int S,
                                  const int32_t* __restrict__ index, float* __restrict__ out, int W) {
    dependents_may_launch();
    wait_for_predecessor();
    const size_t src = (size_t)(index ? index[blockIdx.x] : blockIdx.x) * W;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < W; i += gridDim.y * blockDim.x) {
        float v = 0.0f;
        for (int s = 0; s < S; ++s) v += X[s * stream_stride + src + i];
        out[(size_t)blockIdx.x * W + i] = v;
    }
}

template <typename T>
__global__ void relu_squared_kernel(const T* x, T* y, size_t n) {
    dependents_may_launch();
    wait_for_predecessor();
    constexpr int PER = 16 / sizeof(T);                       // elements of a 16-byte access
    const size_t pieces = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 ? n / PER : 0;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < pieces; e += (size_t)gridDim.x * blockDim.x) {
        uint4 w = reinterpret_cast<const uint4*>(x)[e];
        T* v = reinterpret_cast<T*>(&w);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const float f = fmaxf(ldf(v, j), 0.0f);
            stf(v, j, f * f);
        }
        reinterpret_cast<uint4*>(y)[e] = w;
    }
    for (size_t e = pieces * PER + (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(ldf(x, e), 0.0f);
        stf(y, e, v * v);
    }
}

static int grid_for(size_t n) {
    const size_t blocks = (n + 255) / 256;
    return (int)(blocks < 8192 ? blocks : 8192);
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_hyper_read_norm(const float* X, size_t stream_stride, int streams, const float* w_in,
                                       const float* gain, void* out, int out_dtype, int rows, int width, float eps,
                                       cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (streams < 1 || smem > 200 * 1024) {
        set_last_error("hyper_read_norm: %d streams of width %d", streams, width);
        return kBadShape;
    }
    return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(hyper_read_norm_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // few rows in bfloat16 (decoding): a row is spread over more threads; 32-bit keeps one order of summation
        launch_kernel(hyper_read_norm_kernel<TO>, rows, (sizeof(TO) == 2 && rows < 128 && width >= 2048) ? 1024 : 256, smem, stream, X, stream_stride, streams, w_in, gain, (TO*)out,
                      width, eps);
        return CITLALI_LAUNCH_CHECK();
    });
}

extern "C" int citlali_hyper_write(float* X, size_t stream_stride, int streams, const float* y, const float* w_mix,
                                   const float* w_out, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    if (streams < 1 || streams > kMaxStreams) {
        set_last_error("hyper_write: %d streams (1 to %d are taken)", streams, kMaxStreams);
        return kBadShape;
    }
    launch_kernel(hyper_write_kernel, grid_for(n), 256, 0, stream, X, stream_stride, streams, y, w_mix, w_out, n);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_hyper_write_read_norm(float* X, size_t stream_stride, int streams, const float* y, const float* w_mix,
                                             const float* w_out, const float* w_in, const float* gain, void* out,
                                             int out_dtype, int rows, int width, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (streams < 1 || streams > kMaxStreams || smem > 200 * 1024) {
        set_last_error("hyper_write_read_norm: %d streams of width %d", streams, width);
        return kBadShape;
    }
    return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(hyper_write_read_norm_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_kernel(hyper_write_read_norm_kernel<TO>, rows, (sizeof(TO) == 2 && rows < 128 && width >= 2048) ? 1024 : 256, smem, stream, X, stream_stride, streams, y, w_mix, w_out,
                      w_in, gain, (TO*)out, width, eps);
        return CITLALI_LAUNCH_CHECK();
    });
}

extern "C" int citlali_stream_sum(const float* X, size_t stream_stride, int streams, const int32_t* index, float* out,
                                  int rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    dim3 grid(rows, rows < 64 ? (width + 255) / 256 : 1);          // few rows: a row's columns over several blocks
    launch_kernel(stream_sum_kernel, grid, 256, 0, stream, X, stream_stride, streams, index, out, width);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_relu_squared(const void* x, void* y, int dtype, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    return CITLALI_DISPATCH_FLOAT(dtype, T, [&] {
        launch_kernel(relu_squared_kernel<T>, grid_for(n), 256, 0, stream, (const T*)x, (T*)y, n);
        return CITLALI_LAUNCH_CHECK();
    });
}
