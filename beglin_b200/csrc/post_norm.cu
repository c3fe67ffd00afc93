// The norm on a sublayer's RESULT and the residual sum behind it, for layers of the form x <- x + norm(f(x)):
//   y = sum_p part[p][t]  (a product's result, or its split-K partial sums, added in index order)
//   x[t] += y * rsqrt(mean(y^2) + eps) * w;  lowp[t] = x[t] rounded to the compute type (optional)
// The statistics, the scaling and the sum are float.  The rounded copy is what the next sublayer reads, since it takes
// the stream as it is, un-normed: writing it here saves a kernel of its own.
// One block per row; the row of y is held in shared memory between the two passes.  Every row's sum of squares is
// added up in an order fixed by the width alone, so a row does not depend on what else the step holds.
#include <type_traits>

#include "common.cuh"

namespace bg {

template <typename TY, typename TW, typename TL>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* __restrict__ x, const TY* __restrict__ y, int parts, size_t part_stride, const TW* __restrict__ w,
                   float eps, TL* __restrict__ lowp, int d) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * d;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = sum_parts(y + base + i, parts, part_stride);
        row_buf[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = x[base + i] + row_buf[i] * inv * to_float(w[i]);
        x[base + i] = v;
        if (lowp) lowp[base + i] = from_float<TL>(v);
    }
}

// Float partial sums (or one float tensor) of a width that is a multiple of 4, 16-byte aligned: four features a
// thread, the parts' loads in flight together.
template <typename TW, typename TL>
__global__ void __launch_bounds__(256)
rmsnorm_add_vec4_kernel(float* __restrict__ x, const float* __restrict__ y, int parts, size_t part_stride,
                        const TW* __restrict__ w, float eps, TL* __restrict__ lowp, int d) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * d;
    float ss = 0.0f;
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        const float4 v = sum_parts4(reinterpret_cast<const float4*>(y + base + i), parts, part_stride / 4);
        *reinterpret_cast<float4*>(row_buf + i) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row_buf + i);
        float4 o = *reinterpret_cast<const float4*>(x + base + i);
        o.x += v.x * inv * to_float(w[i]);     o.y += v.y * inv * to_float(w[i + 1]);
        o.z += v.z * inv * to_float(w[i + 2]); o.w += v.w * inv * to_float(w[i + 3]);
        *reinterpret_cast<float4*>(x + base + i) = o;
        if (lowp) {
            if constexpr (std::is_same<TL, float>::value) {
                *reinterpret_cast<float4*>(lowp + base + i) = o;
            } else {
                uint2 raw;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
                h[0] = __floats2bfloat162_rn(o.x, o.y);
                h[1] = __floats2bfloat162_rn(o.z, o.w);
                *reinterpret_cast<uint2*>(lowp + base + i) = raw;
            }
        }
    }
}

// Many rows of a bfloat16 step: a warp per row, the row's values in registers (ITER chunks of eight a lane), one trip to
// memory.  The float32 path keeps ONE kernel for every number of rows, so that a row's statistics are added up in the same
// order whatever else the step holds.
template <typename TY, typename TW, int ITER>
__global__ void __launch_bounds__(256)
rmsnorm_add_warp_kernel(float* __restrict__ x, const TY* __restrict__ y, int parts, size_t part_stride, const TW* __restrict__ w,
                        float eps, __nv_bfloat16* __restrict__ lowp, int n_rows, int d) {
    pdl_launch();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const bool idle = warp >= n_rows;
    const size_t base = (size_t)(idle ? 0 : warp) * d;
    const int d8 = d >> 3;
    pdl_wait();
    if (idle) return;
    float v[ITER][8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = lane + 32 * i;
        if (c < d8) {
            load8(y + base + 8 * c, v[i]);
            for (int pp = 1; pp < parts; ++pp) {
                float u[8];
                load8(y + (size_t)pp * part_stride + base + 8 * c, u);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[i][e] += u[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
        }
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = lane + 32 * i;
        if (c < d8) {
            float xv[8], wv[8];
            load8(x + base + 8 * c, xv);
            load8(w + 8 * c, wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) xv[e] += v[i][e] * inv * wv[e];
            store8(x + base + 8 * c, xv);
            if (lowp) store8(lowp + base + 8 * c, xv);
        }
    }
}

// The same behind routed experts: a token's y is the sum of the rows that its `top` chosen experts produced,
// y[t] = sum_j (weights[a] *) yp[row_of[a]], a = t * top + j, added in rank order; the sum that a kernel of its own would
// write and this one read back is formed here.  `vec`: the width is a multiple of 4 and everything 16-byte aligned.
template <typename TW, typename TL>
__global__ void __launch_bounds__(256)
rmsnorm_add_routed_kernel(float* __restrict__ x, const float* __restrict__ yp, const int* __restrict__ row_of,
                          const float* __restrict__ weights, int top, int scale, const TW* __restrict__ w, float eps,
                          TL* __restrict__ lowp, int d, int vec) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const size_t base = (size_t)t * d;
    float ss = 0.0f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int j = 0; j < top; ++j) {
                const int a = t * top + j;
                const float4 v = *reinterpret_cast<const float4*>(yp + (size_t)row_of[a] * d + i);
                const float f = scale ? weights[a] : 1.0f;
                acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
            }
            *reinterpret_cast<float4*>(row_buf + i) = acc;
            ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float acc = 0.0f;
            for (int j = 0; j < top; ++j) {
                const int a = t * top + j;
                const float v = yp[(size_t)row_of[a] * d + i];
                acc += scale ? weights[a] * v : v;
            }
            row_buf[i] = acc;
            ss += acc * acc;
        }
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = x[base + i] + row_buf[i] * inv * to_float(w[i]);
        x[base + i] = v;
        if (lowp) lowp[base + i] = from_float<TL>(v);
    }
}

template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<TO>(x[i]);
}

}  // namespace bg

using namespace bg;

template <typename TY, typename TW, typename TL>
static int rmsnorm_add_launch(float* x, const void* y, int parts, size_t part_stride, const void* w, float eps, void* lowp,
                              int n_rows, int d, cudaStream_t stream) {
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    const bool vec = std::is_same<TY, float>::value && d % 4 == 0 && part_stride % 4 == 0 && (uintptr_t)x % 16 == 0 &&
                     (uintptr_t)y % 16 == 0 && (uintptr_t)lowp % 8 == 0;
    const bool rows_in_registers = std::is_same<TL, __nv_bfloat16>::value && lowp && n_rows >= 64 && d % 8 == 0 && d <= 8 * 32 * 16 &&
                                   part_stride % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                                   (uintptr_t)lowp % 16 == 0;
    if (rows_in_registers) {
        const int iter = (d / 8 + 31) / 32;
        const unsigned blocks = (unsigned)((n_rows + 7) / 8);
#define BG_NORM_ADD_WARP(IT)                                                                                                \
        launch(rmsnorm_add_warp_kernel<TY, TW, IT>, dim3(blocks), dim3(256), 0, stream, x, (const TY*)y, parts, part_stride,     \
               (const TW*)w, eps, (__nv_bfloat16*)lowp, n_rows, d)
        if (iter <= 2) BG_NORM_ADD_WARP(2);
        else if (iter <= 4) BG_NORM_ADD_WARP(4);
        else if (iter <= 8) BG_NORM_ADD_WARP(8);
        else BG_NORM_ADD_WARP(16);
#undef BG_NORM_ADD_WARP
    } else if (vec) {
        auto kern = rmsnorm_add_vec4_kernel<TW, TL>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int threads = ((d / 4 + 31) / 32) * 32;
        threads = threads > 256 ? 256 : (threads < 32 ? 32 : threads);
        launch(kern, dim3(n_rows), dim3(threads), smem, stream, x, (const float*)y, parts, part_stride, (const TW*)w, eps,
               (TL*)lowp, d);
    } else {
        auto kern = rmsnorm_add_kernel<TY, TW, TL>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kern, dim3(n_rows), dim3(256), smem, stream, x, (const TY*)y, parts, part_stride, (const TW*)w, eps, (TL*)lowp, d);
    }
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// y is [T][d] of y_dtype or float [parts][T][d] with part_stride elements between the parts; lowp may be null.
extern "C" int bg_rmsnorm_add(float* x, const void* y, int y_dtype, int parts, long long part_stride, const void* w,
                              int w_dtype, float eps, void* lowp, int lowp_dtype, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (parts < 1 || d <= 0) return BG_ERR_SHAPE;
    if (!lowp) lowp_dtype = BG_DTYPE_F32;
    BG_DISPATCH_DTYPE(y_dtype, TY, BG_DISPATCH_DTYPE(w_dtype, TW, BG_DISPATCH_DTYPE(lowp_dtype, TL,
        return (rmsnorm_add_launch<TY, TW, TL>(x, y, parts, (size_t)part_stride, w, eps, lowp, n_rows, d, stream)))));
    return BG_OK;
}

// x [T][d] += norm(sum over a token's `top` rows of yp [T * top][d] float) * w; lowp may be null.
extern "C" int bg_rmsnorm_add_routed(float* x, const float* yp, const int* row_of, const float* weights, int top, int scale,
                                     const void* w, int w_dtype, float eps, void* lowp, int lowp_dtype, int n_rows, int d,
                                     cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (top < 1 || d <= 0) return BG_ERR_SHAPE;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    if (!lowp) lowp_dtype = BG_DTYPE_F32;
    const int vec = d % 4 == 0 && (uintptr_t)yp % 16 == 0;
    int threads = ((d / 4 + 31) / 32) * 32;
    threads = threads > 256 ? 256 : (threads < 32 ? 32 : threads);
#define BG_ROUTED(TW, TL)                                                                                                   \
    do {                                                                                                                    \
        auto kern = rmsnorm_add_routed_kernel<TW, TL>;                                                                      \
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        launch(kern, dim3(n_rows), dim3(threads), smem, stream, x, yp, row_of, weights, top, scale, (const TW*)w, eps, (TL*)lowp, d, vec); \
    } while (0)
    BG_DISPATCH_DTYPE(w_dtype, TW, BG_DISPATCH_DTYPE(lowp_dtype, TL, BG_ROUTED(TW, TL)));
#undef BG_ROUTED
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    BG_DISPATCH_DTYPE(out_dtype, TO, launch(cast_rows_kernel<TO>, dim3(blocks), dim3(256), 0, stream, x, (TO*)out, n));
    BG_LAUNCH_CHECK();
    return BG_OK;
}
