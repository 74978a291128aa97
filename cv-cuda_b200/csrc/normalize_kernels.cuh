// Stand-alone Normalize: out = SaturateCast((in - base) * mul * globalScale + shift), mul = scale or
// 1 / sqrt(scale^2 + epsilon), element by element on interleaved images of 1 to 4 channels, dense tensors or
// variable-shape batches on both sides; base and scale are float32 tensors that may be broadcast along any of the
// sample, row, column and channel dimensions (a stride of zero).
//
// Replaces the normalize kernels of the reference (src/cvcuda/priv/legacy/normalize.cu,
// src/cvcuda/priv/legacy/normalize_var_shape.cu); arithmetic follows the reference's CPU golden
// (tests/cvcuda/system/TestOpNormalize.cpp:34-77): float32, un-fused, in source order; rint + clamp is the saturate cast.
// Bound: HBM (every element read once, written once).
#ifndef CVCUDA_B200_NORMALIZE_KERNELS_CUH
#define CVCUDA_B200_NORMALIZE_KERNELS_CUH

#include "device_math.cuh"
#include "plain_resize_kernels.cuh"

namespace b200pp {

struct NormalizeKParams
{
    PlainSide    src, dst;
    int          numSamples, channels;
    int          srcType, dstType, srcElem, dstElem;
    const float *base, *scale;
    long long    baseStride[4], scaleStride[4]; // bytes per step along sample, row, column, channel; 0 = broadcast
    float        gscale, shift, epsilon;
    int          stddev;
};

// One thread per pixel (all channels), two rows per thread for a little more memory-level parallelism.
__global__ void __launch_bounds__(256) normalize_kernel(const NormalizeKParams p)
{
    const int x  = blockIdx.x * blockDim.x + threadIdx.x;
    const int y0 = (blockIdx.y * blockDim.y + threadIdx.y) * 2;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const PlainView S = plain_view(p.src, n), D = plain_view(p.dst, n);
        const int       w = min(S.w, D.w), h = min(S.h, D.h);
        if (x >= w)
            continue;
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const int y = y0 + r;
            if (y >= h)
                break;
            const uint8_t *sp = S.base + y * S.pitch + static_cast<long long>(x) * p.channels * p.srcElem;
            uint8_t       *dp = D.base + y * D.pitch + static_cast<long long>(x) * p.channels * p.dstElem;
            const char    *bp = reinterpret_cast<const char *>(p.base) + n * p.baseStride[0] + y * p.baseStride[1] + x * p.baseStride[2];
            const char    *cp = reinterpret_cast<const char *>(p.scale) + n * p.scaleStride[0] + y * p.scaleStride[1] + x * p.scaleStride[2];
            for (int c = 0; c < p.channels; ++c)
            {
                const float v = load_any(sp + c * p.srcElem, p.srcType);
                const float b = *reinterpret_cast<const float *>(bp + c * p.baseStride[3]);
                const float s = *reinterpret_cast<const float *>(cp + c * p.scaleStride[3]);
                const float m = p.stddev ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(s, s), p.epsilon))) : s;
                store_any(dp + c * p.dstElem, p.dstType, __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, b), m), p.gscale), p.shift));
            }
        }
    }
}

} // namespace b200pp

#endif
