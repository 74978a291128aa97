// Stand-alone ConvertTo: out = SaturateCast<DstT>(alpha * in + beta), element by element, between any two of uint8,
// int8, uint16, int16, int32 and float32, on (N)HWC tensors of equal shape.
//
// Replaces the convertFormat kernel of the reference (src/cvcuda/priv/legacy/convert_to.cu:36-58). The arithmetic is the
// reference test's expectation, tests/cvcuda/system/TestOpConvertTo.cpp:118-133: alpha and beta are doubles, the product
// and the sum are formed in double precision (un-fused), then the saturate cast (round half to even and clamp for the
// integer types, a plain narrowing for float32). Bound: HBM.
#ifndef CVCUDA_B200_CONVERT_KERNELS_CUH
#define CVCUDA_B200_CONVERT_KERNELS_CUH

#include "kparams.h"

namespace b200pp {

struct ConvertKParams
{
    const uint8_t *src;
    uint8_t       *dst;
    long long      sSample, sRow, dSample, dRow;
    int            numSamples, rowElems, height;
    int            srcType, dstType, srcElem, dstElem;
    double         alpha, beta;
};

__device__ __forceinline__ double load_as_double(const uint8_t *p, int dtype)
{
    switch (dtype)
    {
    case B200PP_U8:
        return *p;
    case B200PP_S8:
        return *reinterpret_cast<const signed char *>(p);
    case B200PP_U16:
        return *reinterpret_cast<const unsigned short *>(p);
    case B200PP_S16:
        return *reinterpret_cast<const short *>(p);
    case B200PP_S32:
        return *reinterpret_cast<const int *>(p);
    default:
        return *reinterpret_cast<const float *>(p);
    }
}

__device__ __forceinline__ void store_saturated(uint8_t *p, int dtype, double v)
{
    if (dtype == B200PP_F32)
    {
        *reinterpret_cast<float *>(p) = static_cast<float>(v);
        return;
    }
    const double r = rint(v); // round half to even
    switch (dtype)
    {
    case B200PP_U8:
        *p = static_cast<uint8_t>(fmin(fmax(r, 0.0), 255.0));
        break;
    case B200PP_S8:
        *reinterpret_cast<signed char *>(p) = static_cast<signed char>(fmin(fmax(r, -128.0), 127.0));
        break;
    case B200PP_U16:
        *reinterpret_cast<unsigned short *>(p) = static_cast<unsigned short>(fmin(fmax(r, 0.0), 65535.0));
        break;
    case B200PP_S16:
        *reinterpret_cast<short *>(p) = static_cast<short>(fmin(fmax(r, -32768.0), 32767.0));
        break;
    default:
        *reinterpret_cast<int *>(p) = static_cast<int>(fmin(fmax(r, -2147483648.0), 2147483647.0));
        break;
    }
}

// A thread converts four elements of a row, 32 apart (coalesced across the warp), in each of two rows.
__global__ void __launch_bounds__(256) convert_kernel(const ConvertKParams p)
{
    const int e0 = blockIdx.x * (blockDim.x * 4) + threadIdx.x;
    const int y0 = (blockIdx.y * blockDim.y + threadIdx.y) * 2;
    if (e0 >= p.rowElems)
        return;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const int y = y0 + r;
            if (y >= p.height)
                break;
            const uint8_t *s = p.src + n * p.sSample + y * p.sRow;
            uint8_t       *d = p.dst + n * p.dSample + y * p.dRow;
            double         v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                const int e = min(e0 + 32 * k, p.rowElems - 1);
                v[k]        = load_as_double(s + static_cast<long long>(e) * p.srcElem, p.srcType);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                const int e = e0 + 32 * k;
                if (e < p.rowElems)
                    store_saturated(d + static_cast<long long>(e) * p.dstElem, p.dstType, __dadd_rn(__dmul_rn(p.alpha, v[k]), p.beta));
            }
        }
    }
}

} // namespace b200pp

#endif
