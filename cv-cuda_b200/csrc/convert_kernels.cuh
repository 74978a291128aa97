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

// 8-bit sources: the 256 possible results are computed once per CTA with the arithmetic above and kept in shared
// memory; an element then costs one shared-memory lookup. A thread handles four 4-byte words of source, 32 words apart
// (a warp reads 128 contiguous bytes and writes 128 x DE), in each of two or four rows per pass. DE = destination element bytes. Needs
// source rows on 4-byte and destination rows on 4 x DE-byte boundaries (the caller checks).
template<int DE>
__global__ void __launch_bounds__(256, 5) convert_lut_kernel(const ConvertKParams p)
{
    __shared__ unsigned lut[256];
    {
        const int    t = threadIdx.y * blockDim.x + threadIdx.x; // 256 threads
        const double v = p.srcType == B200PP_U8 ? static_cast<double>(t) : static_cast<double>(static_cast<signed char>(t));
        unsigned     bits = 0;
        store_saturated(reinterpret_cast<uint8_t *>(&bits), p.dstType, __dadd_rn(__dmul_rn(p.alpha, v), p.beta));
        lut[t] = bits;
    }
    __syncthreads();
    constexpr int RPT      = DE == 4 ? 2 : 4; // rows per thread and pass: keeps 32 to 64 bytes of loads in flight per thread
    const int     w0       = blockIdx.x * (blockDim.x * 4) + threadIdx.x;
    const int     rowWords = (p.rowElems + 3) >> 2;
    if (w0 >= rowWords)
        return;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        // the grid's y extent may be smaller than the image: CTAs walk down in steps, so the table is built less often
        for (int yb = blockIdx.y; yb * (blockDim.y * RPT) < p.height; yb += gridDim.y)
        {
            const int y0 = (yb * blockDim.y + threadIdx.y) * RPT;
            unsigned  q[RPT][4];
            // the row's last word may reach up to three bytes past its last element: still inside the aligned word
            // that holds that element, so the load cannot leave the allocation's pages
#pragma unroll
            for (int r = 0; r < RPT; ++r)
            {
                const unsigned *s = reinterpret_cast<const unsigned *>(p.src + n * p.sSample + min(y0 + r, p.height - 1) * p.sRow);
#pragma unroll
                for (int k = 0; k < 4; ++k) q[r][k] = __ldg(s + min(w0 + 32 * k, rowWords - 1));
            }
#pragma unroll
            for (int r = 0; r < RPT; ++r)
            {
                const int y = y0 + r;
                if (y >= p.height)
                    break;
                uint8_t *d = p.dst + n * p.dSample + y * p.dRow;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                {
                    const int w = w0 + 32 * k;
                    if (w >= rowWords)
                        break;
                    const unsigned v  = q[r][k];
                    const unsigned o0 = lut[v & 255u], o1 = lut[(v >> 8) & 255u], o2 = lut[(v >> 16) & 255u], o3 = lut[v >> 24];
                    const int      count = min(4, p.rowElems - 4 * w);
                    uint8_t       *out   = d + static_cast<long long>(w) * (4 * DE);
                    if (count == 4)
                    {
                        if constexpr (DE == 4)
                            *reinterpret_cast<uint4 *>(out) = make_uint4(o0, o1, o2, o3);
                        else if constexpr (DE == 2)
                            *reinterpret_cast<uint2 *>(out) = make_uint2(o0 | (o1 << 16), o2 | (o3 << 16));
                        else
                            *reinterpret_cast<unsigned *>(out) = o0 | (o1 << 8) | (o2 << 16) | (o3 << 24);
                    }
                    else
                    {
                        const unsigned o[3] = {o0, o1, o2};
                        for (int j = 0; j < count; ++j)
                        {
                            if constexpr (DE == 4)
                                reinterpret_cast<unsigned *>(out)[j] = o[j];
                            else if constexpr (DE == 2)
                                reinterpret_cast<unsigned short *>(out)[j] = static_cast<unsigned short>(o[j]);
                            else
                                out[j] = static_cast<uint8_t>(o[j]);
                        }
                    }
                }
            }
        }
    }
}

// float32 sources: a thread converts two groups of four adjacent elements (one 16-byte load each, 32 groups apart) in
// each of two rows and stores each group's results as one word / 8 bytes / 16 bytes, with the arithmetic of
// convert_kernel. DE = destination element bytes. Needs source rows on 16-byte and destination rows on 4 x DE-byte
// boundaries (the caller checks); the ragged end of a row goes element by element.
template<int DE>
__global__ void __launch_bounds__(256) convert_f32_kernel(const ConvertKParams p)
{
    const int g0        = blockIdx.x * (blockDim.x * 2) + threadIdx.x;
    const int y0        = (blockIdx.y * blockDim.y + threadIdx.y) * 2;
    const int rowGroups = (p.rowElems + 3) >> 2;
    if (g0 >= rowGroups)
        return;
    const float alphaF = static_cast<float>(p.alpha), betaF = static_cast<float>(p.beta);
    const float errB   = __fmul_rn(fabsf(betaF), 4.76837158203125e-07f); // |beta| * 2^-21
    const float loF = p.dstType == B200PP_U8 || p.dstType == B200PP_U16 ? 0.0f : (DE == 1 ? -128.0f : -32768.0f);
    const float hiF = p.dstType == B200PP_U8 ? 255.0f : (p.dstType == B200PP_S8 ? 127.0f : (p.dstType == B200PP_U16 ? 65535.0f : 32767.0f));
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        float4 v[2][2];
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const uint8_t *s = p.src + n * p.sSample + min(y0 + r, p.height - 1) * p.sRow;
#pragma unroll
            for (int k = 0; k < 2; ++k)
            {
                const int g = min(g0 + 32 * k, rowGroups - 1);
                if (4 * g + 4 <= p.rowElems)
                    v[r][k] = __ldg(reinterpret_cast<const float4 *>(s) + g);
                else
                {
                    asm volatile("" ::: "memory"); // the ragged end of a row stays a branch, not predicated loads
                    const float *f = reinterpret_cast<const float *>(s) + 4 * g;
                    const int    c = p.rowElems - 4 * g;
                    v[r][k]        = make_float4(f[0], c > 1 ? f[1] : 0.f, c > 2 ? f[2] : 0.f, 0.f);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const int y = y0 + r;
            if (y >= p.height)
                break;
            uint8_t *d = p.dst + n * p.dSample + y * p.dRow;
#pragma unroll
            for (int k = 0; k < 2; ++k)
            {
                const int g = g0 + 32 * k;
                if (g >= rowGroups)
                    break;
                const float in[4] = {v[r][k].x, v[r][k].y, v[r][k].z, v[r][k].w};
                unsigned    o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    o[j] = 0;
                    if constexpr (DE <= 2)
                    {
                        // Integer destinations of 8 or 16 bits: t = alpha * x + beta in float32 first (one fused multiply-add). It
                        // differs from the double-precision value by less than (|alpha x| + |beta| + |t|) * 2^-24 <= err / 4 with
                        // err = (|alpha x| + |beta|) * 2^-21. Clamped to the type's range, t is rounded half to even by adding
                        // 1.5 * 2^23 (the integer is then the low bits of the sum, two's complement for negative results). If t is
                        // further than err from a rounding boundary (and err <= 0.5, which keeps a clamped value clamped), the
                        // double-precision value rounds and clamps to the same integer; everything else -- ties, huge factors,
                        // NaN, infinities (the comparison is false for them) -- is done again in double precision.
                        const float t   = __fmaf_rn(alphaF, in[j], betaF);
                        const float err = __fmaf_rn(fabsf(__fmul_rn(alphaF, in[j])), 4.76837158203125e-07f, errB);
                        const float tc  = fminf(fmaxf(t, loF), hiF);
                        const float rb  = __fadd_rn(tc, 12582912.0f);
                        if (__fadd_rn(fabsf(__fsub_rn(tc, __fsub_rn(rb, 12582912.0f))), err) <= 0.5f)
                        {
                            o[j] = __float_as_uint(rb) & (DE == 1 ? 0xffu : 0xffffu);
                            continue;
                        }
                        asm volatile("" ::: "memory"); // the exact redo stays a branch
                    }
                    store_saturated(reinterpret_cast<uint8_t *>(&o[j]), p.dstType,
                                    __dadd_rn(__dmul_rn(p.alpha, static_cast<double>(in[j])), p.beta));
                }
                const int count = min(4, p.rowElems - 4 * g);
                uint8_t  *out   = d + static_cast<long long>(g) * (4 * DE);
                if (count == 4)
                {
                    if constexpr (DE == 4)
                        *reinterpret_cast<uint4 *>(out) = make_uint4(o[0], o[1], o[2], o[3]);
                    else if constexpr (DE == 2)
                        *reinterpret_cast<uint2 *>(out) = make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
                    else
                        *reinterpret_cast<unsigned *>(out) = o[0] | (o[1] << 8) | (o[2] << 16) | (o[3] << 24);
                }
                else
                {
                    asm volatile("" ::: "memory"); // likewise for the stores
#pragma unroll
                    for (int j = 0; j < 3; ++j)
                        if (j < count)
                        {
                            if constexpr (DE == 4)
                                reinterpret_cast<unsigned *>(out)[j] = o[j];
                            else if constexpr (DE == 2)
                                reinterpret_cast<unsigned short *>(out)[j] = static_cast<unsigned short>(o[j]);
                            else
                                out[j] = static_cast<uint8_t>(o[j]);
                        }
                }
            }
        }
    }
}

} // namespace b200pp

#endif
