// Device-side arithmetic of the fused pre-processing kernels.
//
// Every float operation is an explicit round-to-nearest intrinsic so that nothing is contracted into a fused
// multiply-add: results then equal the reference's CPU golden code bit for bit
// (tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:118-168,
//  tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:86-145).
#ifndef CVCUDA_B200_DEVICE_MATH_CUH
#define CVCUDA_B200_DEVICE_MATH_CUH

#include "kparams.h"

#include <cuda_fp16.h>

namespace b200pp {

// ---- saturating, round-half-to-even conversions (cuda::SaturateCast semantics,
//      cvcuda/cuda_tools/detail/SaturateCastImpl.hpp:118-157)

__device__ __forceinline__ unsigned sat_u8(float v)
{
    unsigned r;
    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ int sat_s8(float v)
{
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ unsigned short sat_u16(float v)
{
    unsigned short r;
    asm("cvt.rni.sat.u16.f32 %0, %1;" : "=h"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ short sat_s16(float v)
{
    short r;
    asm("cvt.rni.sat.s16.f32 %0, %1;" : "=h"(r) : "f"(v));
    return r;
}

// float(byte i of `word`) without a conversion instruction: selector 0x7540 + i makes PRMT build 0x4B0000bb, the float
// 2^23 + bb, and the subtraction of 2^23 is exact.
__device__ __forceinline__ float byte_as_float(unsigned word, unsigned selector)
{
    return __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, selector)), 8388608.0f);
}

// Store one value of the resize path (uint8 / float32 / float16 destinations).
template<int DK>
__device__ __forceinline__ void store_elem(uint8_t *ptr, float v)
{
    if constexpr (DK == DST_F32)
        *reinterpret_cast<float *>(ptr) = v;
    else if constexpr (DK == DST_F16)
        *reinterpret_cast<__half *>(ptr) = __float2half_rn(v);
    else
        *ptr = static_cast<uint8_t>(sat_u8(v));
}

// Store one value of the slice path (any B200PP_* element type, chosen at run time).
__device__ __forceinline__ void store_any(uint8_t *ptr, int dtype, float v)
{
    switch (dtype)
    {
    case B200PP_U8:
        *ptr = static_cast<uint8_t>(sat_u8(v));
        break;
    case B200PP_S8:
        *reinterpret_cast<signed char *>(ptr) = static_cast<signed char>(sat_s8(v));
        break;
    case B200PP_U16:
        *reinterpret_cast<unsigned short *>(ptr) = sat_u16(v);
        break;
    case B200PP_S16:
        *reinterpret_cast<short *>(ptr) = sat_s16(v);
        break;
    case B200PP_U32:
        *reinterpret_cast<unsigned *>(ptr) = __float2uint_rn(v);
        break;
    case B200PP_S32:
        *reinterpret_cast<int *>(ptr) = __float2int_rn(v);
        break;
    case B200PP_F32:
        *reinterpret_cast<float *>(ptr) = v;
        break;
    default:
        *reinterpret_cast<__half *>(ptr) = __float2half_rn(v);
        break;
    }
}

__device__ __forceinline__ float load_any(const uint8_t *ptr, int dtype)
{
    switch (dtype)
    {
    case B200PP_U8:
        return static_cast<float>(*ptr);
    case B200PP_S8:
        return static_cast<float>(*reinterpret_cast<const signed char *>(ptr));
    case B200PP_U16:
        return static_cast<float>(*reinterpret_cast<const unsigned short *>(ptr));
    case B200PP_S16:
        return static_cast<float>(*reinterpret_cast<const short *>(ptr));
    case B200PP_U32:
        return static_cast<float>(*reinterpret_cast<const unsigned *>(ptr));
    case B200PP_S32:
        return static_cast<float>(*reinterpret_cast<const int *>(ptr));
    default:
        return *reinterpret_cast<const float *>(ptr);
    }
}

// ---- sampling coordinates

// Linear taps along one axis for destination coordinate d (crop offset already added):
//   f = scale*(d + 0.5) - 0.5; s0 = floor(f); s1 = min(s0+1, size-1); w1 = f - s0 (before clamping); s0 = max(0, s0).
// The extra clamp of s0 to size-1 never changes a legal case and keeps every read inside the image.
__device__ __forceinline__ void linear_tap(float scale, int d, int size, int &s0, int &s1, float &w1)
{
    const float f  = __fsub_rn(__fmul_rn(scale, __fadd_rn(static_cast<float>(d), 0.5f)), 0.5f);
    const int   i0 = __float2int_rd(f);
    s1             = min(i0 + 1, size - 1);
    w1             = __fsub_rn(f, static_cast<float>(i0));
    s0             = min(max(0, i0), size - 1);
    s1             = max(s1, 0);
}

// Nearest tap: floor(scale*(d + 0.5)), clamped into the image for safety only.
__device__ __forceinline__ int nearest_tap(float scale, int d, int size)
{
    const int s = __float2int_rd(__fmul_rn(scale, __fadd_rn(static_cast<float>(d), 0.5f)));
    return min(max(s, 0), size - 1);
}

// ((p00*wy0)*wx0 + (p01*wy0)*wx1 + (p10*wy1)*wx0 + (p11*wy1)*wx1), left to right.
__device__ __forceinline__ float blend4(float p00, float p01, float p10, float p11, float wx0, float wx1, float wy0,
                                        float wy1)
{
    const float a = __fmul_rn(__fmul_rn(p00, wy0), wx0);
    const float b = __fmul_rn(__fmul_rn(p01, wy0), wx1);
    const float c = __fmul_rn(__fmul_rn(p10, wy1), wx0);
    const float d = __fmul_rn(__fmul_rn(p11, wy1), wx1);
    return __fadd_rn(__fadd_rn(__fadd_rn(a, b), c), d);
}

// scale*v + offset, or (v - base)*mul*gscale + shift, un-fused.
__device__ __forceinline__ float affine(const ResizeKParams &p, int c, float v)
{
    if (!p.perChannel)
        return __fadd_rn(__fmul_rn(p.scale, v), p.offset);
    return __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, p.base[c]), p.mul[c]), p.gscale), p.shift);
}

// Eight float32 values as one 256-bit store (sm_100); `d` is 32-byte aligned.
__device__ __forceinline__ void store_f32x8(uint8_t *d, float a, float b, float c, float e, float f, float g, float h, float i)
{
    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(d), "f"(a), "f"(b), "f"(c), "f"(e), "f"(f), "f"(g),
                 "f"(h), "f"(i)
                 : "memory");
}

// ---- per-sample source geometry

struct Geom
{
    const uint8_t *base;  // first byte of the (sub-view of the) image
    const uint8_t *image; // first byte of the whole image (alignment checks)
    long long      pitch;
    int            w, h;
    int            flip;
    float          scaleW, scaleH;
};

__device__ __forceinline__ Geom load_geom(const ResizeKParams &p, int n)
{
    Geom g;
    if (p.list)
    {
        const B200ppImagePlane &pl = p.list[n].planes[0];
        g.base  = pl.basePtr;
        g.pitch = pl.rowStride;
        g.w     = pl.width;
        g.h     = pl.height;
    }
    else
    {
        g.base  = p.srcBase + static_cast<long long>(n) * p.srcSampleStride;
        g.pitch = p.srcRowStride;
        g.w     = p.srcW;
        g.h     = p.srcH;
    }
    g.image = g.base;
    if (p.roi)
    {
        // The rectangle is intersected with the image before anything is addressed through it; a rectangle that misses the
        // image, or has no area, shrinks to the nearest single pixel. For rectangles inside the image (the contract)
        // nothing changes.
        const int *r  = reinterpret_cast<const int *>(reinterpret_cast<const char *>(p.roi) + n * p.roiStride);
        const int  x0 = min(max(r[0], 0), max(g.w - 1, 0)), y0 = min(max(r[1], 0), max(g.h - 1, 0));
        const int  x1 = min(max(r[0] + max(r[2], 1), x0 + 1), max(g.w, 1)), y1 = min(max(r[1] + max(r[3], 1), y0 + 1), max(g.h, 1));
        g.base += static_cast<long long>(y0) * g.pitch + 3LL * x0;
        g.w = x1 - x0;
        g.h = y1 - y0;
    }
    g.flip = p.flip ? p.flip[n] : 2;
    if (p.list || p.roi)
    {
        g.scaleW = __fdiv_rn(static_cast<float>(g.w), static_cast<float>(p.resizeW));
        g.scaleH = __fdiv_rn(static_cast<float>(g.h), static_cast<float>(p.resizeH));
    }
    else
    {
        g.scaleW = p.denseScaleW;
        g.scaleH = p.denseScaleH;
    }
    return g;
}

} // namespace b200pp

#endif
