// TEST INFRASTRUCTURE ONLY -- never linked into, loaded by, or called from the product library.
//
// C-callable wrapper around the reference project's own CPU golden functions, so that the C
// restatement in preproc_oracle.c can be pinned against the real thing.
//
// The golden functions live inside gtest translation units that cannot be compiled as they are
// (googletest is absent), so build_oracle.py cuts the two function templates out of the reference tree
// at build time into a scratch directory (REF_GOLDEN_RCCR_INC / REF_GOLDEN_CFNR_INC), compiles this
// file against them plus the reference's header-only host helpers, and deletes the scratch files.
// Nothing from the reference is stored in this repository.
//
//   tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:76-172   ResizeCropConvert<DstT,SrcT>
//   tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:43-149   CropFlipNormalizeReformat<T_Src,T_Dst,B>
//   tests/cvcuda/system/ResizeUtils.cpp:189-300                      test::resizedCrop<T> (stand-alone Resize golden)
//   tests/common/InterpUtils.hpp:38-89                               test::ValueAt
//   tests/common/BorderUtils.cpp:24-137                              test::IsInside + border index rules
//   cvcuda/cuda_tools/SaturateCast.hpp                               cuda::SaturateCast (host path)

#include <cuda_runtime.h> // int2, long4 (vector types only; no runtime call is made)

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

// Stand-ins for the two object-model classes the golden code queries. The real ones call into
// libnvcv_types, which is not built here; the golden functions only ask for these two counts.
namespace nvcv {
struct ImageFormat
{
    int channels, planes;

    int numChannels() const
    {
        return channels;
    }

    int numPlanes() const
    {
        return planes;
    }
};

struct Size2D
{
    int w, h;
};
} // namespace nvcv

#include <common/InterpUtils.hpp>
#include <cvcuda/OpNormalize.h> // CVCUDA_NORMALIZE_SCALE_IS_STDDEV
#include <cvcuda/Types.h>
#include <cvcuda/cuda_tools/SaturateCast.hpp>
#include <nvcv/Rect.h>
#include <nvcv/Size.h>

// tests/common/BorderUtils.cpp is a plain source file with no main(): compile it in place.
#include <common/BorderUtils.cpp>

namespace test = nvcv::test;
namespace cuda = nvcv::cuda;

#include REF_GOLDEN_RCCR_INC
#include REF_GOLDEN_CFNR_INC

// tests/cvcuda/system/ResizeUtils.cpp:189-300  nvcv::test::resizedCrop<T> (nearest / linear / cubic), cut by signature
#include <cassert>
#include <limits>
namespace nvcv::test {
#include REF_GOLDEN_RESIZE_INC
} // namespace nvcv::test

namespace {

template<typename S, typename D>
int cfnr_border(int border, std::vector<uint8_t> &hDst, long4 outStrides, std::vector<uint8_t> &hSrc, long4 inStrides,
                nvcv::Size2D srcSize, nvcv::Size2D dstSize, nvcv::ImageFormat fmt, nvcv::ImageFormat dstFmt,
                float borderValue, int flip, NVCVRectI rect, const std::vector<float> &base, nvcv::ImageFormat baseFmt,
                const std::vector<float> &scale, nvcv::ImageFormat scaleFmt, float gScale, float gShift, float eps,
                uint32_t flags)
{
#define CALL(B)                                                                                                      \
    CropFlipNormalizeReformat<S, D, B>(hDst, 0, outStrides, hSrc, 0, inStrides, srcSize, dstSize, fmt, dstFmt,       \
                                       borderValue, flip, rect, base, 0, {1, 1}, baseFmt, scale, 0, {1, 1}, scaleFmt, \
                                       gScale, gShift, eps, flags);                                                  \
    return 0
    switch (border)
    {
    case NVCV_BORDER_CONSTANT:
        CALL(NVCV_BORDER_CONSTANT);
    case NVCV_BORDER_REPLICATE:
        CALL(NVCV_BORDER_REPLICATE);
    case NVCV_BORDER_REFLECT:
        CALL(NVCV_BORDER_REFLECT);
    case NVCV_BORDER_WRAP:
        CALL(NVCV_BORDER_WRAP);
    case NVCV_BORDER_REFLECT101:
        CALL(NVCV_BORDER_REFLECT101);
    }
#undef CALL
    return -1;
}

template<typename S, typename... A>
int cfnr_dst(int dstType, A &&...a)
{
    switch (dstType)
    {
    case 0:
        return cfnr_border<S, uint8_t>(a...);
    case 1:
        return cfnr_border<S, int8_t>(a...);
    case 2:
        return cfnr_border<S, uint16_t>(a...);
    case 3:
        return cfnr_border<S, int16_t>(a...);
    case 4:
        return cfnr_border<S, uint32_t>(a...);
    case 5:
        return cfnr_border<S, int32_t>(a...);
    case 6:
        return cfnr_border<S, float>(a...);
    }
    return -1;
}

const int kTypeSize[7] = {1, 1, 2, 2, 4, 4, 4};

} // namespace

extern "C"
{
// Dense batch of packed (unpadded) interleaved 3-channel uint8 images -> packed output.
// dstIsFloat: 0 = uint8 output, 1 = float32 output.  dstPlanar: 0 = NHWC, 1 = NCHW.
int ref_rccr(void *dst, int dstW, int dstH, int dstPlanar, int dstIsFloat, const uint8_t *src, int srcW, int srcH,
             int numImages, int newW, int newH, int cropX, int cropY, int interp, int manip, float scale,
             float offset, int srcCast)
{
    nvcv::ImageFormat srcFmt{3, 1}, dstFmt{3, dstPlanar ? 3 : 1};
    NVCVSize2D        dstSize{dstW, dstH}, srcSize{srcW, srcH}, newSize{newW, newH};
    int2              crop{cropX, cropY};
    if (dstIsFloat)
        ResizeCropConvert((float *)dst, dstSize, dstFmt, src, srcSize, srcFmt, numImages, newSize, crop,
                          (NVCVInterpolationType)interp, (NVCVChannelManip)manip, scale, offset, srcCast != 0);
    else
        ResizeCropConvert((uint8_t *)dst, dstSize, dstFmt, src, srcSize, srcFmt, numImages, newSize, crop,
                          (NVCVInterpolationType)interp, (NVCVChannelManip)manip, scale, offset, srcCast != 0);
    return 0;
}

// One image. Type codes: 0 u8, 1 s8, 2 u16, 3 s16, 4 u32, 5 s32, 6 f32. Source and destination are
// packed (no row padding); planar flags select CHW vs HWC. base/scale hold baseCh / scaleCh floats.
int ref_cfnr(void *dst, int dstType, int dstPlanar, int dstW, int dstH, const void *src, int srcType, int srcPlanar,
             int srcW, int srcH, int channels, int border, float borderValue, int flip, int cropX, int cropY,
             int cropW, int cropH, const float *base, int baseCh, const float *scale, int scaleCh, float gScale,
             float gShift, float eps, uint32_t flags)
{
    if (dstType < 0 || dstType > 6 || srcType < 0 || srcType > 6)
        return -1;
    const long ss = kTypeSize[srcType], ds = kTypeSize[dstType];
    // A one-channel image has a single plane: the golden code derives planarity from numPlanes() > 1.
    if (channels == 1)
        srcPlanar = dstPlanar = 0;

    std::vector<uint8_t> hSrc((size_t)srcW * srcH * channels * ss), hDst((size_t)dstW * dstH * channels * ds);
    std::memcpy(hSrc.data(), src, hSrc.size());

    // Stride vectors exactly as the reference test driver builds them
    // (TestOpCropFlipNormalizeReformat.cpp:354-388).
    long4 in, out;
    in.x = (long)srcW * srcH * channels * ss;
    if (srcPlanar)
    {
        in.y = (long)srcW * srcH * ss;
        in.z = (long)srcW * ss;
        in.w = ss;
    }
    else
    {
        in.y = (long)srcW * channels * ss;
        in.z = (long)channels * ss;
        in.w = ss;
    }
    out.x = (long)dstW * dstH * channels * ds;
    if (dstPlanar)
    {
        out.y = (long)dstW * dstH * ds;
        out.z = (long)dstW * ds;
        out.w = ds;
    }
    else
    {
        out.y = (long)dstW * channels * ds;
        out.z = (long)channels * ds;
        out.w = ds;
    }

    nvcv::ImageFormat  fmt{channels, srcPlanar ? channels : 1}, dfmt{channels, dstPlanar ? channels : 1};
    nvcv::ImageFormat  bfmt{baseCh, 1}, sfmt{scaleCh, 1};
    std::vector<float> vb(base, base + baseCh), vs(scale, scale + scaleCh);
    NVCVRectI          rect{cropX, cropY, cropW, cropH};
    nvcv::Size2D       ssz{srcW, srcH}, dsz{dstW, dstH};

    int rc = -1;
#define SRC(T)                                                                                                   \
    rc = cfnr_dst<T>(dstType, border, hDst, out, hSrc, in, ssz, dsz, fmt, dfmt, borderValue, flip, rect, vb, bfmt, \
                     vs, sfmt, gScale, gShift, eps, flags)
    switch (srcType)
    {
    case 0:
        SRC(uint8_t);
        break;
    case 1:
        SRC(int8_t);
        break;
    case 2:
        SRC(uint16_t);
        break;
    case 3:
        SRC(int16_t);
        break;
    case 4:
        SRC(uint32_t);
        break;
    case 5:
        SRC(int32_t);
        break;
    case 6:
        SRC(float);
        break;
    }
#undef SRC
    if (rc == 0)
        std::memcpy(dst, hDst.data(), hDst.size());
    return rc;
}

// cuda::SaturateCast host path, exposed so the restated rounding can be compared value by value.
uint8_t ref_sat_u8_f32(float v)
{
    return cuda::SaturateCast<uint8_t>(v);
}

int32_t ref_sat_s32_f32(float v)
{
    return cuda::SaturateCast<int32_t>(v);
}

int16_t ref_sat_s16_f32(float v)
{
    return cuda::SaturateCast<int16_t>(v);
}
}

// tests/cvcuda/system/TestOpCopyMakeBorder.cpp:40-97  CopyMakeBorder<T> (tensor form), cut by signature. It asks the
// destination's data-access object for its extents and strides: a stand-in answers.
namespace nvcv {
struct TensorDataAccessStridedImagePlanar
{
    int  samples, rows, cols, channels;
    long rowBytes, sampleBytes;

    int numSamples() const
    {
        return samples;
    }

    int numRows() const
    {
        return rows;
    }

    int numCols() const
    {
        return cols;
    }

    int numChannels() const
    {
        return channels;
    }

    long rowStride() const
    {
        return rowBytes;
    }

    long sampleStride() const
    {
        return sampleBytes;
    }
};
} // namespace nvcv

#include REF_GOLDEN_BORDER_INC

namespace {
template<typename T>
void ref_border_t(void *dst, const void *src, int n, int dw, int dh, int sw, int sh, int ch, int top, int left, int border,
                  const float *value)
{
    std::vector<T> hSrc(static_cast<const T *>(src), static_cast<const T *>(src) + static_cast<size_t>(n) * sh * sw * ch);
    std::vector<T> hDst(static_cast<size_t>(n) * dh * dw * ch);
    nvcv::TensorDataAccessStridedImagePlanar acc{n, dh, dw, ch, static_cast<long>(dw) * ch * static_cast<long>(sizeof(T)),
                                                 static_cast<long>(dh) * dw * ch * static_cast<long>(sizeof(T))};
    CopyMakeBorder<T>(hDst, hSrc, acc, sw, sh, sw * ch, ch, sh * sw * ch, top, left, static_cast<NVCVBorderType>(border),
                      float4{value[0], value[1], value[2], value[3]});
    std::memcpy(dst, hDst.data(), hDst.size() * sizeof(T));
}
} // namespace

// Packed [n, h, w, ch] tensors; dtype: 0 uint8, 2 uint16, 3 int16, 5 int32, 6 float32.
extern "C" int ref_copy_make_border(void *dst, const void *src, int n, int dw, int dh, int sw, int sh, int ch, int dtype,
                                    int top, int left, int border, const float *value)
{
    switch (dtype)
    {
    case 0:
        ref_border_t<uint8_t>(dst, src, n, dw, dh, sw, sh, ch, top, left, border, value);
        return 0;
    case 2:
        ref_border_t<uint16_t>(dst, src, n, dw, dh, sw, sh, ch, top, left, border, value);
        return 0;
    case 3:
        ref_border_t<int16_t>(dst, src, n, dw, dh, sw, sh, ch, top, left, border, value);
        return 0;
    case 5:
        ref_border_t<int32_t>(dst, src, n, dw, dh, sw, sh, ch, top, left, border, value);
        return 0;
    case 6:
        ref_border_t<float>(dst, src, n, dw, dh, sw, sh, ch, top, left, border, value);
        return 0;
    }
    return -1;
}

// tests/cvcuda/system/TestOpNormalize.cpp:34-77  Normalize (uint8 images, float32 base / scale), cut by signature
#include REF_GOLDEN_NORMALIZE_INC

// One uint8 image of `channels` interleaved channels; base / scale are either one value or a full w x h x channels
// float32 image (the two forms the reference's test uses).
extern "C" int ref_normalize(uint8_t *dst, const uint8_t *src, int w, int h, int channels, const float *base, int baseFull,
                             const float *scale, int scaleFull, float gscale, float shift, float epsilon, uint32_t flags)
{
    std::vector<uint8_t> hSrc(src, src + static_cast<size_t>(w) * h * channels), hDst(hSrc.size());
    std::vector<float>   hBase(base, base + (baseFull ? static_cast<size_t>(w) * h * channels : 1));
    std::vector<float>   hScale(scale, scale + (scaleFull ? static_cast<size_t>(w) * h * channels : 1));
    Normalize(hDst, w * channels, hSrc, w * channels, nvcv::Size2D{w, h}, nvcv::ImageFormat{channels, 1}, hBase,
              baseFull ? w * channels : 1, baseFull ? nvcv::Size2D{w, h} : nvcv::Size2D{1, 1},
              nvcv::ImageFormat{baseFull ? channels : 1, 1}, hScale, scaleFull ? w * channels : 1,
              scaleFull ? nvcv::Size2D{w, h} : nvcv::Size2D{1, 1}, nvcv::ImageFormat{scaleFull ? channels : 1, 1}, gscale,
              shift, epsilon, flags);
    std::memcpy(dst, hDst.data(), hDst.size());
    return 0;
}

namespace {
template<typename T>
void ref_resize_t(void *dst, int dstStepElems, int dstW, int dstH, const void *src, int srcStepElems, int srcW, int srcH,
                  int channels, int interp, const int *rect = nullptr)
{
    if (rect) // the call test::ResizedCrop makes (ResizeUtils.cpp:360-369): left, top, crop_cols, crop_rows
    {
        nvcv::test::resizedCrop<T>(static_cast<T *>(dst), dstStepElems, nvcv::Size2D{dstW, dstH}, static_cast<const T *>(src),
                                   srcStepElems, nvcv::Size2D{srcW, srcH}, rect[1], rect[0], rect[3], rect[2],
                                   nvcv::ImageFormat{channels, 1}, static_cast<NVCVInterpolationType>(interp),
                                   std::numeric_limits<T>::min(), std::numeric_limits<T>::max());
        return;
    }
    // the call test::Resize makes for nearest / linear / cubic (ResizeUtils.cpp:320-323)
    nvcv::test::resizedCrop<T>(static_cast<T *>(dst), dstStepElems, nvcv::Size2D{dstW, dstH}, static_cast<const T *>(src),
                               srcStepElems, nvcv::Size2D{srcW, srcH}, 0, 0, srcH, srcW, nvcv::ImageFormat{channels, 1},
                               static_cast<NVCVInterpolationType>(interp), std::numeric_limits<T>::min(),
                               std::numeric_limits<T>::max());
}
} // namespace

// dtype: 0 uint8, 2 uint16, 3 int16, 6 float32. Steps in elements, as the golden takes them.
extern "C" int ref_resize(void *dst, int dstStepElems, int dstW, int dstH, const void *src, int srcStepElems, int srcW,
                          int srcH, int channels, int dtype, int interp)
{
    switch (dtype)
    {
    case 0:
        ref_resize_t<uint8_t>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp);
        return 0;
    case 2:
        ref_resize_t<uint16_t>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp);
        return 0;
    case 3:
        ref_resize_t<int16_t>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp);
        return 0;
    case 6:
        ref_resize_t<float>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp);
        return 0;
    }
    return -1;
}

extern "C" int ref_resized_crop(void *dst, int dstStepElems, int dstW, int dstH, const void *src, int srcStepElems, int srcW,
                                int srcH, int channels, int dtype, int interp, const int *rect)
{
    switch (dtype)
    {
    case 0:
        ref_resize_t<uint8_t>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp, rect);
        return 0;
    case 2:
        ref_resize_t<uint16_t>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp, rect);
        return 0;
    case 3:
        ref_resize_t<int16_t>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp, rect);
        return 0;
    case 6:
        ref_resize_t<float>(dst, dstStepElems, dstW, dstH, src, srcStepElems, srcW, srcH, channels, interp, rect);
        return 0;
    }
    return -1;
}

// tests/cvcuda/system/TestOpRandomResizedCrop.cpp:39-93  GetCropParams (the test's copy of the operator's rectangle
// generator), cut by signature.
#include <random>
#include REF_GOLDEN_RANDOM_CROP_INC

// The first n rectangles (left, top, width, height) a generator seeded with `seed` yields for rows x cols images.
extern "C" int ref_random_crop_rects(unsigned seed, double minScale, double maxScale, double minRatio, double maxRatio,
                                     const int *rowsCols, int n, int *rects)
{
    std::mt19937 generator(seed);
    for (int i = 0; i < n; ++i)
    {
        int top = 0, left = 0, cropRows = 0, cropCols = 0;
        GetCropParams(generator, minScale, maxScale, minRatio, maxRatio, rowsCols[2 * i], rowsCols[2 * i + 1], &top, &left,
                      &cropRows, &cropCols);
        rects[4 * i + 0] = left;
        rects[4 * i + 1] = top;
        rects[4 * i + 2] = cropCols;
        rects[4 * i + 3] = cropRows;
    }
    return 0;
}
