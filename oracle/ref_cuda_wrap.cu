// TEST / BASELINE INFRASTRUCTURE ONLY -- never linked into, loaded by, or called from the product library.
//
// The reference project's own CUDA kernels for the fused pre-processing path, compiled for sm_100a so that they can be
// timed on the same B200 and cross-checked against the new kernels. build_oracle.py cuts the kernel templates (and the
// DstMap writer they use) out of the reference's operator sources at build time into a scratch directory
// (REF_CUDA_RCCR_INC, REF_CUDA_CFNR_INC) and compiles this file against them plus the reference's header-only device
// accessors (cvcuda/cuda_tools). Nothing from the reference is stored in this repository.
//
//   src/cvcuda/priv/OpResizeCropConvertReformat.cu:47-278   remapC, DstMap, resizeCrop_NN / _bilinear (+ _varShape)
//   src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:38-186   get_*_value, transfer_data, set_data, slice_flip_normalize
//
// The launch shapes below repeat the reference launchers (OpResizeCropConvertReformat.cu:325-347, :387-407,
// OpCropFlipNormalizeReformat.cu:206-251, :267-273). What is NOT taken from the reference is the handle plumbing in
// front of the launch (tensor / image-batch export, argument checks): it needs libnvcv_types, which is not built here,
// and costs no device time.
#include <cuda_runtime.h>

#include <cvcuda/Types.h>
#include <cvcuda/cuda_tools/BorderVarShapeWrap.hpp>
#include <cvcuda/cuda_tools/DropCast.hpp>
#include <cvcuda/cuda_tools/ImageBatchVarShapeWrap.hpp>
#include <cvcuda/cuda_tools/MathOps.hpp>
#include <cvcuda/cuda_tools/MathWrappers.hpp>
#include <cvcuda/cuda_tools/SaturateCast.hpp>
#include <cvcuda/cuda_tools/StaticCast.hpp>
#include <cvcuda/cuda_tools/TensorWrap.hpp>
#include <cvcuda/cuda_tools/TypeTraits.hpp>
#include <nvcv/BorderType.h>
#include <nvcv/ImageBatchData.hpp>
#include <nvcv/Size.h>

#include <cmath>
#include <cstdint>

namespace cuda = nvcv::cuda;

// The header-only object-model classes reference a few C functions of libnvcv_types on their error paths only
// (exception text); this library never takes those paths, the definitions below just let it load on its own.
extern "C" const char *nvcvStatusGetName(NVCVStatus)
{
    return "NVCV_STATUS";
}

extern "C" NVCVStatus nvcvGetLastErrorMessage(char *msg, int32_t len)
{
    if (msg && len > 0)
        msg[0] = 0;
    return NVCV_SUCCESS;
}

extern "C" NVCVStatus nvcvImageFormatGetNumPlanes(NVCVImageFormat, int32_t *out)
{
    if (out)
        *out = 1;
    return NVCV_SUCCESS;
}

namespace refrccr {
#include REF_CUDA_RCCR_INC
} // namespace refrccr

namespace refcfnr {
#include REF_CUDA_CFNR_INC
} // namespace refcfnr

namespace {

inline int div_up(int a, int b)
{
    return (a + b - 1) / b;
}

nvcv::ImageBatchVarShapeDataStridedCuda batch_of(const void *imageList, int numImages)
{
    NVCVImageBatchVarShapeBufferStrided buf{};
    buf.imageList = const_cast<NVCVImageBufferStrided *>(static_cast<const NVCVImageBufferStrided *>(imageList));
    return nvcv::ImageBatchVarShapeDataStridedCuda(numImages, buf);
}

// dstIsFloat / dstPlanar select DstMap<float|uint8_t, 3> and its strides exactly as the reference launcher derives
// them from a densely allocated output tensor (OpResizeCropConvertReformat.cu:314-323).
template<typename DstT>
refrccr::DstMap<DstT, 3> dst_map(void *dst, int dstPlanar, int dstW, int dstH, int manip)
{
    const int    planes = dstPlanar ? 3 : 1;
    const size_t rowEl  = static_cast<size_t>(dstW) * (dstPlanar ? 1 : 3);
    const size_t addC   = planes > 1 ? rowEl * dstH : 1;
    const int    addW   = 3 / planes;
    const int    addH   = static_cast<int>(rowEl);
    const size_t addN   = rowEl * dstH * planes;
    return refrccr::DstMap<DstT, 3>(static_cast<DstT *>(dst), addN, addH, addW, addC,
                                    static_cast<NVCVChannelManip>(manip), dstW, dstH);
}

template<typename DstT>
int rccr_tensor(const uint8_t *src, int n, int srcW, int srcH, long long rowStride, long long sampleStride, void *dst,
                int dstPlanar, int dstW, int dstH, int resizeW, int resizeH, int interp, int cropX, int cropY, int manip,
                float scale, float offset, int srcCast, cudaStream_t stream)
{
    auto   dmap = dst_map<DstT>(dst, dstPlanar, dstW, dstH, manip);
    float2 resize{(float)srcW / resizeW, (float)srcH / resizeH};
    int2   crop{cropX, cropY};
    cuda::Tensor3DWrap<const uchar3, int32_t> swrap(reinterpret_cast<const uchar3 *>(src),
                                                    static_cast<int32_t>(sampleStride), static_cast<int32_t>(rowStride));
    const dim3 block(16, 16, 1), grid(div_up(dstW, 16), div_up(dstH, 16), n);
    if (interp == NVCV_INTERP_NEAREST)
        refrccr::resizeCrop_NN<<<grid, block, 0, stream>>>(dmap, swrap, resize, crop, scale, offset);
    else
        refrccr::resizeCrop_bilinear<<<grid, block, 0, stream>>>(dmap, swrap, srcW, srcH, resize, crop, scale, offset,
                                                                 srcCast != 0);
    return static_cast<int>(cudaPeekAtLastError());
}

template<typename DstT>
int rccr_varshape(const void *imageList, int n, void *dst, int dstPlanar, int dstW, int dstH, int resizeW, int resizeH,
                  int interp, int cropX, int cropY, int manip, float scale, float offset, int srcCast,
                  cudaStream_t stream)
{
    auto       dmap = dst_map<DstT>(dst, dstPlanar, dstW, dstH, manip);
    NVCVSize2D resize{resizeW, resizeH};
    int2       crop{cropX, cropY};
    cuda::ImageBatchVarShapeWrap<const uchar3> swrap(batch_of(imageList, n));
    const dim3 block(8, 32, 1), grid(div_up(dstW, 8), div_up(dstH, 32), n);
    if (interp == NVCV_INTERP_NEAREST)
        refrccr::resizeCrop_NN_varShape<<<grid, block, 0, stream>>>(dmap, swrap, resize, crop, scale, offset);
    else
        refrccr::resizeCrop_bilinear_varShape<<<grid, block, 0, stream>>>(dmap, swrap, resize, crop, scale, offset,
                                                                          srcCast != 0);
    return static_cast<int>(cudaPeekAtLastError());
}

} // namespace

extern "C"
{
// Dense uint8 NHWC source (byte strides; the reference addresses samples with 32-bit offsets), packed output.
int refcuda_rccr_tensor(const uint8_t *src, int n, int srcW, int srcH, long long rowStride, long long sampleStride,
                        void *dst, int dstIsFloat, int dstPlanar, int dstW, int dstH, int resizeW, int resizeH,
                        int interp, int cropX, int cropY, int manip, float scale, float offset, int srcCast,
                        cudaStream_t stream)
{
    if (sampleStride * n > 2147483647LL)
        return -10; // the reference operator refuses such inputs (OpResizeCropConvertReformat.cu:515-519)
    return dstIsFloat ? rccr_tensor<float>(src, n, srcW, srcH, rowStride, sampleStride, dst, dstPlanar, dstW, dstH, resizeW,
                                           resizeH, interp, cropX, cropY, manip, scale, offset, srcCast, stream)
                      : rccr_tensor<uint8_t>(src, n, srcW, srcH, rowStride, sampleStride, dst, dstPlanar, dstW, dstH,
                                             resizeW, resizeH, interp, cropX, cropY, manip, scale, offset, srcCast, stream);
}

// Variable-shape source: device array of NVCVImageBufferStrided descriptors.
int refcuda_rccr_varshape(const void *imageList, int n, void *dst, int dstIsFloat, int dstPlanar, int dstW, int dstH,
                          int resizeW, int resizeH, int interp, int cropX, int cropY, int manip, float scale,
                          float offset, int srcCast, cudaStream_t stream)
{
    return dstIsFloat ? rccr_varshape<float>(imageList, n, dst, dstPlanar, dstW, dstH, resizeW, resizeH, interp, cropX,
                                             cropY, manip, scale, offset, srcCast, stream)
                      : rccr_varshape<uint8_t>(imageList, n, dst, dstPlanar, dstW, dstH, resizeW, resizeH, interp, cropX,
                                               cropY, manip, scale, offset, srcCast, stream);
}
}

// -------------------------------------------------------------------------------------------------- CropFlipNormalizeReformat

namespace {

template<typename T_Dst, NVCVBorderType B>
int cfnr_run(const void *imageList, int n, int channels, void *dst, int dstPlanar, int outW, int outH, const int *cropRect,
             const int *flip, const float *base, int baseCh, const float *scale, int scaleCh, float borderValue,
             float gscale, float shift, float eps, uint32_t flags, cudaStream_t stream)
{
    using SrcT = uint8_t;
    cuda::ImageBatchVarShapeWrapNHWC<const SrcT> srcWrap(batch_of(imageList, n), channels);
    cuda::BorderVarShapeWrapNHWC<const SrcT, B>  srcBorder(srcWrap, static_cast<SrcT>(borderValue));

    // packed output tensor: NCHW strides (sample, plane, row) or NHWC strides (sample, row, pixel), in bytes
    const int32_t es = sizeof(T_Dst);
    const int32_t s0 = es * channels * outW * outH;
    const int32_t s1 = dstPlanar ? es * outW * outH : es * channels * outW;
    const int32_t s2 = dstPlanar ? es * outW : es * channels;
    cuda::Tensor4DWrap<T_Dst, int32_t> dstWrap(static_cast<T_Dst *>(dst), s0, s1, s2);

    cuda::Tensor1DWrap<int, int32_t>   flipWrap(const_cast<int *>(flip));
    cuda::Tensor4DWrap<float, int32_t> baseWrap(const_cast<float *>(base), 4 * baseCh, 4 * baseCh, 4 * baseCh);
    cuda::Tensor4DWrap<float, int32_t> scaleWrap(const_cast<float *>(scale), 4 * scaleCh, 4 * scaleCh, 4 * scaleCh);
    cuda::Tensor4DWrap<int, int32_t>   cropWrap(const_cast<int *>(cropRect), 16, 16, 16);

    const dim3 block(32, 32, 1);
    const dim3 grid(static_cast<unsigned>(std::ceil(outW / 32.f)), static_cast<unsigned>(std::ceil(outH / 32.f)), n);
    refcfnr::slice_flip_normalize<<<grid, block, 0, stream>>>(srcBorder, dstWrap, flipWrap, baseWrap, scaleWrap, cropWrap,
                                                              gscale, shift, eps, flags, channels, baseCh, scaleCh,
                                                              int3{outW, outH, channels}, dstPlanar != 0);
    return static_cast<int>(cudaPeekAtLastError());
}

template<typename T_Dst, typename... A>
int cfnr_border(int border, A... a)
{
    switch (border)
    {
    case NVCV_BORDER_CONSTANT:
        return cfnr_run<T_Dst, NVCV_BORDER_CONSTANT>(a...);
    case NVCV_BORDER_REPLICATE:
        return cfnr_run<T_Dst, NVCV_BORDER_REPLICATE>(a...);
    case NVCV_BORDER_REFLECT:
        return cfnr_run<T_Dst, NVCV_BORDER_REFLECT>(a...);
    case NVCV_BORDER_WRAP:
        return cfnr_run<T_Dst, NVCV_BORDER_WRAP>(a...);
    case NVCV_BORDER_REFLECT101:
        return cfnr_run<T_Dst, NVCV_BORDER_REFLECT101>(a...);
    }
    return -1;
}

} // namespace

// Interleaved uint8 variable-shape source -> packed uint8 / float32 output tensor. cropRect: packed int32 x 4 per sample.
extern "C" int refcuda_cfnr_u8(const void *imageList, int n, int channels, void *dst, int dstIsFloat, int dstPlanar,
                               int outW, int outH, const int *cropRect, const int *flip, const float *base, int baseCh,
                               const float *scale, int scaleCh, int border, float borderValue, float gscale, float shift,
                               float eps, uint32_t flags, cudaStream_t stream)
{
    return dstIsFloat ? cfnr_border<float>(border, imageList, n, channels, dst, dstPlanar, outW, outH, cropRect, flip, base,
                                           baseCh, scale, scaleCh, borderValue, gscale, shift, eps, flags, stream)
                      : cfnr_border<uint8_t>(border, imageList, n, channels, dst, dstPlanar, outW, outH, cropRect, flip,
                                             base, baseCh, scale, scaleCh, borderValue, gscale, shift, eps, flags, stream);
}
