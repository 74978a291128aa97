/*
 * Handle-based operator API: the drop-in replacement for the reference's C operators of the fused pre-processing path.
 *
 * The entry points below have the names, signatures, status codes and ownership rules of the reference library's
 * (libcvcuda) exports, so a program, the reference's C++ wrappers (cvcuda/Op*.hpp) or its Python module can bind to
 * this library instead. Tensor and image-batch handles are unpacked with the object-model library of the reference
 * (libnvcv_types: nvcvTensorExportData, nvcvImageBatchExportData, nvcvDataTypeGet*, nvcvImageFormatGet*,
 * nvcvSetThreadStatus), which is looked up in the running process; then the plain-C layer of preproc.h does the work.
 *
 * Define CVCUDA_B200_USE_NVCV_HEADERS before including this file to take the types from the reference's own headers
 * (<nvcv/...>, <cvcuda/...>); otherwise the ABI-identical minimal declarations below are used.
 */
#ifndef CVCUDA_B200_CVCUDA_OPS_H
#define CVCUDA_B200_CVCUDA_OPS_H

#include "preproc.h"

#include <stdbool.h>
#include <stdint.h>

#if defined(CVCUDA_B200_USE_NVCV_HEADERS)
#    include <cvcuda/OpCropFlipNormalizeReformat.h>
#    include <cvcuda/OpResizeCropConvertReformat.h>
#else

#    if defined(__cplusplus)
extern "C"
{
#    endif

/* ---- types of the reference's object model, restated with identical memory layout -------------------------------- */

typedef int NVCVStatus; /* values: B200PP_* of preproc.h = NVCVStatus of nvcv/Status.h:48-62 */

typedef struct NVCVOperator   *NVCVOperatorHandle;   /* cvcuda/Operator.h:34 */
typedef struct NVCVTensor     *NVCVTensorHandle;     /* nvcv/Tensor.h:43 */
typedef struct NVCVImageBatch *NVCVImageBatchHandle; /* nvcv/ImageBatch.h:54 */
typedef struct NVCVImage      *NVCVImageHandle;      /* nvcv/Image.h */

typedef struct NVCVSize2D /* nvcv/Size.h:33-36 */
{
    int32_t w, h;
} NVCVSize2D;

#    if !defined(__VECTOR_TYPES_H__)
typedef struct __attribute__((aligned(8))) int2 /* CUDA vector type */
{
    int x, y;
} int2;
typedef struct __attribute__((aligned(16))) float4 /* CUDA vector type */
{
    float x, y, z, w;
} float4;
#    endif

typedef int      NVCVInterpolationType; /* cvcuda/Types.h:39-51 */
typedef int      NVCVChannelManip;      /* cvcuda/Types.h:63-67 */
typedef int      NVCVBorderType;        /* nvcv/BorderType.h:36-43 */
typedef uint64_t NVCVDataType;          /* nvcv/DataType.h:52 */
typedef uint64_t NVCVImageFormat;       /* nvcv/ImageFormat.h */

#    define NVCV_TENSOR_MAX_RANK 15 /* nvcv/TensorLayout.h:34 */

typedef struct NVCVTensorLayout /* nvcv/TensorLayout.h */
{
    char    data[NVCV_TENSOR_MAX_RANK + 1];
    int32_t rank;
} NVCVTensorLayout;

typedef struct NVCVTensorData /* nvcv/TensorData.h:31-80 */
{
    NVCVDataType     dtype;
    NVCVTensorLayout layout;
    int32_t          rank;
    int64_t          shape[NVCV_TENSOR_MAX_RANK];
    int32_t          bufferType; /* 1 = NVCV_TENSOR_BUFFER_STRIDED_CUDA */
    struct
    {
        int64_t  strides[NVCV_TENSOR_MAX_RANK];
        uint8_t *basePtr;
    } strided;
} NVCVTensorData;

typedef struct NVCVImageBatchData /* nvcv/ImageBatchData.h:26-111 */
{
    int32_t numImages;
    int32_t bufferType; /* 1 = NVCV_IMAGE_BATCH_VARSHAPE_BUFFER_STRIDED_CUDA */
    struct
    {
        NVCVImageFormat        uniqueFormat;
        int32_t                maxWidth, maxHeight;
        NVCVImageFormat       *formatList;
        const NVCVImageFormat *hostFormatList;
        B200ppImageBuffer     *imageList; /* NVCVImageBufferStrided[], device memory */
    } varShapeStrided;
} NVCVImageBatchData;

/* ---- the exported operator entry points ---------------------------------------------------------------------------- */

/* Replaces cvcudaResizeCropConvertReformatCreate (reference: src/cvcuda/OpResizeCropConvertReformat.cpp:29-42,
 * declared in src/cvcuda/include/cvcuda/OpResizeCropConvertReformat.h:54). NULL handle pointer: INVALID_ARGUMENT.
 * The caller owns the handle and releases it with nvcvOperatorDestroy. */
B200PP_PUBLIC NVCVStatus cvcudaResizeCropConvertReformatCreate(NVCVOperatorHandle *handle);

/* Replaces cvcudaResizeCropConvertReformatSubmit (src/cvcuda/OpResizeCropConvertReformat.cpp:44-56, header :220-223;
 * validation and status codes of src/cvcuda/priv/OpResizeCropConvertReformat.cu:418-554). Asynchronous on `stream`;
 * tensors are borrowed for the duration of the enqueued work. */
B200PP_PUBLIC NVCVStatus cvcudaResizeCropConvertReformatSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                               NVCVTensorHandle in, NVCVTensorHandle out,
                                                               const NVCVSize2D resizeDim,
                                                               const NVCVInterpolationType interpolation,
                                                               const int2 cropPos, const NVCVChannelManip manip,
                                                               const float scale, const float offset,
                                                               const bool srcCast);

/* Replaces cvcudaResizeCropConvertReformatVarShapeSubmit (src/cvcuda/OpResizeCropConvertReformat.cpp:58-71,
 * header :225-228; validation of src/cvcuda/priv/OpResizeCropConvertReformat.cu:556-683). */
B200PP_PUBLIC NVCVStatus cvcudaResizeCropConvertReformatVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                                       NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                                       const NVCVSize2D resizeDim,
                                                                       const NVCVInterpolationType interpolation,
                                                                       const int2 cropPos, const NVCVChannelManip manip,
                                                                       const float scale, const float offset,
                                                                       const bool srcCast);

/* Replaces cvcudaCropFlipNormalizeReformatCreate (src/cvcuda/OpCropFlipNormalizeReformat.cpp:29-42,
 * header src/cvcuda/include/cvcuda/OpCropFlipNormalizeReformat.h:53). */
B200PP_PUBLIC NVCVStatus cvcudaCropFlipNormalizeReformatCreate(NVCVOperatorHandle *handle);

/* Replaces cvcudaCropFlipNormalizeReformatSubmit (src/cvcuda/OpCropFlipNormalizeReformat.cpp:44-60, header :171-174;
 * validation of src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:366-468). */
B200PP_PUBLIC NVCVStatus cvcudaCropFlipNormalizeReformatSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                               NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                               NVCVTensorHandle cropRect, NVCVBorderType borderMode,
                                                               float borderValue, NVCVTensorHandle flipCode,
                                                               NVCVTensorHandle base, NVCVTensorHandle scale,
                                                               float global_scale, float shift, float epsilon,
                                                               uint32_t flags);

/* Replaces nvcvOperatorDestroy (src/cvcuda/Operator.cpp:26-29, header cvcuda/Operator.h:34-36). NULL is ignored. */
B200PP_PUBLIC void nvcvOperatorDestroy(NVCVOperatorHandle handle);

#    if defined(__cplusplus)
}
#    endif
#endif /* CVCUDA_B200_USE_NVCV_HEADERS */

#if defined(__cplusplus)
extern "C"
{
#endif

/* Stand-alone Resize, nearest and linear interpolation (cubic and area: NVCV_ERROR_NOT_IMPLEMENTED).
 * Replace cvcudaResizeCreate / cvcudaResizeSubmit / cvcudaResizeVarShapeSubmit (reference:
 * src/cvcuda/OpResize.cpp:29-71, declared in src/cvcuda/include/cvcuda/OpResize.h:52,115-120; validation and status codes
 * of src/cvcuda/priv/OpResize.cu:501-555). Same ownership, threading and error rules as the entry points above. */
B200PP_PUBLIC NVCVStatus cvcudaResizeCreate(NVCVOperatorHandle *handle);
B200PP_PUBLIC NVCVStatus cvcudaResizeSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                            NVCVTensorHandle out, const NVCVInterpolationType interpolation);
B200PP_PUBLIC NVCVStatus cvcudaResizeVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                    NVCVImageBatchHandle in, NVCVImageBatchHandle out,
                                                    const NVCVInterpolationType interpolation);

/* Stand-alone Normalize. Replace cvcudaNormalizeCreate / cvcudaNormalizeSubmit / cvcudaNormalizeVarShapeSubmit (reference:
 * src/cvcuda/OpNormalize.cpp:29-71, declared in src/cvcuda/include/cvcuda/OpNormalize.h:54,128-163; operator
 * src/cvcuda/priv/OpNormalize.cpp:38-108). base and scale are float32 (N)HWC tensors whose sample, row, column and channel
 * extents are each 1 (broadcast) or the input's. */
B200PP_PUBLIC NVCVStatus cvcudaNormalizeCreate(NVCVOperatorHandle *handle);
B200PP_PUBLIC NVCVStatus cvcudaNormalizeSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                               NVCVTensorHandle base, NVCVTensorHandle scale, NVCVTensorHandle out,
                                               float global_scale, float shift, float epsilon, uint32_t flags);
B200PP_PUBLIC NVCVStatus cvcudaNormalizeVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                       NVCVImageBatchHandle in, NVCVTensorHandle base,
                                                       NVCVTensorHandle scale, NVCVImageBatchHandle out,
                                                       float global_scale, float shift, float epsilon, uint32_t flags);

/* Stand-alone Reformat (NHWC / HWC <-> NCHW / CHW, or a strided copy within one layout). Replace cvcudaReformatCreate /
 * cvcudaReformatSubmit (reference: src/cvcuda/OpReformat.cpp:28-55, declared in src/cvcuda/include/cvcuda/OpReformat.h). */
B200PP_PUBLIC NVCVStatus cvcudaReformatCreate(NVCVOperatorHandle *handle);
B200PP_PUBLIC NVCVStatus cvcudaReformatSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                              NVCVTensorHandle out);

/* Stand-alone ConvertTo: out = SaturateCast(alpha * in + beta). Replace cvcudaConvertToCreate / cvcudaConvertToSubmit
 * (reference: src/cvcuda/OpConvertTo.cpp:28-55, declared in src/cvcuda/include/cvcuda/OpConvertTo.h). */
B200PP_PUBLIC NVCVStatus cvcudaConvertToCreate(NVCVOperatorHandle *handle);
B200PP_PUBLIC NVCVStatus cvcudaConvertToSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                               NVCVTensorHandle out, const double alpha, const double beta);

/* Stand-alone CopyMakeBorder: tensor -> tensor with one (top, left); variable-shape batch -> variable-shape batch, and
 * variable-shape batch -> tensor ("stack"), with int32 top / left tensors holding one value per image along the width.
 * Replace cvcudaCopyMakeBorderCreate / cvcudaCopyMakeBorderSubmit / cvcudaCopyMakeBorderVarShapeSubmit /
 * cvcudaCopyMakeBorderVarShapeStackSubmit (reference: src/cvcuda/OpCopyMakeBorder.cpp:29-82, declared in
 * src/cvcuda/include/cvcuda/OpCopyMakeBorder.h:53-140). */
B200PP_PUBLIC NVCVStatus cvcudaCopyMakeBorderCreate(NVCVOperatorHandle *handle);
B200PP_PUBLIC NVCVStatus cvcudaCopyMakeBorderSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                                    NVCVTensorHandle out, int32_t top, int32_t left,
                                                    NVCVBorderType borderMode, const float4 borderValue);
B200PP_PUBLIC NVCVStatus cvcudaCopyMakeBorderVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                            NVCVImageBatchHandle in, NVCVImageBatchHandle out,
                                                            NVCVTensorHandle top, NVCVTensorHandle left,
                                                            NVCVBorderType borderMode, const float4 borderValue);
B200PP_PUBLIC NVCVStatus cvcudaCopyMakeBorderVarShapeStackSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                                 NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                                 NVCVTensorHandle top, NVCVTensorHandle left,
                                                                 NVCVBorderType borderMode, const float4 borderValue);

/* RandomResizedCrop: one random crop rectangle per image (area fraction in [minScale, maxScale], aspect ratio
 * log-uniform in [minRatio, maxRatio], drawn from a std::mt19937 seeded with `seed`, 0 = random seed) resized to the
 * output's size, nearest or linear (cubic: NVCV_ERROR_NOT_IMPLEMENTED). The handle owns the generator and a device
 * parameter buffer for maxBatchSize images; calls on one handle must not overlap. Replace cvcudaRandomResizedCropCreate /
 * cvcudaRandomResizedCropSubmit / cvcudaRandomResizedCropVarShapeSubmit (reference: src/cvcuda/OpRandomResizedCrop.cpp:29-70,
 * declared in src/cvcuda/include/cvcuda/OpRandomResizedCrop.h). The variable-shape form asks the object-model library for
 * each input image's size (nvcvImageBatchVarShapeGetImages, nvcvImageGetSize), as the reference does through
 * ImageBatchVarShape::operator[]. */
B200PP_PUBLIC NVCVStatus cvcudaRandomResizedCropCreate(NVCVOperatorHandle *handle, double minScale, double maxScale,
                                                       double minRatio, double maxRatio, int32_t maxBatchSize,
                                                       uint32_t seed);
B200PP_PUBLIC NVCVStatus cvcudaRandomResizedCropSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                                       NVCVTensorHandle out, const NVCVInterpolationType interpolation);
B200PP_PUBLIC NVCVStatus cvcudaRandomResizedCropVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                               NVCVImageBatchHandle in, NVCVImageBatchHandle out,
                                                               const NVCVInterpolationType interpolation);

/* Additions (no counterpart in the reference): the whole fused pass -- per-channel normalisation, float16 output,
 * per-sample regions of interest and flip codes, letterbox placement -- on tensor / image-batch handles. `op` is the
 * B200ppResizeOp of preproc.h; its roi / flipCode pointers are device memory. The operator handle is the one
 * cvcudaResizeCropConvertReformatCreate returns. */
B200PP_PUBLIC NVCVStatus cvcudaB200FusedPreprocessSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                         NVCVTensorHandle in, NVCVTensorHandle out,
                                                         const B200ppResizeOp *op);
B200PP_PUBLIC NVCVStatus cvcudaB200FusedPreprocessVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                                 NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                                 const B200ppResizeOp *op);

#if defined(__cplusplus)
}
#endif

#endif /* CVCUDA_B200_CVCUDA_OPS_H */
