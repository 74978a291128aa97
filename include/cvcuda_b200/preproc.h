/*
 * Fused image pre-processing for NVIDIA B200 (sm_100a): plain-C launch layer.
 *
 * These entry points take only pointers, sizes and byte strides. The handle-based operator API of
 * cvcuda_ops.h (the drop-in for the reference's C operators) translates its tensor / image-batch handles
 * into these structs and calls the same functions, and so can any foreign-function binding.
 *
 * All pointers are device-accessible memory unless stated otherwise. All strides are in bytes.
 * Every function is asynchronous with respect to `stream`, allocates nothing and returns an NVCVStatus
 * value (0 = success); the message of the last failure on the calling thread is kept for
 * b200ppGetLastErrorMessage().
 */
#ifndef CVCUDA_B200_PREPROC_H
#define CVCUDA_B200_PREPROC_H

#include <stddef.h>
#include <stdint.h>

#if defined(__cplusplus)
extern "C"
{
#endif

#if !defined(__DRIVER_TYPES_H__) && !defined(__CUDA_RUNTIME_H__)
typedef struct CUstream_st *cudaStream_t;
#endif

#define B200PP_PUBLIC __attribute__((visibility("default")))

/* Status codes: numerically identical to NVCVStatus (reference: src/nvcv/src/include/nvcv/Status.h:48-62). */
enum
{
    B200PP_SUCCESS                = 0,
    B200PP_ERROR_NOT_IMPLEMENTED  = 1,
    B200PP_ERROR_INVALID_ARGUMENT = 2,
    B200PP_ERROR_INTERNAL         = 8,
    B200PP_ERROR_NOT_COMPATIBLE   = 9,
    B200PP_ERROR_OVERFLOW         = 10
};

/* Element types. 0..6 are the types the reference's CropFlipNormalizeReformat dispatches on
 * (src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:335-341,453-458); F16 is an addition, output only. */
enum
{
    B200PP_U8  = 0,
    B200PP_S8  = 1,
    B200PP_U16 = 2,
    B200PP_S16 = 3,
    B200PP_U32 = 4,
    B200PP_S32 = 5,
    B200PP_F32 = 6,
    B200PP_F16 = 7
};

/* Interpolation: NVCVInterpolationType values (src/cvcuda/include/cvcuda/Types.h:39-51). */
enum
{
    B200PP_INTERP_NEAREST = 0,
    B200PP_INTERP_LINEAR  = 1
};

/* Channel manipulation: NVCVChannelManip (Types.h:63-67). */
enum
{
    B200PP_CHANNEL_NO_OP   = 0,
    B200PP_CHANNEL_REVERSE = 1
};

/* Border modes: NVCVBorderType (src/nvcv/src/include/nvcv/BorderType.h:36-43). */
enum
{
    B200PP_BORDER_CONSTANT   = 0,
    B200PP_BORDER_REPLICATE  = 1,
    B200PP_BORDER_REFLECT    = 2,
    B200PP_BORDER_WRAP       = 3,
    B200PP_BORDER_REFLECT101 = 4
};

/* Bit 0 of B200ppSliceOp::flags: `scale` holds standard deviations (CVCUDA_NORMALIZE_SCALE_IS_STDDEV,
 * src/cvcuda/include/cvcuda/OpNormalize.h:43). */
#define B200PP_NORMALIZE_SCALE_IS_STDDEV 1u

/* One plane of one image; same memory layout as NVCVImagePlaneStrided
 * (src/nvcv/src/include/nvcv/ImageData.h:27-50). */
typedef struct B200ppImagePlane
{
    int32_t  width, height;
    int32_t  rowStride;
    uint8_t *basePtr;
} B200ppImagePlane;

/* One image of a variable-shape batch; same memory layout as NVCVImageBufferStrided (ImageData.h:52-66), so the
 * device array an exported NVCVImageBatchVarShape points to can be passed as B200ppSource::imageList unchanged. */
typedef struct B200ppImageBuffer
{
    int32_t          numPlanes;
    B200ppImagePlane planes[6];
} B200ppImageBuffer;

/* Source batch: either one dense tensor (imageList == NULL) or a device array of per-image descriptors. */
typedef struct B200ppSource
{
    int32_t dtype;    /* element type */
    int32_t channels; /* 1..4 */
    int32_t planar;   /* 0: channels interleaved per pixel; 1: one plane per channel */
    int32_t numSamples;

    /* dense tensor */
    const void *base;
    int64_t     sampleStride, rowStride, planeStride;
    int32_t     width, height;

    /* variable-shape batch: device array of numSamples descriptors */
    const B200ppImageBuffer *imageList;
    int32_t maxWidth, maxHeight; /* upper bounds of the image sizes if known, else 0 (a tuning hint only) */
} B200ppSource;

/* Destination tensor: element (n, y, x, c) lives at base + n*sampleStride + y*rowStride + x*pixStride + c*chanStride,
 * which covers NHWC (pixStride = C*elem, chanStride = elem) and NCHW (pixStride = elem, chanStride = plane). */
typedef struct B200ppDest
{
    void   *base;
    int32_t dtype;
    int32_t channels;
    int32_t width, height;
    int64_t sampleStride, rowStride, pixStride, chanStride;
} B200ppDest;

/* Resize -> crop -> (flip) -> affine -> channel map -> cast -> layout, in one pass.
 *
 * With roi = flipCode = NULL, perChannel = 0 and the region equal to the destination this is exactly the reference's
 * ResizeCropConvertReformat (kernels src/cvcuda/priv/OpResizeCropConvertReformat.cu:137-278, golden arithmetic
 * tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:95-171). The other fields are additions the reference's
 * operator cannot express in one call. */
typedef struct B200ppResizeOp
{
    int32_t resizeW, resizeH; /* size each source image (or its roi) is resized to */
    int32_t cropX, cropY;     /* top-left of the crop inside the resized image */
    int32_t interp;           /* B200PP_INTERP_NEAREST or _LINEAR */
    int32_t srcCast;          /* round the interpolated value to uint8 before the affine step */
    int32_t manip;            /* B200PP_CHANNEL_* ; output channel (C-1-c) receives source channel c when reversed */

    int32_t perChannel;       /* 0: out = scale*v + offset          (the reference operator's formula)
                                 1: out = (v - base[c])*mul[c]*gscale + shift, c = source channel */
    float   scale, offset;
    float   base[4], mul[4];
    float   gscale, shift;

    /* Placement of the cropped region inside the destination (letterbox). regionW/H = 0 means "the whole destination".
     * Destination pixels outside the region receive padValue pushed through the same affine step. */
    int32_t dstX, dstY, regionW, regionH;
    float   padValue;

    /* Optional per-sample device arrays. roi: int32 (x, y, w, h) per sample, roiStride bytes apart (0 = packed): the
     * sample's source is that sub-view of its image. Contract: the rectangle lies inside the image and has w, h >= 1; the
     * kernels intersect it with the image before addressing through it (a rectangle that misses the image shrinks to
     * the nearest single pixel), so a bad rectangle gives meaningless pixels but no access outside the image.
     * flipCode: packed int32 per sample, applied to region coordinates
     * after the resize with the reference's codes (1 mirror x, 0 mirror y, -1 both, anything else none). */
    const int32_t *roi;
    int64_t        roiStride;
    const int32_t *flipCode;
} B200ppResizeOp;

/* Crop (with border) -> flip -> per-channel normalise -> cast -> layout: the reference's CropFlipNormalizeReformat
 * (kernel src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:137-186 with :38-116, golden arithmetic
 * tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:57-148). */
typedef struct B200ppSliceOp
{
    const int32_t *cropRect;       /* device: int32 (x, y, w, h) per sample */
    int64_t        cropRectStride; /* bytes between samples (0 = packed 16) */
    const int32_t *flipCode;       /* device: packed int32 per sample */
    int32_t        border;         /* B200PP_BORDER_* */
    float          borderValue;
    const float   *base;  /* device */
    int32_t        baseChannels;  /* 1, or >= source channels */
    int64_t        baseChanStride; /* bytes between channel values (0 = packed 4) */
    const float   *scale; /* device */
    int32_t        scaleChannels;
    int64_t        scaleChanStride;
    float          gscale, shift, epsilon;
    uint32_t       flags;
} B200ppSliceOp;

/* A batch of interleaved images of one element type and channel count, for the stand-alone Resize: a dense tensor
 * [numSamples, height, width, channels] (base and byte strides), or -- when imageList is not NULL -- a device array of
 * numSamples image descriptors with per-image sizes (plane 0 of each is used). */
typedef struct B200ppImageSet
{
    void                    *base;
    const B200ppImageBuffer *imageList;
    int32_t                  dtype;    /* B200PP_U8, _U16, _S16 or _F32 */
    int32_t                  channels; /* 1, 3 or 4 */
    int32_t                  numSamples;
    int32_t                  width, height;       /* dense only */
    int32_t                  maxWidth, maxHeight; /* image lists: upper bounds of the image sizes (sizes the launch) */
    int64_t                  rowStride, sampleStride; /* dense only, bytes */
} B200ppImageSet;

/* Replaces: cvcuda::priv::ResizeCropConvertReformat::operator() (tensor and var-shape),
 * src/cvcuda/priv/OpResizeCropConvertReformat.cu:418-554 and :556-683, minus the handle unpacking.
 * Sources must be interleaved 3-channel uint8; destination uint8, float32 or float16. */
B200PP_PUBLIC int b200ppResizeCropConvertReformat(const B200ppSource *src, const B200ppDest *dst,
                                                  const B200ppResizeOp *op, cudaStream_t stream);

/* Replaces: cvcuda::priv::CropFlipNormalizeReformat::operator(),
 * src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:366-468, minus the handle unpacking. */
B200PP_PUBLIC int b200ppCropFlipNormalizeReformat(const B200ppSource *src, const B200ppDest *dst,
                                                  const B200ppSliceOp *op, cudaStream_t stream);

/* Stand-alone Resize, nearest or linear: dst[i] = src[i] resized to the size of dst[i], element type and channel
 * count unchanged. Replaces cvcuda::priv::Resize::operator() for tensors (src/cvcuda/priv/OpResize.cu:501-560) and for
 * variable-shape batches (src/cvcuda/priv/legacy/resize_var_shape.cu), minus the handle unpacking; results follow the
 * reference's CPU golden (tests/cvcuda/system/ResizeUtils.cpp:189-241) bit for bit for the integer element types.
 * Cubic and area interpolation are not implemented (B200PP_ERROR_NOT_IMPLEMENTED). */
B200PP_PUBLIC int b200ppResize(const B200ppImageSet *src, const B200ppImageSet *dst, int32_t interp, cudaStream_t stream);

/* Resize of one crop rectangle per image: dst[i] = the rectangle cropRects[i] = (left, top, width, height; device, packed
 * int32 x 4 on a 16-byte boundary) of src[i], resized to the size of dst[i]. The resampling step of the reference's
 * RandomResizedCrop (kernels src/cvcuda/priv/legacy/random_resized_crop.cu:92-154, which take top / left / scale per
 * sample), with the arithmetic of the reference's CPU golden for it (test::ResizedCrop,
 * tests/cvcuda/system/ResizeUtils.cpp:189-241 with its crop arguments): sample positions are scaled by crop / output
 * size and shifted by (left, top); taps clamp at the image's edges, not the rectangle's. Nearest and linear. */
B200PP_PUBLIC int b200ppResizedCrop(const B200ppImageSet *src, const B200ppImageSet *dst, const int32_t *cropRects,
                                    int32_t interp, cudaStream_t stream);

/* b200ppResizedCrop for callers that cannot allocate device memory. No counterpart in the reference: its
 * RandomResizedCrop operator allocates its rectangle table with cudaMalloc when the operator is created.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a pre-processing plug-in inside a serving process
 * whose device memory was all handed out at start-up, a GPU shared with a model that fills it, a latency-critical
 * stretch of a pipeline where the device-wide stall of an allocation is not acceptable. Such a caller still owns its
 * images (src, dst: device memory as for b200ppResizedCrop) but has nowhere to put the per-image rectangle table the
 * kernel reads. Here the table is an array built into the library, and the rectangles are passed from the HOST:
 * hostRects = numSamples x (left, top, width, height) int32 in ordinary or page-locked host memory, copied to the
 * built-in table on `stream` ahead of the kernel. The call allocates nothing, on the device or through any library.
 *
 * Limits and rules:
 *  - at most B200PP_NO_ALLOC_MAX_RECTS images per call; more is refused with B200PP_ERROR_INVALID_ARGUMENT (split the
 *    batch). The table costs 64 KiB of device memory on every GPU that loads the library, until the process exits;
 *  - one table per GPU, shared by every call: calls whose GPU work can overlap (different streams, several threads)
 *    race on it and read each other's rectangles. Issue them on one stream, or order them with events. The table keeps
 *    the last call's rectangles; that is harmless, because a call overwrites every entry it reads;
 *  - the first call on each device looks up the table's device address (once, with that device current). Make that first
 *    call outside any stream capture; later calls only enqueue one copy and one kernel;
 *  - hostRects must stay unchanged until the copy has been taken: for pageable memory that is when the call returns,
 *    for page-locked memory when the stream reaches the copy.
 * Results are those of b200ppResizedCrop given the same rectangles. */
#define B200PP_NO_ALLOC_MAX_RECTS 4096
B200PP_PUBLIC int b200ppResizedCropNoAlloc(const B200ppImageSet *src, const B200ppImageSet *dst, const int32_t *hostRects,
                                           int32_t interp, cudaStream_t stream);

/* The crop-rectangle generator of the reference's RandomResizedCrop
 * (src/cvcuda/priv/legacy/random_resized_crop.cu:288-390): a std::mt19937 seeded with `seed` (0 = from the system's
 * random device) and the reference's draw sequence, so equal seeds give the reference's rectangles. Host only, not
 * thread-safe per generator. Next() writes (left, top, width, height) of the next crop of a rows x cols image. */
typedef struct B200ppRandomCrop B200ppRandomCrop;
B200PP_PUBLIC int  b200ppRandomCropCreate(B200ppRandomCrop **gen, double minScale, double maxScale, double minRatio,
                                          double maxRatio, uint32_t seed);
B200PP_PUBLIC void b200ppRandomCropDestroy(B200ppRandomCrop *gen);
B200PP_PUBLIC int  b200ppRandomCropNext(B200ppRandomCrop *gen, int32_t rows, int32_t cols, int32_t rect[4]);

/* Device buffers for per-sample parameters drawn on the host (what an operator object such as RandomResizedCrop owns,
 * src/cvcuda/priv/legacy/random_resized_crop.cu:305-313,459-475): allocate once, upload from pageable host memory on the
 * stream of the launch that reads them. */
B200PP_PUBLIC int  b200ppParamBufferCreate(void **dev, size_t bytes);
B200PP_PUBLIC void b200ppParamBufferDestroy(void *dev);
B200PP_PUBLIC int  b200ppParamBufferUpload(void *dev, const void *host, size_t bytes, cudaStream_t stream);

/* Parameters of the stand-alone Normalize. base and scale are float32 device tensors addressed as
 * ptr + n*stride[0] + y*stride[1] + x*stride[2] + c*stride[3] (bytes); a stride of 0 broadcasts along that dimension. */
typedef struct B200ppNormalizeOp
{
    const float *base;
    int64_t      baseStride[4];
    const float *scale;
    int64_t      scaleStride[4];
    float        gscale, shift, epsilon;
    uint32_t     flags; /* B200PP_NORMALIZE_SCALE_IS_STDDEV: mul = 1 / sqrt(scale^2 + epsilon) */
} B200ppNormalizeOp;

/* Stand-alone Normalize: dst = SaturateCast((src - base) * mul * gscale + shift), same image sizes and channel count on
 * both sides (1 to 4 interleaved channels; uint8, int8, uint16, int16, int32 or float32 elements; the destination may
 * have another element type). Replaces cvcuda::priv::Normalize::operator() for tensors and variable-shape batches
 * (src/cvcuda/priv/OpNormalize.cpp:38-108, kernels src/cvcuda/priv/legacy/normalize.cu), minus the handle unpacking;
 * results follow the reference's CPU golden (tests/cvcuda/system/TestOpNormalize.cpp:34-77) bit for bit. */
B200PP_PUBLIC int b200ppNormalize(const B200ppImageSet *src, const B200ppImageSet *dst, const B200ppNormalizeOp *op,
                                  cudaStream_t stream);

/* Stand-alone Reformat: dst(n, y, x, c) = src(n, y, x, c) for numSamples images; each side is a B200ppDest-style view
 * (base, element type, channels, width, height and the four byte strides), which expresses NHWC / HWC and NCHW / CHW
 * alike. Element type, channel count and image size must agree. Replaces cvcuda::priv::Reformat::operator()
 * (src/cvcuda/priv/OpReformat.cpp:36-60, kernels src/cvcuda/priv/legacy/reformat.cu), minus the handle unpacking; the
 * reference's golden is the same element-wise copy (tests/cvcuda/system/TestOpReformat.cpp:51-69). */
B200PP_PUBLIC int b200ppReformat(const B200ppDest *src, const B200ppDest *dst, int32_t numSamples, cudaStream_t stream);

/* Stand-alone ConvertTo: dst = SaturateCast(alpha * src + beta) element by element on dense (N)HWC tensors of equal
 * shape; element types uint8, int8, uint16, int16, int32, float32 on either side. Replaces
 * cvcuda::priv::ConvertTo::operator() (src/cvcuda/priv/OpConvertTo.cpp, kernel src/cvcuda/priv/legacy/convert_to.cu:36-58),
 * minus the handle unpacking; arithmetic in double precision as the reference's test expects
 * (tests/cvcuda/system/TestOpConvertTo.cpp:118-133). */
B200PP_PUBLIC int b200ppConvertTo(const B200ppImageSet *src, const B200ppImageSet *dst, double alpha, double beta,
                                  cudaStream_t stream);

/* Stand-alone CopyMakeBorder: dst[i] = src[i] placed at (left, top) inside dst[i], every other destination pixel taken
 * by the border rule (B200PP_BORDER_*; the constant rule writes borderValue[c] converted to the element type). Dense
 * tensors or image lists on either side; top / left apply to all samples unless topList and leftList (device arrays, one
 * packed int32 per sample) are given, as the reference's variable-shape forms require. 1 to 4 interleaved channels of
 * uint8, int8, uint16, int16, int32 or float32. Replaces cvcuda::priv::CopyMakeBorder::operator() in its three forms
 * (src/cvcuda/priv/OpCopyMakeBorder.cpp:42-124; kernels src/cvcuda/priv/legacy/copy_make_border.cu and
 * copy_make_border_var_shape.cu), minus the handle unpacking; results follow the reference's CPU golden
 * (tests/cvcuda/system/TestOpCopyMakeBorder.cpp:40-97) bit for bit. */
B200PP_PUBLIC int b200ppCopyMakeBorder(const B200ppImageSet *src, const B200ppImageSet *dst, int32_t top, int32_t left,
                                       const int32_t *topList, const int32_t *leftList, int32_t borderMode,
                                       const float borderValue[4], cudaStream_t stream);

/* Message of the last failed call on this thread ("" if none). Mirrors nvcvPeekAtLastStatusMessage
 * (src/nvcv/src/include/nvcv/Status.h). */
B200PP_PUBLIC const char *b200ppGetLastErrorMessage(void);

/* ---- Test and profiling hooks. Not part of the operator interface: process-wide state that two threads cannot set
 * differently, kept for the tests (which run every kernel on the same inputs) and for profiling runs. The same holds for
 * the B200PP_* environment variables (B200PP_STAGES, _UNIT_ROWS, _TEAMS, _MAX_CONSUMERS, _MAX_CTAS_PER_SM, _BLOCK_UNITS,
 * _WALK_ROWS, and B200PP_PROBE, which makes the staged kernel move its bytes without computing anything), which are read once
 * per process and, PROBE apart, only reshape launches. ---- */

/* Kernel selection: 0 automatic (default), 1 force the per-pixel gather kernels, 2 force the staged (bulk-copy pipelined)
 * kernel where it applies, 3 force the row-walk kernel. Process-wide. Returns the previous value. Test hook. */
B200PP_PUBLIC int b200ppSetKernelPath(int path);

/* Number of kernels this library has launched in this process (all threads). */
B200PP_PUBLIC uint64_t b200ppGetLaunchCount(void);

/* Reads and clears the device-side error word of the current device (blocking). Non-zero means a kernel gave up
 * on a bounded wait; bit layout is documented next to the kernels. A set word is also reported unasked: the kernel writes
 * it through to a page-locked word the host can see, and the next b200ppResizeCropConvertReformat /
 * b200ppCropFlipNormalizeReformat call on that device (hence the next cvcuda...Submit) returns B200PP_ERROR_INTERNAL
 * without launching, until this function has cleared it. No synchronisation is added to any call for this. */
B200PP_PUBLIC int b200ppReadDeviceError(uint32_t *outError);

/* Test hook. Self-test of the kernels' bounded waits: launches one warp that waits, for at most limitMs (1..1000) milliseconds, on a
 * barrier nothing completes. The kernel then returns normally and bit 8 of the device error word is set; the context
 * stays usable. No counterpart in the reference. */
B200PP_PUBLIC int b200ppSelfTestWaitTimeout(uint32_t limitMs, cudaStream_t stream);

#if defined(__cplusplus)
}
#endif

#endif /* CVCUDA_B200_PREPROC_H */
