/* TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement of the reference project's golden code for the fused pre-processing path
 * (ResizeCropConvertReformat and CropFlipNormalizeReformat). It exists to check the CUDA kernels and to be
 * timed as the CPU baseline; the product library never links, loads or calls it.
 *
 * Parity is pinned: tests compare this restatement element-for-element with the reference's own golden
 * functions (compiled from the reference tree into oracle/_ref by build_oracle.py) over the reference's
 * test tables, and with fixtures those functions produced (tests/golden).
 *
 * All strides are in BYTES. All arithmetic is float32, un-fused, in the reference's source order.
 */
#ifndef PREPROC_ORACLE_H
#define PREPROC_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C"
{
#endif

/* element type codes (source and destination) */
enum
{
    ORC_U8  = 0,
    ORC_S8  = 1,
    ORC_U16 = 2,
    ORC_S16 = 3,
    ORC_U32 = 4,
    ORC_S32 = 5,
    ORC_F32 = 6,
    ORC_F16 = 7 /* destination only; not offered by the reference, an extension (round-to-nearest-even) */
};

/* border codes = NVCVBorderType (nvcv/BorderType.h:36-43) */
enum
{
    ORC_BORDER_CONSTANT   = 0,
    ORC_BORDER_REPLICATE  = 1,
    ORC_BORDER_REFLECT    = 2,
    ORC_BORDER_WRAP       = 3,
    ORC_BORDER_REFLECT101 = 4
};

typedef struct OracleImage
{
    const void *base;
    int32_t     width, height;
    int64_t     rowStride;   /* bytes between rows of one plane */
    int64_t     planeStride; /* bytes between planes (planar sources only) */
} OracleImage;

typedef struct OracleDst
{
    void   *base;
    int32_t dtype;
    int32_t width, height; /* full output extent (the canvas) */
    int64_t sampleStride, rowStride, pixStride, chanStride;
} OracleDst;

typedef struct OracleResizeParams
{
    int32_t resizeW, resizeH; /* size the (sub-view of the) source is resized to */
    int32_t cropX, cropY;     /* top-left of the crop inside the resized image */
    int32_t interp;           /* 0 nearest, 1 linear (NVCVInterpolationType) */
    int32_t srcCast;          /* round the interpolated value to uint8 before the affine step */
    int32_t manip;            /* 0 no-op, 1 reverse channel order (NVCVChannelManip) */
    int32_t epilogue;         /* 0: scale*v+offset   1: (v-base[c])*mul[c]*gscale+shift, c = source channel */
    float   scale, offset;
    float   base[4], mul[4];
    float   gscale, shift;
    /* placement of the cropped region inside the output canvas (letterbox); region = canvas when unused */
    int32_t dstX, dstY, regionW, regionH;
    float   padValue; /* source-domain value of pixels outside the region; goes through the epilogue */
} OracleResizeParams;

/* ResizeCropConvertReformat golden, generalised.
 * Follows tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:76-172 exactly when roi == flip == NULL,
 * epilogue == 0, region == canvas and dtype is u8 or f32. Sources are interleaved 3-channel uint8.
 * roi:  optional int32[4*n] (x, y, w, h): the source of sample i is that sub-view of images[i].
 * flip: optional int32[n], CropFlipNormalizeReformat codes applied to region coordinates after the resize
 *       (1 mirror x, 0 mirror y, -1 both, anything else none).
 * nthreads <= 1 runs single-threaded. Returns 0, or -1 on an unsupported argument. */
int oracle_resize_crop(const OracleImage *images, int32_t n, const int32_t *roi, const int32_t *flip,
                       const OracleResizeParams *p, const OracleDst *dst, int32_t nthreads);

typedef struct OracleSliceParams
{
    int32_t srcType, srcPlanar, channels;
    int32_t border;
    float   borderValue;
    const float *base;
    int32_t      baseCh;
    const float *scale;
    int32_t      scaleCh;
    float    gscale, shift, epsilon;
    uint32_t flags; /* bit 0: scale holds standard deviations (CVCUDA_NORMALIZE_SCALE_IS_STDDEV) */
} OracleSliceParams;

/* CropFlipNormalizeReformat golden.
 * Follows tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:43-149, border rules
 * tests/common/BorderUtils.cpp:24-137, ValueAt tests/common/InterpUtils.hpp:74-89.
 * cropRect: int32[4*n] (x, y, w, h); flip: int32[n]. */
int oracle_crop_flip_normalize(const OracleImage *images, int32_t n, const int32_t *cropRect, const int32_t *flip,
                               const OracleSliceParams *p, const OracleDst *dst, int32_t nthreads);

/* Algorithmic source bytes of one sample of the resize path: the number of distinct 32-byte sectors (address
 * taken relative to a 32-byte aligned base, given row stride) that hold at least one byte a tap of the golden
 * formula addresses, times 32. */
int64_t oracle_resize_source_bytes(int32_t srcW, int32_t srcH, int64_t rowStride, const int32_t *roi,
                                   const OracleResizeParams *p);

/* rounding helpers, exported so tests can compare them with cuda::SaturateCast's host path */
uint8_t  oracle_sat_u8(float v);
int16_t  oracle_sat_s16(float v);
int32_t  oracle_sat_s32(float v);
uint16_t oracle_f32_to_f16_bits(float v);

/* Stand-alone CopyMakeBorder golden (tests/cvcuda/system/TestOpCopyMakeBorder.cpp:40-175); images are the
 * OraclePlainImage of resize_oracle.h. top / left hold one value, or one per sample when perSample != 0. */
struct OraclePlainImage;
int oracle_copy_make_border(const struct OraclePlainImage *src, const struct OraclePlainImage *dst, int32_t n,
                            int32_t elemSize, int32_t channels, const int32_t *top, const int32_t *left, int32_t perSample,
                            int32_t border, const uint32_t *fill);

#ifdef __cplusplus
}
#endif
#endif
