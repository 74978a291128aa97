/* TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement of the reference project's golden code for the stand-alone Resize operator, nearest and linear
 * interpolation (tests/cvcuda/system/ResizeUtils.cpp:189-241: `resizedCrop` with top = left = 0 and the crop equal to
 * the whole source, which is what `test::Resize` calls for these two interpolations, :320-330). The product library
 * never links, loads or calls it.
 *
 * Parity is pinned: tests compare this restatement element-for-element with the reference's own function (compiled
 * from the reference tree into oracle/_ref by build_oracle.py) over the shapes of the reference's test table.
 *
 * Element types: 0 = uint8, 2 = uint16, 3 = int16, 6 = float32 (the codes of preproc_oracle.h); 1 to 4 interleaved
 * channels. Strides in BYTES.
 */
#ifndef RESIZE_ORACLE_H
#define RESIZE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C"
{
#endif

typedef struct OraclePlainImage
{
    void   *base;
    int32_t width, height;
    int64_t rowStride;
} OraclePlainImage;

/* dst[i] = resize(src[i]) for i < n. interp: 0 nearest, 1 linear. `goldenFloat`: for float32 elements and linear
 * interpolation the reference golden rounds the blend to an integer and clamps it to [FLT_MIN, FLT_MAX]
 * (ResizeUtils.cpp:226-234 with std::numeric_limits<float>::min()); with goldenFloat == 0 the blend is stored as
 * computed, which is what the reference's CUDA operator does (src/cvcuda/priv/OpResize.cu:228-262) and what the
 * product implements. The same flag covers the golden's other quirk: it rounds fabs(blend) (ResizeUtils.cpp:226), so a
 * negative int16 blend comes out positive; with goldenFloat == 0 the signed blend is rounded and clamped, as the
 * reference's CUDA operators do (their tests run int16 with nearest only, so the golden's sign flip is never
 * exercised). Returns 0, or -1 for arguments it does not cover. */
int oracle_resize_plain(const OraclePlainImage *src, const OraclePlainImage *dst, int32_t n, int32_t dtype,
                        int32_t channels, int32_t interp, int32_t goldenFloat);

/* The same golden with its crop arguments (ResizeUtils.cpp:190-194: top, left, crop_rows, crop_cols), as the
 * RandomResizedCrop test calls it (tests/cvcuda/system/TestOpRandomResizedCrop.cpp:206-208): rects holds
 * (left, top, crop_cols, crop_rows) per image, NULL = whole images. Taps clamp at the image's edges, not the rectangle's. */
int oracle_resized_crop(const OraclePlainImage *src, const OraclePlainImage *dst, int32_t n, int32_t dtype,
                        int32_t channels, int32_t interp, int32_t goldenFloat, const int32_t *rects);

/* Stand-alone Normalize golden (tests/cvcuda/system/TestOpNormalize.cpp:34-77), element types as in preproc_oracle.h
 * (source: U8, S8, U16, S16, S32, F32; destination the same set). base / scale: float32, addressed as
 * ptr + n*stride[0] + y*stride[1] + x*stride[2] + c*stride[3] (bytes; 0 broadcasts). flags bit 0: scale holds standard
 * deviations. Image i of dst has the size of image i of src. */
int oracle_normalize(const OraclePlainImage *src, const OraclePlainImage *dst, int32_t n, int32_t srcType, int32_t dstType,
                     int32_t channels, const float *base, const int64_t *baseStride, const float *scale,
                     const int64_t *scaleStride, float gscale, float shift, float epsilon, uint32_t flags);

#ifdef __cplusplus
}
#endif

#endif
