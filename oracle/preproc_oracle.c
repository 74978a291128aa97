/* TEST INFRASTRUCTURE ONLY -- see preproc_oracle.h. Build: gcc -std=c11 -O2 -ffp-contract=off -shared -fPIC. */
#define _GNU_SOURCE
#include "preproc_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- rounding / casts
 * cuda::SaturateCast host path (cvcuda/cuda_tools/detail/SaturateCastImpl.hpp:31-50 with RoundEvenImpl,
 * detail/MathWrappersImpl.hpp:403-415): round half to even, then clamp to the target range.
 * nearbyintf under the default rounding mode is round-half-to-even. */

static inline float clampf(float v, float lo, float hi)
{
    return v < lo ? lo : (v > hi ? hi : v);
}

uint8_t oracle_sat_u8(float v)
{
    return (uint8_t)clampf(nearbyintf(v), 0.f, 255.f);
}

static inline int8_t sat_s8(float v)
{
    return (int8_t)clampf(nearbyintf(v), -128.f, 127.f);
}

static inline uint16_t sat_u16(float v)
{
    return (uint16_t)clampf(nearbyintf(v), 0.f, 65535.f);
}

int16_t oracle_sat_s16(float v)
{
    return (int16_t)clampf(nearbyintf(v), -32768.f, 32767.f);
}

/* For 32-bit targets the reference clamps to float(INT_MAX) = 2^31 and then converts, which is undefined
 * on the host for the top value; the device instruction saturates. The oracle saturates. */
int32_t oracle_sat_s32(float v)
{
    float r = nearbyintf(v);
    if (!(r > -2147483648.f))
        return r != r ? 0 : INT32_MIN;
    if (r >= 2147483648.f)
        return INT32_MAX;
    return (int32_t)r;
}

static inline uint32_t sat_u32(float v)
{
    float r = nearbyintf(v);
    if (!(r > 0.f))
        return 0u;
    if (r >= 4294967296.f)
        return UINT32_MAX;
    return (uint32_t)r;
}

uint16_t oracle_f32_to_f16_bits(float v)
{
    _Float16 h = (_Float16)v; /* IEEE round-to-nearest-even */
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

static inline void store_cast(void *p, int dtype, float v)
{
    switch (dtype)
    {
    case ORC_U8:
        *(uint8_t *)p = oracle_sat_u8(v);
        break;
    case ORC_S8:
        *(int8_t *)p = sat_s8(v);
        break;
    case ORC_U16:
        *(uint16_t *)p = sat_u16(v);
        break;
    case ORC_S16:
        *(int16_t *)p = oracle_sat_s16(v);
        break;
    case ORC_U32:
        *(uint32_t *)p = sat_u32(v);
        break;
    case ORC_S32:
        *(int32_t *)p = oracle_sat_s32(v);
        break;
    case ORC_F32:
        *(float *)p = v;
        break;
    case ORC_F16:
        *(uint16_t *)p = oracle_f32_to_f16_bits(v);
        break;
    }
}

static const int kElemSize[8] = {1, 1, 2, 2, 4, 4, 4, 2};

static inline float load_as_float(const void *p, int dtype)
{
    switch (dtype)
    {
    case ORC_U8:
        return (float)*(const uint8_t *)p;
    case ORC_S8:
        return (float)*(const int8_t *)p;
    case ORC_U16:
        return (float)*(const uint16_t *)p;
    case ORC_S16:
        return (float)*(const int16_t *)p;
    case ORC_U32:
        return (float)*(const uint32_t *)p;
    case ORC_S32:
        return (float)*(const int32_t *)p;
    default:
        return *(const float *)p;
    }
}

/* static_cast<T_Src>(borderValue) followed by the promotion to float the normalisation performs */
static inline float border_as_src(float bv, int dtype)
{
    switch (dtype)
    {
    case ORC_U8:
        return (float)(uint8_t)bv;
    case ORC_S8:
        return (float)(int8_t)bv;
    case ORC_U16:
        return (float)(uint16_t)bv;
    case ORC_S16:
        return (float)(int16_t)bv;
    case ORC_U32:
        return (float)(uint32_t)bv;
    case ORC_S32:
        return (float)(int32_t)bv;
    default:
        return bv;
    }
}

/* ---------------------------------------------------------------- thread fan-out over (sample,row) */

typedef void (*row_fn)(const void *ctx, int32_t sample, int32_t row);

typedef struct
{
    row_fn      fn;
    const void *ctx;
    int64_t     begin, end;
    int32_t     rowsPerSample;
} Span;

static void *span_main(void *arg)
{
    const Span *s = (const Span *)arg;
    for (int64_t i = s->begin; i < s->end; ++i) s->fn(s->ctx, (int32_t)(i / s->rowsPerSample), (int32_t)(i % s->rowsPerSample));
    return NULL;
}

static void for_rows(row_fn fn, const void *ctx, int32_t n, int32_t rows, int32_t nthreads)
{
    int64_t total = (int64_t)n * rows;
    if (nthreads < 1)
        nthreads = 1;
    if (nthreads > 1024)
        nthreads = 1024;
    if ((int64_t)nthreads > total)
        nthreads = (int32_t)(total > 0 ? total : 1);
    if (nthreads == 1)
    {
        Span s = {fn, ctx, 0, total, rows};
        span_main(&s);
        return;
    }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * nthreads);
    Span      *sp = (Span *)malloc(sizeof(Span) * nthreads);
    for (int t = 0; t < nthreads; ++t)
    {
        sp[t].fn            = fn;
        sp[t].ctx           = ctx;
        sp[t].begin         = total * t / nthreads;
        sp[t].end           = total * (t + 1) / nthreads;
        sp[t].rowsPerSample = rows;
        pthread_create(&th[t], NULL, span_main, &sp[t]);
    }
    for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
    free(th);
    free(sp);
}

/* ---------------------------------------------------------------- resize + crop + convert + reformat */

typedef struct
{
    const OracleImage        *images;
    const int32_t            *roi, *flip;
    const OracleResizeParams *p;
    const OracleDst          *dst;
} ResizeCtx;

static inline float epilogue(const OracleResizeParams *p, int c, float v)
{
    if (p->epilogue == 0)
        return p->scale * v + p->offset; /* TestOpResizeCropConvertReformat.cpp:127,164 */
    return (v - p->base[c]) * p->mul[c] * p->gscale + p->shift; /* TestOpCropFlipNormalizeReformat.cpp:139 */
}

static void resize_row(const void *vctx, int32_t n, int32_t y)
{
    const ResizeCtx          *ctx = (const ResizeCtx *)vctx;
    const OracleResizeParams *p   = ctx->p;
    const OracleDst          *d   = ctx->dst;
    const OracleImage        *im  = &ctx->images[n];

    const uint8_t *srcBase = (const uint8_t *)im->base;
    int32_t        srcW = im->width, srcH = im->height;
    if (ctx->roi)
    {
        const int32_t *r = ctx->roi + 4 * (int64_t)n;
        srcBase += (int64_t)r[1] * im->rowStride + (int64_t)r[0] * 3;
        srcW = r[2];
        srcH = r[3];
    }
    const int fc = ctx->flip ? ctx->flip[n] : 2;

    const int esz = kElemSize[d->dtype];
    (void)esz;
    uint8_t *dstRow = (uint8_t *)d->base + (int64_t)n * d->sampleStride + (int64_t)y * d->rowStride;

    /* TestOpResizeCropConvertReformat.cpp:95-103 */
    int mapC[3] = {0, 1, 2};
    if (p->manip == 1)
        for (int c = 0; c < 3; ++c) mapC[c] = 3 - c - 1;

    const float scaleW = (float)srcW / p->resizeW;
    const float scaleH = (float)srcH / p->resizeH;

    for (int32_t x = 0; x < d->width; ++x)
    {
        uint8_t *dstPix = dstRow + (int64_t)x * d->pixStride;
        int32_t  rx = x - p->dstX, ry = y - p->dstY;

        if (rx < 0 || ry < 0 || rx >= p->regionW || ry >= p->regionH)
        {
            for (int c = 0; c < 3; ++c) store_cast(dstPix + mapC[c] * d->chanStride, d->dtype, epilogue(p, c, p->padValue));
            continue;
        }
        /* flip of region coordinates: TestOpCropFlipNormalizeReformat.cpp:103-122 with the region as the crop */
        int32_t dx = rx, dy = ry;
        if (fc == 1 || fc == -1)
            dx = p->regionW - 1 - rx;
        if (fc == 0 || fc == -1)
            dy = p->regionH - 1 - ry;

        if (p->interp == 0)
        {
            /* :118-129 */
            int sx = (int)floorf(scaleW * ((float)(dx + p->cropX) + 0.5f));
            int sy = (int)floorf(scaleH * ((float)(dy + p->cropY) + 0.5f));

            const uint8_t *s0 = srcBase + (int64_t)sy * im->rowStride + (int64_t)sx * 3;
            for (int c = 0; c < 3; ++c) store_cast(dstPix + mapC[c] * d->chanStride, d->dtype, epilogue(p, c, (float)s0[c]));
        }
        else
        {
            /* :130-168 */
            float fx = scaleW * ((float)(dx + p->cropX) + 0.5f) - 0.5f;
            float fy = scaleH * ((float)(dy + p->cropY) + 0.5f) - 0.5f;

            int sx0 = (int)floorf(fx);
            int sy0 = (int)floorf(fy);
            int sx1 = sx0 + 1 < srcW - 1 ? sx0 + 1 : srcW - 1;
            int sy1 = sy0 + 1 < srcH - 1 ? sy0 + 1 : srcH - 1;

            fx -= (float)sx0;
            fy -= (float)sy0;

            sx0 = sx0 > 0 ? sx0 : 0;
            sy0 = sy0 > 0 ? sy0 : 0;

            const float wx0 = 1 - fx, wx1 = fx, wy0 = 1 - fy, wy1 = fy;

            const uint8_t *r0 = srcBase + (int64_t)sy0 * im->rowStride;
            const uint8_t *r1 = srcBase + (int64_t)sy1 * im->rowStride;
            for (int c = 0; c < 3; ++c)
            {
                float val = (float)r0[sx0 * 3 + c] * wy0 * wx0 + (float)r0[sx1 * 3 + c] * wy0 * wx1
                          + (float)r1[sx0 * 3 + c] * wy1 * wx0 + (float)r1[sx1 * 3 + c] * wy1 * wx1;
                if (p->srcCast)
                    val = (float)oracle_sat_u8(val);
                store_cast(dstPix + mapC[c] * d->chanStride, d->dtype, epilogue(p, c, val));
            }
        }
    }
}

int oracle_resize_crop(const OracleImage *images, int32_t n, const int32_t *roi, const int32_t *flip,
                       const OracleResizeParams *p, const OracleDst *dst, int32_t nthreads)
{
    if (!images || !p || !dst || n < 0)
        return -1;
    if (!(dst->dtype == ORC_U8 || dst->dtype == ORC_F32 || dst->dtype == ORC_F16))
        return -1;
    if (p->interp != 0 && p->interp != 1)
        return -1;
    ResizeCtx ctx = {images, roi, flip, p, dst};
    for_rows(resize_row, &ctx, n, dst->height, nthreads);
    return 0;
}

/* ---------------------------------------------------------------- crop + flip + normalise + reformat */

/* tests/common/BorderUtils.cpp:24-76. Returns 0 when the coordinate stays outside (constant border). */
static inline int border_index(int *c, int size, int mode)
{
    if (*c >= 0 && *c < size)
        return 1;
    switch (mode)
    {
    case ORC_BORDER_CONSTANT:
        return 0;
    case ORC_BORDER_REPLICATE:
        *c = *c < 0 ? 0 : size - 1;
        return 1;
    case ORC_BORDER_WRAP:
        *c = *c % size;
        if (*c < 0)
            *c += size;
        return 1;
    case ORC_BORDER_REFLECT:
        *c = *c % (size * 2);
        if (*c < 0)
            *c += size * 2;
        if (*c >= size)
            *c = size - 1 - (*c - size);
        return 1;
    case ORC_BORDER_REFLECT101:
        if (size == 1)
        {
            *c = 0;
        }
        else
        {
            *c = *c % (2 * size - 2);
            if (*c < 0)
                *c += 2 * size - 2;
            *c = size - 1 - abs(size - 1 - *c);
        }
        return 1;
    }
    return 0;
}

typedef struct
{
    const OracleImage       *images;
    const int32_t           *rect, *flip;
    const OracleSliceParams *p;
    const OracleDst         *dst;
} SliceCtx;

static void slice_row(const void *vctx, int32_t n, int32_t i)
{
    const SliceCtx          *ctx = (const SliceCtx *)vctx;
    const OracleSliceParams *p   = ctx->p;
    const OracleDst         *d   = ctx->dst;
    const OracleImage       *im  = &ctx->images[n];
    const int32_t           *r   = ctx->rect + 4 * (int64_t)n;
    const int32_t cx = r[0], cy = r[1], cw = r[2], ch = r[3];
    const int     fc  = ctx->flip[n];
    const int     ssz = kElemSize[p->srcType];
    const int64_t srcPix  = p->srcPlanar ? ssz : (int64_t)ssz * p->channels;
    const int64_t srcChan = p->srcPlanar ? im->planeStride : ssz;
    const float   bsrc    = border_as_src(p->borderValue, p->srcType);

    uint8_t *dstRow = (uint8_t *)d->base + (int64_t)n * d->sampleStride + (int64_t)i * d->rowStride;

    for (int32_t j = 0; j < d->width; ++j)
    {
        uint8_t *dstPix = dstRow + (int64_t)j * d->pixStride;
        if (i >= ch || j >= cw)
        { /* TestOpCropFlipNormalizeReformat.cpp:66-80 */
            for (int k = 0; k < p->channels; ++k) memset(dstPix + k * d->chanStride, 0, kElemSize[d->dtype]);
            continue;
        }
        int x, y; /* :101-122 */
        if (fc == 1)
        {
            x = cw - 1 - j + cx;
            y = i + cy;
        }
        else if (fc == 0)
        {
            x = j + cx;
            y = ch - 1 - i + cy;
        }
        else if (fc == -1)
        {
            x = cw - 1 - j + cx;
            y = ch - 1 - i + cy;
        }
        else
        {
            x = j + cx;
            y = i + cy;
        }
        /* IsInside remaps both coordinates unless the pixel is inside (BorderUtils.cpp:102-135);
         * for a constant border any outside coordinate yields the border value. */
        int inside;
        if (x >= 0 && x < im->width && y >= 0 && y < im->height)
            inside = 1;
        else if (p->border == ORC_BORDER_CONSTANT)
            inside = 0;
        else
        {
            border_index(&x, im->width, p->border);
            border_index(&y, im->height, p->border);
            inside = 1;
        }
        for (int k = 0; k < p->channels; ++k)
        {
            const int bk = p->baseCh == 1 ? 0 : k;
            const int sk = p->scaleCh == 1 ? 0 : k;
            float     mul;
            if (p->flags & 1u)
            { /* :88-93 */
                float s  = p->scale[sk];
                float xx = s * s + p->epsilon;
                mul      = 1.0f / sqrtf(xx);
            }
            else
                mul = p->scale[sk];
            float base = p->base[bk];
            float out  = inside ? load_as_float((const uint8_t *)im->base + (int64_t)y * im->rowStride + (int64_t)x * srcPix
                                                   + (int64_t)k * srcChan,
                                               p->srcType)
                                : bsrc;
            store_cast(dstPix + k * d->chanStride, d->dtype, (out - base) * mul * p->gscale + p->shift); /* :139 */
        }
    }
}

int oracle_crop_flip_normalize(const OracleImage *images, int32_t n, const int32_t *cropRect, const int32_t *flip,
                               const OracleSliceParams *p, const OracleDst *dst, int32_t nthreads)
{
    if (!images || !cropRect || !flip || !p || !dst || n < 0)
        return -1;
    if (p->srcType < 0 || p->srcType > ORC_F32 || dst->dtype < 0 || dst->dtype > ORC_F16)
        return -1;
    if (p->channels < 1 || p->channels > 4 || p->border < 0 || p->border > 4)
        return -1;
    SliceCtx ctx = {images, cropRect, flip, p, dst};
    for_rows(slice_row, &ctx, n, dst->height, nthreads);
    return 0;
}

/* ---------------------------------------------------------------- algorithmic source bytes */

static inline void mark(uint8_t *bm, int64_t byteAddr, int len)
{
    int64_t a = byteAddr >> 5, b = (byteAddr + len - 1) >> 5;
    for (int64_t s = a; s <= b; ++s) bm[s >> 3] |= (uint8_t)(1u << (s & 7));
}

int64_t oracle_resize_source_bytes(int32_t srcW, int32_t srcH, int64_t rowStride, const int32_t *roi,
                                   const OracleResizeParams *p)
{
    int64_t  total = rowStride * (int64_t)srcH;
    int64_t  nsec  = (total + 31) / 32 + 1;
    uint8_t *bm    = (uint8_t *)calloc((size_t)(nsec / 8 + 2), 1);
    int64_t  off   = 0;
    int32_t  w = srcW, h = srcH;
    if (roi)
    {
        off = (int64_t)roi[1] * rowStride + (int64_t)roi[0] * 3;
        w   = roi[2];
        h   = roi[3];
    }
    const float scaleW = (float)w / p->resizeW, scaleH = (float)h / p->resizeH;
    for (int32_t dy = 0; dy < p->regionH; ++dy)
        for (int32_t dx = 0; dx < p->regionW; ++dx)
        {
            if (p->interp == 0)
            {
                int sx = (int)floorf(scaleW * ((float)(dx + p->cropX) + 0.5f));
                int sy = (int)floorf(scaleH * ((float)(dy + p->cropY) + 0.5f));
                mark(bm, off + (int64_t)sy * rowStride + (int64_t)sx * 3, 3);
            }
            else
            {
                float fx  = scaleW * ((float)(dx + p->cropX) + 0.5f) - 0.5f;
                float fy  = scaleH * ((float)(dy + p->cropY) + 0.5f) - 0.5f;
                int   sx0 = (int)floorf(fx), sy0 = (int)floorf(fy);
                int   sx1 = sx0 + 1 < w - 1 ? sx0 + 1 : w - 1;
                int   sy1 = sy0 + 1 < h - 1 ? sy0 + 1 : h - 1;
                sx0       = sx0 > 0 ? sx0 : 0;
                sy0       = sy0 > 0 ? sy0 : 0;
                mark(bm, off + (int64_t)sy0 * rowStride + (int64_t)sx0 * 3, 3);
                mark(bm, off + (int64_t)sy0 * rowStride + (int64_t)sx1 * 3, 3);
                mark(bm, off + (int64_t)sy1 * rowStride + (int64_t)sx0 * 3, 3);
                mark(bm, off + (int64_t)sy1 * rowStride + (int64_t)sx1 * 3, 3);
            }
        }
    int64_t cnt = 0;
    for (int64_t i = 0; i < nsec / 8 + 2; ++i) cnt += __builtin_popcount(bm[i]);
    free(bm);
    return cnt * 32;
}

/* ---------------------------------------------------------------- stand-alone CopyMakeBorder */

#include "resize_oracle.h"

/* tests/cvcuda/system/TestOpCopyMakeBorder.cpp:40-97 (tensor form) and :99-175 (variable-shape forms): each destination
 * pixel takes the source pixel at (x - left, y - top), or -- outside the source -- the per-channel constant converted
 * with static_cast<T>, or the source pixel the border rule maps to. elemSize 1, 2 or 4; `fill` holds the constants
 * already converted to the element type (low bytes of each 32-bit word). */
int oracle_copy_make_border(const OraclePlainImage *src, const OraclePlainImage *dst, int32_t n, int32_t elemSize,
                            int32_t channels, const int32_t *top, const int32_t *left, int32_t perSample, int32_t border,
                            const uint32_t *fill)
{
    if (channels < 1 || channels > 4 || border < 0 || border > 4 || !(elemSize == 1 || elemSize == 2 || elemSize == 4))
        return -1;
    for (int32_t i = 0; i < n; ++i)
    {
        const int t = top[perSample ? i : 0], l = left[perSample ? i : 0];
        for (int y = 0; y < dst[i].height; ++y)
            for (int x = 0; x < dst[i].width; ++x)
            {
                int       sx = x - l, sy = y - t;
                uint8_t  *d  = (uint8_t *)dst[i].base + y * dst[i].rowStride + (int64_t)x * channels * elemSize;
                const int in = sx >= 0 && sx < src[i].width && sy >= 0 && sy < src[i].height;
                if (!in && border == ORC_BORDER_CONSTANT)
                {
                    for (int c = 0; c < channels; ++c) memcpy(d + c * elemSize, &fill[c], (size_t)elemSize);
                    continue;
                }
                if (!in)
                {
                    border_index(&sx, src[i].width, border);
                    border_index(&sy, src[i].height, border);
                }
                memcpy(d, (const uint8_t *)src[i].base + sy * src[i].rowStride + (int64_t)sx * channels * elemSize,
                       (size_t)channels * elemSize);
            }
    }
    return 0;
}
