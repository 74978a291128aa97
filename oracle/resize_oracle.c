/* TEST INFRASTRUCTURE ONLY -- see resize_oracle.h. */
#include "resize_oracle.h"

#include <float.h>
#include <math.h>
#include <stddef.h>

static double load_elem(const void *p, int32_t dtype)
{
    switch (dtype)
    {
    case 0:
        return *(const uint8_t *)p;
    case 2:
        return *(const uint16_t *)p;
    case 3:
        return *(const int16_t *)p;
    default:
        return *(const float *)p;
    }
}

static int elem_size(int32_t dtype)
{
    return dtype == 0 ? 1 : (dtype == 6 ? 4 : 2);
}

/* `res < MinVal ? MinVal : (res > MaxVal ? MaxVal : res)` then the implicit conversion to T
 * (ResizeUtils.cpp:234), MinVal / MaxVal = std::numeric_limits<T>::min() / max() (:320-322). */
static void store_clamped(void *p, int32_t dtype, double res)
{
    switch (dtype)
    {
    case 0:
        *(uint8_t *)p = (uint8_t)(res < 0 ? 0 : (res > 255 ? 255 : res));
        break;
    case 2:
        *(uint16_t *)p = (uint16_t)(res < 0 ? 0 : (res > 65535 ? 65535 : res));
        break;
    case 3:
        *(int16_t *)p = (int16_t)(res < -32768 ? -32768 : (res > 32767 ? 32767 : res));
        break;
    default:
        *(float *)p = (float)(res < FLT_MIN ? FLT_MIN : (res > FLT_MAX ? FLT_MAX : res));
        break;
    }
}

static void copy_elem(void *d, const void *s, int es)
{
    for (int i = 0; i < es; ++i) ((uint8_t *)d)[i] = ((const uint8_t *)s)[i];
}

int oracle_resize_plain(const OraclePlainImage *src, const OraclePlainImage *dst, int32_t n, int32_t dtype,
                        int32_t channels, int32_t interp, int32_t goldenFloat)
{
    return oracle_resized_crop(src, dst, n, dtype, channels, interp, goldenFloat, 0);
}

int oracle_resized_crop(const OraclePlainImage *src, const OraclePlainImage *dst, int32_t n, int32_t dtype,
                        int32_t channels, int32_t interp, int32_t goldenFloat, const int32_t *rects)
{
    if (!(dtype == 0 || dtype == 2 || dtype == 3 || dtype == 6) || channels < 1 || channels > 4 || (interp != 0 && interp != 1))
        return -1;
    const int es = elem_size(dtype);
    for (int32_t i = 0; i < n; ++i)
    {
        const OraclePlainImage *S = &src[i], *D = &dst[i];
        /* ResizeUtils.cpp:193-194: float scale factors */
        const int   left = rects ? rects[4 * i + 0] : 0, top = rects ? rects[4 * i + 1] : 0;
        const int   cropW = rects ? rects[4 * i + 2] : S->width, cropH = rects ? rects[4 * i + 3] : S->height;
        const float scaleH = (float)cropH / D->height;
        const float scaleW = (float)cropW / D->width;
        for (int dy = 0; dy < D->height; ++dy)
        {
            for (int dx = 0; dx < D->width; ++dx)
            {
                uint8_t *dpix = (uint8_t *)D->base + dy * D->rowStride + (int64_t)dx * channels * es;
                if (interp == 0)
                {
                    /* :204-220: float arithmetic */
                    const float fy = scaleH * (dy + 0.5f) + top;
                    const float fx = scaleW * (dx + 0.5f) + left;
                    int         sy = (int)floorf(fy);
                    int         sx = (int)floorf(fx);
                    sy             = sy < S->height - 1 ? sy : S->height - 1;
                    sx             = sx < S->width - 1 ? sx : S->width - 1;
                    const uint8_t *spix = (const uint8_t *)S->base + sy * S->rowStride + (int64_t)sx * channels * es;
                    for (int c = 0; c < channels; ++c) copy_elem(dpix + c * es, spix + c * es, es);
                }
                else
                {
                    /* :222-241: the float scale is promoted, everything else is double */
                    double fy = scaleH * (dy + 0.5) - 0.5 + top;
                    double fx = scaleW * (dx + 0.5) - 0.5 + left;
                    int    sy = (int)floor(fy);
                    int    sx = (int)floor(fx);
                    fy        = (sy < 0) ? 0 : ((sy > S->height - 2) ? 1 : fy - sy);
                    fx        = (sx < 0) ? 0 : ((sx > S->width - 2) ? 1 : fx - sx);
                    {
                        const int ty = sy < S->height - 2 ? sy : S->height - 2;
                        const int tx = sx < S->width - 2 ? sx : S->width - 2;
                        sy           = ty > 0 ? ty : 0;
                        sx           = tx > 0 ? tx : 0;
                    }
                    const double wy[2] = {1 - fy, fy};
                    const double wx[2] = {1 - fx, fx};
                    const uint8_t *r0 = (const uint8_t *)S->base + sy * S->rowStride;
                    const uint8_t *r1 = r0 + S->rowStride;
                    for (int c = 0; c < channels; ++c)
                    {
                        const size_t o0 = ((size_t)sx * channels + c) * es, o1 = ((size_t)(sx + 1) * channels + c) * es;
                        const double sum = load_elem(r0 + o0, dtype) * wy[0] * wx[0] + load_elem(r1 + o0, dtype) * wy[1] * wx[0]
                                         + load_elem(r0 + o1, dtype) * wy[0] * wx[1] + load_elem(r1 + o1, dtype) * wy[1] * wx[1];
                        if (dtype == 6 && !goldenFloat)
                            *(float *)(dpix + c * es) = (float)sum;
                        else if (dtype == 3 && !goldenFloat)
                            /* the reference's CUDA operators saturate-cast the signed blend
                             * (src/cvcuda/priv/OpResize.cu:228-262); the golden's fabs (ResizeUtils.cpp:226) would
                             * flip the sign of negative int16 results, which its own tests never produce */
                            store_clamped(dpix + c * es, dtype, rint(sum));
                        else
                            store_clamped(dpix + c * es, dtype, rint(fabs(sum)));
                    }
                }
            }
        }
    }
    return 0;
}
