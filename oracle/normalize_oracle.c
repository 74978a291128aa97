/* TEST INFRASTRUCTURE ONLY -- see resize_oracle.h for the rules; declared there too.
 *
 * CPU restatement of the reference's Normalize golden (tests/cvcuda/system/TestOpNormalize.cpp:34-77): float32,
 * un-fused, in source order. The reference golden covers uint8 RGBA only; other element types use the reference's
 * saturate cast (round half to even, clamp), restated in preproc_oracle.c. */
#include "preproc_oracle.h"
#include "resize_oracle.h"

#include <math.h>

static float load_f(const void *p, int32_t dtype)
{
    switch (dtype)
    {
    case ORC_U8:
        return *(const uint8_t *)p;
    case ORC_S8:
        return *(const int8_t *)p;
    case ORC_U16:
        return *(const uint16_t *)p;
    case ORC_S16:
        return *(const int16_t *)p;
    case ORC_S32:
        return (float)*(const int32_t *)p;
    default:
        return *(const float *)p;
    }
}

static int esize(int32_t dtype)
{
    return (dtype == ORC_U8 || dtype == ORC_S8) ? 1 : ((dtype == ORC_U16 || dtype == ORC_S16) ? 2 : 4);
}

static void store_sat(void *p, int32_t dtype, float v)
{
    switch (dtype)
    {
    case ORC_U8:
        *(uint8_t *)p = oracle_sat_u8(v);
        break;
    case ORC_S8:
    {
        float r = rintf(v);
        *(int8_t *)p = (int8_t)(r < -128.f ? -128.f : (r > 127.f ? 127.f : r));
        break;
    }
    case ORC_U16:
    {
        float r = rintf(v);
        *(uint16_t *)p = (uint16_t)(r < 0.f ? 0.f : (r > 65535.f ? 65535.f : r));
        break;
    }
    case ORC_S16:
        *(int16_t *)p = oracle_sat_s16(v);
        break;
    case ORC_S32:
        *(int32_t *)p = oracle_sat_s32(v);
        break;
    default:
        *(float *)p = v;
        break;
    }
}

int oracle_normalize(const OraclePlainImage *src, const OraclePlainImage *dst, int32_t n, int32_t srcType, int32_t dstType,
                     int32_t channels, const float *base, const int64_t *baseStride, const float *scale,
                     const int64_t *scaleStride, float gscale, float shift, float epsilon, uint32_t flags)
{
    if (channels < 1 || channels > 4)
        return -1;
    const int se = esize(srcType), de = esize(dstType);
    for (int32_t i = 0; i < n; ++i)
        for (int y = 0; y < src[i].height; ++y)
            for (int x = 0; x < src[i].width; ++x)
                for (int c = 0; c < channels; ++c)
                {
                    const float v = load_f((const uint8_t *)src[i].base + y * src[i].rowStride + ((int64_t)x * channels + c) * se, srcType);
                    const float b = *(const float *)((const char *)base + i * baseStride[0] + y * baseStride[1] + x * baseStride[2] + c * baseStride[3]);
                    const float s = *(const float *)((const char *)scale + i * scaleStride[0] + y * scaleStride[1] + x * scaleStride[2] + c * scaleStride[3]);
                    float       mul;
                    if (flags & 1u)
                    {
                        const float t = s * s + epsilon; /* TestOpNormalize.cpp:58-60 */
                        mul           = 1.0f / sqrtf(t);
                    }
                    else
                        mul = s;
                    const float res = (v - b) * mul * gscale + shift; /* :67-70 */
                    store_sat((uint8_t *)dst[i].base + y * dst[i].rowStride + ((int64_t)x * channels + c) * de, dstType, res);
                }
    return 0;
}
