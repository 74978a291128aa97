// Stand-alone Resize (nearest / linear) for interleaved images of 1, 3 or 4 channels of uint8, uint16, int16 or float32,
// dense tensors or variable-shape image batches on either side.
//
// Replaces NearestResize / LinearResize of the reference (src/cvcuda/priv/OpResize.cu:141-166, 303-342) and the
// variable-shape resize it delegates to (src/cvcuda/priv/legacy/resize_var_shape.cu); arithmetic follows the
// reference's CPU golden (tests/cvcuda/system/ResizeUtils.cpp:189-241) operation by operation, including its use of
// double precision for the linear weights and products, so integer element types come out bit-exact (B200 runs double
// precision at half the float32 rate and the operator is bound by HBM, not by arithmetic).
//
// A thread produces a 4 x 4 patch of destination pixels (columns 32 apart, rows 8 apart). Pixels of 1, 2 or 4 elements
// move as one vector when their addresses allow it. uint8 linear blends run in float32 with an exact double-precision
// redo of the rare values that land near a rounding boundary, so the result is still the golden's, bit for bit.
#ifndef CVCUDA_B200_PLAIN_RESIZE_KERNELS_CUH
#define CVCUDA_B200_PLAIN_RESIZE_KERNELS_CUH

#include "kparams.h"

namespace b200pp {

// One side of a stand-alone resize: dense [N, H, W, C] or a device array of image descriptors.
struct PlainSide
{
    uint8_t                 *base;
    const B200ppImageBuffer *list;
    long long                sampleStride, rowStride;
    int                      width, height;
};

struct PlainResizeKParams
{
    PlainSide src, dst;
    int       numSamples;
};

struct PlainView
{
    uint8_t  *base;
    long long pitch;
    int       w, h;
};

__device__ __forceinline__ PlainView plain_view(const PlainSide &s, int n)
{
    PlainView v;
    if (s.list)
    {
        const B200ppImagePlane &pl = s.list[n].planes[0];
        v.base  = const_cast<uint8_t *>(pl.basePtr);
        v.pitch = pl.rowStride;
        v.w     = pl.width;
        v.h     = pl.height;
    }
    else
    {
        v.base  = s.base + static_cast<long long>(n) * s.sampleStride;
        v.pitch = s.rowStride;
        v.w     = s.width;
        v.h     = s.height;
    }
    return v;
}

template<typename T, int C>
struct alignas(sizeof(T) * (C == 3 ? 1 : C)) PlainPixel
{
    T v[C];
};

template<typename T, int C>
__device__ __forceinline__ PlainPixel<T, C> load_plain(const uint8_t *p, bool vector)
{
    PlainPixel<T, C> px;
    if (C != 3 && vector)
    {
        px = *reinterpret_cast<const PlainPixel<T, C> *>(p);
    }
    else
    {
#pragma unroll
        for (int c = 0; c < C; ++c) px.v[c] = reinterpret_cast<const T *>(p)[c];
    }
    return px;
}

template<typename T, int C>
__device__ __forceinline__ void store_plain(uint8_t *p, const PlainPixel<T, C> &px, bool vector)
{
    if (C != 3 && vector)
    {
        *reinterpret_cast<PlainPixel<T, C> *>(p) = px;
    }
    else
    {
#pragma unroll
        for (int c = 0; c < C; ++c) reinterpret_cast<T *>(p)[c] = px.v[c];
    }
}

// rint(|sum|) clamped to the element type's range (ResizeUtils.cpp:226-234); float32 elements keep the blend as it is,
// like the reference's CUDA operator.
template<typename T>
__device__ __forceinline__ T finish_linear(double sum)
{
    if constexpr (sizeof(T) == 4)
        return static_cast<float>(sum);
    else
    {
        const double r  = rint(fabs(sum));
        const double lo = T(-1) < T(0) ? -32768.0 : 0.0;
        const double hi = sizeof(T) == 1 ? 255.0 : (T(-1) < T(0) ? 32767.0 : 65535.0);
        return static_cast<T>(r < lo ? lo : (r > hi ? hi : r));
    }
}

// Work per thread: lane L of a warp produces columns L, L + 32, L + 64, L + 96 of a 128-column tile (every load and
// store instruction stays coalesced across the warp) in four rows, eight apart. The column taps and weights are worked
// out once and reused down the rows -- the int<->float conversions they need run on a pipe with an eighth of the
// float32 rate and were the bottleneck when every pixel paid for its own -- and a thread has 16 (nearest: 4)
// independent loads in flight per row.
constexpr int kPlainCols = 4;
constexpr int kPlainRows = 4;

// float(a - b) for two bytes without a conversion instruction: the difference becomes the low mantissa bits of
// 1.5 * 2^23.
__device__ __forceinline__ float diff_to_float(uint8_t a, uint8_t b)
{
    return __fsub_rn(__int_as_float(0x4B400000 + static_cast<int>(a) - static_cast<int>(b)), 12582912.0f);
}

// float(b) for a byte without a conversion instruction: the byte becomes the low mantissa bits of 2^23.
__device__ __forceinline__ float byte_to_float(uint8_t b)
{
    return __fsub_rn(__uint_as_float(0x4B000000u | b), 8388608.0f);
}

__device__ __forceinline__ bool is_multiple_of_2_to_minus_8(double w)
{
    const double t = __dmul_rn(w, 256.0);
    return t == rint(t);
}

// One channel of the linear blend in double precision, exactly as the golden writes it.
template<typename T>
__device__ __forceinline__ T blend_exact(T p00, T p10, T p01, T p11, double wy0, double wy1, double wx0, double wx1)
{
    const double a = __dmul_rn(__dmul_rn(static_cast<double>(p00), wy0), wx0);
    const double b = __dmul_rn(__dmul_rn(static_cast<double>(p10), wy1), wx0);
    const double d = __dmul_rn(__dmul_rn(static_cast<double>(p01), wy0), wx1);
    const double e = __dmul_rn(__dmul_rn(static_cast<double>(p11), wy1), wx1);
    return finish_linear<T>(__dadd_rn(__dadd_rn(__dadd_rn(a, b), d), e));
}

// The golden's linear tap along one axis (ResizeUtils.cpp:224-234): first tap index (clamped), second tap index, and
// the weight of the second tap, in double precision.
__device__ __forceinline__ void linear_tap_exact(float scale, int d, int size, int &s0, int &s1, double &w1)
{
    double f = __dsub_rn(__dmul_rn(static_cast<double>(scale), __dadd_rn(static_cast<double>(d), 0.5)), 0.5);
    int    s = __double2int_rd(f);
    w1       = (s < 0) ? 0.0 : ((s > size - 2) ? 1.0 : __dsub_rn(f, static_cast<double>(s)));
    s0       = max(0, min(s, size - 2));
    // sources one pixel wide or high: the golden would read outside them; here the second tap is the first
    s1       = min(s0 + 1, size - 1);
}

template<typename T, int C, int INTERP>
__global__ void __launch_bounds__(256) resize_plain_kernel(const PlainResizeKParams p)
{
    const int     dx0  = blockIdx.x * (32 * kPlainCols) + threadIdx.x;
    const int     dy0  = blockIdx.y * (8 * kPlainRows) + threadIdx.y;
    constexpr int kPix = sizeof(T) * C;
    constexpr bool kFast = INTERP == B200PP_INTERP_LINEAR && sizeof(T) == 1; // uint8: float32 blend with exact redo

    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const PlainView S = plain_view(p.src, n), D = plain_view(p.dst, n);
        if (dx0 >= D.w || dy0 >= D.h || S.w < 1 || S.h < 1)
            continue;
        // float scale factors, as the golden computes them (ResizeUtils.cpp:193-194)
        const float scaleW = __fdiv_rn(static_cast<float>(S.w), static_cast<float>(D.w));
        const float scaleH = __fdiv_rn(static_cast<float>(S.h), static_cast<float>(D.h));
        // whole-pixel vector accesses when every address involved is a multiple of the pixel size
        const bool vector = C != 3
                         && ((reinterpret_cast<unsigned long long>(S.base) | reinterpret_cast<unsigned long long>(D.base)
                              | static_cast<unsigned long long>(S.pitch) | static_cast<unsigned long long>(D.pitch))
                             & (kPix - 1))
                                == 0;

        // ---- columns: source byte offsets and weights, once per thread and sample
        int    off0[kPlainCols], off1[kPlainCols];
        float  wx0f[kPlainCols], wx1f[kPlainCols];  // uint8 fast path
        double wx1d[kPlainCols];                    // other element types
        unsigned exactCols = 0; // bit k: column k's weights are multiples of 2^-8
#pragma unroll
        for (int k = 0; k < kPlainCols; ++k)
        {
            const int dx = min(dx0 + 32 * k, D.w - 1); // columns past the end repeat the last one and are not stored
            if constexpr (INTERP == B200PP_INTERP_NEAREST)
            {
                // :204-220, float arithmetic
                off0[k] = max(min(__float2int_rd(__fmul_rn(scaleW, __fadd_rn(static_cast<float>(dx), 0.5f))), S.w - 1), 0) * kPix;
            }
            else
            {
                int    s0, s1;
                double w1;
                linear_tap_exact(scaleW, dx, S.w, s0, s1, w1);
                off0[k] = s0 * kPix;
                off1[k] = s1 * kPix;
                if constexpr (kFast)
                {
                    wx0f[k] = static_cast<float>(__dsub_rn(1.0, w1));
                    wx1f[k] = static_cast<float>(w1);
                    if (is_multiple_of_2_to_minus_8(w1))
                        exactCols |= 1u << k;
                }
                else
                    wx1d[k] = w1;
            }
        }

        // ---- rows
#pragma unroll 1
        for (int j = 0; j < kPlainRows; ++j)
        {
            const int dy = dy0 + 8 * j;
            if (dy >= D.h)
                break;
            uint8_t *drow = D.base + dy * D.pitch;
            if constexpr (INTERP == B200PP_INTERP_NEAREST)
            {
                const int sy = max(min(__float2int_rd(__fmul_rn(scaleH, __fadd_rn(static_cast<float>(dy), 0.5f))), S.h - 1), 0);
                const uint8_t   *srow = S.base + sy * S.pitch;
                PlainPixel<T, C> px[kPlainCols];
#pragma unroll
                for (int k = 0; k < kPlainCols; ++k) px[k] = load_plain<T, C>(srow + off0[k], vector);
#pragma unroll
                for (int k = 0; k < kPlainCols; ++k)
                    if (dx0 + 32 * k < D.w)
                        store_plain<T, C>(drow + static_cast<long long>(dx0 + 32 * k) * kPix, px[k], vector);
            }
            else
            {
                // :222-241: products and sum in double precision, left to right
                int    sy, sy1;
                double fy;
                linear_tap_exact(scaleH, dy, S.h, sy, sy1, fy);
                const double   wy0 = __dsub_rn(1.0, fy);
                const uint8_t *r0 = S.base + sy * S.pitch, *r1 = S.base + sy1 * S.pitch;

                PlainPixel<T, C> p00[kPlainCols], p10[kPlainCols], p01[kPlainCols], p11[kPlainCols];
#pragma unroll
                for (int k = 0; k < kPlainCols; ++k)
                {
                    p00[k] = load_plain<T, C>(r0 + off0[k], vector);
                    p10[k] = load_plain<T, C>(r1 + off0[k], vector);
                    p01[k] = load_plain<T, C>(r0 + off1[k], vector);
                    p11[k] = load_plain<T, C>(r1 + off1[k], vector);
                }
                [[maybe_unused]] const float wy0f = static_cast<float>(wy0), wy1f = static_cast<float>(fy);
                // Weights that are multiples of 2^-8 on both axes (whole-number and simple fractional scale factors)
                // make the float32 blend exact (8 + 8 + 8 bits; a fused multiply-add rounds once), ties included:
                // nothing to redo.
                [[maybe_unused]] const unsigned exactHere = is_multiple_of_2_to_minus_8(fy) ? exactCols : 0u;
#pragma unroll
                for (int k = 0; k < kPlainCols; ++k)
                {
                    PlainPixel<T, C> out;
                    if constexpr (kFast)
                    {
                        // Blend in float32 first. Its error against the golden's double-precision sum is below 2.4e-4
                        // (three fused multiply-adds on values of at most 255 and three rounded weights), so unless the
                        // float32 sum lies within 2^-10 of a rounding boundary both round to the same integer; the
                        // values that do are blended again exactly -- unless the weights make the float32 blend exact
                        // anyway (with a 1.5x reduction one value in sixteen is an exact tie). Adding 1.5 * 2^23 rounds half-to-even and leaves the
                        // integer in the low mantissa bits: no conversion instruction.
#pragma unroll
                        for (int c = 0; c < C; ++c)
                        {
                            // separable form with fused multiply-adds: cheaper than the golden's order and just as
                            // good here, where only the size of the error matters (and exact when the weights are)
                            const float f00 = byte_to_float(p00[k].v[c]), f10 = byte_to_float(p10[k].v[c]);
                            const float top = __fmaf_rn(wx1f[k], diff_to_float(p01[k].v[c], p00[k].v[c]), f00);
                            const float bot = __fmaf_rn(wx1f[k], diff_to_float(p11[k].v[c], p10[k].v[c]), f10);
                            const float sum = __fmaf_rn(wy1f, __fsub_rn(bot, top), top);
                            const float biased = __fadd_rn(sum, 12582912.0f);
                            const float r      = __fsub_rn(biased, 12582912.0f);
                            out.v[c]           = static_cast<uint8_t>(__float_as_uint(biased) & 0xffu);
                            if (fabsf(__fsub_rn(sum, r)) > 0.5f - 0.0009765625f && !((exactHere >> k) & 1u))
                            {
                                // a real branch: the empty asm keeps the compiler from turning the redo into a select,
                                // which would run the double-precision blend for every value
                                asm volatile("" ::: "memory");
                                int    s0, s1;
                                double w1;
                                linear_tap_exact(scaleW, min(dx0 + 32 * k, D.w - 1), S.w, s0, s1, w1);
                                out.v[c] = blend_exact<T>(p00[k].v[c], p10[k].v[c], p01[k].v[c], p11[k].v[c], wy0, fy,
                                                          __dsub_rn(1.0, w1), w1);
                            }
                        }
                    }
                    else
                    {
                        const double wx0 = __dsub_rn(1.0, wx1d[k]);
#pragma unroll
                        for (int c = 0; c < C; ++c)
                            out.v[c] = blend_exact<T>(p00[k].v[c], p10[k].v[c], p01[k].v[c], p11[k].v[c], wy0, fy, wx0, wx1d[k]);
                    }
                    if (dx0 + 32 * k < D.w)
                        store_plain<T, C>(drow + static_cast<long long>(dx0 + 32 * k) * kPix, out, vector);
                }
            }
        }
    }
}

} // namespace b200pp

#endif
