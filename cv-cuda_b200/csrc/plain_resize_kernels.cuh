// Stand-alone Resize (nearest / linear) for interleaved images of 1, 3 or 4 channels of uint8, uint16, int16 or float32,
// dense tensors or variable-shape image batches on either side.
//
// Replaces NearestResize / LinearResize of the reference (src/cvcuda/priv/OpResize.cu:141-166, 303-342) and the
// variable-shape resize it delegates to (src/cvcuda/priv/legacy/resize_var_shape.cu); arithmetic follows the
// reference's CPU golden (tests/cvcuda/system/ResizeUtils.cpp:189-241) operation by operation, including its use of
// double precision for the linear weights and products, so integer element types come out bit-exact (B200 runs double
// precision at half the float32 rate and the operator is bound by HBM, not by arithmetic).
//
// A thread produces four destination pixels of one row (all channels), 32 columns apart. Pixels of 1, 2 or 4 elements
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

// Destination columns per thread: lane L of a warp produces columns L, L + 32, L + 64, ... of a tile, so that every load
// and store instruction stays coalesced across the warp while each thread has several pixels' worth of independent
// loads in flight (one pixel per thread left HBM idle: 2.3 TB/s on a nearest-neighbour 1.5x reduction): eight pixels
// for nearest (one load each), four for linear (four loads each).
template<int INTERP>
constexpr int kPlainCols = INTERP == B200PP_INTERP_NEAREST ? 8 : 4;

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

template<typename T, int C, int INTERP>
__global__ void __launch_bounds__(256) resize_plain_kernel(const PlainResizeKParams p)
{
    constexpr int kCols = kPlainCols<INTERP>;
    const int     dx0   = blockIdx.x * (32 * kCols) + threadIdx.x;
    const int dy  = blockIdx.y * blockDim.y + threadIdx.y;
    constexpr int kPix = sizeof(T) * C;

    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const PlainView S = plain_view(p.src, n), D = plain_view(p.dst, n);
        if (dx0 >= D.w || dy >= D.h || S.w < 1 || S.h < 1)
            continue;
        // float scale factors, as the golden computes them (ResizeUtils.cpp:193-194)
        const float scaleW = __fdiv_rn(static_cast<float>(S.w), static_cast<float>(D.w));
        const float scaleH = __fdiv_rn(static_cast<float>(S.h), static_cast<float>(D.h));
        uint8_t    *drow   = D.base + dy * D.pitch;
        // whole-pixel vector accesses when every address involved is a multiple of the pixel size
        const bool vector = C != 3
                         && ((reinterpret_cast<unsigned long long>(S.base) | reinterpret_cast<unsigned long long>(D.base)
                              | static_cast<unsigned long long>(S.pitch) | static_cast<unsigned long long>(D.pitch))
                             & (kPix - 1))
                                == 0;

        if constexpr (INTERP == B200PP_INTERP_NEAREST)
        {
            // :204-220, float arithmetic
            const int sy = max(min(__float2int_rd(__fmul_rn(scaleH, __fadd_rn(static_cast<float>(dy), 0.5f))), S.h - 1), 0);
            const uint8_t   *srow = S.base + sy * S.pitch;
            PlainPixel<T, C> px[kCols];
#pragma unroll
            for (int k = 0; k < kCols; ++k)
            {
                const int dx = dx0 + 32 * k;
                if (dx < D.w)
                {
                    const int sx = max(min(__float2int_rd(__fmul_rn(scaleW, __fadd_rn(static_cast<float>(dx), 0.5f))), S.w - 1), 0);
                    px[k]        = load_plain<T, C>(srow + static_cast<long long>(sx) * kPix, vector);
                }
            }
#pragma unroll
            for (int k = 0; k < kCols; ++k)
            {
                const int dx = dx0 + 32 * k;
                if (dx < D.w)
                    store_plain<T, C>(drow + static_cast<long long>(dx) * kPix, px[k], vector);
            }
        }
        else
        {
            // :222-241, the float scale promoted to double, everything else double, products left to right
            double fy = __dsub_rn(__dmul_rn(static_cast<double>(scaleH), __dadd_rn(static_cast<double>(dy), 0.5)), 0.5);
            int    sy = __double2int_rd(fy);
            fy        = (sy < 0) ? 0.0 : ((sy > S.h - 2) ? 1.0 : __dsub_rn(fy, static_cast<double>(sy)));
            sy        = max(0, min(sy, S.h - 2));
            // sources one pixel wide or high: the golden would read outside them; here the second tap is the first
            const int      sy1 = min(sy + 1, S.h - 1);
            const double   wy0 = __dsub_rn(1.0, fy);
            const uint8_t *r0 = S.base + sy * S.pitch, *r1 = S.base + sy1 * S.pitch;

            PlainPixel<T, C> p00[kCols], p10[kCols], p01[kCols], p11[kCols];
            double           fxs[kCols];
#pragma unroll
            for (int k = 0; k < kCols; ++k)
            {
                const int dx = dx0 + 32 * k;
                fxs[k]       = 0.0;
                if (dx < D.w)
                {
                    double fx = __dsub_rn(__dmul_rn(static_cast<double>(scaleW), __dadd_rn(static_cast<double>(dx), 0.5)), 0.5);
                    int    sx = __double2int_rd(fx);
                    fx        = (sx < 0) ? 0.0 : ((sx > S.w - 2) ? 1.0 : __dsub_rn(fx, static_cast<double>(sx)));
                    sx        = max(0, min(sx, S.w - 2));
                    const int sx1 = min(sx + 1, S.w - 1);
                    fxs[k]        = fx;
                    p00[k]        = load_plain<T, C>(r0 + static_cast<long long>(sx) * kPix, vector);
                    p10[k]        = load_plain<T, C>(r1 + static_cast<long long>(sx) * kPix, vector);
                    p01[k]        = load_plain<T, C>(r0 + static_cast<long long>(sx1) * kPix, vector);
                    p11[k]        = load_plain<T, C>(r1 + static_cast<long long>(sx1) * kPix, vector);
                }
            }
#pragma unroll
            for (int k = 0; k < kCols; ++k)
            {
                const int dx = dx0 + 32 * k;
                if (dx >= D.w)
                    continue;
                const double     fx = fxs[k], wx0 = __dsub_rn(1.0, fx);
                PlainPixel<T, C> out;
                if constexpr (sizeof(T) == 1)
                {
                    // uint8: blend in float32 first. Its error against the golden's double-precision sum is below
                    // 2.4e-4 (four products of at most 255 with three roundings each, three additions), so unless the
                    // float32 sum lies within 2^-10 of a rounding boundary both round to the same integer; the few
                    // values that do are blended again exactly.
                    const float wy0f = static_cast<float>(wy0), wy1f = static_cast<float>(fy);
                    const float wx0f = static_cast<float>(wx0), wx1f = static_cast<float>(fx);
#pragma unroll
                    for (int c = 0; c < C; ++c)
                    {
                        const float sum = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(__fmul_rn(p00[k].v[c], wy0f), wx0f),
                                                                        __fmul_rn(__fmul_rn(p10[k].v[c], wy1f), wx0f)),
                                                              __fmul_rn(__fmul_rn(p01[k].v[c], wy0f), wx1f)),
                                                    __fmul_rn(__fmul_rn(p11[k].v[c], wy1f), wx1f));
                        const float r   = rintf(sum);
                        out.v[c]        = static_cast<T>(fminf(r, 255.0f));
                        if (fabsf(__fsub_rn(sum, r)) > 0.5f - 0.0009765625f)
                        {
                            // a real branch: the empty asm keeps the compiler from turning the redo into a select,
                            // which would run the double-precision blend for every value
                            asm volatile("" ::: "memory");
                            out.v[c] = blend_exact<T>(p00[k].v[c], p10[k].v[c], p01[k].v[c], p11[k].v[c], wy0, fy, wx0, fx);
                        }
                    }
                }
                else
                {
#pragma unroll
                    for (int c = 0; c < C; ++c)
                        out.v[c] = blend_exact<T>(p00[k].v[c], p10[k].v[c], p01[k].v[c], p11[k].v[c], wy0, fy, wx0, fx);
                }
                store_plain<T, C>(drow + static_cast<long long>(dx) * kPix, out, vector);
            }
        }
    }
}

} // namespace b200pp

#endif
