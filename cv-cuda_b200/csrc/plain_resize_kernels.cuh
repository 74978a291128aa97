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

#include <type_traits>

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
    PlainSide  src, dst;
    int        numSamples;
    const int *cropRects; // device, (left, top, width, height) per sample: the golden's crop arguments; null = whole images
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

// The blend rounded half to even and clamped to the element type's range (ResizeUtils.cpp:226-234). The golden rounds
// |sum|; for unsigned types that is the same thing, and for int16 the sign is kept, as the reference's CUDA operators
// do (src/cvcuda/priv/OpResize.cu:228-262 saturate-cast the signed blend) -- the golden's fabs would turn a negative
// blend positive, which its own tests never reach (int16 rows are nearest only). float32 elements keep the blend as it
// is, like the reference's CUDA operator.
template<typename T>
__device__ __forceinline__ T finish_linear(double sum)
{
    if constexpr (sizeof(T) == 4)
        return static_cast<float>(sum);
    else
    {
        const double r  = rint(T(-1) < T(0) ? sum : fabs(sum));
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

// uint8 pixels of 1, 3 or 4 channels as one packed word (channel c in byte c): a quarter of the registers of
// unpacked bytes, and a byte goes from the word into a float's mantissa with a single byte permute.
template<int C>
__device__ __forceinline__ unsigned load_packed(const uint8_t *p, bool vector)
{
    if (C == 4 && vector)
        return *reinterpret_cast<const unsigned *>(p);
    if (C == 3 && vector)
    {
        // rows on word boundaries: the aligned word that holds the pixel's first byte and, only when the pixel runs past
        // it, the next one (which then holds the pixel's last byte, so it lies inside the image); byte 3 is not used
        const unsigned  shift = static_cast<unsigned>(reinterpret_cast<unsigned long long>(p) & 3ull);
        const unsigned *w     = reinterpret_cast<const unsigned *>(p - shift);
        const unsigned  lo    = w[0];
        const unsigned  hi    = shift >= 2 ? w[1] : 0u;
        return __funnelshift_r(lo, hi, shift * 8);
    }
    unsigned w = p[0];
    if (C > 1)
        w |= static_cast<unsigned>(p[1]) << 8 | static_cast<unsigned>(p[2]) << 16;
    if (C > 3)
        w |= static_cast<unsigned>(p[3]) << 24;
    return w;
}

// The C bytes of one uint8 pixel, each zero-extended into a word of its own: one word load and a byte permute per channel
// for four channels at aligned addresses, one-byte loads otherwise.
template<int C>
__device__ __forceinline__ void load_taps(const uint8_t *p, bool vector, unsigned (&b)[C])
{
    if (C == 4 && vector)
    {
        const unsigned w = *reinterpret_cast<const unsigned *>(p);
        b[0]             = w & 0xffu;
        if constexpr (C == 4)
        {
            b[1] = __byte_perm(w, 0u, 0x4441);
            b[2] = __byte_perm(w, 0u, 0x4442);
            b[3] = w >> 24;
        }
    }
    else
    {
#pragma unroll
        for (int c = 0; c < C; ++c) b[c] = p[c];
    }
}

template<int C>
__device__ __forceinline__ void store_packed(uint8_t *p, unsigned w, bool vector)
{
    if (C == 4 && vector)
    {
        *reinterpret_cast<unsigned *>(p) = w;
        return;
    }
#pragma unroll
    for (int c = 0; c < C; ++c) p[c] = static_cast<uint8_t>(w >> (8 * c));
}

// float(byte c of w): the byte becomes the low mantissa bits of 2^23
template<int CH>
__device__ __forceinline__ float packed_byte_to_float(unsigned w)
{
    return __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 | CH)), 8388608.0f);
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
__device__ __forceinline__ void linear_tap_exact(float scale, int d, int size, int origin, int &s0, int &s1, double &w1)
{
    double f = __dadd_rn(__dsub_rn(__dmul_rn(static_cast<double>(scale), __dadd_rn(static_cast<double>(d), 0.5)), 0.5),
                         static_cast<double>(origin));
    int    s = __double2int_rd(f);
    w1       = (s < 0) ? 0.0 : ((s > size - 2) ? 1.0 : __dsub_rn(f, static_cast<double>(s)));
    s0       = max(0, min(s, size - 2));
    // sources one pixel wide or high: the golden would read outside them; here the second tap is the first
    s1       = min(s0 + 1, size - 1);
}

// SINGLE: compiled with the single-tap shortcut for rows and columns whose second taps all weigh exactly zero (launched when
// the host sees odd whole-number scale factors; the shortcut still checks the weights, so a wrong guess only costs time).
// The shortcut is kept out of the general instantiation, where its extra live ranges cost 8-17 % (spills at 80 registers).
// Resident CTAs per SM for the uint8 linear kernels: three for one and three channels (80 registers, no spills; four CTAs were
// 16 % slower on 1080p -> 224 x 224), four for four channels (64 registers with a few spills, 5 % faster on 1080p -> 720p).
template<typename T, int C, int INTERP, bool SINGLE = false>
__global__ void __launch_bounds__(256, INTERP == B200PP_INTERP_LINEAR && sizeof(T) == 1 ? (C == 4 ? 4 : 3) : 1) resize_plain_kernel(const PlainResizeKParams p)
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
        // over the crop rectangle when there is one (:190-194); taps clamp at the image's edges either way
        int left = 0, top = 0, cropW = S.w, cropH = S.h;
        if (p.cropRects)
        {
            const int4 r = *reinterpret_cast<const int4 *>(p.cropRects + 4 * n);
            left = r.x, top = r.y, cropW = r.z, cropH = r.w;
        }
        const float scaleW = __fdiv_rn(static_cast<float>(cropW), static_cast<float>(D.w));
        const float scaleH = __fdiv_rn(static_cast<float>(cropH), static_cast<float>(D.h));
        // whole-pixel vector accesses when every address involved is a multiple of the pixel size
        // (three uint8 channels: word loads need the source rows on 4-byte boundaries; stores stay byte by byte)
        const bool vectorFlag = C != 3 ? ((reinterpret_cast<unsigned long long>(S.base) | reinterpret_cast<unsigned long long>(D.base)
                                           | static_cast<unsigned long long>(S.pitch) | static_cast<unsigned long long>(D.pitch))
                                          & (kPix - 1))
                                             == 0
                                       : (kFast && ((reinterpret_cast<unsigned long long>(S.base) | static_cast<unsigned long long>(S.pitch)) & 3ull) == 0);

        // ---- columns: source byte offsets and weights, once per thread and sample
        int    off0[kPlainCols], off1[kPlainCols];
        float  wx0s[kPlainCols], wx1s[kPlainCols];  // uint8 fast path: the two weights * 2^127
        double wx1d[kPlainCols];                    // other element types
        unsigned exactCols = 0; // bit k: column k's weights are multiples of 2^-8
        unsigned zeroCols  = 0; // bit k: column k's second tap has weight exactly zero (it is then not even read)
#pragma unroll
        for (int k = 0; k < kPlainCols; ++k)
        {
            const int dx = min(dx0 + 32 * k, D.w - 1); // columns past the end repeat the last one and are not stored
            if constexpr (INTERP == B200PP_INTERP_NEAREST)
            {
                // :204-220, float arithmetic
                const float fx = __fadd_rn(__fmul_rn(scaleW, __fadd_rn(static_cast<float>(dx), 0.5f)), static_cast<float>(left));
                off0[k]        = max(min(__float2int_rd(fx), S.w - 1), 0) * kPix;
            }
            else
            {
                int    s0, s1;
                double w1;
                linear_tap_exact(scaleW, dx, S.w, left, s0, s1, w1);
                off0[k] = s0 * kPix;
                off1[k] = s1 * kPix;
                if constexpr (kFast)
                {
                    wx1s[k] = __fmul_rn(static_cast<float>(w1), 1.7014118346046923e38f);
                    wx0s[k] = __fmul_rn(static_cast<float>(__dsub_rn(1.0, w1)), 1.7014118346046923e38f);
                    if (is_multiple_of_2_to_minus_8(w1))
                        exactCols |= 1u << k;
                    if constexpr (SINGLE)
                        if (w1 == 0.0)
                            zeroCols |= 1u << k;
                }
                else
                    wx1d[k] = w1;
            }
        }

        // ---- rows. The body is compiled twice, with the vector-access decision as a constant: as a run-time flag both
        // forms of every load and store were issued under predicates, a quarter of all issue slots.
        auto rows = [&](auto vectorTag) {
            constexpr bool vector = decltype(vectorTag)::value;
#pragma unroll 1
        for (int j = 0; j < kPlainRows; ++j)
        {
            const int dy = dy0 + 8 * j;
            if (dy >= D.h)
                break;
            uint8_t *drow = D.base + dy * D.pitch;
            if constexpr (INTERP == B200PP_INTERP_NEAREST)
            {
                const float fy = __fadd_rn(__fmul_rn(scaleH, __fadd_rn(static_cast<float>(dy), 0.5f)), static_cast<float>(top));
                const int   sy = max(min(__float2int_rd(fy), S.h - 1), 0);
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
                linear_tap_exact(scaleH, dy, S.h, top, sy, sy1, fy);
                const double   wy0 = __dsub_rn(1.0, fy);
                const uint8_t *r0 = S.base + sy * S.pitch, *r1 = S.base + sy1 * S.pitch;

                if constexpr (kFast)
                {
                    // uint8. Blend in float32 first (separable form, fused multiply-adds). Its error against the
                    // golden's double-precision sum is below 2.4e-4 (three fused multiply-adds on values of at most 255
                    // and three rounded weights), so unless the float32 sum lies within 2^-10 of a rounding boundary
                    // both round to the same integer; the values that do are blended again exactly -- unless the
                    // weights make the float32 blend exact anyway (with a 1.5x reduction one value in sixteen is an
                    // exact tie). Adding 1.5 * 2^23 rounds half-to-even and leaves the integer in the low mantissa
                    // bits: no conversion instruction anywhere.
                    unsigned q00[kPlainCols];
                    // All second taps of weight exactly zero (whole-number scale factors: 1080p -> 640x360): the blend of
                    // every pixel is its first tap, exactly, in float32 and in double precision alike, so the row is a
                    // gather of single pixels -- one tap of four read, one source row of two. Decided per thread (the
                    // same for all threads when the scale factor is a whole number); anything else takes all four taps.
                    if (SINGLE && fy == 0.0 && zeroCols == (1u << kPlainCols) - 1u)
                    {
#pragma unroll
                        for (int k = 0; k < kPlainCols; ++k) q00[k] = load_packed<C>(r0 + off0[k], vector);
#pragma unroll
                        for (int k = 0; k < kPlainCols; ++k)
                            if (dx0 + 32 * k < D.w)
                                store_packed<C>(drow + static_cast<long long>(dx0 + 32 * k) * kPix, q00[k], vector);
                        continue;
                    }
                    // Every tapped byte is used as the float whose bit pattern it is (the denormal b * 2^-149): with the
                    // horizontal weights pre-multiplied by 2^127 the separable blend needs no conversion at all -- ten
                    // float32 instructions per channel, rounding included.
                    const float    wy1f = static_cast<float>(fy), wy0f = static_cast<float>(wy0);
                    // Weights that are multiples of 2^-8 on both axes (whole-number and simple fractional scale
                    // factors) make the float32 blend exact (8 + 8 + 8 bits), ties included: nothing to redo.
                    const unsigned exactHere = is_multiple_of_2_to_minus_8(fy) ? exactCols : 0u;
                    constexpr int  kGroup    = 2; // columns whose taps are requested together (four at once: slower, spills)
#pragma unroll
                    for (int kb = 0; kb < kPlainCols; kb += kGroup)
                    {
                        unsigned t[kGroup][4][C]; // [column][tap: upper left, upper right, lower left, lower right][channel]
#pragma unroll
                        for (int i = 0; i < kGroup; ++i)
                        {
                            load_taps<C>(r0 + off0[kb + i], vector, t[i][0]);
                            load_taps<C>(r0 + off1[kb + i], vector, t[i][1]);
                            load_taps<C>(r1 + off0[kb + i], vector, t[i][2]);
                            load_taps<C>(r1 + off1[kb + i], vector, t[i][3]);
                        }
#pragma unroll
                        for (int i = 0; i < kGroup; ++i)
                        {
                            const int k = kb + i;
                            unsigned  u[4] = {0u, 0u, 0u, 0u};
                            bool      nearTie = false;
#pragma unroll
                            for (int c = 0; c < C; ++c)
                            {
                                const float top = __fmaf_rn(__uint_as_float(t[i][1][c]), wx1s[k], __fmul_rn(__uint_as_float(t[i][0][c]), wx0s[k]));
                                const float bot = __fmaf_rn(__uint_as_float(t[i][3][c]), wx1s[k], __fmul_rn(__uint_as_float(t[i][2][c]), wx0s[k]));
                                const float sum = __fmaf_rn(bot, wy1f, __fmul_rn(top, wy0f)); // the blend * 2^-22
                                const float biased = __fmaf_rn(sum, 4194304.0f, 12582912.0f); // integer in the low mantissa bits
                                u[c]               = __float_as_uint(biased);
                                nearTie |= fabsf(__fmaf_rn(sum, 4194304.0f, __fsub_rn(12582912.0f, biased))) > 0.5f - 0.0009765625f;
                            }
                            if (nearTie && !((exactHere >> k) & 1u))
                            {
                                // a real branch: the empty asm keeps the compiler from turning the redo into selects,
                                // which would run the double-precision blend for every pixel
                                asm volatile("" ::: "memory");
                                int    s0, s1;
                                double w1;
                                linear_tap_exact(scaleW, min(dx0 + 32 * k, D.w - 1), S.w, left, s0, s1, w1);
#pragma unroll
                                for (int c = 0; c < C; ++c)
                                    u[c] = blend_exact<uint8_t>(static_cast<uint8_t>(t[i][0][c]), static_cast<uint8_t>(t[i][2][c]),
                                                                static_cast<uint8_t>(t[i][1][c]), static_cast<uint8_t>(t[i][3][c]), wy0, fy,
                                                                __dsub_rn(1.0, w1), w1);
                            }
                            if (dx0 + 32 * k < D.w)
                            {
                                uint8_t *d = drow + static_cast<long long>(dx0 + 32 * k) * kPix;
                                if (C == 4 && vector) // byte 0 of each of the four words, gathered with byte permutes
                                    *reinterpret_cast<unsigned *>(d) = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
                                else
                                {
#pragma unroll
                                    for (int c = 0; c < C; ++c) d[c] = static_cast<uint8_t>(u[c]);
                                }
                            }
                        }
                    }
                }
                else
                {
                    PlainPixel<T, C> p00[kPlainCols], p10[kPlainCols], p01[kPlainCols], p11[kPlainCols];
#pragma unroll
                    for (int k = 0; k < kPlainCols; ++k)
                    {
                        p00[k] = load_plain<T, C>(r0 + off0[k], vector);
                        p10[k] = load_plain<T, C>(r1 + off0[k], vector);
                        p01[k] = load_plain<T, C>(r0 + off1[k], vector);
                        p11[k] = load_plain<T, C>(r1 + off1[k], vector);
                    }
#pragma unroll
                    for (int k = 0; k < kPlainCols; ++k)
                    {
                        PlainPixel<T, C> out;
                        const double     wx0 = __dsub_rn(1.0, wx1d[k]);
#pragma unroll
                        for (int c = 0; c < C; ++c)
                            out.v[c] = blend_exact<T>(p00[k].v[c], p10[k].v[c], p01[k].v[c], p11[k].v[c], wy0, fy, wx0, wx1d[k]);
                        if (dx0 + 32 * k < D.w)
                            store_plain<T, C>(drow + static_cast<long long>(dx0 + 32 * k) * kPix, out, vector);
                    }
                }
            }
        }
        };
        if (vectorFlag)
            rows(std::true_type{});
        else
            rows(std::false_type{});
    }
}

} // namespace b200pp

#endif
