// Stand-alone CopyMakeBorder: every destination image is its source image placed at (left, top) inside it, the rest
// filled by a border rule (constant value per channel, replicate, reflect, wrap, reflect-101). Dense tensors or
// variable-shape batches on either side (batch -> batch, or batch -> tensor: the reference's "stack" form), top / left
// one pair for all samples or one per sample from device arrays. Pixels of 1 to 16 bytes are copied bit for bit.
//
// Replaces the copy_make_border kernels of the reference (src/cvcuda/priv/legacy/copy_make_border.cu,
// copy_make_border_var_shape.cu); follows the reference's CPU golden (tests/cvcuda/system/TestOpCopyMakeBorder.cpp:40-97)
// and its border index rules (tests/common/BorderUtils.cpp:24-137, restated in slice_kernels.cuh: border_index).
// Bound: HBM.
#ifndef CVCUDA_B200_BORDER_KERNELS_CUH
#define CVCUDA_B200_BORDER_KERNELS_CUH

#include "plain_resize_kernels.cuh"
#include <type_traits>
#include "slice_kernels.cuh"

namespace b200pp {

struct BorderKParams
{
    PlainSide  src, dst;
    int        numSamples;
    int        top, left;          // used when the lists are null
    const int *topList, *leftList; // one value per sample
    int        border;
    unsigned   fill[4]; // constant border: one pixel's bytes (channel values already converted to the element type)
};

constexpr int kBorderRows = 4; // destination rows per thread, blockDim.y apart

struct BorderSample
{
    PlainView S, D;
    int       top, left, rowBytes;
    bool      constant, aligned; // aligned: all four row starts and pitches on 4-byte boundaries
};

// Byte `within` of the constant border's pixel pattern.
__device__ __forceinline__ unsigned border_fill_byte(const BorderKParams &p, int within)
{
    return (p.fill[within >> 2] >> (8 * (within & 3))) & 255u;
}

// Source row of destination row y, or -1 where the constant rule applies.
__device__ __forceinline__ int border_source_row(const BorderKParams &p, const BorderSample &s, int y)
{
    const int sy = y - s.top;
    if (sy >= 0 && sy < s.S.h)
        return sy;
    return s.constant ? -1 : border_index(sy, s.S.h, p.border);
}

// One 4-byte group of kBorderRows destination rows (PB = bytes per pixel). The group's bytes are mapped to source bytes
// once; where they are four consecutive source bytes a row costs one or two aligned word loads, a funnel shift and one
// word store, otherwise (next to the left / right border, at the row's ragged end, rows off 4-byte boundaries) it goes
// byte by byte.
template<int PB>
__device__ __forceinline__ void border_word(const BorderKParams &p, const BorderSample &s, int b0, int y0, int yStep)
{
    const int nb = min(4, s.rowBytes - b0);
    int       sb[4]; // source byte offset within a row, -1: border value
    unsigned  fillWord = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k)
    {
        const int b = b0 + k, x = b / PB, within = b - x * PB;
        int       sx = x - s.left;
        if (sx < 0 || sx >= s.S.w)
            sx = s.constant ? -1 : border_index(sx, s.S.w, p.border);
        sb[k] = (sx < 0 || k >= nb) ? -1 : sx * PB + within;
        fillWord |= border_fill_byte(p, within) << (8 * k);
    }
    const bool run   = s.aligned && nb == 4 && sb[0] >= 0 && sb[1] == sb[0] + 1 && sb[2] == sb[0] + 2 && sb[3] == sb[0] + 3;
    const int  shift = (sb[0] & 3) * 8;

    unsigned v[kBorderRows];
#pragma unroll
    for (int r = 0; r < kBorderRows; ++r)
    {
        const int y = y0 + r * yStep;
        v[r]        = fillWord;
        if (y >= s.D.h)
            continue;
        const int sy = border_source_row(p, s, y);
        if (sy < 0)
            continue;
        const uint8_t *srow = s.S.base + sy * s.S.pitch;
        if (run)
        {
            const unsigned *w  = reinterpret_cast<const unsigned *>(srow + (sb[0] & ~3));
            const unsigned  lo = __ldg(w);
            v[r]               = shift ? __funnelshift_r(lo, __ldg(w + 1), shift) : lo;
        }
        else
        {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (sb[k] >= 0)
                    v[r] = (v[r] & ~(255u << (8 * k))) | (static_cast<unsigned>(__ldg(srow + sb[k])) << (8 * k));
        }
    }
#pragma unroll
    for (int r = 0; r < kBorderRows; ++r)
    {
        const int y = y0 + r * yStep;
        if (y >= s.D.h)
            continue;
        uint8_t *d = s.D.base + y * s.D.pitch + b0;
        if (s.aligned && nb == 4)
            *reinterpret_cast<unsigned *>(d) = v[r];
        else
            for (int k = 0; k < nb; ++k) d[k] = static_cast<uint8_t>(v[r] >> (8 * k));
    }
}

// One thread per 16-byte group of a destination row, kBorderRows rows per thread. A group whose bytes are sixteen
// consecutive source bytes (everything but the groups that touch the left / right border or the row's ragged end) is
// moved with four or five aligned word loads, funnel shifts and one 16-byte store per row; destination rows outside the
// source follow the row rule (another source row, or the constant pattern). Other groups, and images whose destination
// rows do not start on 16-byte boundaries, go through border_word.
template<int PB>
__global__ void __launch_bounds__(256, 6) copy_make_border_kernel(const BorderKParams p)
{
    const int b0 = (blockIdx.x * blockDim.x + threadIdx.x) * 16;
    const int y0 = blockIdx.y * (blockDim.y * kBorderRows) + threadIdx.y;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        BorderSample s;
        s.S        = plain_view(p.src, n);
        s.D        = plain_view(p.dst, n);
        s.rowBytes = s.D.w * PB;
        if (b0 >= s.rowBytes || y0 >= s.D.h)
            continue;
        s.top      = p.topList ? p.topList[n] : p.top;
        s.left     = p.leftList ? p.leftList[n] : p.left;
        s.constant = p.border == B200PP_BORDER_CONSTANT || s.S.w < 1 || s.S.h < 1;
        const uintptr_t sBits = reinterpret_cast<uintptr_t>(s.S.base) | static_cast<uintptr_t>(s.S.pitch);
        const uintptr_t dBits = reinterpret_cast<uintptr_t>(s.D.base) | static_cast<uintptr_t>(s.D.pitch);
        s.aligned             = ((sBits | dBits) & 3) == 0;

        // first and last byte of the group inside the source columns and 15 apart: all sixteen are consecutive
        const int  x0 = b0 / PB, x1 = (b0 + 15) / PB;
        const int  sx0 = x0 - s.left, sx1 = x1 - s.left;
        const int  sb0 = sx0 * PB + (b0 - x0 * PB);
        // ... or, with the constant rule, all sixteen lie left or right of the source: the pattern in every row
        const bool outside = s.constant && (sx1 < 0 || sx0 >= s.S.w);
        const bool run     = s.aligned && (dBits & 15) == 0 && b0 + 16 <= s.rowBytes && ((sx0 >= 0 && sx1 < s.S.w) || outside);
        if (!run)
        {
#pragma unroll 1
            for (int j = 0; j < 16 && b0 + j < s.rowBytes; j += 4) border_word<PB>(p, s, b0 + j, y0, blockDim.y);
            continue;
        }
        const int shift = (sb0 & 3) * 8;
        int       sy[kBorderRows];
        bool      anyFill = false;
#pragma unroll
        for (int r = 0; r < kBorderRows; ++r)
        {
            const int y = y0 + r * blockDim.y;
            sy[r]       = y < s.D.h ? (outside ? -1 : border_source_row(p, s, y)) : -2; // -2: no such row, -1: pattern
            anyFill     = anyFill || sy[r] == -1;
        }
        uint4 fill = make_uint4(0, 0, 0, 0);
        if (anyFill)
        {
            unsigned f[4] = {0, 0, 0, 0};
            int      within = b0 % PB;
#pragma unroll
            for (int k = 0; k < 16; ++k)
            {
                f[k >> 2] |= border_fill_byte(p, within) << (8 * (k & 3));
                within = within + 1 == PB ? 0 : within + 1;
            }
            fill = make_uint4(f[0], f[1], f[2], f[3]);
        }
        uint4 v[kBorderRows];
        // The loads are compiled twice: sixteen source bytes on a 16-byte boundary are one vector load, anything else four or
        // five words and funnel shifts (as one loop with run-time flags every row issued all of them under predicates).
        auto loadRows = [&](auto vecTag) {
            constexpr bool VEC = decltype(vecTag)::value;
#pragma unroll
            for (int r = 0; r < kBorderRows; ++r)
            {
                v[r] = fill;
                if (sy[r] < 0)
                    continue;
                if constexpr (VEC)
                    v[r] = __ldg(reinterpret_cast<const uint4 *>(s.S.base + sy[r] * s.S.pitch + sb0));
                else
                {
                    const unsigned *w = reinterpret_cast<const unsigned *>(s.S.base + sy[r] * s.S.pitch + (sb0 & ~3));
                    const unsigned  w0 = __ldg(w), w1 = __ldg(w + 1), w2 = __ldg(w + 2), w3 = __ldg(w + 3);
                    const unsigned  w4 = shift ? __ldg(w + 4) : 0u;
                    v[r] = make_uint4(__funnelshift_r(w0, w1, shift), __funnelshift_r(w1, w2, shift), __funnelshift_r(w2, w3, shift),
                                      __funnelshift_r(w3, w4, shift));
                }
            }
        };
        if ((sBits & 15) == 0 && (sb0 & 15) == 0)
            loadRows(std::true_type{});
        else
            loadRows(std::false_type{});
#pragma unroll
        for (int r = 0; r < kBorderRows; ++r)
            if (sy[r] != -2)
                *reinterpret_cast<uint4 *>(s.D.base + (y0 + r * blockDim.y) * s.D.pitch + b0) = v[r];
    }
}

} // namespace b200pp

#endif
