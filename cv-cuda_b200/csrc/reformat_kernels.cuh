// Stand-alone Reformat: dst(n, y, x, c) = src(n, y, x, c) between any two of the NHWC / HWC / NCHW / CHW layouts (each
// side given by its four byte strides), elements of 1, 2, 4 or 8 bytes copied bit for bit.
//
// Replaces the reformat kernels of the reference (src/cvcuda/priv/legacy/reformat.cu); the reference's CPU golden is the
// same element-wise copy (tests/cvcuda/system/TestOpReformat.cpp:51-69). Bound: HBM.
#ifndef CVCUDA_B200_REFORMAT_KERNELS_CUH
#define CVCUDA_B200_REFORMAT_KERNELS_CUH

#include "kparams.h"

namespace b200pp {

struct ReformatKParams
{
    const uint8_t *src;
    uint8_t       *dst;
    long long      sSample, sRow, sPix, sChan;
    long long      dSample, dRow, dPix, dChan;
    int            numSamples, channels, width, height;
};

// A thread copies all channels of 4 / sizeof(E) adjacent pixels (one 32-bit word per channel) in each of four rows, 8
// apart. On a side whose pixels of one channel are adjacent in memory (planar) the word moves with one aligned 32-bit
// access; on the other side (interleaved) its elements are gathered or scattered one by one, which the L1 merges:
// a warp reads or writes one contiguous span. Ragged row ends and unaligned rows go element by element.
template<typename E>
__global__ void __launch_bounds__(256) reformat_kernel(const ReformatKParams p)
{
    constexpr int PX = 4 / sizeof(E);
    const int     x  = (blockIdx.x * blockDim.x + threadIdx.x) * PX;
    const int     y0 = blockIdx.y * (blockDim.y * 4) + threadIdx.y;
    if (x >= p.width)
        return;
    const bool whole  = x + PX <= p.width;
    const bool sPlane = PX > 1 && p.sPix == static_cast<long long>(sizeof(E));
    const bool dPlane = PX > 1 && p.dPix == static_cast<long long>(sizeof(E));
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
#pragma unroll
        for (int r = 0; r < 4; ++r)
        {
            const int y = y0 + r * blockDim.y;
            if (y >= p.height)
                break;
            const uint8_t *s = p.src + n * p.sSample + y * p.sRow + x * p.sPix;
            uint8_t       *d = p.dst + n * p.dSample + y * p.dRow + x * p.dPix;
            for (int c = 0; c < p.channels; ++c)
            {
                const uint8_t *sc = s + c * p.sChan;
                uint8_t       *dc = d + c * p.dChan;
                if (PX == 1 || !whole)
                {
                    for (int k = 0; k < PX && x + k < p.width; ++k)
                        *reinterpret_cast<E *>(dc + k * p.dPix) = *reinterpret_cast<const E *>(sc + k * p.sPix);
                    continue;
                }
                unsigned w = 0;
                if (sPlane && (reinterpret_cast<unsigned long long>(sc) & 3ull) == 0)
                    w = *reinterpret_cast<const unsigned *>(sc);
                else
                {
#pragma unroll
                    for (int k = 0; k < PX; ++k)
                        w |= static_cast<unsigned>(*reinterpret_cast<const E *>(sc + k * p.sPix)) << (8 * sizeof(E) * k);
                }
                if (dPlane && (reinterpret_cast<unsigned long long>(dc) & 3ull) == 0)
                    *reinterpret_cast<unsigned *>(dc) = w;
                else
                {
#pragma unroll
                    for (int k = 0; k < PX; ++k)
                        *reinterpret_cast<E *>(dc + k * p.dPix) = static_cast<E>(w >> (8 * sizeof(E) * k));
                }
            }
        }
    }
}

// Three 8-bit channels, packed interleaved on one side (pixel stride 3, channel stride 1) and planar on the other
// (pixel stride 1), every row and plane on a 16-byte boundary: the common RGB8 NHWC <-> NCHW case. A thread moves 16
// pixels of two rows: three 16-byte vectors on the interleaved side, one 16-byte vector per plane on the other, shuffled
// in registers with byte permutes (six per four pixels). TO_PLANAR: interleaved source. The ragged end of a row (width
// not a multiple of 16) goes byte by byte.
template<bool TO_PLANAR>
__global__ void __launch_bounds__(256) reformat_u8x3_kernel(const ReformatKParams p)
{
    const int x  = (blockIdx.x * blockDim.x + threadIdx.x) * 16;
    const int y0 = (blockIdx.y * blockDim.y + threadIdx.y) * 2;
    if (x >= p.width)
        return;
    const long long iSample = TO_PLANAR ? p.sSample : p.dSample, iRow = TO_PLANAR ? p.sRow : p.dRow;
    const long long pSample = TO_PLANAR ? p.dSample : p.sSample, pRow = TO_PLANAR ? p.dRow : p.sRow;
    const long long pChan   = TO_PLANAR ? p.dChan : p.sChan;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        if (x + 16 > p.width)
        {
            for (int r = 0; r < 2 && y0 + r < p.height; ++r)
                for (int k = x; k < p.width; ++k)
                    for (int c = 0; c < 3; ++c)
                        p.dst[n * p.dSample + (y0 + r) * p.dRow + k * p.dPix + c * p.dChan]
                            = p.src[n * p.sSample + (y0 + r) * p.sRow + k * p.sPix + c * p.sChan];
            continue;
        }
        unsigned in[2][12];
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const int y = min(y0 + r, p.height - 1);
            if constexpr (TO_PLANAR)
            {
                const uint4 *s = reinterpret_cast<const uint4 *>(p.src + n * iSample + y * iRow + x * 3);
#pragma unroll
                for (int v = 0; v < 3; ++v)
                {
                    const uint4 q = __ldg(s + v);
                    in[r][4 * v + 0] = q.x, in[r][4 * v + 1] = q.y, in[r][4 * v + 2] = q.z, in[r][4 * v + 3] = q.w;
                }
            }
            else
            {
#pragma unroll
                for (int c = 0; c < 3; ++c)
                {
                    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(p.src + n * pSample + c * pChan + y * pRow + x));
                    in[r][4 * c + 0] = q.x, in[r][4 * c + 1] = q.y, in[r][4 * c + 2] = q.z, in[r][4 * c + 3] = q.w;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const int y = y0 + r;
            if (y >= p.height)
                break;
            unsigned out[12];
#pragma unroll
            for (int j = 0; j < 4; ++j) // four pixels = twelve bytes = words a, b, c interleaved / one word per plane
            {
                if constexpr (TO_PLANAR)
                {
                    const unsigned a = in[r][3 * j], b = in[r][3 * j + 1], c = in[r][3 * j + 2];
                    out[0 + j] = __byte_perm(__byte_perm(a, b, 0x0630), c, 0x5210); // bytes 0, 3, 6, 9
                    out[4 + j] = __byte_perm(__byte_perm(a, b, 0x0741), c, 0x6210); // bytes 1, 4, 7, 10
                    out[8 + j] = __byte_perm(__byte_perm(a, b, 0x0052), c, 0x7410); // bytes 2, 5, 8, 11
                }
                else
                {
                    const unsigned c0 = in[r][j], c1 = in[r][4 + j], c2 = in[r][8 + j];
                    out[3 * j + 0] = __byte_perm(__byte_perm(c0, c1, 0x1040), c2, 0x3410); // r0 g0 b0 r1
                    out[3 * j + 1] = __byte_perm(__byte_perm(c0, c1, 0x6205), c2, 0x3250); // g1 b1 r2 g2
                    out[3 * j + 2] = __byte_perm(__byte_perm(c0, c1, 0x0730), c2, 0x7216); // b2 r3 g3 b3
                }
            }
            if constexpr (TO_PLANAR)
            {
#pragma unroll
                for (int c = 0; c < 3; ++c)
                    *reinterpret_cast<uint4 *>(p.dst + n * pSample + c * pChan + y * pRow + x)
                        = make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
            }
            else
            {
                uint4 *d = reinterpret_cast<uint4 *>(p.dst + n * iSample + y * iRow + x * 3);
#pragma unroll
                for (int v = 0; v < 3; ++v) d[v] = make_uint4(out[4 * v], out[4 * v + 1], out[4 * v + 2], out[4 * v + 3]);
            }
        }
    }
}

// Three 32-bit channels, packed interleaved on one side (pixel stride 12, channel stride 4) and planar on the other
// (pixel stride 4), every row and plane on a 16-byte boundary: float32 / int32 RGB NHWC <-> NCHW. A thread moves four
// pixels of each of two rows: three 16-byte vectors on the interleaved side, one per plane on the other; the shuffle is
// a renaming of registers. The ragged end of a row goes element by element.
template<bool TO_PLANAR>
__global__ void __launch_bounds__(256) reformat_w32x3_kernel(const ReformatKParams p)
{
    const int x  = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int y0 = (blockIdx.y * blockDim.y + threadIdx.y) * 2;
    if (x >= p.width)
        return;
    const long long iSample = TO_PLANAR ? p.sSample : p.dSample, iRow = TO_PLANAR ? p.sRow : p.dRow;
    const long long pSample = TO_PLANAR ? p.dSample : p.sSample, pRow = TO_PLANAR ? p.dRow : p.sRow;
    const long long pChan   = TO_PLANAR ? p.dChan : p.sChan;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        if (x + 4 > p.width)
        {
            for (int r = 0; r < 2 && y0 + r < p.height; ++r)
                for (int k = x; k < p.width; ++k)
                    for (int c = 0; c < 3; ++c)
                        *reinterpret_cast<unsigned *>(p.dst + n * p.dSample + (y0 + r) * p.dRow + k * p.dPix + c * p.dChan)
                            = *reinterpret_cast<const unsigned *>(p.src + n * p.sSample + (y0 + r) * p.sRow + k * p.sPix + c * p.sChan);
            continue;
        }
        uint4 in[2][3];
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const int y = min(y0 + r, p.height - 1);
#pragma unroll
            for (int v = 0; v < 3; ++v)
                in[r][v] = TO_PLANAR ? __ldg(reinterpret_cast<const uint4 *>(p.src + n * iSample + y * iRow + x * 12ll) + v)
                                     : __ldg(reinterpret_cast<const uint4 *>(p.src + n * pSample + v * pChan + y * pRow + x * 4ll));
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            const int y = y0 + r;
            if (y >= p.height)
                break;
            const uint4 a = in[r][0], b = in[r][1], c = in[r][2];
            if constexpr (TO_PLANAR)
            {
                // a = r0 g0 b0 r1, b = g1 b1 r2 g2, c = b2 r3 g3 b3
                uint8_t *d = p.dst + n * pSample + y * pRow + x * 4ll;
                *reinterpret_cast<uint4 *>(d)             = make_uint4(a.x, a.w, b.z, c.y);
                *reinterpret_cast<uint4 *>(d + pChan)     = make_uint4(a.y, b.x, b.w, c.z);
                *reinterpret_cast<uint4 *>(d + 2 * pChan) = make_uint4(a.z, b.y, c.x, c.w);
            }
            else
            {
                // a = r0..r3, b = g0..g3, c = b0..b3
                uint4 *d = reinterpret_cast<uint4 *>(p.dst + n * iSample + y * iRow + x * 12ll);
                d[0]     = make_uint4(a.x, b.x, c.x, a.y);
                d[1]     = make_uint4(b.y, c.y, a.z, b.z);
                d[2]     = make_uint4(c.z, a.w, b.w, c.w);
            }
        }
    }
}

} // namespace b200pp

#endif
