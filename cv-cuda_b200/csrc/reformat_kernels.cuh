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

} // namespace b200pp

#endif
