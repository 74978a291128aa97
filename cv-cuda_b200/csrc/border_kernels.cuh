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

// One thread per 4-byte group of a destination row (PB = bytes per pixel), kBorderRows rows per thread. A group's four
// bytes are mapped to source bytes once per thread; where they are four consecutive source bytes (everywhere except
// next to the left / right border and at the row's ragged end) a row costs one or two aligned word loads, a funnel
// shift and one word store. Rows and groups outside the source take the border rule. Images whose rows do not start on
// 4-byte boundaries go byte by byte.
template<int PB>
__global__ void __launch_bounds__(256) copy_make_border_kernel(const BorderKParams p)
{
    const int b0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int y0 = blockIdx.y * (blockDim.y * kBorderRows) + threadIdx.y;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const PlainView S = plain_view(p.src, n), D = plain_view(p.dst, n);
        const int       rowBytes = D.w * PB;
        if (b0 >= rowBytes || y0 >= D.h)
            continue;
        const int  top = p.topList ? p.topList[n] : p.top, left = p.leftList ? p.leftList[n] : p.left;
        const bool constant = p.border == B200PP_BORDER_CONSTANT || S.w < 1 || S.h < 1;
        const bool aligned
            = ((reinterpret_cast<uintptr_t>(S.base) | static_cast<uintptr_t>(S.pitch) | reinterpret_cast<uintptr_t>(D.base)
                | static_cast<uintptr_t>(D.pitch))
               & 3)
           == 0;
        const int nb = min(4, rowBytes - b0);

        int      sb[4]; // source byte offset within a row, -1: border value
        unsigned fillWord = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k)
        {
            const int b = b0 + k, x = b / PB, within = b - x * PB;
            int       sx = x - left;
            if (sx < 0 || sx >= S.w)
                sx = constant ? -1 : border_index(sx, S.w, p.border);
            sb[k] = (sx < 0 || k >= nb) ? -1 : sx * PB + within;
            fillWord |= ((p.fill[within >> 2] >> (8 * (within & 3))) & 255u) << (8 * k);
        }
        const bool run = aligned && nb == 4 && sb[0] >= 0 && sb[1] == sb[0] + 1 && sb[2] == sb[0] + 2 && sb[3] == sb[0] + 3;
        const int  shift = (sb[0] & 3) * 8;

        unsigned v[kBorderRows];
#pragma unroll
        for (int r = 0; r < kBorderRows; ++r)
        {
            const int y = y0 + r * blockDim.y;
            v[r]        = fillWord;
            if (y >= D.h)
                continue;
            int sy = y - top;
            if (sy < 0 || sy >= S.h)
            {
                if (constant)
                    continue;
                sy = border_index(sy, S.h, p.border);
            }
            const uint8_t *srow = S.base + sy * S.pitch;
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
            const int y = y0 + r * blockDim.y;
            if (y >= D.h)
                continue;
            uint8_t *d = D.base + y * D.pitch + b0;
            if (aligned && nb == 4)
                *reinterpret_cast<unsigned *>(d) = v[r];
            else
                for (int k = 0; k < nb; ++k) d[k] = static_cast<uint8_t>(v[r] >> (8 * k));
        }
    }
}

} // namespace b200pp

#endif
