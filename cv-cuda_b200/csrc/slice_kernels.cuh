// Crop (with border) + flip + per-channel normalise + cast + layout kernel.
//
// Replaces slice_flip_normalize / transfer_data / set_data of the reference
// (src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:38-186); arithmetic follows the reference's CPU golden
// (tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:57-148) and its border rules
// (tests/common/BorderUtils.cpp:24-137, the same rules as cvcuda/cuda_tools/BorderWrap.hpp:76-127).
#ifndef CVCUDA_B200_SLICE_KERNELS_CUH
#define CVCUDA_B200_SLICE_KERNELS_CUH

#include "device_math.cuh"

namespace b200pp {

// Maps a coordinate that lies outside [0, size) back inside for the non-constant border modes.
__device__ __forceinline__ int border_index(int c, int size, int mode)
{
    switch (mode)
    {
    case B200PP_BORDER_REPLICATE:
        return c < 0 ? 0 : (c >= size ? size - 1 : c);
    case B200PP_BORDER_WRAP:
        c = c % size;
        return c < 0 ? c + size : c;
    case B200PP_BORDER_REFLECT:
        c = c % (size * 2);
        if (c < 0)
            c += size * 2;
        return c >= size ? size - 1 - (c - size) : c;
    default: // B200PP_BORDER_REFLECT101
        if (size == 1)
            return 0;
        c = c % (2 * size - 2);
        if (c < 0)
            c += 2 * size - 2;
        return size - 1 - abs(size - 1 - c);
    }
}

template<int MAXC>
__global__ void __launch_bounds__(256) slice_gather_kernel(const SliceKParams p, const int srcType, const int dstType,
                                                           const int srcElem, const int dstElem)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int i = blockIdx.y * blockDim.y + threadIdx.y;
    if (j >= p.dstW || i >= p.dstH)
        return;

    // per-channel constants, identical for every pixel of the launch
    float base[MAXC], mul[MAXC];
#pragma unroll
    for (int k = 0; k < MAXC; ++k)
    {
        if (k < p.channels)
        {
            const int bk = p.baseCh == 1 ? 0 : k;
            const int sk = p.scaleCh == 1 ? 0 : k;
            base[k]      = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.base) + bk * p.baseChanStride);
            const float s = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.scale) + sk * p.scaleChanStride);
            mul[k]        = p.stddev ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(s, s), p.epsilon))) : s;
        }
    }

    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        uint8_t *dstPix = p.dst + n * p.dSample + i * p.dRow + j * p.dPix;

        const int *rect = reinterpret_cast<const int *>(reinterpret_cast<const char *>(p.cropRect) + n * p.cropRectStride);
        const int  cx = rect[0], cy = rect[1], cw = rect[2], ch = rect[3];
        if (i >= ch || j >= cw)
        {
#pragma unroll
            for (int k = 0; k < MAXC; ++k)
                if (k < p.channels)
                    store_any(dstPix + k * p.dChan, dstType, 0.f);
            continue;
        }
        const int fc = p.flip[n];
        int       x  = (fc == 1 || fc == -1) ? cw - 1 - j + cx : j + cx;
        int       y  = (fc == 0 || fc == -1) ? ch - 1 - i + cy : i + cy;

        const uint8_t *img;
        long long      pitch, planeStride;
        int            w, h;
        if (p.list)
        {
            const B200ppImageBuffer &b = p.list[n];
            img   = b.planes[0].basePtr;
            pitch = b.planes[0].rowStride;
            w     = b.planes[0].width;
            h     = b.planes[0].height;
            planeStride = 0;
        }
        else
        {
            img         = p.srcBase + n * p.srcSampleStride;
            pitch       = p.srcRowStride;
            planeStride = p.srcPlaneStride;
            w           = p.srcW;
            h           = p.srcH;
        }

        bool inside = (x >= 0 && x < w && y >= 0 && y < h);
        if (!inside && p.border != B200PP_BORDER_CONSTANT)
        {
            x      = border_index(x, w, p.border);
            y      = border_index(y, h, p.border);
            inside = true;
        }
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
        {
            if (k < p.channels)
            {
                float v = p.borderAsSrc;
                if (inside)
                {
                    const uint8_t *src;
                    if (p.srcPlanar)
                    {
                        const uint8_t *plane = p.list ? p.list[n].planes[k].basePtr : img + k * planeStride;
                        const long long pp   = p.list ? p.list[n].planes[k].rowStride : pitch;
                        src                  = plane + y * pp + static_cast<long long>(x) * srcElem;
                    }
                    else
                    {
                        src = img + y * pitch + (static_cast<long long>(x) * p.channels + k) * srcElem;
                    }
                    v = load_any(src, srcType);
                }
                const float o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, base[k]), mul[k]), p.gscale), p.shift);
                store_any(dstPix + k * p.dChan, dstType, o);
            }
        }
    }
}

} // namespace b200pp

#endif
