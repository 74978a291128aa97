// Crop (with border) + flip + per-channel normalise + cast + layout kernel.
//
// Replaces slice_flip_normalize / transfer_data / set_data of the reference
// (src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:38-186); arithmetic follows the reference's CPU golden
// (tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:57-148) and its border rules
// (tests/common/BorderUtils.cpp:24-137, the same rules as cvcuda/cuda_tools/BorderWrap.hpp:76-127).
#ifndef CVCUDA_B200_SLICE_KERNELS_CUH
#define CVCUDA_B200_SLICE_KERNELS_CUH

#include "device_math.cuh"
#include <type_traits>

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

// Per-channel constants of a launch: base value and multiplier (scale, or 1/sqrt(scale^2 + epsilon)).
template<int MAXC>
__device__ __forceinline__ void load_constants(const SliceKParams &p, float (&base)[MAXC], float (&mul)[MAXC])
{
#pragma unroll
    for (int k = 0; k < MAXC; ++k)
    {
        base[k] = 0.f;
        mul[k]  = 0.f;
        if (k < p.channels)
        {
            const int bk  = p.baseCh == 1 ? 0 : k;
            const int sk  = p.scaleCh == 1 ? 0 : k;
            base[k]       = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.base) + bk * p.baseChanStride);
            const float s = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.scale) + sk * p.scaleChanStride);
            mul[k]        = p.stddev ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(s, s), p.epsilon))) : s;
        }
    }
}

// What a sample's descriptors say, read once per thread and sample.
struct SliceSample
{
    const uint8_t *img;
    long long      pitch, planeStride;
    int            w, h;
    int            cx, cy, cw, ch, flip;
};

__device__ __forceinline__ SliceSample load_slice_sample(const SliceKParams &p, int n)
{
    SliceSample s;
    const int  *rect = reinterpret_cast<const int *>(reinterpret_cast<const char *>(p.cropRect) + n * p.cropRectStride);
    s.cx   = rect[0];
    s.cy   = rect[1];
    s.cw   = rect[2];
    s.ch   = rect[3];
    s.flip = p.flip[n];
    if (p.list)
    {
        const B200ppImagePlane &pl = p.list[n].planes[0];
        s.img         = pl.basePtr;
        s.pitch       = pl.rowStride;
        s.w           = pl.width;
        s.h           = pl.height;
        s.planeStride = 0;
    }
    else
    {
        s.img         = p.srcBase + n * p.srcSampleStride;
        s.pitch       = p.srcRowStride;
        s.planeStride = p.srcPlaneStride;
        s.w           = p.srcW;
        s.h           = p.srcH;
    }
    return s;
}

// One destination pixel (j, i) of sample n, any element types, layout and border mode.
template<int MAXC>
__device__ __forceinline__ void slice_pixel(const SliceKParams &p, const SliceSample &s, int n, int i, int j, int srcType,
                                            int dstType, int srcElem, const float (&base)[MAXC], const float (&mul)[MAXC])
{
    uint8_t *dstPix = p.dst + n * p.dSample + i * p.dRow + j * p.dPix;
    if (i >= s.ch || j >= s.cw)
    {
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
            if (k < p.channels)
                store_any(dstPix + k * p.dChan, dstType, 0.f);
        return;
    }
    int x = (s.flip == 1 || s.flip == -1) ? s.cw - 1 - j + s.cx : j + s.cx;
    int y = (s.flip == 0 || s.flip == -1) ? s.ch - 1 - i + s.cy : i + s.cy;

    bool inside = (x >= 0 && x < s.w && y >= 0 && y < s.h);
    // an empty image has no pixel to replicate, wrap or reflect: every rule then answers with the constant
    if (!inside && p.border != B200PP_BORDER_CONSTANT && s.w >= 1 && s.h >= 1)
    {
        x      = border_index(x, s.w, p.border);
        y      = border_index(y, s.h, p.border);
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
                    const uint8_t  *plane = p.list ? p.list[n].planes[k].basePtr : s.img + k * s.planeStride;
                    const long long pp    = p.list ? p.list[n].planes[k].rowStride : s.pitch;
                    src                   = plane + y * pp + static_cast<long long>(x) * srcElem;
                }
                else
                {
                    src = s.img + y * s.pitch + (static_cast<long long>(x) * p.channels + k) * srcElem;
                }
                v = load_any(src, srcType);
            }
            const float o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, base[k]), mul[k]), p.gscale), p.shift);
            store_any(dstPix + k * p.dChan, dstType, o);
        }
    }
}

// Generic kernel: one thread per destination pixel.
template<int MAXC>
__global__ void __launch_bounds__(256) slice_gather_kernel(const SliceKParams p, const int srcType, const int dstType,
                                                           const int srcElem)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int i = blockIdx.y * blockDim.y + threadIdx.y;
    if (j >= p.dstW || i >= p.dstH)
        return;
    float base[MAXC], mul[MAXC];
    load_constants<MAXC>(p, base, mul);
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const SliceSample s = load_slice_sample(p, n);
        slice_pixel<MAXC>(p, s, n, i, j, srcType, dstType, srcElem, base, mul);
    }
}

// Fast kernel for the pre-processing case: interleaved 3-channel uint8 sources to uint8 / float32 / float16.
// A thread produces four adjacent destination pixels in each of kSliceRowsPerThread rows (the per-launch constants and
// the sample's descriptors are fetched once per thread, not once per pixel group). When the four pixels all lie
// inside the crop and their source pixels inside the image, the twelve source bytes come in as aligned words, bytes
// become floats with one PRMT and one exact subtraction each, and -- for planar, suitably aligned destinations -- each
// channel leaves as one vector store (a warp writes 512 contiguous bytes per channel). Anything else (crop edge,
// border, ragged end of a row) goes through slice_pixel.
constexpr int kSliceRowsPerThread = 4;

template<int DK>
__device__ __forceinline__ void store_four(uint8_t *d, float a, float b, float c, float e)
{
    if constexpr (DK == DST_F32)
        *reinterpret_cast<float4 *>(d) = make_float4(a, b, c, e);
    else if constexpr (DK == DST_F16)
    {
        const __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, e);
        uint2         v;
        v.x = *reinterpret_cast<const unsigned *>(&lo);
        v.y = *reinterpret_cast<const unsigned *>(&hi);
        *reinterpret_cast<uint2 *>(d) = v;
    }
    else
        *reinterpret_cast<unsigned *>(d) = sat_u8(a) | sat_u8(b) << 8 | sat_u8(c) << 16 | sat_u8(e) << 24;
}

template<int DK>
__global__ void __launch_bounds__(256, 4) slice_u8x3_kernel(const SliceKParams p, const int dstType, const int vecStore)
{
    const int j0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int iBase = blockIdx.y * (blockDim.y * kSliceRowsPerThread) + threadIdx.y;
    if (j0 >= p.dstW || iBase >= p.dstH)
        return;
    float base[3], mul[3];
    load_constants<3>(p, base, mul);
    const int cols = min(4, p.dstW - j0);

    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const SliceSample s = load_slice_sample(p, n);

        const bool flipX = (s.flip == 1 || s.flip == -1);
        const bool flipY = (s.flip == 0 || s.flip == -1);
        const int  xlo   = flipX ? s.cw - 1 - (j0 + 3) + s.cx : j0 + s.cx; // leftmost of the four source pixels
        const bool colsFast = cols == 4 && j0 + 3 < s.cw && xlo >= 0 && xlo + 3 < s.w;
        const bool rowAligned = (reinterpret_cast<unsigned long long>(s.img) & 3ull) == 0 && (s.pitch & 3ll) == 0;

        // Pass 1: the aligned source words of all of the thread's rows are requested before any arithmetic, so that
        // sixteen loads are in flight per thread instead of four. mode: 0 no such row, 1 words loaded, 2 fast but
        // unaligned (bytes, pass 2), 3 edge / border (slice_pixel, pass 2).
        unsigned tw[kSliceRowsPerThread][4];
        int      mode[kSliceRowsPerThread];
        unsigned shiftBits = 0;
#pragma unroll
        for (int r = 0; r < kSliceRowsPerThread; ++r)
        {
            const int i = iBase + r * blockDim.y;
            const int y = flipY ? s.ch - 1 - i + s.cy : i + s.cy;
            mode[r]     = i >= p.dstH ? 0 : ((colsFast && i < s.ch && y >= 0 && y < s.h) ? 2 : 3);
            tw[r][0] = tw[r][1] = tw[r][2] = tw[r][3] = 0;
            if (mode[r] == 2)
            {
                const uint8_t           *rowPtr = s.img + y * s.pitch;
                const unsigned long long addr   = reinterpret_cast<unsigned long long>(rowPtr + 3ll * xlo);
                if (rowAligned && (addr & ~3ull) + 16 <= reinterpret_cast<unsigned long long>(rowPtr) + static_cast<unsigned long long>(s.pitch))
                {
                    // aligned window of four words inside the row's pitch
                    const unsigned *wp = reinterpret_cast<const unsigned *>(addr & ~3ull);
                    shiftBits          = static_cast<unsigned>(addr & 3ull) * 8; // the same for every row: pitch % 4 == 0
                    tw[r][0] = __ldg(wp), tw[r][1] = __ldg(wp + 1), tw[r][2] = __ldg(wp + 2), tw[r][3] = __ldg(wp + 3);
                    mode[r] = 1;
                }
            }
        }

#pragma unroll
        for (int r = 0; r < kSliceRowsPerThread; ++r)
        {
            const int i = iBase + r * blockDim.y;
            if (mode[r] == 0)
                break;
            if (mode[r] == 3)
            {
                for (int q = 0; q < cols; ++q) slice_pixel<3>(p, s, n, i, j0 + q, B200PP_U8, dstType, 1, base, mul);
                continue;
            }
            // twelve source bytes as three words, byte 3q+c = channel c of source pixel xlo+q
            unsigned w0, w1, w2;
            if (mode[r] == 1)
            {
                w0 = __funnelshift_r(tw[r][0], tw[r][1], shiftBits);
                w1 = __funnelshift_r(tw[r][1], tw[r][2], shiftBits);
                w2 = __funnelshift_r(tw[r][2], tw[r][3], shiftBits);
            }
            else
            {
                const int      y = flipY ? s.ch - 1 - i + s.cy : i + s.cy;
                const uint8_t *a = s.img + y * s.pitch + 3ll * xlo;
                unsigned       b[12];
#pragma unroll
                for (int k = 0; k < 12; ++k) b[k] = a[k];
                w0 = b[0] | b[1] << 8 | b[2] << 16 | b[3] << 24;
                w1 = b[4] | b[5] << 8 | b[6] << 16 | b[7] << 24;
                w2 = b[8] | b[9] << 8 | b[10] << 16 | b[11] << 24;
            }
            const unsigned words[3] = {w0, w1, w2};

            float o[4][3]; // [source pixel q][channel]
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int c = 0; c < 3; ++c)
                {
                    const int   byte = 3 * q + c;
                    const float v    = byte_as_float(words[byte >> 2], 0x7540u + (byte & 3));
                    o[q][c] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, base[c]), mul[c]), p.gscale), p.shift);
                }

            // source pixel q lands in destination column q, or 3-q when mirrored: the stores are compiled once per direction
            // (as a run-time flag inside the unrolled loop both orders of every store were issued under predicates)
            uint8_t *dst = p.dst + n * p.dSample + i * p.dRow + j0 * p.dPix;
            auto     emit = [&](auto flipTag) {
                constexpr bool FLIP = decltype(flipTag)::value;
                if (vecStore)
                {
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                        store_four<DK>(dst + c * p.dChan, o[FLIP ? 3 : 0][c], o[FLIP ? 2 : 1][c], o[FLIP ? 1 : 2][c], o[FLIP ? 0 : 3][c]);
                }
                else
                {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int c = 0; c < 3; ++c)
                            store_elem<DK>(dst + (FLIP ? 3 - q : q) * p.dPix + c * p.dChan, o[q][c]);
                }
            };
            if (flipX)
                emit(std::true_type{});
            else
                emit(std::false_type{});
        }
    }
}

// Typed kernel for the common element types other than interleaved RGB uint8: uint8 or float32 sources of 1, 3 or 4
// channels, planar or interleaved, to uint8 or float32. Same shape of work as slice_u8x3_kernel -- a thread produces four
// adjacent destination pixels in each of kSliceRowsPerThread rows, all loads of all rows requested before the arithmetic
// -- with the element types and the channel count as template arguments, so that no choice is made per element. Four
// pixels that lie inside the crop with their source pixels inside the image take the fast path; crop edges, borders and
// ragged row ends go through slice_pixel. S, D: float or uint8_t.
template<typename S>
__device__ __forceinline__ float slice_load(const uint8_t *p)
{
    if constexpr (sizeof(S) == 4)
        return __ldg(reinterpret_cast<const float *>(p));
    else // float(byte) through the mantissa of 2^23: no conversion instruction
        return __fsub_rn(__uint_as_float(0x4B000000u | __ldg(p)), 8388608.0f);
}

// Four finished values as four uint8 in one word: round half to even and clamp without a conversion instruction (clamp,
// then add 1.5 * 2^23: the rounded value is the low byte of the sum's bit pattern; NaN clamps to 0 like cvt.sat), two byte
// permutes to gather.
__device__ __forceinline__ unsigned pack_sat_u8x4(float a, float b, float c, float e)
{
    const unsigned ua = __float_as_uint(__fadd_rn(fminf(fmaxf(a, 0.0f), 255.0f), 12582912.0f));
    const unsigned ub = __float_as_uint(__fadd_rn(fminf(fmaxf(b, 0.0f), 255.0f), 12582912.0f));
    const unsigned uc = __float_as_uint(__fadd_rn(fminf(fmaxf(c, 0.0f), 255.0f), 12582912.0f));
    const unsigned ue = __float_as_uint(__fadd_rn(fminf(fmaxf(e, 0.0f), 255.0f), 12582912.0f));
    return __byte_perm(__byte_perm(ua, ub, 0x0040), __byte_perm(uc, ue, 0x0040), 0x5410);
}

// Four finished values to four consecutive elements; `vec`: the address is a multiple of the four elements' size.
template<typename D>
__device__ __forceinline__ void slice_store4(uint8_t *d, float a, float b, float c, float e, bool vec)
{
    if constexpr (sizeof(D) == 4)
    {
        if (vec)
            *reinterpret_cast<float4 *>(d) = make_float4(a, b, c, e);
        else
        {
            float *f = reinterpret_cast<float *>(d);
            f[0] = a, f[1] = b, f[2] = c, f[3] = e;
        }
    }
    else
    {
        const unsigned w = pack_sat_u8x4(a, b, c, e);
        if (vec)
            *reinterpret_cast<unsigned *>(d) = w;
        else
            d[0] = static_cast<uint8_t>(w), d[1] = static_cast<uint8_t>(w >> 8), d[2] = static_cast<uint8_t>(w >> 16),
            d[3] = static_cast<uint8_t>(w >> 24);
    }
}

// Rows per thread: four for one channel and for four-byte pixels (kept as one word per pixel until they are written), two for
// the rest (the loaded values of all rows live in registers as floats).
__host__ __device__ constexpr int slice_typed_rows(int channels, bool srcU8)
{
    return channels == 1 || (channels == 4 && srcU8) ? 4 : 2;
}

template<typename S, typename D, int C>
__global__ void __launch_bounds__(256, C == 1 ? 4 : 3) slice_typed_kernel(const SliceKParams p, const int srcType, const int dstType)
{
    constexpr int  kRows = slice_typed_rows(C, sizeof(S) == 1);
    constexpr bool kRaw  = sizeof(S) == 1 && C == 4; // interleaved four-byte pixels: a word per pixel, converted when written
    const int      j0    = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int     iBase = blockIdx.y * (blockDim.y * kRows) + threadIdx.y;
    if (j0 >= p.dstW || iBase >= p.dstH)
        return;
    float base[C], mul[C];
    load_constants<C>(p, base, mul);
    const int  cols     = min(4, p.dstW - j0);
    const bool dstPacked = p.dPix == C * static_cast<long long>(sizeof(D)) && p.dChan == static_cast<long long>(sizeof(D)); // interleaved
    const bool dstPlanes = p.dPix == static_cast<long long>(sizeof(D));                                                   // planar

    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const SliceSample s     = load_slice_sample(p, n);
        const bool        flipX = (s.flip == 1 || s.flip == -1);
        const bool        flipY = (s.flip == 0 || s.flip == -1);
        const int         xlo   = flipX ? s.cw - 1 - (j0 + 3) + s.cx : j0 + s.cx; // leftmost of the four source pixels
        const bool        colsFast = cols == 4 && j0 + 3 < s.cw && xlo >= 0 && xlo + 3 < s.w;

        float    v[kRaw ? 1 : kRows][4 * C]; // [row][source pixel q * C + channel]
        unsigned raw[kRaw ? kRows : 1][4];   // [row][source pixel]
        int      mode[kRows];                // 0 no such row, 1 loaded, 3 edge / border
#pragma unroll
        for (int r = 0; r < kRows; ++r)
        {
            const int i = iBase + r * blockDim.y;
            const int y = flipY ? s.ch - 1 - i + s.cy : i + s.cy;
            mode[r]     = i >= p.dstH ? 0 : ((colsFast && i < s.ch && y >= 0 && y < s.h) ? 1 : 3);
            if constexpr (kRaw)
            {
                if (mode[r] == 1)
                {
                    const uint8_t *a = s.img + y * s.pitch + static_cast<long long>(xlo) * 4;
                    if (p.srcPlanar || (reinterpret_cast<unsigned long long>(a) & 3ull) != 0)
                        mode[r] = 3; // planes, or pixels off word boundaries: pixel by pixel
                    else if ((reinterpret_cast<unsigned long long>(a) & 15ull) == 0)
                    {
                        const uint4 q4 = __ldg(reinterpret_cast<const uint4 *>(a));
                        raw[r][0] = q4.x, raw[r][1] = q4.y, raw[r][2] = q4.z, raw[r][3] = q4.w;
                    }
                    else
                    {
#pragma unroll
                        for (int q = 0; q < 4; ++q) raw[r][q] = __ldg(reinterpret_cast<const unsigned *>(a) + q);
                    }
                }
            }
            else if (mode[r] == 1)
            {
                if (p.srcPlanar)
                {
#pragma unroll
                    for (int k = 0; k < C; ++k)
                    {
                        const uint8_t  *plane = p.list ? p.list[n].planes[k].basePtr : s.img + k * s.planeStride;
                        const long long pp    = p.list ? p.list[n].planes[k].rowStride : s.pitch;
                        const uint8_t  *a     = plane + y * pp + static_cast<long long>(xlo) * sizeof(S);
#pragma unroll
                        for (int q = 0; q < 4; ++q) v[r][q * C + k] = slice_load<S>(a + q * sizeof(S));
                    }
                }
                else
                {
                    const uint8_t *a = s.img + y * s.pitch + static_cast<long long>(xlo) * (C * sizeof(S));
                    if (sizeof(S) == 1 && C == 4 && (reinterpret_cast<unsigned long long>(a) & 3ull) == 0)
                    {
                        // four-byte pixels on word boundaries: one load per pixel, the bytes picked out with permutes
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                        {
                            const unsigned word = __ldg(reinterpret_cast<const unsigned *>(a) + q);
#pragma unroll
                            for (int k = 0; k < C; ++k) v[r][q * C + k] = byte_as_float(word, 0x7540u + (k & 3));
                        }
                    }
                    else
                    {
#pragma unroll
                        for (int e = 0; e < 4 * C; ++e) v[r][e] = slice_load<S>(a + e * sizeof(S));
                    }
                }
            }
        }

#pragma unroll
        for (int r = 0; r < kRows; ++r)
        {
            const int i = iBase + r * blockDim.y;
            if (mode[r] == 0)
                break;
            if (mode[r] == 3)
            {
                for (int q = 0; q < cols; ++q) slice_pixel<C>(p, s, n, i, j0 + q, srcType, dstType, sizeof(S), base, mul);
                continue;
            }
            // The row is written by code compiled once per flip direction (the reversal is then a renaming of registers, not
            // sixteen selects) and with the vector-store decision taken once per row, not inside every store: as a run-time
            // flag both forms of every store were issued under predicates.
            auto emitRow = [&](auto flipTag) {
                constexpr bool FLIP = decltype(flipTag)::value;
                float          o[4][C]; // [destination column][channel]
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                    for (int k = 0; k < C; ++k)
                    {
                        float in;
                        if constexpr (kRaw)
                            in = byte_as_float(raw[r][q], 0x7540u + (k & 3));
                        else
                            in = v[r][q * C + k];
                        o[FLIP ? 3 - q : q][k] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(in, base[k]), mul[k]), p.gscale), p.shift);
                    }

                uint8_t *dst = p.dst + n * p.dSample + i * p.dRow + j0 * p.dPix;
                if (dstPlanes)
                {
                    if (((reinterpret_cast<unsigned long long>(dst) | static_cast<unsigned long long>(p.dChan)) & (4 * sizeof(D) - 1)) == 0)
                    {
#pragma unroll
                        for (int k = 0; k < C; ++k) slice_store4<D>(dst + k * p.dChan, o[0][k], o[1][k], o[2][k], o[3][k], true);
                    }
                    else
                    {
                        asm volatile("" ::: "memory"); // keeps this a branch
#pragma unroll
                        for (int k = 0; k < C; ++k) slice_store4<D>(dst + k * p.dChan, o[0][k], o[1][k], o[2][k], o[3][k], false);
                    }
                }
                else if (dstPacked)
                {
                    float f[4 * C];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int k = 0; k < C; ++k) f[q * C + k] = o[q][k];
                    const unsigned long long da = reinterpret_cast<unsigned long long>(dst);
                    if (sizeof(D) == 4 && C == 3 && (da & 15ull) == 0)
                    {
                        // twelve float32 results = 48 consecutive bytes per lane, i.e. three sectors per pair of lanes. As three
                        // 16-byte stores every instruction wrote half-sectors 48 bytes apart. Instead: one 256-bit store of the
                        // lane's sector-aligned 32 bytes (the first eight values in lanes that start on a sector boundary, the
                        // last eight in the others), then one 16-byte store of the rest -- the two halves of the sector a pair
                        // of lanes shares then leave in the same instruction.
                        const bool odd = (da & 31ull) != 0;
                        store_f32x8(dst + (odd ? 16 : 0), odd ? f[4] : f[0], odd ? f[5] : f[1], odd ? f[6] : f[2], odd ? f[7] : f[3],
                                    odd ? f[8] : f[4], odd ? f[9] : f[5], odd ? f[10] : f[6], odd ? f[11] : f[7]);
                        slice_store4<D>(dst + (odd ? 0 : 32), odd ? f[0] : f[8], odd ? f[1] : f[9], odd ? f[2] : f[10], odd ? f[3] : f[11], true);
                    }
                    else if ((da & (4 * sizeof(D) - 1)) == 0)
                    {
#pragma unroll
                        for (int g = 0; g < C; ++g)
                            slice_store4<D>(dst + 4 * g * sizeof(D), f[4 * g], f[4 * g + 1], f[4 * g + 2], f[4 * g + 3], true);
                    }
                    else
                    {
                        asm volatile("" ::: "memory");
#pragma unroll
                        for (int g = 0; g < C; ++g)
                            slice_store4<D>(dst + 4 * g * sizeof(D), f[4 * g], f[4 * g + 1], f[4 * g + 2], f[4 * g + 3], false);
                    }
                }
                else
                {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int k = 0; k < C; ++k)
                        {
                            uint8_t *d = dst + q * p.dPix + k * p.dChan;
                            if constexpr (sizeof(D) == 4)
                                *reinterpret_cast<float *>(d) = o[q][k];
                            else
                                *d = static_cast<uint8_t>(sat_u8(o[q][k]));
                        }
                }
            };
            if (flipX)
                emitRow(std::true_type{});
            else
                emitRow(std::false_type{});
        }
    }
}

// Single-plane kernel: one-channel images, and planar sources written to planar destinations (every channel is then an
// independent one-channel problem: blockIdx.z runs over sample x channel). A thread produces kPix adjacent destination
// pixels -- sixteen uint8 or four float32 sources, i.e. sixteen source bytes, fetched as aligned words -- in each of kRows
// rows, all rows' loads first. With four one-byte loads per thread, as the typed kernel would issue, a thread has far too
// few bytes in flight to cover the memory latency (measured 125 us for 32 one-channel 1080p uint8 images).
constexpr int kSlicePlaneIters = 4;

// Rows per thread and row block, and adjacent pixels per thread: sixteen source bytes per thread and row (four float32 or
// sixteen uint8 pixels) in four / two rows. Measured on 32 planar RGB8 1080p images -> float32: sixteen pixels x two rows
// 212.8 us, x four rows 222.5 us, four pixels (one 16-byte store per lane and row) x four rows 216.8 us.
__host__ __device__ constexpr int slice_plane_rows(bool srcF32, bool /*dstF32*/)
{
    return srcF32 ? 4 : 2;
}

__host__ __device__ constexpr int slice_plane_pix(bool srcF32, bool /*dstF32*/)
{
    return srcF32 ? 4 : 16;
}

template<typename S, typename D>
__global__ void __launch_bounds__(256, 4) slice_plane_kernel(const SliceKParams p, const int srcType, const int dstType,
                                                             const int planes)
{
    constexpr int kPix   = slice_plane_pix(sizeof(S) == 4, sizeof(D) == 4);
    constexpr int kWords = kPix * static_cast<int>(sizeof(S)) / 4; // source words of a thread's pixels in one row
    constexpr int kRows = slice_plane_rows(sizeof(S) == 4, sizeof(D) == 4);
    const int     j0    = (blockIdx.x * blockDim.x + threadIdx.x) * kPix;
    const int     iFirst = blockIdx.y * (blockDim.y * kRows * kSlicePlaneIters) + threadIdx.y;
    if (j0 >= p.dstW || iFirst >= p.dstH)
        return;
    const int cols = min(kPix, p.dstW - j0);

    for (int z = blockIdx.z; z < p.numSamples * planes; z += gridDim.z)
    {
        const int         n = z / planes, k = z - n * planes;
        const SliceSample s = load_slice_sample(p, n);
        const uint8_t    *img;
        long long         pitch;
        if (planes > 1)
        {
            img   = p.list ? p.list[n].planes[k].basePtr : s.img + k * s.planeStride;
            pitch = p.list ? p.list[n].planes[k].rowStride : s.pitch;
        }
        else
        {
            img   = s.img;
            pitch = s.pitch;
        }
        // per-channel constants of this plane (load_constants for one channel)
        const int   bk   = p.baseCh == 1 ? 0 : k, sk = p.scaleCh == 1 ? 0 : k;
        const float base = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.base) + bk * p.baseChanStride);
        const float sc   = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.scale) + sk * p.scaleChanStride);
        const float mul  = p.stddev ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(sc, sc), p.epsilon))) : sc;

        const bool flipX = (s.flip == 1 || s.flip == -1);
        const bool flipY = (s.flip == 0 || s.flip == -1);
        const int  xlo   = flipX ? s.cw - 1 - (j0 + kPix - 1) + s.cx : j0 + s.cx; // leftmost of the source pixels
        const bool colsFast = cols == kPix && j0 + kPix - 1 < s.cw && xlo >= 0 && xlo + kPix - 1 < s.w;
        const bool rowAligned = (reinterpret_cast<unsigned long long>(img) & 3ull) == 0 && (pitch & 3ll) == 0;

        // A CTA walks down kSlicePlaneIters blocks of rows: what a thread has to find out about its sample (three dependent
        // loads) is then paid once per 64 or more rows, not once per 16.
        for (int it = 0; it < kSlicePlaneIters; ++it)
        {
        const int iBase = iFirst + it * (blockDim.y * kRows);
        if (iBase >= p.dstH)
            break;
        // float32 sources: L2 is asked for the next block's source rows while this block is converted and stored, so that its
        // loads wait for L2, not for HBM (88.3 -> 82.6 us on 32 one-channel 1080p images; uint8 sources, a quarter of the bytes per
        // row, were 1-3 % slower with it).
        if (sizeof(S) == 4 && it + 1 < kSlicePlaneIters && colsFast)
        {
#pragma unroll
            for (int r = 0; r < kRows; ++r)
            {
                const int i2 = iBase + (kRows + r) * blockDim.y;
                const int y2 = flipY ? s.ch - 1 - i2 + s.cy : i2 + s.cy;
                if (i2 < p.dstH && i2 < s.ch && y2 >= 0 && y2 < s.h)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(img + y2 * pitch + static_cast<long long>(xlo) * sizeof(S)));
            }
        }
        unsigned w[kRows][kWords + 1];
        int      mode[kRows]; // 0 no such row, 1 words loaded, 3 anything else (per pixel)
        unsigned shiftBits = 0;
#pragma unroll
        for (int r = 0; r < kRows; ++r)
        {
            const int i = iBase + r * blockDim.y;
            const int y = flipY ? s.ch - 1 - i + s.cy : i + s.cy;
            mode[r]     = i >= p.dstH ? 0 : 3;
            if (mode[r] == 3 && colsFast && rowAligned && i < s.ch && y >= 0 && y < s.h)
            {
                const uint8_t           *rowPtr = img + y * pitch;
                const unsigned long long addr   = reinterpret_cast<unsigned long long>(rowPtr + static_cast<long long>(xlo) * sizeof(S));
                const bool               extra  = (addr & 3ull) != 0; // only uint8 rows can start inside a word
                if ((addr & ~3ull) + 4 * (kWords + (extra ? 1 : 0)) <= reinterpret_cast<unsigned long long>(rowPtr) + static_cast<unsigned long long>(pitch))
                {
                    const unsigned *wp = reinterpret_cast<const unsigned *>(addr & ~3ull);
                    shiftBits          = static_cast<unsigned>(addr & 3ull) * 8;
                    bool loaded        = false;
                    if constexpr (kWords == 4)
                    {
                        if ((addr & 15ull) == 0)
                        {
                            const uint4 q = __ldg(reinterpret_cast<const uint4 *>(wp));
                            w[r][0] = q.x, w[r][1] = q.y, w[r][2] = q.z, w[r][3] = q.w, w[r][4] = 0;
                            loaded = true;
                        }
                    }
                    if (!loaded)
                    {
#pragma unroll
                        for (int g = 0; g < kWords; ++g) w[r][g] = __ldg(wp + g);
                        w[r][kWords] = extra ? __ldg(wp + kWords) : 0u;
                    }
                    mode[r] = 1;
                }
            }
        }

#pragma unroll
        for (int r = 0; r < kRows; ++r)
        {
            const int i = iBase + r * blockDim.y;
            if (mode[r] == 0)
                break;
            uint8_t *dst = p.dst + n * p.dSample + k * p.dChan + i * p.dRow + j0 * p.dPix;
            if (mode[r] == 3)
            {
                // per pixel, with the crop, border and flip rules of slice_pixel, for this plane only
                for (int q = 0; q < cols; ++q)
                {
                    const int j = j0 + q;
                    float     o = 0.f;
                    if (i < s.ch && j < s.cw)
                    {
                        int  x = flipX ? s.cw - 1 - j + s.cx : j + s.cx;
                        int  y = flipY ? s.ch - 1 - i + s.cy : i + s.cy;
                        bool inside = (x >= 0 && x < s.w && y >= 0 && y < s.h);
                        if (!inside && p.border != B200PP_BORDER_CONSTANT && s.w >= 1 && s.h >= 1)
                        {
                            x      = border_index(x, s.w, p.border);
                            y      = border_index(y, s.h, p.border);
                            inside = true;
                        }
                        const float v = inside ? load_any(img + y * pitch + static_cast<long long>(x) * sizeof(S), srcType) : p.borderAsSrc;
                        o             = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, base), mul), p.gscale), p.shift);
                    }
                    store_any(dst + q * p.dPix, dstType, o);
                }
                continue;
            }
            float t[kPix]; // by source pixel
            if constexpr (sizeof(S) == 4)
            {
#pragma unroll
                for (int q = 0; q < kPix; ++q) t[q] = __uint_as_float(w[r][q]);
            }
            else
            {
#pragma unroll
                for (int g = 0; g < kPix / 4; ++g)
                {
                    const unsigned word = __funnelshift_r(w[r][g], w[r][g + 1], shiftBits);
#pragma unroll
                    for (int b = 0; b < 4; ++b) t[4 * g + b] = byte_as_float(word, 0x7540u + b);
                }
            }
#pragma unroll
            for (int q = 0; q < kPix; ++q) t[q] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(t[q], base), mul), p.gscale), p.shift);
            float o[kPix]; // by destination column: the reversal is a renaming of registers under a uniform branch
            if (flipX)
            {
#pragma unroll
                for (int q = 0; q < kPix; ++q) o[q] = t[kPix - 1 - q];
            }
            else
            {
#pragma unroll
                for (int q = 0; q < kPix; ++q) o[q] = t[q];
            }
            if (p.dPix == static_cast<long long>(sizeof(D)))
            {
                const unsigned long long da = reinterpret_cast<unsigned long long>(dst);
                if constexpr (sizeof(D) == 4)
                {
                    // one decision per row: as a flag inside slice_store4 both forms of every store were issued under predicates
                    if (kPix == 16 && (da & 31ull) == 0)
                    {
                        // sixteen float32 results per lane: two 32-byte stores, each a whole sector (as four 16-byte stores every
                        // store instruction wrote half-sectors 64 bytes apart, twice the transactions on the way to L2)
#pragma unroll
                        for (int h = 0; h < kPix / 8; ++h)
                            store_f32x8(dst + 32 * h, o[8 * h], o[8 * h + 1], o[8 * h + 2], o[8 * h + 3], o[8 * h + 4], o[8 * h + 5],
                                        o[8 * h + 6], o[8 * h + 7]);
                    }
                    else if ((da & 15ull) == 0)
                    {
#pragma unroll
                        for (int g = 0; g < kPix / 4; ++g)
                            slice_store4<D>(dst + 16 * g, o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3], true);
                    }
                    else
                    {
                        asm volatile("" ::: "memory"); // keeps this a branch
#pragma unroll
                        for (int g = 0; g < kPix / 4; ++g)
                            slice_store4<D>(dst + 16 * g, o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3], false);
                    }
                }
                else
                {
                    unsigned pk[kPix / 4];
#pragma unroll
                    for (int g = 0; g < kPix / 4; ++g)
                        pk[g] = pack_sat_u8x4(o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3]);
                    if constexpr (kPix == 16)
                    {
                        if ((da & 15ull) == 0)
                        {
                            *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            continue;
                        }
                    }
#pragma unroll
                    for (int g = 0; g < kPix / 4; ++g)
                    {
                        if ((da & 3ull) == 0)
                            reinterpret_cast<unsigned *>(dst)[g] = pk[g];
                        else
                        {
#pragma unroll
                            for (int b = 0; b < 4; ++b) dst[4 * g + b] = static_cast<uint8_t>(pk[g] >> (8 * b));
                        }
                    }
                }
            }
            else
            {
#pragma unroll
                for (int q = 0; q < kPix; ++q)
                {
                    if constexpr (sizeof(D) == 4)
                        *reinterpret_cast<float *>(dst + q * p.dPix) = o[q];
                    else
                        dst[q * p.dPix] = static_cast<uint8_t>(sat_u8(o[q]));
                }
            }
        }
        }
    }
}

} // namespace b200pp

#endif
