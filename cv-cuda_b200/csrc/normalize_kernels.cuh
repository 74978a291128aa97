// Stand-alone Normalize: out = SaturateCast((in - base) * mul * globalScale + shift), mul = scale or
// 1 / sqrt(scale^2 + epsilon), element by element on interleaved images of 1 to 4 channels, dense tensors or
// variable-shape batches on both sides; base and scale are float32 tensors that may be broadcast along any of the
// sample, row, column and channel dimensions (a stride of zero).
//
// Replaces the normalize kernels of the reference (src/cvcuda/priv/legacy/normalize.cu,
// src/cvcuda/priv/legacy/normalize_var_shape.cu); arithmetic follows the reference's CPU golden
// (tests/cvcuda/system/TestOpNormalize.cpp:34-77): float32, un-fused, in source order; rint + clamp is the saturate cast.
// Bound: HBM (every element read once, written once).
#ifndef CVCUDA_B200_NORMALIZE_KERNELS_CUH
#define CVCUDA_B200_NORMALIZE_KERNELS_CUH

#include "device_math.cuh"
#include <type_traits>
#include "plain_resize_kernels.cuh"

namespace b200pp {

struct NormalizeKParams
{
    PlainSide    src, dst;
    int          numSamples, channels;
    int          srcType, dstType, srcElem, dstElem;
    const float *base, *scale;
    long long    baseStride[4], scaleStride[4]; // bytes per step along sample, row, column, channel; 0 = broadcast
    float        gscale, shift, epsilon;
    int          stddev;
};

__device__ __forceinline__ float normalize_mul(const NormalizeKParams &p, float s)
{
    return p.stddev ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(s, s), p.epsilon))) : s;
}

// A thread produces kNormRows x kNormCols pixels (rows 8 apart, columns 32 apart, so that loads and stores stay
// coalesced across the warp). When base and scale vary only by channel -- the usual mean / standard-deviation case --
// the per-channel constants, including the division and square root of the standard-deviation form, are worked out
// once per thread instead of once per element. uint8 pixels of four channels move as one word.
constexpr int kNormRows = 4;
constexpr int kNormCols = 2;

// SRC / DST: the element type when it is one of the common ones (B200PP_U8 source with B200PP_U8 or B200PP_F32
// destination; B200PP_F32 to B200PP_F32, the normalisation step after a float32 resize), which removes the run-time type
// dispatch and the conversion instructions from the element loop; -1: any.
template<int SRC, int DST>
__global__ void __launch_bounds__(256) normalize_kernel(const NormalizeKParams p)
{
    const int x0 = blockIdx.x * (32 * kNormCols) + threadIdx.x;
    const int y0 = blockIdx.y * (8 * kNormRows) + threadIdx.y;
    const bool perChannel = (p.baseStride[0] | p.baseStride[1] | p.baseStride[2] | p.scaleStride[0] | p.scaleStride[1]
                             | p.scaleStride[2])
                         == 0;
    float cb[4] = {0.f, 0.f, 0.f, 0.f}, cm[4] = {0.f, 0.f, 0.f, 0.f};
    if (perChannel)
    {
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (c < p.channels)
            {
                cb[c] = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.base) + c * p.baseStride[3]);
                cm[c] = normalize_mul(p, *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.scale) + c * p.scaleStride[3]));
            }
    }
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const PlainView S = plain_view(p.src, n), D = plain_view(p.dst, n);
        const int       w = min(S.w, D.w), h = min(S.h, D.h);
        const bool      words = SRC == B200PP_U8 && p.channels == 4
                        && ((reinterpret_cast<unsigned long long>(S.base) | static_cast<unsigned long long>(S.pitch)) & 3ull) == 0;
        const bool      wordsOut = DST == B200PP_U8 && p.channels == 4
                           && ((reinterpret_cast<unsigned long long>(D.base) | static_cast<unsigned long long>(D.pitch)) & 3ull) == 0;
        // uint8 sources: all of the thread's pixels are loaded (as packed words) before any arithmetic, so that eight
        // loads are in flight per thread instead of one
        unsigned packed[kNormRows][kNormCols];
        if constexpr (SRC == B200PP_U8)
        {
#pragma unroll
            for (int r = 0; r < kNormRows; ++r)
#pragma unroll
                for (int k = 0; k < kNormCols; ++k)
                {
                    const int y = min(y0 + 8 * r, h - 1), x = min(x0 + 32 * k, w - 1); // clamped, stored only if inside
                    const uint8_t *sp = S.base + y * S.pitch + static_cast<long long>(x) * p.channels;
                    unsigned       v  = 0;
                    if (w > 0 && h > 0)
                    {
                        if (words)
                            v = *reinterpret_cast<const unsigned *>(sp);
                        else
                            for (int c = 0; c < p.channels; ++c) v |= static_cast<unsigned>(sp[c]) << (8 * c);
                    }
                    packed[r][k] = v;
                }
        }
#pragma unroll
        for (int r = 0; r < kNormRows; ++r)
        {
            const int y = y0 + 8 * r;
            if (y >= h)
                break;
#pragma unroll
            for (int k = 0; k < kNormCols; ++k)
            {
                const int x = x0 + 32 * k;
                if (x >= w)
                    continue;
                const uint8_t *sp = S.base + y * S.pitch + static_cast<long long>(x) * p.channels * p.srcElem;
                uint8_t       *dp = D.base + y * D.pitch + static_cast<long long>(x) * p.channels * p.dstElem;
                const char    *bp = reinterpret_cast<const char *>(p.base) + n * p.baseStride[0] + y * p.baseStride[1] + x * p.baseStride[2];
                const char    *cp = reinterpret_cast<const char *>(p.scale) + n * p.scaleStride[0] + y * p.scaleStride[1] + x * p.scaleStride[2];
                unsigned       outWord = 0;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                {
                    if (c >= p.channels)
                        break;
                    float v;
                    if constexpr (SRC == B200PP_U8)
                        // float(byte) without a conversion instruction: the byte becomes the low mantissa bits of 2^23
                        v = __fsub_rn(__uint_as_float(0x4B000000u | ((packed[r][k] >> (8 * c)) & 0xffu)), 8388608.0f);
                    else if constexpr (SRC == B200PP_F32)
                        v = __ldg(reinterpret_cast<const float *>(sp) + c);
                    else
                        v = load_any(sp + c * p.srcElem, p.srcType);
                    const float b = perChannel ? cb[c] : *reinterpret_cast<const float *>(bp + c * p.baseStride[3]);
                    const float m = perChannel ? cm[c] : normalize_mul(p, *reinterpret_cast<const float *>(cp + c * p.scaleStride[3]));
                    const float o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, b), m), p.gscale), p.shift);
                    if constexpr (DST == B200PP_U8)
                    {
                        // round half to even + clamp through the mantissa of 1.5 * 2^23
                        const unsigned b8 = __float_as_uint(__fadd_rn(fminf(fmaxf(o, 0.0f), 255.0f), 12582912.0f)) & 0xffu;
                        if (wordsOut)
                            outWord |= b8 << (8 * c);
                        else
                            dp[c] = static_cast<uint8_t>(b8);
                    }
                    else if constexpr (DST == B200PP_F32)
                        reinterpret_cast<float *>(dp)[c] = o;
                    else
                        store_any(dp + c * p.dstElem, p.dstType, o);
                }
                if (wordsOut)
                    *reinterpret_cast<unsigned *>(dp) = outWord;
            }
        }
    }
}

// float32 -> float32 with base and scale that vary by channel only (the normalisation step after a float32 resize): a
// copy with four floating-point operations per element, so it is written like one. A thread handles four adjacent pixels
// = C 16-byte vectors in each of two rows, all loads first; which channel an element of a vector belongs to is known at
// compile time (for three channels the pattern repeats every three vectors). Rows that do not start on 16-byte boundaries
// go element by element.
template<int C>
__global__ void __launch_bounds__(256, 4) normalize_f32_kernel(const NormalizeKParams p)
{
    constexpr int kRows = 2;
    const int     g  = blockIdx.x * blockDim.x + threadIdx.x; // group of four pixels
    const int     y0 = blockIdx.y * (blockDim.y * kRows) + threadIdx.y;
    float         cb[C], cm[C];
#pragma unroll
    for (int c = 0; c < C; ++c)
    {
        cb[c] = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.base) + c * p.baseStride[3]);
        cm[c] = normalize_mul(p, *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.scale) + c * p.scaleStride[3]));
    }
    // element 0 of lane L's first vector is element 4 L of the span: channel (4 L) mod C = L mod C for C = 3, 0 for C = 1, 4
    float rb[C], rm[C];
#pragma unroll
    for (int j = 0; j < C; ++j)
    {
        const int c = (static_cast<int>(threadIdx.x) * 4 + j) % C;
        rb[j] = cb[0], rm[j] = cm[0];
#pragma unroll
        for (int q = 1; q < C; ++q)
            if (c == q)
                rb[j] = cb[q], rm[j] = cm[q];
    }
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const PlainView S = plain_view(p.src, n), D = plain_view(p.dst, n);
        const int       w = min(S.w, D.w), h = min(S.h, D.h);
        // A warp's 128 pixels are 32 x C consecutive 16-byte vectors of the row: lane L takes vectors L, L + 32, ... of them, so
        // that every load and store instruction of the warp covers 512 consecutive bytes (with C vectors side by side per lane
        // each instruction touched 16-byte pieces 16 x C bytes apart: half-filled sectors). The channel of element i of a
        // lane's k-th vector is (L + (32 k mod C) * 4 + i) mod C; with the constants rotated by L mod C once per thread it is
        // known at compile time. Vectors past the row's end are skipped; a row's last one to three elements, where its length
        // is not a multiple of four, are done by the lane whose vector they would have been.
        const int  vb    = blockIdx.x * (32 * C); // first vector of the warp's span
        const int  elems = w * C, fullVecs = elems >> 2;
        const bool vec   = ((reinterpret_cast<unsigned long long>(S.base) | reinterpret_cast<unsigned long long>(D.base)
                           | static_cast<unsigned long long>(S.pitch) | static_cast<unsigned long long>(D.pitch)) & 15ull) == 0;
        if (vec ? vb + static_cast<int>(threadIdx.x) > fullVecs : 4 * g >= w)
            continue; // nothing of this row belongs to the thread
        float4 v[kRows][C];
        if (vec)
        {
#pragma unroll
            for (int r = 0; r < kRows; ++r)
            {
                const int y = min(y0 + r * blockDim.y, h - 1);
                const float4 *sp = reinterpret_cast<const float4 *>(S.base + y * S.pitch) + vb + threadIdx.x;
#pragma unroll
                for (int k = 0; k < C; ++k)
                    if (vb + static_cast<int>(threadIdx.x) + 32 * k < fullVecs)
                        v[r][k] = __ldg(sp + 32 * k);
            }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r)
        {
            const int y = y0 + r * blockDim.y;
            if (y >= h)
                break;
            if (vec)
            {
                float4 *dp = reinterpret_cast<float4 *>(D.base + y * D.pitch) + vb + threadIdx.x;
#pragma unroll
                for (int k = 0; k < C; ++k)
                {
                    float e[4] = {v[r][k].x, v[r][k].y, v[r][k].z, v[r][k].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                    {
                        constexpr int kDummy = 0;
                        const int     c      = (128 * k + i) % C + kDummy; // compile-time after unrolling; rotated constants
                        e[i] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(e[i], rb[c]), rm[c]), p.gscale), p.shift);
                    }
                    const int vi = vb + static_cast<int>(threadIdx.x) + 32 * k;
                    if (vi < fullVecs)
                        dp[32 * k] = make_float4(e[0], e[1], e[2], e[3]);
                    else if (vi == fullVecs)
                    {
                        // the row's ragged end, from the source: these elements were not loaded as a vector
                        const float *se = reinterpret_cast<const float *>(S.base + y * S.pitch);
                        float       *de = reinterpret_cast<float *>(D.base + y * D.pitch);
                        for (int x = 4 * vi; x < elems; ++x)
                        {
                            const int c = x % C;
                            de[x] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(se[x], cb[c]), cm[c]), p.gscale), p.shift);
                        }
                    }
                }
            }
            else
            {
                const float *sp = reinterpret_cast<const float *>(S.base + y * S.pitch);
                float       *dp = reinterpret_cast<float *>(D.base + y * D.pitch);
                for (int x = 4 * g; x < min(4 * g + 4, w); ++x)
#pragma unroll
                    for (int c = 0; c < C; ++c)
                        dp[x * C + c] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(sp[x * C + c], cb[c]), cm[c]), p.gscale), p.shift);
            }
        }
    }
}

// uint8 sources with base and scale that vary by channel only (the usual mean / standard-deviation case): the 256
// possible results per channel are computed once per CTA with the arithmetic above and kept in shared memory; an element
// then costs one shared-memory lookup. A thread handles four 4-byte words of a source row, 32 words apart (a warp reads 128
// contiguous bytes and writes 128 x DE), in each of two or four rows per pass; DE = destination element bytes. Images whose rows are not
// on word (source) or 4 x DE-byte (destination) boundaries go byte by byte / element by element.
template<int DE>
__global__ void __launch_bounds__(256, 5) normalize_lut_kernel(const NormalizeKParams p)
{
    __shared__ unsigned lut[4 * 256];
    {
        const int   t = threadIdx.y * blockDim.x + threadIdx.x; // 256 threads
        const float v = static_cast<float>(t);
        for (int c = 0; c < p.channels; ++c)
        {
            const float b = *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.base) + c * p.baseStride[3]);
            const float m = normalize_mul(p, *reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.scale) + c * p.scaleStride[3]));
            const float o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v, b), m), p.gscale), p.shift);
            unsigned    bits = 0;
            store_any(reinterpret_cast<uint8_t *>(&bits), p.dstType, o);
            lut[c * 256 + t] = bits;
        }
    }
    __syncthreads();
    constexpr int RPT = DE == 4 ? 2 : 4; // rows per thread and pass: keeps 32 to 64 bytes of loads in flight per thread
    const int     w0  = blockIdx.x * (blockDim.x * 4) + threadIdx.x;
    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        const PlainView S = plain_view(p.src, n), D = plain_view(p.dst, n);
        const int       rowElems = min(S.w, D.w) * p.channels, h = min(S.h, D.h);
        const int       rowWords = (rowElems + 3) >> 2;
        if (w0 >= rowWords)
            continue;
        const bool alignedS = ((reinterpret_cast<uintptr_t>(S.base) | static_cast<uintptr_t>(S.pitch)) & 3) == 0;
        const bool alignedD = ((reinterpret_cast<uintptr_t>(D.base) | static_cast<uintptr_t>(D.pitch)) & (4 * DE - 1)) == 0;
        // the grid's y extent may be smaller than the image: CTAs walk down in steps, so the table is built less often
        // The pass is compiled twice, with "every row on its vector boundaries" as a constant: as run-time flags inside the
        // unrolled loops both forms of every load and store were issued under predicates.
        auto pass = [&](auto alignedTag) {
        constexpr bool ALIGNED = decltype(alignedTag)::value;
        for (int yb = blockIdx.y; yb * (blockDim.y * RPT) < h; yb += gridDim.y)
        {
            const int y0 = (yb * blockDim.y + threadIdx.y) * RPT;
            unsigned  q[RPT][4];
#pragma unroll
            for (int r = 0; r < RPT; ++r)
            {
                const uint8_t *s = S.base + min(y0 + r, h - 1) * S.pitch;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                {
                    const int w = min(w0 + 32 * k, rowWords - 1);
                    if (ALIGNED || alignedS)
                    {
                        // the row's last word may reach up to three bytes past its last element: still inside the
                        // aligned word that holds that element, so the load cannot leave the allocation's pages
                        q[r][k] = __ldg(reinterpret_cast<const unsigned *>(s) + w);
                    }
                    else
                    {
                        q[r][k] = 0;
                        for (int j = 0; j < 4 && 4 * w + j < rowElems; ++j)
                            q[r][k] |= static_cast<unsigned>(__ldg(s + 4 * w + j)) << (8 * j);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < RPT; ++r)
            {
                const int y = y0 + r;
                if (y >= h)
                    break;
                uint8_t *d = D.base + y * D.pitch;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                {
                    const int w = w0 + 32 * k;
                    if (w >= rowWords)
                        break;
                    unsigned o[4];
                    int      c = (4 * w) % p.channels;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                    {
                        o[j] = lut[c * 256 + ((q[r][k] >> (8 * j)) & 255u)];
                        c    = c + 1 == p.channels ? 0 : c + 1;
                    }
                    const int count = min(4, rowElems - 4 * w);
                    uint8_t  *out   = d + static_cast<long long>(w) * (4 * DE);
                    if (count == 4 && (ALIGNED || alignedD))
                    {
                        if constexpr (DE == 4)
                            *reinterpret_cast<uint4 *>(out) = make_uint4(o[0], o[1], o[2], o[3]);
                        else if constexpr (DE == 2)
                            *reinterpret_cast<uint2 *>(out) = make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
                        else
                            *reinterpret_cast<unsigned *>(out) = o[0] | (o[1] << 8) | (o[2] << 16) | (o[3] << 24);
                    }
                    else
                    {
                        asm volatile("" ::: "memory"); // the ragged end of a row stays a branch, not predicated stores
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (j < count)
                            {
                                if constexpr (DE == 4)
                                    reinterpret_cast<unsigned *>(out)[j] = o[j];
                                else if constexpr (DE == 2)
                                    reinterpret_cast<unsigned short *>(out)[j] = static_cast<unsigned short>(o[j]);
                                else
                                    out[j] = static_cast<uint8_t>(o[j]);
                            }
                    }
                }
            }
        }
        };
        if (alignedS && alignedD)
            pass(std::true_type{});
        else
            pass(std::false_type{});
    }
}

} // namespace b200pp

#endif
