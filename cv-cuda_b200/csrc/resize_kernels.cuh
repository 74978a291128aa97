// Resize + crop + flip + affine + channel map + cast + layout kernels (3-channel interleaved uint8 sources).
//
//  * resize_gather_kernel  -- one thread per destination pixel, taps read straight from global memory.
//                             Handles every argument combination; the fallback and the cross-check.
//  * resize_staged_kernel  -- persistent, warp-specialised pipeline. A work unit is one destination row segment of
//                             one sample. A producer thread copies the one or two source row segments that the unit
//                             taps into a shared-memory ring with bulk asynchronous copies (cp.async.bulk, completion
//                             on an mbarrier); the consumer warps interpolate out of shared memory and write
//                             warp-contiguous destination rows. HBM sees only long contiguous reads and full-sector
//                             writes; the byte-granular gather happens in shared memory.
//
// Replaces resizeCrop_NN / resizeCrop_bilinear / *_varShape of the reference
// (src/cvcuda/priv/OpResizeCropConvertReformat.cu:137-278); arithmetic follows the reference's CPU golden
// (tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:95-171).
#ifndef CVCUDA_B200_RESIZE_KERNELS_CUH
#define CVCUDA_B200_RESIZE_KERNELS_CUH

#include "device_math.cuh"

namespace b200pp {

// Device error word. Bits: 1 = a consumer gave up waiting for a staged row, 2 = the producer gave up waiting
// for a free ring slot, 4 = the producer gave up draining its copies at exit.
__device__ unsigned int g_deviceError;

constexpr int kProducerThreads = 32;
constexpr unsigned long long kWaitLimitNs = 2000000000ull; // 2 s

// ------------------------------------------------------------------------------------------------ pixel maths

// One destination pixel of the linear path. r0/r1 point at byte 0 of the two tapped source rows in whatever
// memory they are staged in; o0/o1 are the byte offsets of the left/right tap pixel.
template<int DK>
__device__ __forceinline__ void linear_pixel(const ResizeKParams &p, const uint8_t *r0, const uint8_t *r1, int o0,
                                             int o1, float wx1, float wy1, uint8_t *dstPix)
{
    const float wx0 = __fsub_rn(1.0f, wx1);
    const float wy0 = __fsub_rn(1.0f, wy1);
#pragma unroll
    for (int c = 0; c < 3; ++c)
    {
        float v = blend4(static_cast<float>(r0[o0 + c]), static_cast<float>(r0[o1 + c]),
                         static_cast<float>(r1[o0 + c]), static_cast<float>(r1[o1 + c]), wx0, wx1, wy0, wy1);
        if (p.srcCast)
            v = static_cast<float>(sat_u8(v));
        store_elem<DK>(dstPix + p.mapC[c] * p.dChan, affine(p, c, v));
    }
}

template<int DK>
__device__ __forceinline__ void nearest_pixel(const ResizeKParams &p, const uint8_t *r0, int o0, uint8_t *dstPix)
{
#pragma unroll
    for (int c = 0; c < 3; ++c) store_elem<DK>(dstPix + p.mapC[c] * p.dChan, affine(p, c, static_cast<float>(r0[o0 + c])));
}

template<int DK>
__device__ __forceinline__ void pad_pixel(const ResizeKParams &p, uint8_t *dstPix)
{
#pragma unroll
    for (int c = 0; c < 3; ++c) store_elem<DK>(dstPix + p.mapC[c] * p.dChan, affine(p, c, p.padValue));
}

// ------------------------------------------------------------------------------------------------ gather kernel

template<int INTERP, int DK>
__global__ void __launch_bounds__(256) resize_gather_kernel(const ResizeKParams p)
{
    const int x = blockIdx.x * blockDim.x + threadIdx.x;
    const int y = blockIdx.y * blockDim.y + threadIdx.y;
    if (x >= p.dstW || y >= p.dstH)
        return;

    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        uint8_t *dstPix = p.dst + n * p.dSample + y * p.dRow + x * p.dPix;
        const int rx = x - p.dstX, ry = y - p.dstY;
        if (rx < 0 || ry < 0 || rx >= p.regionW || ry >= p.regionH)
        {
            pad_pixel<DK>(p, dstPix);
            continue;
        }
        const Geom g  = load_geom(p, n);
        const int  dx = ((g.flip == 1 || g.flip == -1) ? p.regionW - 1 - rx : rx) + p.cropX;
        const int  dy = ((g.flip == 0 || g.flip == -1) ? p.regionH - 1 - ry : ry) + p.cropY;

        if constexpr (INTERP == B200PP_INTERP_NEAREST)
        {
            const int sx = nearest_tap(g.scaleW, dx, g.w);
            const int sy = nearest_tap(g.scaleH, dy, g.h);
            nearest_pixel<DK>(p, g.base + sy * g.pitch, 3 * sx, dstPix);
        }
        else
        {
            int   sx0, sx1, sy0, sy1;
            float wx1, wy1;
            linear_tap(g.scaleW, dx, g.w, sx0, sx1, wx1);
            linear_tap(g.scaleH, dy, g.h, sy0, sy1, wy1);
            linear_pixel<DK>(p, g.base + sy0 * g.pitch, g.base + sy1 * g.pitch, 3 * sx0, 3 * sx1, wx1, wy1, dstPix);
        }
    }
}

// ------------------------------------------------------------------------------------------------ mbarrier / bulk copy

__device__ __forceinline__ unsigned smem_addr(const void *p)
{
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool mbar_try_wait(unsigned addr, unsigned parity)
{
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait for the phase with the given parity: gives up (returns false) after kWaitLimitNs of wall time.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity)
{
    const unsigned addr = smem_addr(bar);
    if (mbar_try_wait(addr, parity))
        return true;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned spin = 1;; ++spin)
    {
        if (mbar_try_wait(addr, parity))
            return true;
        if ((spin & 63u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs)
            return false;
    }
}

// Bulk asynchronous copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load(void *smemDst, const void *gmemSrc, unsigned bytes, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(smemDst)),
                 "l"(gmemSrc), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// ------------------------------------------------------------------------------------------------ staged kernel

// What the producer tells the consumers about the unit staged in one ring slot.
struct UnitInfo
{
    int            mode; // 0: nothing to sample (row outside the region); 1: rows staged in shared memory; 2: read global
    int            y, x0, x1;
    int            flipX;
    int            srcW;
    int            segOrigin; // source-row byte offset that shared-memory offset 0 of the slot corresponds to
    int            sameRow;   // linear: both taps come from one source row
    float          scaleW;
    float          wy1;
    long long      dstRowOff;
    const uint8_t *g0, *g1; // tapped source rows in global memory (byte 0 of the row of the sub-view)
};

enum
{
    UNIT_PAD    = 0,
    UNIT_STAGED = 1,
    UNIT_DIRECT = 2
};

// Columns [x0, x1) of one destination row, strided over the consumer threads so that a warp writes 32 adjacent pixels.
template<int INTERP, int DK>
__device__ __forceinline__ void consume_columns(const ResizeKParams &p, const UnitInfo &info, const uint8_t *r0,
                                                const uint8_t *r1, int origin, uint8_t *dstRow, int ct,
                                                int consumerThreads)
{
    for (int x = info.x0 + ct; x < info.x1; x += consumerThreads)
    {
        uint8_t  *dstPix = dstRow + x * p.dPix;
        const int rx     = x - p.dstX;
        if (rx < 0 || rx >= p.regionW)
        {
            pad_pixel<DK>(p, dstPix);
            continue;
        }
        const int dx = (info.flipX ? p.regionW - 1 - rx : rx) + p.cropX;
        if constexpr (INTERP == B200PP_INTERP_NEAREST)
        {
            nearest_pixel<DK>(p, r0, 3 * nearest_tap(info.scaleW, dx, info.srcW) - origin, dstPix);
        }
        else
        {
            int   sx0, sx1;
            float wx1;
            linear_tap(info.scaleW, dx, info.srcW, sx0, sx1, wx1);
            linear_pixel<DK>(p, r0, r1, 3 * sx0 - origin, 3 * sx1 - origin, wx1, info.wy1, dstPix);
        }
    }
}

template<int INTERP, int DK>
__global__ void __launch_bounds__(512) resize_staged_kernel(const ResizeKParams p, const StagedCfg cfg)
{
    extern __shared__ __align__(128) unsigned char smemRaw[];

    const int       S         = cfg.stages;
    const long long slotBytes = static_cast<long long>(cfg.rowsPerStage) * cfg.segBytes;
    unsigned char  *ring      = smemRaw;
    UnitInfo       *infos     = reinterpret_cast<UnitInfo *>(ring + S * slotBytes);
    auto           *full      = reinterpret_cast<unsigned long long *>(infos + S);
    unsigned long long *empty = full + S;

    const int consumerThreads = blockDim.x - kProducerThreads;
    const int consumerWarps   = consumerThreads / 32;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < S; ++s)
        {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], consumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // contiguous range of units per CTA: a CTA mostly stays inside one sample
    const long long uBegin = cfg.totalUnits * blockIdx.x / gridDim.x;
    const long long uEnd   = cfg.totalUnits * (blockIdx.x + 1) / gridDim.x;
    const long long unitsPerSample = static_cast<long long>(p.dstH) * cfg.chunksPerRow;

    if (threadIdx.x < kProducerThreads)
    {
        // ===================================================================== producer (one thread)
        if (threadIdx.x != 0)
            return;
        int       cachedN = -1;
        Geom      g{};
        bool      aligned = false;
        long long k       = 0;
        bool      failed  = false;
        for (long long u = uBegin; u < uEnd; ++u, ++k)
        {
            const int s = static_cast<int>(k % S);
            if (k >= S && !mbar_wait(&empty[s], static_cast<unsigned>((k / S - 1) & 1)))
            {
                atomicOr(&g_deviceError, 2u);
                failed = true;
                break;
            }
            const int n     = static_cast<int>(u / unitsPerSample);
            const int rem   = static_cast<int>(u - n * unitsPerSample);
            const int y     = rem / cfg.chunksPerRow;
            const int chunk = rem - y * cfg.chunksPerRow;
            if (n != cachedN)
            {
                g       = load_geom(p, n);
                aligned = ((reinterpret_cast<unsigned long long>(g.image) | static_cast<unsigned long long>(g.pitch)) & 15ull) == 0;
                cachedN = n;
            }
            UnitInfo &info = infos[s];
            info.y         = y;
            info.x0        = chunk * cfg.chunkCols;
            info.x1        = min(info.x0 + cfg.chunkCols, p.dstW);
            info.dstRowOff = n * p.dSample + y * p.dRow;
            info.flipX     = (g.flip == 1 || g.flip == -1);
            info.srcW      = g.w;
            info.scaleW    = g.scaleW;

            const int ry  = y - p.dstY;
            const int rx0 = max(info.x0 - p.dstX, 0);
            const int rx1 = min(info.x1 - p.dstX, p.regionW) - 1; // inclusive
            if (ry < 0 || ry >= p.regionH || rx1 < rx0)
            {
                info.mode = UNIT_PAD;
                mbar_arrive(&full[s]);
                continue;
            }
            const int dy  = ((g.flip == 0 || g.flip == -1) ? p.regionH - 1 - ry : ry) + p.cropY;
            const int dlo = (info.flipX ? p.regionW - 1 - rx1 : rx0) + p.cropX;
            const int dhi = (info.flipX ? p.regionW - 1 - rx0 : rx1) + p.cropX;

            int sy0, sy1, sxmin, sxmax;
            if constexpr (INTERP == B200PP_INTERP_NEAREST)
            {
                sy0 = sy1 = nearest_tap(g.scaleH, dy, g.h);
                info.wy1  = 0.f;
                sxmin     = nearest_tap(g.scaleW, dlo, g.w);
                sxmax     = nearest_tap(g.scaleW, dhi, g.w);
            }
            else
            {
                float w;
                int   t;
                linear_tap(g.scaleH, dy, g.h, sy0, sy1, info.wy1);
                linear_tap(g.scaleW, dlo, g.w, sxmin, t, w);
                linear_tap(g.scaleW, dhi, g.w, t, sxmax, w);
            }
            info.g0      = g.base + sy0 * g.pitch;
            info.g1      = g.base + sy1 * g.pitch;
            info.sameRow = (sy0 == sy1);

            const unsigned long long a0 = reinterpret_cast<unsigned long long>(info.g0) + 3ull * sxmin;
            const unsigned long long a1 = reinterpret_cast<unsigned long long>(info.g0) + 3ull * (sxmax + 1);
            const unsigned long long s0 = a0 & ~15ull;
            const unsigned long long s1 = (a1 + 15ull) & ~15ull;
            const unsigned           nb = static_cast<unsigned>(s1 - s0);
            if (!aligned || nb > static_cast<unsigned>(cfg.segBytes))
            {
                info.mode = UNIT_DIRECT;
                mbar_arrive(&full[s]);
                continue;
            }
            info.mode      = UNIT_STAGED;
            info.segOrigin = 3 * sxmin - static_cast<int>(a0 & 15ull);

            unsigned char *slot   = ring + s * slotBytes;
            const bool     twoRow = (INTERP == B200PP_INTERP_LINEAR) && !info.sameRow;
            mbar_arrive_expect_tx(&full[s], twoRow ? 2u * nb : nb);
            bulk_load(slot, reinterpret_cast<const void *>(s0), nb, &full[s]);
            if (twoRow)
                bulk_load(slot + cfg.segBytes, reinterpret_cast<const void *>(s0 + (sy1 - sy0) * g.pitch), nb, &full[s]);
        }
        if (failed)
        {
            // Consumers have stopped releasing slots. Give the copies already issued a bounded time to land before
            // the CTA's shared memory goes away.
            for (long long j = (k > S ? k - S : 0); j < k; ++j)
                if (!mbar_wait(&full[j % S], static_cast<unsigned>((j / S) & 1)))
                {
                    atomicOr(&g_deviceError, 4u);
                    break;
                }
        }
        return;
    }

    // ========================================================================= consumers
    const int ct   = threadIdx.x - kProducerThreads;
    const int lane = threadIdx.x & 31;
    long long k    = 0;
    for (long long u = uBegin; u < uEnd; ++u, ++k)
    {
        const int s = static_cast<int>(k % S);
        if (!mbar_wait(&full[s], static_cast<unsigned>((k / S) & 1)))
        {
            atomicOr(&g_deviceError, 1u);
            return;
        }
        const UnitInfo info = infos[s];
        uint8_t       *dstRow = p.dst + info.dstRowOff;

        if (info.mode == UNIT_PAD)
        {
            for (int x = info.x0 + ct; x < info.x1; x += consumerThreads) pad_pixel<DK>(p, dstRow + x * p.dPix);
        }
        else if (info.mode == UNIT_STAGED)
        {
            // Kept as its own call site so that the row pointers visibly derive from the shared-memory ring and the
            // tap reads compile to shared-memory loads.
            const uint8_t *r0 = ring + s * slotBytes;
            consume_columns<INTERP, DK>(p, info, r0, info.sameRow ? r0 : r0 + cfg.segBytes, info.segOrigin, dstRow, ct,
                                        consumerThreads);
        }
        else
        {
            consume_columns<INTERP, DK>(p, info, info.g0, info.g1, 0, dstRow, ct, consumerThreads);
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(&empty[s]);
    }
}

} // namespace b200pp

#endif
