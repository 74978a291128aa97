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
// for a free ring slot, 4 = the producer gave up draining its copies at exit, 8 = the wait self-test gave up (expected).
__device__ unsigned int g_deviceError;

constexpr int                kProducerThreads = 32;
constexpr unsigned long long kWaitLimitNs     = 2000000000ull; // 2 s
// Upper bound of one hardware-suspended wait: a waiting warp sleeps instead of burning issue slots in a poll loop.
constexpr unsigned           kSuspendHintNs   = 4000;

// ------------------------------------------------------------------------------------------------ pixel maths
//
// Integer <-> float conversion instructions run at a fraction of the FP32 rate and the straightforward kernel would
// issue fifteen of them per pixel. None is needed:
//
//  * A source byte b is loaded zero-extended and its bit pattern is used AS a float: the denormal b * 2^-149. The
//    vertical weights are pre-multiplied by 2^127 and the horizontal ones by 2^22 (exact, once per row / per column).
//    (b*2^-149) * (wy*2^127) is the normal number (b*wy) * 2^-22 with exactly the mantissa rounding of the golden's
//    b*wy, and multiplying by wx*2^22 gives exactly the golden's (b*wy)*wx. Denormal operands run at full rate.
//  * Round-half-even + clamp to [0, 255] (the uint8 saturate cast) is clamp, then add and subtract 1.5 * 2^23.

constexpr float kTwo127 = 1.7014118346046923e38f; // 2^127
constexpr float kTwo22  = 4194304.0f;             // 2^22
constexpr float kRound  = 12582912.0f;            // 1.5 * 2^23

__device__ __forceinline__ float raw_byte(const uint8_t *p)
{
    return __uint_as_float(static_cast<unsigned>(*p));
}

// float(SaturateCast<uint8_t>(v)) for finite v
__device__ __forceinline__ float round_sat_u8(float v)
{
    v = fminf(fmaxf(v, 0.0f), 255.0f);
    return __fsub_rn(__fadd_rn(v, kRound), kRound);
}

// Byte offsets of the three destination channels of a pixel (channel map applied).
struct ChanOff
{
    long long c[3];
};

__device__ __forceinline__ ChanOff chan_offsets(const ResizeKParams &p)
{
    ChanOff o;
#pragma unroll
    for (int c = 0; c < 3; ++c) o.c[c] = p.mapC[c] * p.dChan;
    return o;
}

// Cast + store of one finished value.
template<int DK>
__device__ __forceinline__ void store_value(float v, uint8_t *dst)
{
    if constexpr (DK == DST_U8)
        *dst = static_cast<uint8_t>(__float_as_uint(__fadd_rn(fminf(fmaxf(v, 0.0f), 255.0f), kRound)));
    else
        store_elem<DK>(dst, v);
}

// The affine step on the three channels of one pixel (v[c] belongs to source channel c). The two forms are separate
// code paths so that the choice costs one uniform branch per pixel, not one per channel.
__device__ __forceinline__ void affine3(const ResizeKParams &p, float (&v)[3])
{
    if (p.perChannel)
    {
#pragma unroll
        for (int c = 0; c < 3; ++c)
            v[c] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v[c], p.base[c]), p.mul[c]), p.gscale), p.shift);
    }
    else
    {
#pragma unroll
        for (int c = 0; c < 3; ++c) v[c] = __fadd_rn(__fmul_rn(p.scale, v[c]), p.offset);
    }
}

// Final values of one destination pixel of the linear path. r0/r1 point at byte 0 of the two tapped source rows in
// whatever memory they live in; o0/o1 are the byte offsets of the left/right tap pixel. Weights are pre-scaled:
// wy*s = wy * 2^127, wx*s = wx * 2^22.
__device__ __forceinline__ void linear_values(const ResizeKParams &p, const uint8_t *r0, const uint8_t *r1, int o0, int o1,
                                              float wx0s, float wx1s, float wy0s, float wy1s, float (&v)[3])
{
    // A tap whose weight is exactly zero contributes +0 to the golden's left-to-right sum of non-negative products, so
    // it is neither read nor multiplied (integer scale factors: every second tap; the producer does not even fetch a
    // source row whose weight is zero).
    if (wy1s == 0.0f)
    {
        if (wx1s == 0.0f)
        {
#pragma unroll
            for (int c = 0; c < 3; ++c) v[c] = __fmul_rn(__fmul_rn(raw_byte(r0 + o0 + c), wy0s), wx0s);
        }
        else
        {
#pragma unroll
            for (int c = 0; c < 3; ++c)
                v[c] = __fadd_rn(__fmul_rn(__fmul_rn(raw_byte(r0 + o0 + c), wy0s), wx0s),
                                 __fmul_rn(__fmul_rn(raw_byte(r0 + o1 + c), wy0s), wx1s));
        }
    }
    else if (wx1s == 0.0f)
    {
#pragma unroll
        for (int c = 0; c < 3; ++c)
            v[c] = __fadd_rn(__fmul_rn(__fmul_rn(raw_byte(r0 + o0 + c), wy0s), wx0s),
                             __fmul_rn(__fmul_rn(raw_byte(r1 + o0 + c), wy1s), wx0s));
    }
    else
    {
#pragma unroll
        for (int c = 0; c < 3; ++c)
            v[c] = blend4(raw_byte(r0 + o0 + c), raw_byte(r0 + o1 + c), raw_byte(r1 + o0 + c), raw_byte(r1 + o1 + c),
                          wx0s, wx1s, wy0s, wy1s);
    }
    if (p.srcCast)
    {
#pragma unroll
        for (int c = 0; c < 3; ++c) v[c] = round_sat_u8(v[c]);
    }
    affine3(p, v);
}

__device__ __forceinline__ void nearest_values(const ResizeKParams &p, const uint8_t *r0, int o0, float (&v)[3])
{
#pragma unroll
    for (int c = 0; c < 3; ++c) v[c] = __fmul_rn(__fmul_rn(raw_byte(r0 + o0 + c), kTwo127), kTwo22);
    affine3(p, v);
}

// Destination values of a pixel outside the placed region: the pad value pushed through the affine step, the same for
// every such pixel of a launch, so each thread works them out once.
struct PadValues
{
    float v[3];
};

__device__ __forceinline__ PadValues pad_values(const ResizeKParams &p)
{
    PadValues pv;
#pragma unroll
    for (int c = 0; c < 3; ++c) pv.v[c] = p.padValue;
    affine3(p, pv.v);
    return pv;
}

// Cast + store of the three channels of one pixel through the generic strides (any layout).
template<int DK>
__device__ __forceinline__ void store_pixel(const float (&v)[3], const ChanOff &co, uint8_t *dstPix)
{
#pragma unroll
    for (int c = 0; c < 3; ++c) store_value<DK>(v[c], dstPix + co.c[c]);
}

// Interleaved (NHWC) destinations: a warp's 32 pixels are 96 consecutive elements in memory, but each lane holds the
// three channels of one pixel. The channels are transposed across the warp with shuffles so that every store
// instruction writes consecutive 32-bit words: three fully coalesced stores for float32 (lane L writes elements L,
// 32+L, 64+L), one for uint8 (lanes 0..23 write the 96 bytes as 24 words). `warpBase` is the address of lane 0's pixel.
// All 32 lanes must call this.
template<int DK>
__device__ __forceinline__ void store_interleaved_warp(const float (&d)[3] /* destination channel order */,
                                                       uint8_t *warpBase, int lane)
{
    if constexpr (DK == DST_F32)
    {
#pragma unroll
        for (int k = 0; k < 3; ++k)
        {
            const int   e   = 32 * k + lane; // element index within the warp's 96
            const int   src = (e * 43) >> 7; // e / 3 for e < 128
            const int   c   = e - 3 * src;
            const float a = __shfl_sync(0xffffffffu, d[0], src), b = __shfl_sync(0xffffffffu, d[1], src),
                        g = __shfl_sync(0xffffffffu, d[2], src);
            reinterpret_cast<float *>(warpBase)[e] = c == 0 ? a : (c == 1 ? b : g);
        }
    }
    else
    {
        // pack this lane's pixel into 24 bits, then word j = bytes 4j..4j+3 straddles pixels p0 = 4j/3 and p0+1
        const unsigned w = (__float_as_uint(__fadd_rn(fminf(fmaxf(d[0], 0.0f), 255.0f), kRound)) & 0xffu)
                         | (__float_as_uint(__fadd_rn(fminf(fmaxf(d[1], 0.0f), 255.0f), kRound)) & 0xffu) << 8
                         | (__float_as_uint(__fadd_rn(fminf(fmaxf(d[2], 0.0f), 255.0f), kRound)) & 0xffu) << 16;
        const int      b0  = 4 * lane;
        const int      p0  = (b0 * 43) >> 7; // b0 / 3 (b0 < 128)
        const int      off = b0 - 3 * p0;
        const unsigned lo  = __shfl_sync(0xffffffffu, w, p0 & 31);
        const unsigned hi  = __shfl_sync(0xffffffffu, w, (p0 + 1) & 31);
        if (lane < 24)
            reinterpret_cast<unsigned *>(warpBase)[lane] = (lo >> (8 * off)) | (hi << (8 * (3 - off)));
    }
}

// ------------------------------------------------------------------------------------------------ gather kernel

template<int INTERP, int DK>
__global__ void __launch_bounds__(256) resize_gather_kernel(const ResizeKParams p)
{
    const int x = blockIdx.x * blockDim.x + threadIdx.x;
    const int y = blockIdx.y * blockDim.y + threadIdx.y;
    if (x >= p.dstW || y >= p.dstH)
        return;
    const ChanOff   co = chan_offsets(p);
    const PadValues pv = pad_values(p);

    for (int n = blockIdx.z; n < p.numSamples; n += gridDim.z)
    {
        uint8_t  *dstPix = p.dst + n * p.dSample + y * p.dRow + x * p.dPix;
        const int rx = x - p.dstX, ry = y - p.dstY;
        if (rx < 0 || ry < 0 || rx >= p.regionW || ry >= p.regionH)
        {
            store_pixel<DK>(pv.v, co, dstPix);
            continue;
        }
        const Geom g  = load_geom(p, n);
        const int  dx = ((g.flip == 1 || g.flip == -1) ? p.regionW - 1 - rx : rx) + p.cropX;
        const int  dy = ((g.flip == 0 || g.flip == -1) ? p.regionH - 1 - ry : ry) + p.cropY;

        if constexpr (INTERP == B200PP_INTERP_NEAREST)
        {
            const int sx = nearest_tap(g.scaleW, dx, g.w);
            const int sy = nearest_tap(g.scaleH, dy, g.h);
            float v[3];
            nearest_values(p, g.base + sy * g.pitch, 3 * sx, v);
            store_pixel<DK>(v, co, dstPix);
        }
        else
        {
            int   sx0, sx1, sy0, sy1;
            float wx1, wy1;
            linear_tap(g.scaleW, dx, g.w, sx0, sx1, wx1);
            linear_tap(g.scaleH, dy, g.h, sy0, sy1, wy1);
            float v[3];
            linear_values(p, g.base + sy0 * g.pitch, g.base + sy1 * g.pitch, 3 * sx0, 3 * sx1,
                          __fmul_rn(__fsub_rn(1.0f, wx1), kTwo22), __fmul_rn(wx1, kTwo22),
                          __fmul_rn(__fsub_rn(1.0f, wy1), kTwo127), __fmul_rn(wy1, kTwo127), v);
            store_pixel<DK>(v, co, dstPix);
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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return done != 0;
}

// Bounded wait for the phase with the given parity: gives up (returns false) after `limitNs` of wall time.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity,
                                          unsigned long long limitNs = kWaitLimitNs)
{
    const unsigned addr = smem_addr(bar);
    if (mbar_try_wait(addr, parity))
        return true;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned spin = 1;; ++spin)
    {
        if (mbar_try_wait(addr, parity))
            return true;
        if ((spin & 63u) == 0 && globaltimer_ns() - t0 > limitNs)
            return false;
    }
}

// Self-test of the bounded wait: one warp waits on a barrier that nothing ever completes, with a short limit, and
// must come back with the give-up bit (8) set in the device error word -- the same code path a stuck pipeline takes.
__global__ void wait_timeout_probe_kernel(unsigned long long limitNs)
{
    __shared__ unsigned long long bar;
    if (threadIdx.x == 0)
    {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (!mbar_wait(&bar, 0, limitNs) && threadIdx.x == 0)
        atomicOr(&g_deviceError, 8u);
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
    int            mode; // UNIT_*
    int            x0, x1;
    int            flipX;
    int            srcW;
    int            segOrigin; // source-row byte offset that shared-memory offset 0 of the slot corresponds to
    int            sameRow;   // linear: both taps come from one source row
    float          scaleW;
    float          wy0s, wy1s; // vertical weights * 2^127
    long long      dstRowOff;
    long long      tapKey; // units with equal keys have identical column taps (same sample geometry, chunk and flip)
    const uint8_t *g0, *g1; // tapped source rows in global memory (byte 0 of the row of the sub-view)
};

enum
{
    UNIT_PAD    = 0, // nothing to sample: the row lies outside the placed region
    UNIT_STAGED = 1, // rows are in the shared-memory slot
    UNIT_DIRECT = 2  // read the rows from global memory (unaligned image, or a segment larger than a slot)
};

// Horizontal taps of one destination column: byte offsets of the left/right source pixel within the source row
// (o0 < 0 marks a column outside the placed region), the weights * 2^22 and the column's destination byte offset.
struct ColTap
{
    int       o0, o1;
    float     wx0s, wx1s;
    long long dstOff;
};

template<int INTERP>
__device__ __forceinline__ ColTap make_tap(const ResizeKParams &p, const UnitInfo &info, int x)
{
    ColTap t;
    t.dstOff     = x * p.dPix;
    t.wx0s       = 0.f;
    t.wx1s       = 0.f;
    const int rx = x - p.dstX;
    if (rx < 0 || rx >= p.regionW)
    {
        t.o0 = t.o1 = -1;
        return t;
    }
    const int dx = (info.flipX ? p.regionW - 1 - rx : rx) + p.cropX;
    if constexpr (INTERP == B200PP_INTERP_NEAREST)
    {
        t.o0 = t.o1 = 3 * nearest_tap(info.scaleW, dx, info.srcW);
    }
    else
    {
        int   s0, s1;
        float wx1;
        linear_tap(info.scaleW, dx, info.srcW, s0, s1, wx1);
        t.o0   = 3 * s0;
        t.o1   = 3 * s1;
        t.wx0s = __fmul_rn(__fsub_rn(1.0f, wx1), kTwo22);
        t.wx1s = __fmul_rn(wx1, kTwo22);
    }
    return t;
}

// Final values of one destination pixel from rows r0/r1 whose first byte is source-row byte `origin`.
template<int INTERP>
__device__ __forceinline__ void pixel_values(const ResizeKParams &p, const PadValues &pv, const UnitInfo &info,
                                             const ColTap &t, const uint8_t *r0, const uint8_t *r1, int origin,
                                             float (&v)[3])
{
    if (t.o0 < 0)
    {
#pragma unroll
        for (int c = 0; c < 3; ++c) v[c] = pv.v[c];
    }
    else if constexpr (INTERP == B200PP_INTERP_NEAREST)
        nearest_values(p, r0, t.o0 - origin, v);
    else
        linear_values(p, r0, r1, t.o0 - origin, t.o1 - origin, t.wx0s, t.wx1s, info.wy0s, info.wy1s, v);
}

// How a consumer warp writes its pixels.
struct StorePlan
{
    ChanOff co;
    bool    interleaved; // destination has the three channels of a pixel adjacent: transpose across the warp
    bool    reversed;    // channel order reversed
};

// Stores one pixel per lane of a warp. `x` is this lane's column (lanes hold consecutive columns), `valid` whether it
// exists. Every lane of the warp must call this.
template<int DK, bool IL>
__device__ __forceinline__ void store_warp(const ResizeKParams &p, const StorePlan &plan, const float (&v)[3],
                                           uint8_t *dstRow, int x, bool valid, int lane)
{
    if constexpr (IL && DK != DST_F16)
    {
        uint8_t   *warpBase = dstRow + (x - lane) * p.dPix;
        const bool full     = __all_sync(0xffffffffu, valid) && (reinterpret_cast<unsigned long long>(warpBase) & 3ull) == 0;
        if (full)
        {
            const float d[3] = {plan.reversed ? v[2] : v[0], v[1], plan.reversed ? v[0] : v[2]};
            store_interleaved_warp<DK>(d, warpBase, lane);
            return;
        }
    }
    if (valid)
        store_pixel<DK>(v, plan.co, dstRow + x * p.dPix);
}

// Columns [x0, x1) of one destination row, strided over the consumer threads so that a warp writes 32 adjacent pixels.
// The taps of a thread's first KC columns stay in registers while consecutive units share a tap key, which for a dense
// batch is the whole launch. KC is a template parameter because every cached column costs six registers.
// Loop trip counts are uniform across a warp (the stores vote and shuffle). IL selects the transposing store for
// interleaved destinations; planar destinations compile without it.
template<int INTERP, int DK, int KC, bool IL>
__device__ __forceinline__ void consume_columns(const ResizeKParams &p, const StorePlan &plan, const PadValues &pv,
                                                const UnitInfo &info, const uint8_t *r0, const uint8_t *r1, int origin,
                                                uint8_t *dstRow, int ct, int lane, int consumerThreads,
                                                ColTap (&cache)[KC], bool refresh)
{
#pragma unroll
    for (int k = 0; k < KC; ++k)
    {
        const int  x     = info.x0 + ct + k * consumerThreads;
        const bool valid = x < info.x1;
        float      v[3]  = {0.f, 0.f, 0.f};
        if (valid)
        {
            if (refresh)
                cache[k] = make_tap<INTERP>(p, info, x);
            pixel_values<INTERP>(p, pv, info, cache[k], r0, r1, origin, v);
        }
        store_warp<DK, IL>(p, plan, v, dstRow, x, valid, lane);
    }
    for (int xw = info.x0 + (ct - lane) + KC * consumerThreads; xw < info.x1; xw += consumerThreads)
    {
        const int  x     = xw + lane;
        const bool valid = x < info.x1;
        float      v[3]  = {0.f, 0.f, 0.f};
        if (valid)
        {
            const ColTap t = make_tap<INTERP>(p, info, x);
            pixel_values<INTERP>(p, pv, info, t, r0, r1, origin, v);
        }
        store_warp<DK, IL>(p, plan, v, dstRow, x, valid, lane);
    }
}

// Units are dealt to CTAs in blocks of cfg.blockUnits consecutive units, round-robin over the CTAs.
// Block size 1 keeps all CTAs on neighbouring destination rows (dense batches); a large block keeps a CTA inside one
// sample so that per-sample column taps stay cached (variable-shape batches).
struct UnitWalk
{
    long long blockUnits, stride; // stride = gridDim.x * blockUnits
    long long first;              // first unit of this CTA
    long long count;              // units this CTA processes

    __device__ __forceinline__ UnitWalk(const StagedCfg &cfg)
    {
        blockUnits = cfg.blockUnits;
        stride     = static_cast<long long>(gridDim.x) * blockUnits;
        first      = static_cast<long long>(blockIdx.x) * blockUnits;
        const long long blocks = (cfg.totalUnits + blockUnits - 1) / blockUnits;
        const long long mine   = blockIdx.x < blocks ? (blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        count                  = mine * blockUnits;
        if (mine > 0 && (blocks - 1) % gridDim.x == blockIdx.x)
            count -= blocks * blockUnits - cfg.totalUnits; // the last block of the launch may be short
    }

    // global index of this CTA's k-th unit
    __device__ __forceinline__ long long unit(long long k) const
    {
        const long long j = k / blockUnits;
        return first + j * stride + (k - j * blockUnits);
    }
};

// IL: the destination is interleaved (three adjacent channels per pixel) and is written with the transposing store.
template<int INTERP, int DK, int KC, bool IL>
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
    const int lane            = threadIdx.x & 31;

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

    const UnitWalk walk(cfg);

    if (threadIdx.x < kProducerThreads)
    {
        // ===================================================================== producer warp
        // Geometry of 32 consecutive units is worked out by the 32 lanes side by side (sample descriptors, row taps,
        // tapped span, copy addresses); the lanes then take turns, in unit order, to claim a ring slot, publish the
        // unit and issue its bulk copies.
        const bool perSampleTaps = p.list != nullptr || p.roi != nullptr;
        const int  unitsPerSample = p.dstH * cfg.chunksPerRow;
        int        s           = 0;
        unsigned   emptyParity = 1; // phase the consumers complete when they release the slot's previous use
        bool       failed      = false;
        long long  issued      = 0;

        for (long long kb = 0; kb < walk.count && !failed; kb += 32)
        {
            const long long k     = kb + lane;
            const bool      valid = k < walk.count;
            UnitInfo           info{};
            unsigned long long copySrc = 0;
            long long          rowDelta = 0;
            unsigned           nb = 0;
            if (valid)
            {
                const long long u     = walk.unit(k);
                const int       n     = static_cast<int>(u / unitsPerSample);
                const int       rem   = static_cast<int>(u - static_cast<long long>(n) * unitsPerSample);
                const int       y     = rem / cfg.chunksPerRow;
                const int       chunk = rem - y * cfg.chunksPerRow;
                const Geom      g     = load_geom(p, n);
                const bool      aligned
                    = ((reinterpret_cast<unsigned long long>(g.image) | static_cast<unsigned long long>(g.pitch)) & 15ull) == 0;

                info.x0        = chunk * cfg.chunkCols;
                info.x1        = min(info.x0 + cfg.chunkCols, p.dstW);
                info.dstRowOff = n * p.dSample + y * p.dRow;
                info.flipX     = (g.flip == 1 || g.flip == -1);
                info.tapKey    = ((perSampleTaps ? static_cast<long long>(n) + 1 : 0) * cfg.chunksPerRow + chunk) * 2 + info.flipX;
                info.srcW      = g.w;
                info.scaleW    = g.scaleW;

                const int ry  = y - p.dstY;
                const int rx0 = max(info.x0 - p.dstX, 0);
                const int rx1 = min(info.x1 - p.dstX, p.regionW) - 1; // inclusive
                if (ry < 0 || ry >= p.regionH || rx1 < rx0)
                {
                    info.mode = UNIT_PAD;
                }
                else
                {
                    const int dy  = ((g.flip == 0 || g.flip == -1) ? p.regionH - 1 - ry : ry) + p.cropY;
                    const int dlo = (info.flipX ? p.regionW - 1 - rx1 : rx0) + p.cropX;
                    const int dhi = (info.flipX ? p.regionW - 1 - rx0 : rx1) + p.cropX;
                    int       sy0, sy1, sxmin, sxmax;
                    if constexpr (INTERP == B200PP_INTERP_NEAREST)
                    {
                        sy0 = sy1 = nearest_tap(g.scaleH, dy, g.h);
                        sxmin     = nearest_tap(g.scaleW, dlo, g.w);
                        sxmax     = nearest_tap(g.scaleW, dhi, g.w);
                    }
                    else
                    {
                        float w, wy1;
                        int   t;
                        linear_tap(g.scaleH, dy, g.h, sy0, sy1, wy1);
                        info.wy0s = __fmul_rn(__fsub_rn(1.0f, wy1), kTwo127);
                        info.wy1s = __fmul_rn(wy1, kTwo127);
                        linear_tap(g.scaleW, dlo, g.w, sxmin, t, w);
                        linear_tap(g.scaleW, dhi, g.w, t, sxmax, w);
                    }
                    info.g0      = g.base + sy0 * g.pitch;
                    info.g1      = g.base + sy1 * g.pitch;
                    info.sameRow = (sy0 == sy1) || info.wy1s == 0.0f; // a lower row of weight zero is never read
                    rowDelta     = (sy1 - sy0) * g.pitch;

                    const unsigned long long a0 = reinterpret_cast<unsigned long long>(info.g0) + 3ull * sxmin;
                    const unsigned long long a1 = reinterpret_cast<unsigned long long>(info.g0) + 3ull * (sxmax + 1);
                    copySrc                     = a0 & ~15ull;
                    nb                          = static_cast<unsigned>(((a1 + 15ull) & ~15ull) - copySrc);
                    if (!aligned || nb > static_cast<unsigned>(cfg.segBytes))
                    {
                        info.mode = UNIT_DIRECT;
                    }
                    else
                    {
                        info.mode      = UNIT_STAGED;
                        info.segOrigin = 3 * sxmin - static_cast<int>(a0 & 15ull);
                    }
                }
            }

            const int batch = static_cast<int>(min(32ll, walk.count - kb));
            for (int j = 0; j < batch; ++j)
            {
                bool bad = false;
                if (lane == j)
                {
                    if (kb + j >= S && !mbar_wait(&empty[s], emptyParity))
                    {
                        atomicOr(&g_deviceError, 2u);
                        bad = true;
                    }
                    else
                    {
                        infos[s] = info;
                        if (info.mode == UNIT_STAGED)
                        {
                            unsigned char *slot   = ring + s * slotBytes;
                            const bool     twoRow = (INTERP == B200PP_INTERP_LINEAR) && !info.sameRow;
                            mbar_arrive_expect_tx(&full[s], twoRow ? 2u * nb : nb);
                            bulk_load(slot, reinterpret_cast<const void *>(copySrc), nb, &full[s]);
                            if (twoRow)
                                bulk_load(slot + cfg.segBytes, reinterpret_cast<const void *>(copySrc + rowDelta), nb, &full[s]);
                        }
                        else
                        {
                            mbar_arrive(&full[s]);
                        }
                    }
                }
                if (__any_sync(0xffffffffu, bad))
                {
                    failed = true;
                    break;
                }
                ++issued;
                if (++s == S)
                {
                    s = 0;
                    emptyParity ^= 1u;
                }
            }
        }
        if (failed && lane == 0)
        {
            // Consumers have stopped releasing slots. Give the copies already issued a bounded time to land before
            // the CTA's shared memory goes away.
            for (long long j = (issued > S ? issued - S : 0); j < issued; ++j)
                if (!mbar_wait(&full[j % S], static_cast<unsigned>((j / S) & 1)))
                {
                    atomicOr(&g_deviceError, 4u);
                    break;
                }
        }
        return;
    }

    // ========================================================================= consumers
    const int     ct         = threadIdx.x - kProducerThreads;
    const PadValues pv       = pad_values(p);
    StorePlan       plan;
    plan.co          = chan_offsets(p);
    plan.interleaved = IL;
    plan.reversed    = p.mapC[0] == 2;
    long long     cachedKey  = -1;
    int           s          = 0;
    unsigned      fullParity = 0;
    ColTap        cache[KC];
    for (long long k = 0; k < walk.count; ++k)
    {
        if (!mbar_wait(&full[s], fullParity))
        {
            atomicOr(&g_deviceError, 1u);
            return;
        }
        const UnitInfo info   = infos[s];
        uint8_t       *dstRow = p.dst + info.dstRowOff;

        if (info.mode == UNIT_PAD)
        {
            for (int xw = info.x0 + (ct - lane); xw < info.x1; xw += consumerThreads)
                store_warp<DK, IL>(p, plan, pv.v, dstRow, xw + lane, xw + lane < info.x1, lane);
        }
        else
        {
            const bool refresh = info.tapKey != cachedKey;
            cachedKey          = info.tapKey;
            if (info.mode == UNIT_STAGED)
            {
                // Its own call site: the row pointers visibly derive from the shared-memory ring, so the tap reads
                // compile to shared-memory loads.
                const uint8_t *r0 = ring + s * slotBytes;
                const uint8_t *r1 = info.sameRow ? r0 : r0 + cfg.segBytes;
                consume_columns<INTERP, DK, KC, IL>(p, plan, pv, info, r0, r1, info.segOrigin, dstRow, ct, lane,
                                                    consumerThreads, cache, refresh);
            }
            else
            {
                consume_columns<INTERP, DK, KC, IL>(p, plan, pv, info, info.g0, info.g1, 0, dstRow, ct, lane,
                                                    consumerThreads, cache, refresh);
            }
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(&empty[s]);
        if (++s == S)
        {
            s = 0;
            fullParity ^= 1u;
        }
    }
}

} // namespace b200pp

#endif
