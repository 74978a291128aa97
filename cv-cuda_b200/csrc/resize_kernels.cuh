// Resize + crop + flip + affine + channel map + cast + layout kernels (3-channel interleaved uint8 sources).
//
//  * resize_gather_kernel  -- one thread per destination pixel, taps read straight from global memory.
//                             Handles every argument combination; the fallback and the cross-check.
//  * resize_rowwalk_kernel -- a thread keeps one destination column's taps in registers and walks down a group of
//                             rows, reading from global memory through the L1. No pipeline to fill or drain: the kernel
//                             for batches with per-sample geometry (image lists, regions of interest).
//  * resize_staged_kernel  -- persistent, warp-specialised pipeline for dense batches. A work unit is one to four
//                             destination rows of one column chunk of one sample. A producer warp describes units 32
//                             at a time and publishes them in order: the source row segments a unit taps go into a
//                             shared-memory ring by bulk asynchronous copies (cp.async.bulk, completion counted in
//                             bytes on an mbarrier). Consumer warps interpolate out of shared memory, four adjacent
//                             pixels per thread, and write the rows with 4-element vector stores. HBM sees only long
//                             contiguous reads and full-sector writes; the byte-granular gather happens in shared
//                             memory.
//
// Replaces resizeCrop_NN / resizeCrop_bilinear / *_varShape of the reference
// (src/cvcuda/priv/OpResizeCropConvertReformat.cu:137-278); arithmetic follows the reference's CPU golden
// (tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:95-171).
#ifndef CVCUDA_B200_RESIZE_KERNELS_CUH
#define CVCUDA_B200_RESIZE_KERNELS_CUH

#include "device_math.cuh"

namespace b200pp {

// Device error word. Bits: 1 = a consumer gave up waiting for a staged row, 2 = the producer gave up waiting
// for a free ring slot, 4 = the producer gave up draining its copies at exit, 8 = the wait self-test gave up (expected),
// 16 = the staged kernel was launched with a shape it refuses (nothing was written).
__device__ unsigned int g_deviceError;
// Where the host can see the word without synchronising: a page-locked, device-mapped copy that the library sets up once per
// device (null until then). The entry points look at it before they launch, so a kernel that gave up on a wait turns the
// NEXT call on that device into B200PP_ERROR_INTERNAL instead of going unnoticed.
__device__ unsigned int *g_deviceErrorMirror;

__device__ __forceinline__ void raise_device_error(unsigned bits)
{
    atomicOr(&g_deviceError, bits);
    if (g_deviceErrorMirror)
    {
        atomicOr_system(g_deviceErrorMirror, bits);
        __threadfence_system();
    }
}

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

// A tapped source row segment: either a 32-bit shared-memory address (staged rows; explicit ld.shared with the channel
// as an immediate offset, 32-bit address arithmetic) or a pointer into global memory.
struct SmemRow
{
    unsigned a;
};

__device__ __forceinline__ SmemRow operator+(SmemRow r, int byteOff)
{
    return SmemRow{r.a + static_cast<unsigned>(byteOff)};
}

// The three channel bytes of the pixel at `r`, each as the float whose bit pattern is the byte.
__device__ __forceinline__ void tap3(SmemRow r, float (&b)[3])
{
    unsigned x, y, z;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(x) : "r"(r.a));
    asm volatile("ld.shared.u8 %0, [%1+1];" : "=r"(y) : "r"(r.a));
    asm volatile("ld.shared.u8 %0, [%1+2];" : "=r"(z) : "r"(r.a));
    b[0] = __uint_as_float(x);
    b[1] = __uint_as_float(y);
    b[2] = __uint_as_float(z);
}

__device__ __forceinline__ void tap3(const uint8_t *r, float (&b)[3])
{
#pragma unroll
    for (int c = 0; c < 3; ++c) b[c] = __uint_as_float(static_cast<unsigned>(r[c]));
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

// Final values of one destination pixel of the linear path. r0/r1 address byte 0 of the two tapped source rows in
// whatever memory they live in (SmemRow or a global pointer); o0/o1 are the byte offsets of the left/right tap pixel.
// Weights are pre-scaled: wy*s = wy * 2^127, wx*s = wx * 2^22.
// Two float32 values in one 64-bit register and their packed product (sm_100: mul.rn.f32x2 issues at the rate of one scalar
// multiply and rounds each half like the scalar instruction).
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ unsigned long long mul_f32x2(unsigned long long a, unsigned long long b)
{
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

template<bool PACKED = false, class Row>
__device__ __forceinline__ void linear_values(const ResizeKParams &p, Row r0, Row r1, int o0, int o1, float wx0s,
                                              float wx1s, float wy0s, float wy1s, float (&v)[3])
{
    // A tap whose weight is exactly zero contributes +0 to the golden's left-to-right sum of non-negative products, so
    // it is neither read nor multiplied (integer scale factors: every second tap; the producer does not even fetch a
    // source row whose weight is zero).
    float a[3], b[3];
    if (wy1s == 0.0f)
    {
        tap3(r0 + o0, a);
        if (wx1s == 0.0f)
        {
#pragma unroll
            for (int c = 0; c < 3; ++c) v[c] = __fmul_rn(__fmul_rn(a[c], wy0s), wx0s);
        }
        else
        {
            tap3(r0 + o1, b);
#pragma unroll
            for (int c = 0; c < 3; ++c)
                v[c] = __fadd_rn(__fmul_rn(__fmul_rn(a[c], wy0s), wx0s), __fmul_rn(__fmul_rn(b[c], wy0s), wx1s));
        }
    }
    else if (wx1s == 0.0f)
    {
        tap3(r0 + o0, a);
        tap3(r1 + o0, b);
#pragma unroll
        for (int c = 0; c < 3; ++c)
            v[c] = __fadd_rn(__fmul_rn(__fmul_rn(a[c], wy0s), wx0s), __fmul_rn(__fmul_rn(b[c], wy1s), wx0s));
    }
    else
    {
        float c2[3], d[3];
        tap3(r0 + o0, a);
        tap3(r0 + o1, b);
        tap3(r1 + o0, c2);
        tap3(r1 + o1, d);
        if constexpr (PACKED)
        {
            // the eight products of a channel as four packed multiplies: (left, right) of a row by that row's weight, then by
            // the (left, right) horizontal weights; the sum in the golden's order
            const unsigned long long wy0p = pack_f32x2(wy0s, wy0s), wy1p = pack_f32x2(wy1s, wy1s), wxp = pack_f32x2(wx0s, wx1s);
#pragma unroll
            for (int c = 0; c < 3; ++c)
            {
                float t00, t01, t10, t11;
                unpack_f32x2(mul_f32x2(mul_f32x2(pack_f32x2(a[c], b[c]), wy0p), wxp), t00, t01);
                unpack_f32x2(mul_f32x2(mul_f32x2(pack_f32x2(c2[c], d[c]), wy1p), wxp), t10, t11);
                v[c] = __fadd_rn(__fadd_rn(__fadd_rn(t00, t01), t10), t11);
            }
        }
        else
        {
#pragma unroll
            for (int c = 0; c < 3; ++c) v[c] = blend4(a[c], b[c], c2[c], d[c], wx0s, wx1s, wy0s, wy1s);
        }
    }
    if (p.srcCast)
    {
#pragma unroll
        for (int c = 0; c < 3; ++c) v[c] = round_sat_u8(v[c]);
    }
    affine3(p, v);
}

template<class Row>
__device__ __forceinline__ void nearest_values(const ResizeKParams &p, Row r0, int o0, float (&v)[3])
{
    float a[3];
    tap3(r0 + o0, a);
#pragma unroll
    for (int c = 0; c < 3; ++c) v[c] = __fmul_rn(__fmul_rn(a[c], kTwo127), kTwo22);
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
// 32+L, 64+L), one for uint8 (lanes 0..23 write the 96 bytes as 24 words). `lanePtr` is the address of word `lane` of
// the warp's segment (the address of lane 0's pixel + 4*lane). All 32 lanes must call this.
template<int DK>
__device__ __forceinline__ void store_interleaved_warp(const float (&d)[3] /* destination channel order */,
                                                       uint8_t *lanePtr, int lane)
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
            reinterpret_cast<float *>(lanePtr)[32 * k] = c == 0 ? a : (c == 1 ? b : g);
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
            *reinterpret_cast<unsigned *>(lanePtr) = (lo >> (8 * off)) | (hi << (8 * (3 - off)));
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

// Adds to the bytes the current phase waits for, without arriving.
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ bool mbar_wait_addr(unsigned addr, unsigned parity, unsigned long long limitNs = kWaitLimitNs)
{
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

__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity,
                                          unsigned long long limitNs = kWaitLimitNs)
{
    return mbar_wait_addr(smem_addr(bar), parity, limitNs);
}

__device__ __forceinline__ void mbar_arrive_addr(unsigned addr)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
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
        raise_device_error(8u);
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

enum
{
    UNIT_PAD    = 0, // nothing to sample: the row lies outside the placed region
    UNIT_STAGED = 1, // rows are in the shared-memory slot
    UNIT_DIRECT = 2  // read the rows from global memory (unaligned image, or a segment larger than a slot)
};

// A work unit is up to kMaxUnitRows consecutive destination rows of one column chunk of one sample. Rows are grouped
// so that one ring slot (one barrier phase) moves 10 KB or more: below that the per-phase cost of the pipeline, not
// HBM, sets the pace.
constexpr int kMaxUnitRows = 4;

// One destination row of a unit (two 16-byte words; consumers read the second only for UNIT_DIRECT rows).
struct alignas(16) RowInfo
{
    int            mode;       // UNIT_* in bits 0-7; bit 8: the second tap row has its own segment (off0 + segBytes)
    int            off0;       // byte offset of the row's first segment inside the slot
    float          wy0s, wy1s; // vertical weights * 2^127
    const uint8_t *g0, *g1;    // tapped source rows in global memory (byte 0 of the row of the sub-view)
};

// What the producer tells the consumers about the unit staged in one ring slot: three 16-byte header words (the third
// is read only when cached column taps go stale) and one RowInfo per destination row.
struct alignas(16) UnitInfo
{
    // word 0
    int x0, x1;   // destination columns [x0, x1)
    int origin;   // source-row byte offset that offset 0 of a staged segment corresponds to (0 for UNIT_DIRECT)
    int flipRows; // bit 0: horizontal flip; bit 1: at least one row is sampled; bits 8..: number of rows
    // word 1
    long long dstRowOff; // of the unit's first row
    long long tapKey;    // units with equal keys have identical column taps (sample geometry, chunk, flip, origin)
    // word 2
    int   srcW;
    float scaleW;
    int   pad0, pad1;
    RowInfo row[kMaxUnitRows];
};

static_assert(sizeof(RowInfo) == 32 && sizeof(UnitInfo) == 48 + 32 * kMaxUnitRows, "UnitInfo layout is read by offset");

__device__ __forceinline__ uint4 lds128(unsigned addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ long long join64(unsigned lo, unsigned hi)
{
    return static_cast<long long>((static_cast<unsigned long long>(hi) << 32) | lo);
}

// Horizontal taps of one destination column: byte offsets of the left/right source pixel relative to the unit's
// origin (or one of the two codes below), the weights * 2^22 and the column's destination byte offset.
struct ColTap
{
    int       rel0, rel1;
    float     wx0s, wx1s;
    long long dstOff;
};

enum
{
    TAP_PAD  = -1, // column outside the placed region: gets the pad value
    TAP_NONE = -2  // the thread has no such column
};

template<int INTERP>
__device__ __forceinline__ ColTap make_tap(const ResizeKParams &p, int flipX, int srcW, float scaleW, int origin, int x)
{
    ColTap t;
    t.dstOff     = x * p.dPix;
    t.wx0s       = 0.f;
    t.wx1s       = 0.f;
    const int rx = x - p.dstX;
    if (rx < 0 || rx >= p.regionW)
    {
        t.rel0 = t.rel1 = TAP_PAD;
        return t;
    }
    const int dx = (flipX ? p.regionW - 1 - rx : rx) + p.cropX;
    if constexpr (INTERP == B200PP_INTERP_NEAREST)
    {
        t.rel0 = t.rel1 = 3 * nearest_tap(scaleW, dx, srcW) - origin;
    }
    else
    {
        int   s0, s1;
        float wx1;
        linear_tap(scaleW, dx, srcW, s0, s1, wx1);
        t.rel0 = 3 * s0 - origin;
        t.rel1 = 3 * s1 - origin;
        t.wx0s = __fmul_rn(__fsub_rn(1.0f, wx1), kTwo22);
        t.wx1s = __fmul_rn(wx1, kTwo22);
    }
    return t;
}

// Final values of one destination pixel from rows r0/r1 (addressed from the unit's origin).
template<int INTERP, bool PACKED = false, class Row>
__device__ __forceinline__ void pixel_values(const ResizeKParams &p, const PadValues &pv, const ColTap &t, Row r0, Row r1,
                                             float wy0s, float wy1s, float (&v)[3])
{
    if (t.rel0 < 0)
    {
#pragma unroll
        for (int c = 0; c < 3; ++c) v[c] = pv.v[c];
    }
    else if constexpr (INTERP == B200PP_INTERP_NEAREST)
        nearest_values(p, r0, t.rel0, v);
    else
        linear_values<PACKED>(p, r0, r1, t.rel0, t.rel1, t.wx0s, t.wx1s, wy0s, wy1s, v);
}

// How a thread of the row-walk kernel writes its pixels.
struct StorePlan
{
    ChanOff   co;
    bool      reversed; // channel order reversed
    long long ilAdj;    // interleaved destinations: from a lane's pixel address to the word(s) it writes in the
                        // transposed warp store (-8*lane for float32, +lane for uint8)
};

// The cached columns of one row (row-walk kernel): taps, validity and the choice of store were settled when the cache
// was filled.
template<int INTERP, int DK, int KC, bool IL, class Row>
__device__ __forceinline__ void consume_cached(const ResizeKParams &p, const StorePlan &plan, const PadValues &pv, Row r0,
                                               Row r1, float wy0s, float wy1s, uint8_t *dstRow, const ColTap (&cache)[KC],
                                               unsigned fastMask, int lane)
{
#pragma unroll
    for (int k = 0; k < KC; ++k)
    {
        float v[3];
        // planar destinations: the blend's products as packed multiplies (3 % on an L2-resident batch, nothing lost elsewhere);
        // the interleaved variants, already spilling at the kernel's 40 registers, keep the scalar form
        pixel_values<INTERP, !IL>(p, pv, cache[k], r0, r1, wy0s, wy1s, v);
        uint8_t *pix = dstRow + cache[k].dstOff;
        if constexpr (IL && DK != DST_F16)
        {
            if (fastMask & (1u << k)) // uniform across the warp
            {
                const float d[3] = {plan.reversed ? v[2] : v[0], v[1], plan.reversed ? v[0] : v[2]};
                store_interleaved_warp<DK>(d, pix + plan.ilAdj, lane);
                continue;
            }
        }
        if (cache[k].rel0 != TAP_NONE)
            store_pixel<DK>(v, plan.co, pix);
    }
}

// ------------------------------------------------------------------------------------------------ quads
//
// A consumer thread of the staged kernel produces four adjacent destination pixels of one row (a quad): the per-row
// and per-unit bookkeeping is shared by four pixels, and the twelve finished values leave as vectors -- one 4-element
// store per channel into planar destinations, three into interleaved ones -- with no cross-lane traffic.

// Horizontal taps of a quad. rel0[i]: byte offset of column i's left source pixel relative to the unit's origin, or
// TAP_PAD / TAP_NONE; the right source pixel is the same one or the next (bit i of `flags`). Bit 8 of `flags`: all
// four columns exist.
struct QuadTaps
{
    int       rel0[4];
    float     wx0s[4], wx1s[4]; // horizontal weights * 2^22
    unsigned  flags;
    long long dstOff; // destination byte offset of column 0 within the row
};

constexpr unsigned kQuadFull = 0x100u;

template<int INTERP>
__device__ __forceinline__ void make_quad(const ResizeKParams &p, int flipX, int srcW, float scaleW, int origin, int xq,
                                          int x1, QuadTaps &q)
{
    q.dstOff = xq * p.dPix;
    q.flags  = xq + 3 < x1 ? kQuadFull : 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        if (xq + i < x1)
        {
            const ColTap t = make_tap<INTERP>(p, flipX, srcW, scaleW, origin, xq + i);
            q.rel0[i]      = t.rel0;
            q.wx0s[i]      = t.wx0s;
            q.wx1s[i]      = t.wx1s;
            if (t.rel1 != t.rel0)
                q.flags |= 1u << i;
        }
        else
        {
            q.rel0[i] = TAP_NONE;
            q.wx0s[i] = q.wx1s[i] = 0.f;
        }
    }
}

// Taps of a quad in a row that is all padding: only validity and the destination offset matter.
__device__ __forceinline__ void make_pad_quad(const ResizeKParams &p, int xq, int x1, QuadTaps &q)
{
    q.dstOff = xq * p.dPix;
    q.flags  = xq + 3 < x1 ? kQuadFull : 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        q.rel0[i] = xq + i < x1 ? TAP_PAD : TAP_NONE;
        q.wx0s[i] = q.wx1s[i] = 0.f;
    }
}

// The finished values of the four pixels of a quad: v[i][c], c = source channel.
template<int INTERP, class Row>
__device__ __forceinline__ void quad_values(const ResizeKParams &p, const PadValues &pv, const QuadTaps &q, Row r0, Row r1,
                                            float wy0s, float wy1s, float (&v)[4][3])
{
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        if (q.rel0[i] < 0)
        {
#pragma unroll
            for (int c = 0; c < 3; ++c) v[i][c] = pv.v[c];
        }
        else if constexpr (INTERP == B200PP_INTERP_NEAREST)
            nearest_values(p, r0, q.rel0[i], v[i]);
        else
            linear_values(p, r0, r1, q.rel0[i], q.rel0[i] + ((q.flags >> i) & 1u ? 3 : 0), q.wx0s[i], q.wx1s[i], wy0s, wy1s,
                          v[i]);
    }
}

// Four finished values as one vector of the destination element type; `dst` is aligned to the vector size.
template<int DK>
__device__ __forceinline__ void store_vec4(uint8_t *dst, float a, float b, float c, float d)
{
    if constexpr (DK == DST_F32)
    {
        *reinterpret_cast<float4 *>(dst) = make_float4(a, b, c, d);
    }
    else if constexpr (DK == DST_F16)
    {
        const __half2 lo = __halves2half2(__float2half_rn(a), __float2half_rn(b));
        const __half2 hi = __halves2half2(__float2half_rn(c), __float2half_rn(d));
        uint2         w;
        w.x = *reinterpret_cast<const unsigned *>(&lo);
        w.y = *reinterpret_cast<const unsigned *>(&hi);
        *reinterpret_cast<uint2 *>(dst) = w;
    }
    else
    {
        // round-half-even + clamp leaves the byte in bits 0-7 of each sum; two byte permutes gather the four
        const unsigned ua = __float_as_uint(__fadd_rn(fminf(fmaxf(a, 0.0f), 255.0f), kRound));
        const unsigned ub = __float_as_uint(__fadd_rn(fminf(fmaxf(b, 0.0f), 255.0f), kRound));
        const unsigned uc = __float_as_uint(__fadd_rn(fminf(fmaxf(c, 0.0f), 255.0f), kRound));
        const unsigned ud = __float_as_uint(__fadd_rn(fminf(fmaxf(d, 0.0f), 255.0f), kRound));
        *reinterpret_cast<unsigned *>(dst) = __byte_perm(__byte_perm(ua, ub, 0x0040), __byte_perm(uc, ud, 0x0040), 0x5410);
    }
}

template<int DK>
__device__ __forceinline__ constexpr int elem_bytes()
{
    return DK == DST_F32 ? 4 : (DK == DST_F16 ? 2 : 1);
}

// How a consumer thread writes its quads.
struct QuadStore
{
    ChanOff co;
    bool    reversed;  // channel order reversed
    bool    planarVec; // channels are planes whose distance keeps vector alignment, pixels of a row are adjacent
};

// Writes a quad. IL: the destination has the three channels of a pixel adjacent (twelve consecutive elements).
template<int DK, bool IL>
__device__ __forceinline__ void store_quad(const ResizeKParams &p, const QuadStore &qs, const QuadTaps &q,
                                           const float (&v)[4][3], uint8_t *dstRow)
{
    constexpr int      kVec = 4 * elem_bytes<DK>();
    uint8_t           *base = dstRow + q.dstOff;
    const bool         aligned = (q.flags & kQuadFull) && (reinterpret_cast<unsigned long long>(base) & (kVec - 1)) == 0;
    if constexpr (IL)
    {
        if (aligned)
        {
            // destination order: pixel-major, channel-minor
            float e[12];
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                e[3 * i + 0] = qs.reversed ? v[i][2] : v[i][0];
                e[3 * i + 1] = v[i][1];
                e[3 * i + 2] = qs.reversed ? v[i][0] : v[i][2];
            }
#pragma unroll
            for (int k = 0; k < 3; ++k) store_vec4<DK>(base + k * kVec, e[4 * k], e[4 * k + 1], e[4 * k + 2], e[4 * k + 3]);
            return;
        }
    }
    else
    {
        if (aligned && qs.planarVec)
        {
#pragma unroll
            for (int c = 0; c < 3; ++c) store_vec4<DK>(base + qs.co.c[c], v[0][c], v[1][c], v[2][c], v[3][c]);
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (q.rel0[i] != TAP_NONE)
            store_pixel<DK>(v[i], qs.co, base + i * p.dPix);
}

// A unit as the producer stages it: the description the consumers get, plus what the copies need.
struct alignas(16) Staged
{
    UnitInfo  info;
    long long colOff;  // from byte 0 of a tapped source row to the 16-byte aligned start of the copied span
    unsigned  nb;      // bytes per copied row segment
    unsigned  txBytes; // bytes all copies of the unit deliver
};

static_assert(sizeof(Staged) == sizeof(UnitInfo) + 16, "Staged tail is read as one 16-byte word");

__device__ __forceinline__ void sts128(unsigned addr, uint4 v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Everything about work unit `u`: which sample, rows and columns, what they tap and where the tapped bytes lie.
template<int INTERP>
__device__ __forceinline__ void describe_unit(const ResizeKParams &p, const StagedCfg &cfg, long long u, bool perSampleTaps,
                                              int unitsPerSample, Staged &out)
{
    // 64-bit division is a long subroutine; launches of fewer than 2^31 units (all but absurd ones) do without
    const int  n     = u < 0x7fffffffll ? static_cast<int>(static_cast<unsigned>(u) / static_cast<unsigned>(unitsPerSample))
                                         : static_cast<int>(u / unitsPerSample);
    const int  rem   = static_cast<int>(u - static_cast<long long>(n) * unitsPerSample);
    const int  yg    = rem / cfg.chunksPerRow;
    const int  chunk = rem - yg * cfg.chunksPerRow;
    const Geom g     = load_geom(p, n);
    const bool aligned
        = ((reinterpret_cast<unsigned long long>(g.image) | static_cast<unsigned long long>(g.pitch)) & 15ull) == 0;

    const int  y0    = yg * cfg.unitRows;
    const int  nRows = min(cfg.unitRows, p.dstH - y0);
    const int  x0    = chunk * cfg.chunkCols;
    const int  x1    = min(x0 + cfg.chunkCols, p.dstW);
    const int  flipX = (g.flip == 1 || g.flip == -1);
    const bool flipY = (g.flip == 0 || g.flip == -1);
    long long  tapKey = (((perSampleTaps ? static_cast<long long>(n) + 1 : 0) * cfg.chunksPerRow + chunk) * 2 + flipX) * 32;
    int        unitMode = UNIT_PAD, origin = 0;
    long long  colOff = 0;
    unsigned   nb     = 0;

    const int rx0 = max(x0 - p.dstX, 0);
    const int rx1 = min(x1 - p.dstX, p.regionW) - 1; // inclusive
    if (rx1 >= rx0)
    {
        const int dlo = (flipX ? p.regionW - 1 - rx1 : rx0) + p.cropX;
        const int dhi = (flipX ? p.regionW - 1 - rx0 : rx1) + p.cropX;
        int       sxmin, sxmax;
        if constexpr (INTERP == B200PP_INTERP_NEAREST)
        {
            sxmin = nearest_tap(g.scaleW, dlo, g.w);
            sxmax = nearest_tap(g.scaleW, dhi, g.w);
        }
        else
        {
            float w;
            int   t;
            linear_tap(g.scaleW, dlo, g.w, sxmin, t, w);
            linear_tap(g.scaleW, dhi, g.w, t, sxmax, w);
        }
        // with a 16-byte aligned image and pitch the low address bits are the same in every row
        const unsigned long long a0 = reinterpret_cast<unsigned long long>(g.base) + 3ull * sxmin;
        const unsigned long long a1 = reinterpret_cast<unsigned long long>(g.base) + 3ull * (sxmax + 1);
        colOff                      = 3ll * sxmin - static_cast<long long>(a0 & 15ull);
        nb                          = static_cast<unsigned>(((a1 + 15ull) & ~15ull) - (a0 & ~15ull));
        if (!aligned || nb > static_cast<unsigned>(cfg.segBytes))
        {
            unitMode = UNIT_DIRECT;
        }
        else
        {
            unitMode = UNIT_STAGED;
            origin   = static_cast<int>(colOff);
            // cached taps are relative to the origin, whose alignment part is not implied by the geometry
            tapKey += 16 + static_cast<long long>(a0 & 15ull);
        }
    }

    const int      rowBytes  = cfg.rowsPerStage * cfg.segBytes;
    int            sampled   = 0;
    unsigned       txBytes   = 0;
    for (int r = 0; r < nRows; ++r)
    {
        RowInfo   ri{};
        const int ry = y0 + r - p.dstY;
        ri.mode      = UNIT_PAD;
        ri.off0      = r * rowBytes;
        if (unitMode != UNIT_PAD && ry >= 0 && ry < p.regionH)
        {
            const int dy = (flipY ? p.regionH - 1 - ry : ry) + p.cropY;
            int       sy0, sy1;
            bool      twoRow = false;
            if constexpr (INTERP == B200PP_INTERP_NEAREST)
            {
                sy0 = sy1 = nearest_tap(g.scaleH, dy, g.h);
            }
            else
            {
                float wy1;
                linear_tap(g.scaleH, dy, g.h, sy0, sy1, wy1);
                ri.wy0s = __fmul_rn(__fsub_rn(1.0f, wy1), kTwo127);
                ri.wy1s = __fmul_rn(wy1, kTwo127);
                twoRow  = sy0 != sy1 && ri.wy1s != 0.0f; // a lower row of weight zero is never read
            }
            ri.g0   = g.base + sy0 * g.pitch;
            ri.g1   = g.base + sy1 * g.pitch;
            ri.mode = unitMode | (twoRow && unitMode == UNIT_STAGED ? 0x100 : 0);
            sampled = 2;
            if (unitMode == UNIT_STAGED)
                txBytes += twoRow ? 2u * nb : nb;
        }
        out.info.row[r] = ri;
    }
    out.info.x0        = x0;
    out.info.x1        = x1;
    out.info.origin    = origin;
    out.info.flipRows  = flipX | sampled | (nRows << 8);
    out.info.dstRowOff = n * p.dSample + y0 * p.dRow;
    out.info.tapKey    = tapKey;
    out.info.srcW      = g.w;
    out.info.scaleW    = g.scaleW;
    out.colOff         = colOff;
    out.nb             = nb;
    out.txBytes        = txBytes;
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
        if (blockUnits == 1)
            return first + k * stride;
        const long long j = k / blockUnits;
        return first + j * stride + (k - j * blockUnits);
    }
};

// IL: the destination is interleaved (three adjacent channels per pixel) and is written with the transposing store.
template<int INTERP, int DK, bool IL>
__global__ void __launch_bounds__(288, INTERP == B200PP_INTERP_NEAREST ? 3 : 2) resize_staged_kernel(const ResizeKParams p, const StagedCfg cfg)
{
    extern __shared__ __align__(128) unsigned char smemRaw[];

    // Shared memory: the ring of cfg.stages slots (each holds the row segments of one unit), then per slot a UnitInfo
    // and a full / empty barrier pair, then the producer's staging array.
    const int           S         = cfg.stages;
    const long long     slotBytes = static_cast<long long>(cfg.unitRows) * cfg.rowsPerStage * cfg.segBytes;
    unsigned char      *ring      = smemRaw;
    UnitInfo           *infos     = reinterpret_cast<UnitInfo *>(ring + S * slotBytes);
    unsigned long long *full      = reinterpret_cast<unsigned long long *>(infos + S);
    unsigned long long *empty     = full + S;

    const int consumerThreads = blockDim.x - kProducerThreads;
    const int consumerWarps   = consumerThreads / 32;
    const int lane            = threadIdx.x & 31;

    // A ring slot must always be consumed by the same team (see the host code): refuse any other shape.
    if (cfg.teams < 1 || S % cfg.teams != 0 || consumerWarps % cfg.teams != 0
        || (consumerWarps / cfg.teams) % cfg.colBlocks != 0)
    {
        if (threadIdx.x == 0)
            raise_device_error(16u);
        return;
    }

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < S; ++s)
        {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], consumerWarps / cfg.teams); // a unit is consumed by one team of warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const UnitWalk walk(cfg);

    if (threadIdx.x < kProducerThreads)
    {
        // ===================================================================== producer warp
        // Phase A: the 32 lanes describe 32 consecutive units side by side (sample descriptor, column span, row taps,
        // copy addresses) into a staging array in shared memory. Phase B: unit by unit, in order, lane 0 claims a ring
        // slot, eleven lanes move the description into the slot's UnitInfo and up to eight lanes issue one bulk copy
        // each; lane 0 then arrives on the slot's barrier.
        Staged    *staging        = reinterpret_cast<Staged *>(empty + S);
        const bool perSampleTaps  = p.list != nullptr || p.roi != nullptr;
        const int  groupsPerImage = (p.dstH + cfg.unitRows - 1) / cfg.unitRows;
        const int  unitsPerSample = groupsPerImage * cfg.chunksPerRow;
        int        s           = 0;
        unsigned   emptyParity = 1; // phase the consumers complete when they release the slot's previous use
        bool       failed      = false;
        long long  issued      = 0;

        for (long long kb = 0; kb < walk.count && !failed; kb += 32)
        {
            const long long k = kb + lane;
            if (k < walk.count)
                describe_unit<INTERP>(p, cfg, walk.unit(k), perSampleTaps, unitsPerSample, staging[lane]);
            __syncwarp();

            const int batch = static_cast<int>(min(32ll, walk.count - kb));
            for (int j = 0; j < batch; ++j)
            {
                // Everything the publication needs is read from the staging array before the wait for the slot, so
                // that the copies go out as soon as the slot is free.
                const unsigned from = smem_addr(&staging[j]), to = smem_addr(&infos[s]);
                const uint4    word = lds128(from + 16u * min(lane, static_cast<int>(sizeof(Staged) / 16) - 1));
                const int      r = (lane >> 1) & (kMaxUnitRows - 1), second = lane & 1;
                const uint4    ra   = lds128(from + 48u + 32u * r);
                const uint4    rb   = lds128(from + 64u + 32u * r);
                const uint4    tail = lds128(from + static_cast<unsigned>(sizeof(UnitInfo)));
                const int      rows = static_cast<int>(lds128(from).w >> 8);
                // lane 2r copies the first tapped row of destination row r, lane 2r+1 the second
                const bool copies = lane < 2 * kMaxUnitRows && r < rows && (ra.x & 0xffu) == UNIT_STAGED
                                 && (!second || (ra.x & 0x100u));
                const void *src = reinterpret_cast<const void *>((second ? join64(rb.z, rb.w) : join64(rb.x, rb.y))
                                                                 + join64(tail.x, tail.y));
                unsigned char *dstSeg = ring + s * slotBytes + ra.y + (second ? cfg.segBytes : 0);

                bool bad = false;
                if (lane == 0 && kb + j >= S && !mbar_wait(&empty[s], emptyParity))
                {
                    raise_device_error(2u);
                    bad = true;
                }
                if (__any_sync(0xffffffffu, bad))
                {
                    failed = true;
                    break;
                }
                if (lane < static_cast<int>(sizeof(UnitInfo) / 16))
                    sts128(to + 16u * lane, word);
                if (copies)
                    bulk_load(dstSeg, src, tail.z, &full[s]);
                __syncwarp();
                // One arrival carrying the byte count of all the unit's copies: the phase completes once it and the
                // bytes are in (bytes that land before it only run the transaction count negative for a moment).
                if (lane == 0)
                {
                    if (tail.w)
                        mbar_arrive_expect_tx(&full[s], tail.w);
                    else
                        mbar_arrive(&full[s]);
                }
                ++issued;
                if (++s == S)
                {
                    s = 0;
                    emptyParity ^= 1u;
                }
            }
            __syncwarp();
        }
        if (failed && lane == 0)
        {
            // Consumers have stopped releasing slots. Give the copies already issued a bounded time to land before
            // the CTA's shared memory goes away.
            for (long long j = (issued > S ? issued - S : 0); j < issued; ++j)
                if (!mbar_wait(&full[j % S], static_cast<unsigned>((j / S) & 1)))
                {
                    raise_device_error(4u);
                    break;
                }
        }
        return;
    }

    // ========================================================================= consumers
    // The consumer warps form cfg.teams teams; team t consumes units t, t + teams, ... of this CTA, so that several
    // ring slots are worked on at once. Within a team, warp w works on column block w % colBlocks (128 columns, four
    // per lane) of the unit's rows w / colBlocks, + teamWarps/colBlocks, ... A unit's header arrives in two vector loads
    // and each row in one; the taps of the thread's four columns stay in registers while consecutive units share a tap
    // key, which for a dense batch is the whole launch.
    const int       teamWarps = consumerWarps / cfg.teams;
    const int       cwarp     = (threadIdx.x - kProducerThreads) >> 5;
    const int       team      = cwarp / teamWarps;
    const int       warp      = cwarp - team * teamWarps;
    const int       cb        = warp % cfg.colBlocks;
    const int       rowLane   = warp / cfg.colBlocks;
    const int       rowStep   = teamWarps / cfg.colBlocks;
    const PadValues pv      = pad_values(p);
    QuadStore       qs;
    qs.co        = chan_offsets(p);
    qs.reversed  = p.mapC[0] == 2;
    qs.planarVec = p.dPix == elem_bytes<DK>() && (p.dChan & (4 * elem_bytes<DK>() - 1)) == 0;

    const unsigned ringA = smem_addr(ring), infoA = smem_addr(infos), fullA = smem_addr(full), emptyA = smem_addr(empty);
    const unsigned slotStep = static_cast<unsigned>(slotBytes);
    const unsigned segStep  = static_cast<unsigned>(cfg.segBytes);

    long long cachedKey  = -1;
    int       s          = team % S; // slot of unit `team`
    unsigned  fullParity = static_cast<unsigned>(team / S) & 1u;
    QuadTaps  quad;
    for (long long k = team; k < walk.count; k += cfg.teams)
    {
        if (!mbar_wait_addr(fullA + 8u * s, fullParity))
        {
            raise_device_error(1u);
            return;
        }
        const unsigned infoAddr = infoA + static_cast<unsigned>(s) * static_cast<unsigned>(sizeof(UnitInfo));
        const unsigned slotA    = ringA + static_cast<unsigned>(s) * slotStep;
        const uint4    w0       = lds128(infoAddr);
        const uint4    w1       = lds128(infoAddr + 16);
        const int      x1 = static_cast<int>(w0.y), nRows = static_cast<int>(w0.w >> 8);
        const int      xq = static_cast<int>(w0.x) + 128 * cb + 4 * lane; // first column of this thread's quad
        uint8_t       *dstBase = p.dst + join64(w1.x, w1.y);

        if (w0.w & 2u) // some row is sampled: the cached taps must match this unit
        {
            const long long key = join64(w1.z, w1.w);
            if (key != cachedKey) // uniform across the CTA
            {
                cachedKey      = key;
                const uint4 w2 = lds128(infoAddr + 32);
                make_quad<INTERP>(p, static_cast<int>(w0.w & 1u), static_cast<int>(w2.x), __uint_as_float(w2.y),
                                  static_cast<int>(w0.z), xq, x1, quad);
            }
        }

        for (int r = rowLane; r < nRows; r += rowStep)
        {
            const uint4 ra     = lds128(infoAddr + 48u + 32u * r);
            const int   mode   = static_cast<int>(ra.x & 0xffu);
            uint8_t    *dstRow = dstBase + r * p.dRow;
            float       v[4][3];
            if (mode == UNIT_PAD)
            {
                QuadTaps padQuad;
                make_pad_quad(p, xq, x1, padQuad);
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 3; ++c) v[i][c] = pv.v[c];
                store_quad<DK, IL>(p, qs, padQuad, v, dstRow);
                continue;
            }
            const float wy0s = __uint_as_float(ra.z), wy1s = __uint_as_float(ra.w);
            if (mode == UNIT_STAGED)
            {
                const SmemRow r0{slotA + ra.y};
                const SmemRow r1{r0.a + ((ra.x & 0x100u) ? segStep : 0u)};
                if (cfg.probe) // memory-only run: every copy and every store of the real launch, no taps, no arithmetic
                {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int c = 0; c < 3; ++c) v[i][c] = pv.v[c];
                }
                else
                    quad_values<INTERP>(p, pv, quad, r0, r1, wy0s, wy1s, v);
            }
            else
            {
                const uint4    rb = lds128(infoAddr + 64u + 32u * r);
                const uint8_t *g0 = reinterpret_cast<const uint8_t *>(join64(rb.x, rb.y));
                const uint8_t *g1 = reinterpret_cast<const uint8_t *>(join64(rb.z, rb.w));
                quad_values<INTERP>(p, pv, quad, g0, g1, wy0s, wy1s, v);
            }
            store_quad<DK, IL>(p, qs, quad, v, dstRow);
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive_addr(emptyA + 8u * s);
        s += cfg.teams;
        while (s >= S)
        {
            s -= S;
            fullParity ^= 1u;
        }
    }
}

// ------------------------------------------------------------------------------------------------ row-walk kernel
//
// One CTA = up to blockDim.x destination columns x `rowsPerCta` consecutive destination rows of one sample. A thread
// keeps the taps of its column in registers and walks down the rows, reading the tapped bytes straight from global
// memory: a warp's 32 columns touch one short contiguous span per source row, which the L1 fetches sector by sector,
// once. No pipeline machinery, so the fewest instructions per destination pixel of the three kernels; it wins where the
// staged kernel is bound by instruction issue rather than by HBM (small element types, nearest neighbour).
constexpr int kWalkRowsMax = 16;

__device__ __forceinline__ void prefetch_l2(const void *p)
{
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

struct alignas(16) WalkRow
{
    long long off0, off1; // byte offsets of the two tapped rows from the first byte of the sample's (sub-)image
    float     wy0s, wy1s; // vertical weights * 2^127
    int       mode;       // UNIT_PAD or UNIT_DIRECT
    int       pad;
};

template<int INTERP, int DK, bool IL>
__global__ void __launch_bounds__(256, 6) resize_rowwalk_kernel(const ResizeKParams p, const int rowsPerCta, const int chunksPerRow)
{
    __shared__ WalkRow rows[kWalkRowsMax];

    const int chunk = blockIdx.x % chunksPerRow;
    const int y0    = (blockIdx.x / chunksPerRow) * rowsPerCta;
    const int nRows = min(rowsPerCta, p.dstH - y0);
    const int lane  = threadIdx.x & 31;
    const int x     = chunk * blockDim.x + threadIdx.x;
    const bool valid = x < p.dstW;

    const PadValues pv = pad_values(p);
    StorePlan       plan;
    plan.co       = chan_offsets(p);
    plan.reversed = p.mapC[0] == 2;
    plan.ilAdj    = DK == DST_F32 ? -8 * lane : lane;
    const unsigned fullMask = __all_sync(0xffffffffu, valid) ? 1u : 0u;

    for (int n = blockIdx.y; n < p.numSamples; n += gridDim.y)
    {
        const Geom g     = load_geom(p, n);
        const int  flipX = (g.flip == 1 || g.flip == -1);
        if (threadIdx.x < nRows)
        {
            WalkRow   wr{};
            const int ry = y0 + static_cast<int>(threadIdx.x) - p.dstY;
            wr.mode      = UNIT_PAD;
            if (ry >= 0 && ry < p.regionH)
            {
                const int dy = ((g.flip == 0 || g.flip == -1) ? p.regionH - 1 - ry : ry) + p.cropY;
                int       sy0, sy1;
                if constexpr (INTERP == B200PP_INTERP_NEAREST)
                {
                    sy0 = sy1 = nearest_tap(g.scaleH, dy, g.h);
                }
                else
                {
                    float wy1;
                    linear_tap(g.scaleH, dy, g.h, sy0, sy1, wy1);
                    wr.wy0s = __fmul_rn(__fsub_rn(1.0f, wy1), kTwo127);
                    wr.wy1s = __fmul_rn(wy1, kTwo127);
                }
                wr.off0 = sy0 * g.pitch;
                wr.off1 = sy1 * g.pitch;
                wr.mode = UNIT_DIRECT;
            }
            rows[threadIdx.x] = wr;
        }
        ColTap cache[1];
        if (valid)
            cache[0] = make_tap<INTERP>(p, flipX, g.w, g.scaleW, 0, x);
        else
        {
            cache[0].rel0 = cache[0].rel1 = TAP_NONE;
            cache[0].wx0s = cache[0].wx1s = 0.f;
            cache[0].dstOff               = 0;
        }
        __syncthreads();

        // L2 is asked for the NEXT row's tapped sectors before this row is blended: the next row's one-byte loads then find
        // them at L2 latency instead of HBM latency, at no cost in registers (holding two rows' bytes in flight instead cost a
        // CTA per SM and was slower; asking two or three rows ahead was slower too). Only where consecutive destination rows
        // tap different source rows (vertical reduction of 1.5 or more): elsewhere the next row's sectors are mostly this
        // row's, and the two extra requests per pixel only cost issue slots (48.2 us without this condition). Measured on a
        // 128-image batch of random rectangles: 53.6 -> 43.6 us; not slower where the whole source already sits in L2.
        const bool prefetch = g.scaleH >= 1.5f && cache[0].rel0 >= 0;
        uint8_t   *dstRow   = p.dst + n * p.dSample + y0 * p.dRow;
        WalkRow    wr       = rows[0];
        for (int r = 0; r < nRows; ++r, dstRow += p.dRow)
        {
            WalkRow nx = wr;
            if (r + 1 < nRows)
            {
                nx = rows[r + 1];
                if (prefetch && nx.mode != UNIT_PAD)
                {
                    prefetch_l2(g.base + nx.off0 + cache[0].rel0);
                    if constexpr (INTERP == B200PP_INTERP_LINEAR)
                        prefetch_l2(g.base + nx.off1 + cache[0].rel0);
                }
            }
            if (wr.mode == UNIT_PAD)
            {
                if (valid)
                    store_pixel<DK>(pv.v, plan.co, dstRow + cache[0].dstOff);
            }
            else
            {
                unsigned fastMask = 0;
                if constexpr (IL && DK != DST_F16)
                {
                    // the transposing store needs word-aligned warp segments; lane 0 of every warp sits 32*m columns from 0
                    fastMask = (reinterpret_cast<unsigned long long>(dstRow) & 3ull) == 0 ? fullMask : 0u;
                }
                consume_cached<INTERP, DK, 1, IL>(p, plan, pv, g.base + wr.off0, g.base + wr.off1, wr.wy0s, wr.wy1s, dstRow, cache,
                                                  fastMask, lane);
            }
            wr = nx;
        }
        __syncthreads();
    }
}

} // namespace b200pp

#endif
