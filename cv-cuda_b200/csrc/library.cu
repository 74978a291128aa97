// Host side of the plain-C launch layer: argument validation, kernel selection and launch.
// The single translation unit that contains all device code of the library.
#include "border_kernels.cuh"
#include "convert_kernels.cuh"
#include "normalize_kernels.cuh"
#include "plain_resize_kernels.cuh"
#include "reformat_kernels.cuh"
#include "resize_kernels.cuh"
#include "slice_kernels.cuh"

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

namespace b200pp {

// ------------------------------------------------------------------------------------------------ error state

static thread_local char t_lastError[512] = "";

int fail(int status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_lastError, sizeof(t_lastError), fmt, ap);
    va_end(ap);
    return status;
}

static std::atomic<int>      g_kernelPath{0};
static std::atomic<uint64_t> g_launchCount{0};

static int check_launch(const char *what)
{
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess)
    {
        cudaGetLastError();
        return fail(B200PP_ERROR_INTERNAL, "%s: kernel launch failed: %s", what, cudaGetErrorString(e));
    }
    g_launchCount.fetch_add(1, std::memory_order_relaxed);
    return B200PP_SUCCESS;
}

static int elem_size(int dtype)
{
    switch (dtype)
    {
    case B200PP_U8:
    case B200PP_S8:
        return 1;
    case B200PP_U16:
    case B200PP_S16:
    case B200PP_F16:
        return 2;
    case B200PP_U32:
    case B200PP_S32:
    case B200PP_F32:
        return 4;
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------ device facts

struct DeviceFacts
{
    int                    smCount      = 0;
    int                    maxSmemOptin = 0;
    volatile unsigned int *errorMirror  = nullptr; // host view of the device error word (see raise_device_error)
};

static const DeviceFacts &device_facts(int dev)
{
    static std::mutex                 mu;
    static std::map<int, DeviceFacts> cache;
    std::lock_guard<std::mutex>       lock(mu);
    auto                              it = cache.find(dev);
    if (it == cache.end())
    {
        DeviceFacts f;
        cudaDeviceGetAttribute(&f.smCount, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&f.maxSmemOptin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        // One page-locked, device-mapped word per device, made the first time the library is used on it (the one thing this
        // library ever allocates on its own; it lives until the process ends). Without it the error word is still there
        // for b200ppReadDeviceError, only nothing reports it unasked.
        unsigned int *host = nullptr, *mapped = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void **>(&host), sizeof(unsigned int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess)
        {
            *host = 0;
            if (cudaHostGetDevicePointer(reinterpret_cast<void **>(&mapped), host, 0) == cudaSuccess
                && cudaMemcpyToSymbol(g_deviceErrorMirror, &mapped, sizeof(mapped)) == cudaSuccess)
                f.errorMirror = host;
            else
                cudaFreeHost(host);
        }
        cudaGetLastError();
        it = cache.emplace(dev, f).first;
    }
    return it->second;
}

// A kernel of an earlier call on the current device gave up on one of its bounded waits: say so now (no synchronisation;
// the word is page-locked host memory the kernel wrote through). It stays set until b200ppReadDeviceError clears it.
static int pending_device_error()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess)
    {
        cudaGetLastError();
        return B200PP_SUCCESS; // no device yet: the launch below reports that
    }
    const volatile unsigned int *w = device_facts(dev).errorMirror;
    if (w && *w != 0)
        return fail(B200PP_ERROR_INTERNAL,
                    "An earlier launch on device %d gave up on a bounded internal wait (error word 0x%x); its output is "
                    "incomplete. b200ppReadDeviceError reads and clears the word",
                    dev, *w);
    return B200PP_SUCCESS;
}

// Resident CTAs per SM of one staged-kernel instantiation for a block size and dynamic shared-memory size. The first
// use of a kernel on a device raises its dynamic shared-memory limit to the device maximum, once, so that launches with
// different ring sizes never lower it again.
template<typename K>
static int staged_occupancy(K kernel, int dev, int kernelId, int block, int smemBytes, int maxSmemOptin)
{
    static std::mutex                                     mu;
    static std::map<std::tuple<int, int, int, int>, int> cache;
    static std::map<std::pair<int, int>, bool>           raised;
    std::lock_guard<std::mutex>                           lock(mu);
    auto rk = std::make_pair(dev, kernelId);
    if (raised.find(rk) == raised.end())
    {
        const bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, maxSmemOptin) == cudaSuccess;
        if (!ok)
            cudaGetLastError();
        raised[rk] = ok;
    }
    if (!raised[rk])
        return 0;
    auto key = std::make_tuple(dev, kernelId, block, smemBytes);
    auto it  = cache.find(key);
    if (it == cache.end())
    {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, block, smemBytes) != cudaSuccess)
        {
            cudaGetLastError();
            n = 0;
        }
        it = cache.emplace(key, n).first;
    }
    return it->second;
}

// Launch-shape overrides for tuning runs, read once from the environment:
// B200PP_STAGES (ring depth), B200PP_MAX_CTAS_PER_SM (cap on resident CTAs per SM of the staged kernel) and
// B200PP_BLOCK_UNITS (consecutive units dealt to a CTA at a time), B200PP_MAX_CONSUMERS (consumer threads per CTA),
// B200PP_UNIT_ROWS (destination rows per work unit of the staged kernel), B200PP_WALK_ROWS (rows per CTA of the
// row-walk kernel), B200PP_PROBE (1: the staged kernel's consumers skip the taps and the arithmetic and store the pad
// value -- the launch then moves exactly the real launch's bytes and nothing else, which measures the floor of its copy and
// store pattern; results are meaningless).
struct Tuning
{
    int stages       = 0;
    int maxCtasPerSm = 0;
    int blockUnits   = 0;
    int maxConsumers = 0;
    int unitRows     = 0;
    int walkRows     = 0;
    int teams        = 0;
    int probe        = 0;
    int chunkCols    = 0;
};

static const Tuning &tuning()
{
    static const Tuning t = [] {
        Tuning      v;
        const char *s = getenv("B200PP_STAGES");
        const char *c = getenv("B200PP_MAX_CTAS_PER_SM");
        if (s)
            v.stages = atoi(s);
        if (c)
            v.maxCtasPerSm = atoi(c);
        if (const char *b = getenv("B200PP_BLOCK_UNITS"))
            v.blockUnits = atoi(b);
        if (const char *m = getenv("B200PP_MAX_CONSUMERS"))
            v.maxConsumers = atoi(m);
        if (const char *r = getenv("B200PP_UNIT_ROWS"))
            v.unitRows = atoi(r);
        if (const char *w = getenv("B200PP_WALK_ROWS"))
            v.walkRows = atoi(w);
        if (const char *t = getenv("B200PP_TEAMS"))
            v.teams = atoi(t);
        if (const char *pr = getenv("B200PP_PROBE"))
            v.probe = atoi(pr);
        if (const char *cc = getenv("B200PP_CHUNK_COLS"))
            v.chunkCols = atoi(cc);
        return v;
    }();
    return t;
}

// ------------------------------------------------------------------------------------------------ resize dispatch

template<int INTERP, int DK>
static int launch_resize_gather(const ResizeKParams &kp, cudaStream_t stream)
{
    dim3 block(32, 8);
    dim3 grid((kp.dstW + 31) / 32, (kp.dstH + 7) / 8, std::min(kp.numSamples, 32768));
    resize_gather_kernel<INTERP, DK><<<grid, block, 0, stream>>>(kp);
    return check_launch("ResizeCropConvertReformat (gather)");
}

template<int INTERP, int DK>
static int launch_resize_rowwalk(const ResizeKParams &kp, cudaStream_t stream)
{
    const int block  = std::min(256, (kp.dstW + 31) / 32 * 32);
    const int chunks = (kp.dstW + block - 1) / block;
    int       rows   = tuning().walkRows > 0 ? tuning().walkRows : 8;
    rows             = std::max(1, std::min({rows, kWalkRowsMax, kp.dstH}));
    const long long gx = static_cast<long long>(chunks) * ((kp.dstH + rows - 1) / rows);
    if (gx > 0x7fffffffll)
        return launch_resize_gather<INTERP, DK>(kp, stream);
    const int  elem = DK == DST_F32 ? 4 : (DK == DST_F16 ? 2 : 1);
    const bool il   = DK != DST_F16 && kp.dPix == 3 * elem && kp.dChan == elem;
    dim3       grid(static_cast<unsigned>(gx), static_cast<unsigned>(std::min(kp.numSamples, 65535)));
    if (il)
        resize_rowwalk_kernel<INTERP, DK, true><<<grid, block, 0, stream>>>(kp, rows, chunks);
    else
        resize_rowwalk_kernel<INTERP, DK, false><<<grid, block, 0, stream>>>(kp, rows, chunks);
    return check_launch("ResizeCropConvertReformat (row walk)");
}

// Returns 1 when the staged kernel was launched, 0 when it does not apply (caller falls back), <0 never.
template<int INTERP, int DK>
static int launch_resize_staged(const ResizeKParams &kp, int srcWBound, cudaStream_t stream, int *status)
{
    int dev = 0;
    cudaGetDevice(&dev);
    const DeviceFacts &facts = device_facts(dev);

    StagedCfg cfg{};
    cfg.rowsPerStage = INTERP == B200PP_INTERP_LINEAR ? 2 : 1;

    // Shared-memory bytes one staged source row may need for `cols` destination columns: the tapped span is at most
    // cols*srcW/resizeW + 2 pixels, plus alignment slack on both ends.
    auto seg_for = [&](int cols) {
        long long span = (static_cast<long long>(cols) * srcWBound + kp.resizeW - 1) / kp.resizeW + 3;
        span           = std::min<long long>(span, srcWBound);
        long long b    = span * 3 + 48; // 16 + 16 bytes of alignment slack, 16 for the word-wise tap reads
        return static_cast<int>((b + 127) / 128 * 128);
    };
    const int kMaxSeg = 32 * 1024;
    cfg.chunkCols     = kp.dstW;
    if (tuning().chunkCols >= 32)
        cfg.chunkCols = std::min(kp.dstW, (tuning().chunkCols + 3) / 4 * 4);
    // a consumer warp covers 128 columns (four per lane) and a CTA has at most eight consumer warps
    while (cfg.chunkCols > 32 && (cfg.chunkCols > 1024 || seg_for(cfg.chunkCols) > kMaxSeg))
        cfg.chunkCols = ((cfg.chunkCols + 1) / 2 + 3) / 4 * 4;
    cfg.segBytes     = std::min(seg_for(cfg.chunkCols), kMaxSeg);
    cfg.chunksPerRow = (kp.dstW + cfg.chunkCols - 1) / cfg.chunkCols;

    // Destination rows per unit: a ring slot (one barrier phase) should move 10 KB or more, about 20 KB where rows are
    // short. Measured on B200 with 5 KB row segments (1080p -> 224, nearest): 96 / 77 / 71 / 68 us at 1 / 2 / 3 / 4 rows.
    // Planar float32 output (the classification case) measured best with larger units and eight consumer warps:
    // 118.8 us against 121.1 us for 256 1080p images.
    const int  elemBytes  = DK == DST_F32 ? 4 : (DK == DST_F16 ? 2 : 1);
    const bool planarF32  = DK == DST_F32 && kp.dPix == elemBytes && cfg.chunkCols <= 256;
    const int  rowBytes   = cfg.segBytes * cfg.rowsPerStage;
    // Rows wider than 512 destination columns with linear interpolation (the letterbox case: 640 columns, five consumer warps
    // side by side, one row at a time): measured best with three rows per unit and three slots, 92.3 us against 96.6 us for
    // 64 1080p images into 640x640 (two rows, two slots); chunking such rows was slower at every size tried (109-184 us).
    const bool wideLinear = INTERP == B200PP_INTERP_LINEAR && cfg.chunkCols > 512;
    const int  unitTarget = (planarF32 ? 40 : (wideLinear ? 36 : 24)) * 1024;
    cfg.unitRows          = std::max(1, std::min({kMaxUnitRows, (unitTarget + rowBytes / 2) / rowBytes, kp.dstH}));
    if (tuning().unitRows > 0)
        cfg.unitRows = std::max(1, std::min({kMaxUnitRows, tuning().unitRows, kp.dstH}));
    cfg.totalUnits = static_cast<long long>(kp.numSamples) * ((kp.dstH + cfg.unitRows - 1) / cfg.unitRows) * cfg.chunksPerRow;

    const int stageBytes = rowBytes * cfg.unitRows;
    // About 30-40 KB of copies in flight per CTA (four CTAs per SM): measured best on B200; deeper rings were slower.
    cfg.stages           = std::max(wideLinear ? 3 : 2, std::min(8, (32 * 1024) / stageBytes));
    if (tuning().stages > 0)
        cfg.stages = std::max(2, std::min(16, tuning().stages));
    const int smemBytes  = cfg.stages * stageBytes + cfg.stages * (int)sizeof(UnitInfo) + cfg.stages * 16
                         + kProducerThreads * (int)sizeof(Staged) + 128;
    if (smemBytes > facts.maxSmemOptin)
        return 0;

    // Consumer warps: a team has one warp per 128-column block, times as many rows of a unit as fit; teams (each on
    // its own unit) fill the CTA up to its warp budget. The budget keeps four CTAs resident per SM for the linear
    // kernels (about 90 registers per thread) and three for the nearest ones (72).
    cfg.colBlocks          = (cfg.chunkCols + 127) / 128;
    const int budget       = INTERP == B200PP_INTERP_LINEAR && !planarF32 ? 4 : 8;
    const int maxWarps     = std::max(cfg.colBlocks, tuning().maxConsumers > 0 ? std::min(8, tuning().maxConsumers / 32) : budget);
    const int rowWarps     = std::max(1, std::min(cfg.unitRows, maxWarps / cfg.colBlocks));
    cfg.teams              = std::max(1, std::min(cfg.stages / 2, maxWarps / (cfg.colBlocks * rowWarps)));
    if (tuning().teams > 0)
        cfg.teams = std::max(1, std::min({cfg.stages, tuning().teams, 8 / (cfg.colBlocks * rowWarps)}));
    // A ring slot must always be consumed by the same team: a team that did not consume a slot's previous phase could
    // run two phases ahead of it, and a parity wait cannot tell those apart. So the team count divides the ring depth.
    while (cfg.stages % cfg.teams != 0) --cfg.teams;
    const int block        = kProducerThreads + 32 * cfg.colBlocks * rowWarps * cfg.teams;
    // interleaved destinations: the three channels of a pixel are adjacent
    const int  elem   = DK == DST_F32 ? 4 : (DK == DST_F16 ? 2 : 1);
    const bool il     = kp.dPix == 3 * elem && kp.dChan == elem;
    auto       kernel = il ? resize_staged_kernel<INTERP, DK, true> : resize_staged_kernel<INTERP, DK, false>;
    const int occ = staged_occupancy(kernel, dev, (INTERP * 4 + DK) * 2 + (il ? 1 : 0), block, smemBytes,
                                     facts.maxSmemOptin);
    if (occ <= 0)
        return 0;
    const int       perSm = tuning().maxCtasPerSm > 0 ? std::min(occ, tuning().maxCtasPerSm) : occ;
    const long long grid  = std::min<long long>(cfg.totalUnits, static_cast<long long>(facts.smCount) * perSm);
    // Dense batches: deal single units round-robin, so that all CTAs sweep neighbouring rows. Per-sample geometry
    // (image list or regions of interest): one contiguous range per CTA, so that column taps stay cached.
    const bool perSample = kp.list != nullptr || kp.roi != nullptr;
    cfg.blockUnits       = perSample ? (cfg.totalUnits + grid - 1) / grid : 1;
    if (tuning().blockUnits > 0)
        cfg.blockUnits = tuning().blockUnits;
    cfg.probe = tuning().probe != 0;
    kernel<<<static_cast<unsigned>(grid), block, smemBytes, stream>>>(kp, cfg);
    *status = check_launch("ResizeCropConvertReformat (staged)");
    return 1;
}

template<int INTERP, int DK>
static int run_resize(const ResizeKParams &kp, int srcWBound, cudaStream_t stream)
{
    const int path = g_kernelPath.load(std::memory_order_relaxed);
    // The staged kernel works on 128-column blocks of destination rows with vector stores; tiny outputs gain nothing.
    // It also fetches whole row segments: beyond a 32x horizontal reduction (96 source bytes per destination column)
    // the taps skip whole 32-byte sectors and the per-pixel gather moves fewer bytes.
    const bool sparseTaps = static_cast<long long>(srcWBound) > 32ll * kp.resizeW;
    // Batches with per-sample geometry (image lists, regions of interest) have short, uneven runs of units per CTA:
    // the row-walk kernel, with no pipeline to fill and drain, is the faster one there (measured 45 vs 65 us on a
    // 64-image random-crop batch).
    const bool perSample = kp.list != nullptr || kp.roi != nullptr;
    if (path == 3 || (path == 0 && perSample && kp.dstW >= 32))
        return launch_resize_rowwalk<INTERP, DK>(kp, stream);
    const bool wantStaged = path == 2 || (path == 0 && kp.dstW >= 32 && !sparseTaps);
    if (wantStaged)
    {
        int status = B200PP_SUCCESS;
        if (launch_resize_staged<INTERP, DK>(kp, srcWBound, stream, &status))
            return status;
    }
    return launch_resize_gather<INTERP, DK>(kp, stream);
}

template<int INTERP>
static int run_resize_dk(int dk, const ResizeKParams &kp, int srcWBound, cudaStream_t stream)
{
    switch (dk)
    {
    case DST_U8:
        return run_resize<INTERP, DST_U8>(kp, srcWBound, stream);
    case DST_F32:
        return run_resize<INTERP, DST_F32>(kp, srcWBound, stream);
    default:
        return run_resize<INTERP, DST_F16>(kp, srcWBound, stream);
    }
}

} // namespace b200pp

namespace b200pp {

template<typename S, typename D>
static void launch_slice_typed_sd(int channels, dim3 grid, dim3 block, cudaStream_t stream, const SliceKParams &kp, int srcType,
                                  int dstType)
{
    if (channels == 1)
        slice_typed_kernel<S, D, 1><<<grid, block, 0, stream>>>(kp, srcType, dstType);
    else if (channels == 3)
        slice_typed_kernel<S, D, 3><<<grid, block, 0, stream>>>(kp, srcType, dstType);
    else
        slice_typed_kernel<S, D, 4><<<grid, block, 0, stream>>>(kp, srcType, dstType);
}

static void launch_slice_typed(bool srcFloat, bool dstFloat, int channels, dim3 grid, dim3 block, cudaStream_t stream,
                               const SliceKParams &kp, int srcType, int dstType)
{
    if (srcFloat && dstFloat)
        launch_slice_typed_sd<float, float>(channels, grid, block, stream, kp, srcType, dstType);
    else if (srcFloat)
        launch_slice_typed_sd<float, uint8_t>(channels, grid, block, stream, kp, srcType, dstType);
    else if (dstFloat)
        launch_slice_typed_sd<uint8_t, float>(channels, grid, block, stream, kp, srcType, dstType);
    else
        launch_slice_typed_sd<uint8_t, uint8_t>(channels, grid, block, stream, kp, srcType, dstType);
}

} // namespace b200pp

using namespace b200pp;

// ================================================================================================ C entry points

extern "C" int b200ppResizeCropConvertReformat(const B200ppSource *src, const B200ppDest *dst, const B200ppResizeOp *op,
                                               cudaStream_t stream)
{
    if (!src || !dst || !op)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    if (src->numSamples != 0 && (!dst->base || (!src->base && !src->imageList)))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be cuda-accessible, pitch-linear memory");

    // Same checks, order and status codes as the reference operator
    // (src/cvcuda/priv/OpResizeCropConvertReformat.cu:446-539 and :591-668).
    if (src->channels != dst->channels)
        return fail(B200PP_ERROR_NOT_COMPATIBLE,
                    "Input and output must have same number of channels: Provided %d input and %d output channels",
                    src->channels, dst->channels);
    if (src->channels != 3)
        return fail(B200PP_ERROR_NOT_COMPATIBLE,
                    "Only three-channel input is currently supported: Provided %d input channels", src->channels);
    if (src->dtype != B200PP_U8)
        return fail(B200PP_ERROR_NOT_COMPATIBLE, "Input must be of data type uchar.");
    if (dst->dtype != B200PP_U8 && dst->dtype != B200PP_F32 && dst->dtype != B200PP_F16)
        return fail(B200PP_ERROR_NOT_COMPATIBLE, "Output must be of data type uchar, float or half.");
    if (src->planar)
        return fail(B200PP_ERROR_NOT_COMPATIBLE, "Input must be non-planar (i.e., interleaved).");
    if (op->resizeW <= 1 || op->resizeH <= 1)
        return fail(B200PP_ERROR_INVALID_ARGUMENT,
                    "Invalid resize dimensions: width x hight = %d x %d dimensions must be larger than 1.", op->resizeW,
                    op->resizeH);

    const bool wholeDst = (op->regionW == 0 && op->regionH == 0);
    const int  regionW = wholeDst ? dst->width : op->regionW, regionH = wholeDst ? dst->height : op->regionH;
    const int  dstX = wholeDst ? 0 : op->dstX, dstY = wholeDst ? 0 : op->dstY;
    if (dst->width < 1 || dst->height < 1 || regionW < 1 || regionH < 1 || dstX < 0 || dstY < 0
        || static_cast<long long>(dstX) + regionW > dst->width || static_cast<long long>(dstY) + regionH > dst->height)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid placement: region (%d, %d, %d, %d) does not fit the %d x %d output",
                    dstX, dstY, regionW, regionH, dst->width, dst->height);
    if (op->cropX < 0 || op->cropY < 0 || static_cast<long long>(op->cropX) + regionW > op->resizeW
        || static_cast<long long>(op->cropY) + regionH > op->resizeH)
        return fail(B200PP_ERROR_INVALID_ARGUMENT,
                    "Invalid crop region: crop region(x, y, w, h) = (%d, %d, %d, %d) extends beyond bounds of resized tensor",
                    op->cropX, op->cropY, regionW, regionH);
    if (op->interp != B200PP_INTERP_NEAREST && op->interp != B200PP_INTERP_LINEAR)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, op->interp == 2   ? "Interpolation not implemented: NVCV_INTERP_CUBIC"
                                                   : op->interp == 3 ? "Interpolation not implemented: NVCV_INTERP_AREA"
                                                                     : "Invalid interpolation");
    if (op->manip != B200PP_CHANNEL_NO_OP && op->manip != B200PP_CHANNEL_REVERSE)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid channel manipulation");
    if (src->numSamples < 0)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Negative batch size");
    if (!src->imageList && (src->width < 1 || src->height < 1))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input size");
    if (src->numSamples == 0)
        return B200PP_SUCCESS;

    ResizeKParams kp{};
    kp.srcBase         = static_cast<const uint8_t *>(src->base);
    kp.srcSampleStride = src->sampleStride;
    kp.srcRowStride    = src->rowStride;
    kp.srcW            = src->width;
    kp.srcH            = src->height;
    kp.list            = src->imageList;
    kp.roi             = op->roi;
    kp.roiStride       = op->roiStride ? op->roiStride : 16;
    kp.flip            = op->flipCode;
    kp.numSamples      = src->numSamples;
    kp.denseScaleW     = static_cast<float>(src->width) / static_cast<float>(op->resizeW);
    kp.denseScaleH     = static_cast<float>(src->height) / static_cast<float>(op->resizeH);
    kp.resizeW         = op->resizeW;
    kp.resizeH         = op->resizeH;
    kp.cropX           = op->cropX;
    kp.cropY           = op->cropY;
    kp.srcCast         = op->srcCast != 0;
    kp.dstX            = dstX;
    kp.dstY            = dstY;
    kp.regionW         = regionW;
    kp.regionH         = regionH;
    kp.padValue        = op->padValue;
    kp.perChannel      = op->perChannel != 0;
    kp.scale           = op->scale;
    kp.offset          = op->offset;
    for (int c = 0; c < 3; ++c)
    {
        kp.base[c] = op->base[c];
        kp.mul[c]  = op->mul[c];
        kp.mapC[c] = op->manip == B200PP_CHANNEL_REVERSE ? 2 - c : c;
    }
    kp.gscale  = op->gscale;
    kp.shift   = op->shift;
    kp.dst     = static_cast<uint8_t *>(dst->base);
    kp.dSample = dst->sampleStride;
    kp.dRow    = dst->rowStride;
    kp.dPix    = dst->pixStride;
    kp.dChan   = dst->chanStride;
    kp.dstW    = dst->width;
    kp.dstH    = dst->height;

    const int dk        = dst->dtype == B200PP_U8 ? DST_U8 : (dst->dtype == B200PP_F32 ? DST_F32 : DST_F16);
    const int srcWBound = src->imageList ? (src->maxWidth > 0 ? src->maxWidth : 3840) : src->width;
    if (const int st = pending_device_error())
        return st;
    if (op->interp == B200PP_INTERP_NEAREST)
        return run_resize_dk<B200PP_INTERP_NEAREST>(dk, kp, srcWBound, stream);
    return run_resize_dk<B200PP_INTERP_LINEAR>(dk, kp, srcWBound, stream);
}

extern "C" int b200ppCropFlipNormalizeReformat(const B200ppSource *src, const B200ppDest *dst, const B200ppSliceOp *op,
                                               cudaStream_t stream)
{
    if (!src || !dst || !op)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    if (src->numSamples != 0 && (!dst->base || (!src->base && !src->imageList)))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be cuda-accessible, pitch-linear memory");
    if (!op->cropRect || !op->flipCode || !op->base || !op->scale)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "cropRect, flipCode, base and scale must be cuda-accessible tensors");

    // Checks of the reference operator (src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:430-464, :304-317, :342-356).
    const int channels = src->channels;
    if (channels < 1 || channels > 4)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input must have 1 to 4 channels");
    if (!(op->baseChannels == 1 || op->baseChannels >= channels))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Channel of base tensor must be 1 or >= input/output tensor channels");
    if (!(op->scaleChannels == 1 || op->scaleChannels >= channels))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Channel of scale tensor must be 1 or >= input/output tensor channels");
    if (src->dtype < B200PP_U8 || src->dtype > B200PP_F32)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Unsupported input data type");
    if (dst->dtype < B200PP_U8 || dst->dtype > B200PP_F16)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Unsupported output data type");
    if (op->border < B200PP_BORDER_CONSTANT || op->border > B200PP_BORDER_REFLECT101)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Unsupported border mode");
    if (dst->channels != channels)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must have the same number of channels");
    if (src->numSamples < 0 || dst->width < 1 || dst->height < 1)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid batch or output size");
    if (src->numSamples == 0)
        return B200PP_SUCCESS;

    SliceKParams kp{};
    kp.srcBase         = static_cast<const uint8_t *>(src->base);
    kp.srcSampleStride = src->sampleStride;
    kp.srcRowStride    = src->rowStride;
    kp.srcPlaneStride  = src->planeStride;
    kp.srcW            = src->width;
    kp.srcH            = src->height;
    kp.list            = src->imageList;
    kp.srcPlanar       = src->planar != 0 && channels > 1;
    kp.channels        = channels;
    kp.numSamples      = src->numSamples;
    kp.cropRect        = op->cropRect;
    kp.cropRectStride  = op->cropRectStride ? op->cropRectStride : 16;
    kp.flip            = op->flipCode;
    kp.border          = op->border;
    // static_cast<T_Src>(borderValue), then the promotion to float that the normalisation applies to every source value
    switch (src->dtype)
    {
    case B200PP_U8:
        kp.borderAsSrc = static_cast<float>(static_cast<uint8_t>(op->borderValue));
        break;
    case B200PP_S8:
        kp.borderAsSrc = static_cast<float>(static_cast<int8_t>(op->borderValue));
        break;
    case B200PP_U16:
        kp.borderAsSrc = static_cast<float>(static_cast<uint16_t>(op->borderValue));
        break;
    case B200PP_S16:
        kp.borderAsSrc = static_cast<float>(static_cast<int16_t>(op->borderValue));
        break;
    case B200PP_U32:
        kp.borderAsSrc = static_cast<float>(static_cast<uint32_t>(op->borderValue));
        break;
    case B200PP_S32:
        kp.borderAsSrc = static_cast<float>(static_cast<int32_t>(op->borderValue));
        break;
    default:
        kp.borderAsSrc = op->borderValue;
        break;
    }
    kp.base            = op->base;
    kp.baseChanStride  = op->baseChanStride ? op->baseChanStride : 4;
    kp.baseCh          = op->baseChannels;
    kp.scale           = op->scale;
    kp.scaleChanStride = op->scaleChanStride ? op->scaleChanStride : 4;
    kp.scaleCh         = op->scaleChannels;
    kp.gscale          = op->gscale;
    kp.shift           = op->shift;
    kp.epsilon         = op->epsilon;
    // The reference kernel receives the whole flags word as a bool
    // (src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:46,73): any set bit selects the standard-deviation formula.
    kp.stddev  = op->flags != 0;
    kp.dst     = static_cast<uint8_t *>(dst->base);
    kp.dSample = dst->sampleStride;
    kp.dRow    = dst->rowStride;
    kp.dPix    = dst->pixStride;
    kp.dChan   = dst->chanStride;
    kp.dstW    = dst->width;
    kp.dstH    = dst->height;

    dim3 block(32, 8);
    const int  path     = g_kernelPath.load(std::memory_order_relaxed);
    const bool fastCase = src->dtype == B200PP_U8 && channels == 3 && !kp.srcPlanar
                       && (dst->dtype == B200PP_U8 || dst->dtype == B200PP_F32 || dst->dtype == B200PP_F16);
    if (const int st = pending_device_error())
        return st;
    if (fastCase && path != 1)
    {
        // four destination pixels per thread; one vector store per channel when the destination is planar and every
        // address involved is a multiple of the vector size
        const long long vec      = 4ll * elem_size(dst->dtype);
        const int       vecStore = kp.dPix == elem_size(dst->dtype)
                           && ((reinterpret_cast<unsigned long long>(kp.dst) | static_cast<unsigned long long>(kp.dRow)
                                | static_cast<unsigned long long>(kp.dChan) | static_cast<unsigned long long>(kp.dSample))
                               % vec)
                                  == 0;
        const int rowsPerBlock = 8 * kSliceRowsPerThread;
        dim3      grid((kp.dstW + 127) / 128, (kp.dstH + rowsPerBlock - 1) / rowsPerBlock, std::min(kp.numSamples, 32768));
        if (dst->dtype == B200PP_F32)
            slice_u8x3_kernel<DST_F32><<<grid, block, 0, stream>>>(kp, dst->dtype, vecStore);
        else if (dst->dtype == B200PP_F16)
            slice_u8x3_kernel<DST_F16><<<grid, block, 0, stream>>>(kp, dst->dtype, vecStore);
        else
            slice_u8x3_kernel<DST_U8><<<grid, block, 0, stream>>>(kp, dst->dtype, vecStore);
        return check_launch("CropFlipNormalizeReformat (uint8 x 3)");
    }
    // uint8 / float32 on both sides, 1, 3 or 4 channels: the typed kernel (element types and channel count compiled in)
    const bool typedCase = (src->dtype == B200PP_U8 || src->dtype == B200PP_F32) && (dst->dtype == B200PP_U8 || dst->dtype == B200PP_F32)
                        && (channels == 1 || channels == 3 || channels == 4);
    // ... and among those the single-plane cases: one channel, or planar source to planar destination
    const bool planeCase = typedCase && (channels == 1 || (kp.srcPlanar && kp.dPix == elem_size(dst->dtype)));
    if (planeCase && path != 1)
    {
        const bool sf = src->dtype == B200PP_F32, df = dst->dtype == B200PP_F32;
        const int  pix = slice_plane_pix(sf, df), rowsPerBlock = 8 * slice_plane_rows(sf, df) * kSlicePlaneIters;
        dim3       grid((kp.dstW + 32 * pix - 1) / (32 * pix), (kp.dstH + rowsPerBlock - 1) / rowsPerBlock,
                        static_cast<unsigned>(std::min<long long>(static_cast<long long>(kp.numSamples) * channels, 32768)));
        if (sf && df)
            slice_plane_kernel<float, float><<<grid, block, 0, stream>>>(kp, src->dtype, dst->dtype, channels);
        else if (sf)
            slice_plane_kernel<float, uint8_t><<<grid, block, 0, stream>>>(kp, src->dtype, dst->dtype, channels);
        else if (df)
            slice_plane_kernel<uint8_t, float><<<grid, block, 0, stream>>>(kp, src->dtype, dst->dtype, channels);
        else
            slice_plane_kernel<uint8_t, uint8_t><<<grid, block, 0, stream>>>(kp, src->dtype, dst->dtype, channels);
        return check_launch("CropFlipNormalizeReformat (planes)");
    }
    if (typedCase && path != 1)
    {
        const int rowsPerBlock = 8 * slice_typed_rows(channels, src->dtype == B200PP_U8);
        dim3      grid((kp.dstW + 127) / 128, (kp.dstH + rowsPerBlock - 1) / rowsPerBlock, std::min(kp.numSamples, 32768));
        launch_slice_typed(src->dtype == B200PP_F32, dst->dtype == B200PP_F32, channels, grid, block, stream, kp, src->dtype, dst->dtype);
        return check_launch("CropFlipNormalizeReformat (typed)");
    }
    dim3 grid((kp.dstW + 31) / 32, (kp.dstH + 7) / 8, std::min(kp.numSamples, 32768));
    slice_gather_kernel<4><<<grid, block, 0, stream>>>(kp, src->dtype, dst->dtype, elem_size(src->dtype));
    return check_launch("CropFlipNormalizeReformat");
}

// ================================================================================================ stand-alone Resize

namespace b200pp {

template<typename T, int C>
static void launch_plain(int interp, bool singleTap, dim3 grid, dim3 block, cudaStream_t stream, const PlainResizeKParams &kp)
{
    if (interp == B200PP_INTERP_NEAREST)
        resize_plain_kernel<T, C, B200PP_INTERP_NEAREST><<<grid, block, 0, stream>>>(kp);
    else if (sizeof(T) == 1 && singleTap)
        resize_plain_kernel<T, C, B200PP_INTERP_LINEAR, true><<<grid, block, 0, stream>>>(kp);
    else
        resize_plain_kernel<T, C, B200PP_INTERP_LINEAR><<<grid, block, 0, stream>>>(kp);
}

template<typename T>
static void launch_plain_channels(int channels, int interp, bool singleTap, dim3 grid, dim3 block, cudaStream_t stream,
                                  const PlainResizeKParams &kp)
{
    if (channels == 1)
        launch_plain<T, 1>(interp, singleTap, grid, block, stream, kp);
    else if (channels == 3)
        launch_plain<T, 3>(interp, singleTap, grid, block, stream, kp);
    else
        launch_plain<T, 4>(interp, singleTap, grid, block, stream, kp);
}

static PlainSide plain_side(const B200ppImageSet *s)
{
    PlainSide p{};
    p.base         = static_cast<uint8_t *>(s->base);
    p.list         = s->imageList;
    p.sampleStride = s->sampleStride;
    p.rowStride    = s->rowStride;
    p.width        = s->width;
    p.height       = s->height;
    return p;
}

} // namespace b200pp

static int resize_common(const B200ppImageSet *src, const B200ppImageSet *dst, int32_t interp, const int32_t *cropRects,
                         cudaStream_t stream)
{
    if (!src || !dst)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    if (reinterpret_cast<uintptr_t>(cropRects) & 15)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Crop rectangles must be packed int32 x 4 on a 16-byte boundary");
    // Checks, order and status codes of the reference operator (src/cvcuda/priv/OpResize.cu:501-555, :455-486).
    if (src->dtype != dst->dtype)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output data type are different");
    if (src->numSamples != dst->numSamples)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output samples are different");
    if (src->channels != dst->channels)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output channels are different");
    if (src->channels > 4 || src->channels < 1)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid number of channels");
    if (interp == 2 /* NVCV_INTERP_CUBIC */ || interp == 3 /* NVCV_INTERP_AREA */)
        return fail(B200PP_ERROR_NOT_IMPLEMENTED, "Interpolation not implemented: %s",
                    interp == 2 ? "NVCV_INTERP_CUBIC" : "NVCV_INTERP_AREA");
    if (interp != B200PP_INTERP_NEAREST && interp != B200PP_INTERP_LINEAR)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid interpolation");
    const bool knownType = src->dtype == B200PP_U8 || src->dtype == B200PP_U16 || src->dtype == B200PP_S16
                        || src->dtype == B200PP_F32;
    if (!knownType || src->channels == 2)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input data type");
    if (src->numSamples < 0)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Negative batch size");
    if (src->numSamples == 0)
        return B200PP_SUCCESS;
    if ((!src->base && !src->imageList) || (!dst->base && !dst->imageList))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be cuda-accessible, pitch-linear memory");
    if ((!src->imageList && (src->width < 1 || src->height < 1)) || (!dst->imageList && (dst->width < 1 || dst->height < 1)))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid image size");

    PlainResizeKParams kp{};
    kp.src        = plain_side(src);
    kp.dst        = plain_side(dst);
    kp.numSamples = src->numSamples;
    kp.cropRects  = cropRects;
    const int gw = dst->imageList ? dst->maxWidth : dst->width, gh = dst->imageList ? dst->maxHeight : dst->height;
    if (gw < 1 || gh < 1)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Output image list needs its maximum width and height");
    dim3 block(32, 8);
    dim3 grid((gw + 32 * kPlainCols - 1) / (32 * kPlainCols), (gh + 8 * kPlainRows - 1) / (8 * kPlainRows),
              std::min(src->numSamples, 65535));
    if (grid.y > 65535u)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
    // Odd whole-number scale factors on both axes (1080p -> 640x360 is 3 x 3) put every sample position on a source pixel:
    // all second taps weigh exactly zero and the uint8 kernel may take its single-tap shortcut.
    auto oddMultiple = [](int s, int d) { return d > 0 && s % d == 0 && ((s / d) & 1) == 1; };
    const bool singleTap = !src->imageList && !dst->imageList && !cropRects && oddMultiple(src->width, dst->width)
                        && oddMultiple(src->height, dst->height);
    switch (src->dtype)
    {
    case B200PP_U8:
        launch_plain_channels<uint8_t>(src->channels, interp, singleTap, grid, block, stream, kp);
        break;
    case B200PP_U16:
        launch_plain_channels<uint16_t>(src->channels, interp, singleTap, grid, block, stream, kp);
        break;
    case B200PP_S16:
        launch_plain_channels<int16_t>(src->channels, interp, singleTap, grid, block, stream, kp);
        break;
    default:
        launch_plain_channels<float>(src->channels, interp, singleTap, grid, block, stream, kp);
        break;
    }
    return check_launch("Resize");
}

extern "C" int b200ppResize(const B200ppImageSet *src, const B200ppImageSet *dst, int32_t interp, cudaStream_t stream)
{
    return resize_common(src, dst, interp, nullptr, stream);
}

extern "C" int b200ppResizedCrop(const B200ppImageSet *src, const B200ppImageSet *dst, const int32_t *cropRects,
                                 int32_t interp, cudaStream_t stream)
{
    if (!cropRects)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null crop rectangles");
    return resize_common(src, dst, interp, cropRects, stream);
}

// ------------------------------------------------------------------------------------------------------------------------
// b200ppResizedCropNoAlloc: the resized crop for callers that must not allocate device memory.
//
// A crop-and-resize launch reads one rectangle per image from a device table. b200ppResizedCrop leaves that table to the
// caller, who normally gets it from cudaMalloc (or from b200ppParamBufferCreate, which calls cudaMalloc). Some callers
// cannot do that: a plug-in that runs inside an inference server's request path where every byte of device memory was
// handed out at start-up, a process that shares its GPU with a model sized to fill it, code between two points of a
// pipeline where a cudaMalloc would stall every stream of the device. For them the table lives in the library image
// itself, in the fixed array below, and the rectangles arrive as an ordinary host array.
//
// The price: the array has a fixed capacity (B200PP_NO_ALLOC_MAX_RECTS rectangles = 64 KiB, held by every GPU that loads
// the library until the process exits), and there is only one per GPU, so two such calls whose GPU work overlaps (on
// two streams, or from two threads) overwrite each other's rectangles. Calls on one stream are ordered and safe.
// Nothing in the table has to start at zero: a call overwrites the entries it uses before its kernel reads them and
// never reads further; whatever an earlier call left beyond them is ignored.
static __device__ __align__(256) int32_t g_noAllocRects[B200PP_NO_ALLOC_MAX_RECTS * 4];

namespace {
// In host code `g_noAllocRects` names a host-side shadow, not device memory: the device address has to be asked for,
// once per device with that device current. Cached here per device ordinal.
constexpr int kNoAllocMaxDevices = 64;
std::mutex    g_noAllocMutex;
int32_t      *g_noAllocRectsDev[kNoAllocMaxDevices] = {};
} // namespace

extern "C" int b200ppResizedCropNoAlloc(const B200ppImageSet *src, const B200ppImageSet *dst, const int32_t *hostRects,
                                        int32_t interp, cudaStream_t stream)
{
    if (!src || !dst || !hostRects)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    if (src->numSamples > B200PP_NO_ALLOC_MAX_RECTS)
        return fail(B200PP_ERROR_INVALID_ARGUMENT,
                    "b200ppResizedCropNoAlloc takes at most %d images per call (%d given): split the batch, or use "
                    "b200ppResizedCrop with a rectangle table of your own",
                    B200PP_NO_ALLOC_MAX_RECTS, src->numSamples);
    if (src->numSamples <= 0) // nothing to upload; the common checks decide between "empty batch" and "negative size"
        return b200ppResize(src, dst, interp, stream);
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kNoAllocMaxDevices)
    {
        cudaGetLastError();
        return fail(B200PP_ERROR_INTERNAL, "No current CUDA device (or its ordinal is above %d)", kNoAllocMaxDevices - 1);
    }
    int32_t *table = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noAllocMutex);
        if (!g_noAllocRectsDev[device])
        {
            // first call on this device: look the array's device address up
            void             *addr = nullptr;
            const cudaError_t e    = cudaGetSymbolAddress(&addr, g_noAllocRects);
            if (e != cudaSuccess || !addr)
            {
                cudaGetLastError();
                return fail(B200PP_ERROR_INTERNAL, "Cannot locate the built-in rectangle table on device %d: %s", device,
                            cudaGetErrorString(e));
            }
            g_noAllocRectsDev[device] = static_cast<int32_t *>(addr);
        }
        table = g_noAllocRectsDev[device];
    }
    // Pageable or page-locked host memory alike; ordered on `stream` before the kernel below.
    const cudaError_t e = cudaMemcpyAsync(table, hostRects, sizeof(int32_t) * 4 * static_cast<size_t>(src->numSamples),
                                          cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess)
    {
        cudaGetLastError();
        return fail(B200PP_ERROR_INTERNAL, "Upload of the crop rectangles failed: %s", cudaGetErrorString(e));
    }
    return resize_common(src, dst, interp, table, stream);
}

// Rows of CTAs for the table kernels (Normalize, ConvertTo): one per block of rows, up to the grid limit (the kernels
// walk down the image in steps of the grid's height beyond it). Fewer, longer-lived CTAs were slower (227 vs 193 us on
// 32 x 1080p RGB uint8 -> float32 with sixteen CTAs per SM): the table costs little next to the tail it creates.
static unsigned lut_grid_rows(int height, int rowsPerCta, unsigned long long /*ctasPerRow*/)
{
    const unsigned long long needed = static_cast<unsigned long long>((height + rowsPerCta - 1) / rowsPerCta);
    return static_cast<unsigned>(std::max(1ull, std::min(needed, 65535ull)));
}

// ================================================================================================ stand-alone Normalize

extern "C" int b200ppNormalize(const B200ppImageSet *src, const B200ppImageSet *dst, const B200ppNormalizeOp *op,
                               cudaStream_t stream)
{
    if (!src || !dst || !op)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    // Checks of the reference operator (src/cvcuda/priv/legacy/normalize.cu:314-373): same layout on both sides is
    // implied by the argument types here; channel count and element types as there.
    if (src->numSamples != dst->numSamples)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output samples are different");
    if (src->channels != dst->channels)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output channels are different");
    if (src->channels > 4 || src->channels < 1)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid channel number %d", src->channels);
    auto known = [](int t) {
        return t == B200PP_U8 || t == B200PP_S8 || t == B200PP_U16 || t == B200PP_S16 || t == B200PP_S32 || t == B200PP_F32;
    };
    if (!known(src->dtype) || !known(dst->dtype))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataType");
    if (src->numSamples < 0)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Negative batch size");
    if (src->numSamples == 0)
        return B200PP_SUCCESS;
    if (!op->base || !op->scale)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input base and scale must be cuda-accessible, pitch-linear tensors");
    if ((!src->base && !src->imageList) || (!dst->base && !dst->imageList))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be cuda-accessible, pitch-linear memory");
    if (!src->imageList && !dst->imageList && (src->width != dst->width || src->height != dst->height))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output sizes are different");

    NormalizeKParams kp{};
    kp.src        = plain_side(src);
    kp.dst        = plain_side(dst);
    kp.numSamples = src->numSamples;
    kp.channels   = src->channels;
    kp.srcType    = src->dtype;
    kp.dstType    = dst->dtype;
    kp.srcElem    = elem_size(src->dtype);
    kp.dstElem    = elem_size(dst->dtype);
    kp.base       = op->base;
    kp.scale      = op->scale;
    for (int k = 0; k < 4; ++k)
    {
        kp.baseStride[k]  = op->baseStride[k];
        kp.scaleStride[k] = op->scaleStride[k];
    }
    kp.gscale  = op->gscale;
    kp.shift   = op->shift;
    kp.epsilon = op->epsilon;
    kp.stddev  = (op->flags & B200PP_NORMALIZE_SCALE_IS_STDDEV) != 0;
    const int gw = dst->imageList ? dst->maxWidth : dst->width, gh = dst->imageList ? dst->maxHeight : dst->height;
    if (gw < 1 || gh < 1)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid image size");
    dim3 block(32, 8);
    dim3 grid((gw + 32 * kNormCols - 1) / (32 * kNormCols), (gh + 8 * kNormRows - 1) / (8 * kNormRows),
              std::min(src->numSamples, 65535));
    if (grid.y > 65535u)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
    const bool perChannel = (kp.baseStride[0] | kp.baseStride[1] | kp.baseStride[2] | kp.scaleStride[0] | kp.scaleStride[1]
                             | kp.scaleStride[2])
                         == 0;
    if (src->dtype == B200PP_U8 && perChannel && g_kernelPath.load(std::memory_order_relaxed) != 1)
    {
        // table of the 256 results per channel; one thread per four words of a row x two rows
        const long long rowWords = (static_cast<long long>(gw) * src->channels + 3) / 4;
        dim3            lutGrid(static_cast<unsigned>((rowWords + 127) / 128), 1, grid.z);
        lutGrid.y = lut_grid_rows(gh, kp.dstElem == 4 ? 16 : 32, lutGrid.x * lutGrid.z);
        if (kp.dstElem == 4)
            normalize_lut_kernel<4><<<lutGrid, block, 0, stream>>>(kp);
        else if (kp.dstElem == 2)
            normalize_lut_kernel<2><<<lutGrid, block, 0, stream>>>(kp);
        else
            normalize_lut_kernel<1><<<lutGrid, block, 0, stream>>>(kp);
        return check_launch("Normalize");
    }
    if (src->dtype == B200PP_F32 && dst->dtype == B200PP_F32 && perChannel && src->channels != 2
        && g_kernelPath.load(std::memory_order_relaxed) != 1)
    {
        // four pixels x two rows per thread
        dim3 fgrid((gw + 127) / 128, (gh + 15) / 16, grid.z);
        if (fgrid.y > 65535u)
            return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
        if (src->channels == 1)
            normalize_f32_kernel<1><<<fgrid, block, 0, stream>>>(kp);
        else if (src->channels == 3)
            normalize_f32_kernel<3><<<fgrid, block, 0, stream>>>(kp);
        else
            normalize_f32_kernel<4><<<fgrid, block, 0, stream>>>(kp);
        return check_launch("Normalize (float32)");
    }
    if (src->dtype == B200PP_U8 && dst->dtype == B200PP_U8)
        normalize_kernel<B200PP_U8, B200PP_U8><<<grid, block, 0, stream>>>(kp);
    else if (src->dtype == B200PP_U8 && dst->dtype == B200PP_F32)
        normalize_kernel<B200PP_U8, B200PP_F32><<<grid, block, 0, stream>>>(kp);
    else if (src->dtype == B200PP_F32 && dst->dtype == B200PP_F32 && g_kernelPath.load(std::memory_order_relaxed) != 1)
        normalize_kernel<B200PP_F32, B200PP_F32><<<grid, block, 0, stream>>>(kp);
    else
        normalize_kernel<-1, -1><<<grid, block, 0, stream>>>(kp);
    return check_launch("Normalize");
}

// ================================================================================================ stand-alone Reformat

extern "C" int b200ppReformat(const B200ppDest *src, const B200ppDest *dst, int32_t numSamples, cudaStream_t stream)
{
    if (!src || !dst)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    if (src->dtype != dst->dtype)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output data type are different");
    if (src->channels != dst->channels || src->width != dst->width || src->height != dst->height)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output shapes are different");
    if (src->dtype < B200PP_U8 || src->dtype > B200PP_F16)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataType");
    if (numSamples < 0 || src->channels < 1 || src->width < 0 || src->height < 0)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid shape");
    if (numSamples == 0 || src->width == 0 || src->height == 0)
        return B200PP_SUCCESS;
    if (!src->base || !dst->base)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be cuda-accessible, pitch-linear memory");
    ReformatKParams kp{};
    kp.src        = static_cast<const uint8_t *>(src->base);
    kp.dst        = static_cast<uint8_t *>(dst->base);
    kp.sSample    = src->sampleStride;
    kp.sRow       = src->rowStride;
    kp.sPix       = src->pixStride;
    kp.sChan      = src->chanStride;
    kp.dSample    = dst->sampleStride;
    kp.dRow       = dst->rowStride;
    kp.dPix       = dst->pixStride;
    kp.dChan      = dst->chanStride;
    kp.numSamples = numSamples;
    kp.channels   = src->channels;
    kp.width      = src->width;
    kp.height     = src->height;
    dim3 block(32, 8);
    // RGB8 between packed interleaved and planar, everything on 16-byte boundaries: the vector kernel
    if (elem_size(src->dtype) == 1 && kp.channels == 3 && g_kernelPath.load(std::memory_order_relaxed) != 1)
    {
        const bool toPlanar   = kp.sPix == 3 && kp.sChan == 1 && kp.dPix == 1;
        const bool fromPlanar = kp.dPix == 3 && kp.dChan == 1 && kp.sPix == 1;
        const uintptr_t bits  = reinterpret_cast<uintptr_t>(kp.src) | reinterpret_cast<uintptr_t>(kp.dst)
                             | static_cast<uintptr_t>(kp.sSample) | static_cast<uintptr_t>(kp.sRow)
                             | static_cast<uintptr_t>(kp.dSample) | static_cast<uintptr_t>(kp.dRow)
                             | static_cast<uintptr_t>(toPlanar ? kp.dChan : kp.sChan);
        if ((toPlanar || fromPlanar) && (bits & 15) == 0)
        {
            dim3 vgrid((kp.width + 511) / 512, (kp.height + 15) / 16, std::min(numSamples, 65535));
            if (vgrid.y > 65535u)
                return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
            if (toPlanar)
                reformat_u8x3_kernel<true><<<vgrid, block, 0, stream>>>(kp);
            else
                reformat_u8x3_kernel<false><<<vgrid, block, 0, stream>>>(kp);
            return check_launch("Reformat");
        }
    }
    // the same for 32-bit elements (float32 / int32 RGB)
    if (elem_size(src->dtype) == 4 && kp.channels == 3 && g_kernelPath.load(std::memory_order_relaxed) != 1)
    {
        const bool toPlanar   = kp.sPix == 12 && kp.sChan == 4 && kp.dPix == 4;
        const bool fromPlanar = kp.dPix == 12 && kp.dChan == 4 && kp.sPix == 4;
        const uintptr_t bits  = reinterpret_cast<uintptr_t>(kp.src) | reinterpret_cast<uintptr_t>(kp.dst)
                             | static_cast<uintptr_t>(kp.sSample) | static_cast<uintptr_t>(kp.sRow)
                             | static_cast<uintptr_t>(kp.dSample) | static_cast<uintptr_t>(kp.dRow)
                             | static_cast<uintptr_t>(toPlanar ? kp.dChan : kp.sChan);
        if ((toPlanar || fromPlanar) && (bits & 15) == 0)
        {
            dim3 vgrid((kp.width + 127) / 128, (kp.height + 15) / 16, std::min(numSamples, 65535));
            if (vgrid.y > 65535u)
                return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
            if (toPlanar)
                reformat_w32x3_kernel<true><<<vgrid, block, 0, stream>>>(kp);
            else
                reformat_w32x3_kernel<false><<<vgrid, block, 0, stream>>>(kp);
            return check_launch("Reformat");
        }
    }
    const int perThread = 4 / std::min(4, elem_size(src->dtype)); // pixels per thread: one 32-bit word per channel
    dim3      grid((kp.width + 32 * perThread - 1) / (32 * perThread), (kp.height + 31) / 32, std::min(numSamples, 65535));
    if (grid.y > 65535u)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
    switch (elem_size(src->dtype))
    {
    case 1:
        reformat_kernel<uint8_t><<<grid, block, 0, stream>>>(kp);
        break;
    case 2:
        reformat_kernel<uint16_t><<<grid, block, 0, stream>>>(kp);
        break;
    default:
        reformat_kernel<uint32_t><<<grid, block, 0, stream>>>(kp);
        break;
    }
    return check_launch("Reformat");
}

// ================================================================================================ stand-alone ConvertTo

extern "C" int b200ppConvertTo(const B200ppImageSet *src, const B200ppImageSet *dst, double alpha, double beta,
                               cudaStream_t stream)
{
    if (!src || !dst)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    // checks of src/cvcuda/priv/legacy/convert_to.cu:140-188
    if (src->imageList || dst->imageList)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "ConvertTo works on tensors");
    auto known = [](int t) {
        return t == B200PP_U8 || t == B200PP_S8 || t == B200PP_U16 || t == B200PP_S16 || t == B200PP_S32 || t == B200PP_F32;
    };
    if (!known(src->dtype))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input DataType");
    if (!known(dst->dtype))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid output DataType");
    if (src->numSamples != dst->numSamples || src->width != dst->width || src->height != dst->height
        || src->channels != dst->channels)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input/output shape: the shapes must be equal");
    if (src->channels < 1 || src->channels > 4)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid channel number %d", src->channels);
    if (src->numSamples < 0 || src->width < 0 || src->height < 0)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid shape");
    if (src->numSamples == 0 || src->width == 0 || src->height == 0)
        return B200PP_SUCCESS;
    if (!src->base || !dst->base)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be cuda-accessible, pitch-linear memory");
    ConvertKParams kp{};
    kp.src        = static_cast<const uint8_t *>(src->base);
    kp.dst        = static_cast<uint8_t *>(dst->base);
    kp.sSample    = src->sampleStride;
    kp.sRow       = src->rowStride;
    kp.dSample    = dst->sampleStride;
    kp.dRow       = dst->rowStride;
    kp.numSamples = src->numSamples;
    kp.rowElems   = src->width * src->channels;
    kp.height     = src->height;
    kp.srcType    = src->dtype;
    kp.dstType    = dst->dtype;
    kp.srcElem    = elem_size(src->dtype);
    kp.dstElem    = elem_size(dst->dtype);
    kp.alpha      = alpha;
    kp.beta       = beta;
    dim3 block(32, 8);
    dim3 grid((kp.rowElems + 127) / 128, (kp.height + 15) / 16, std::min(src->numSamples, 65535));
    if (grid.y > 65535u)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
    // 8-bit sources go through a 256-entry table of results when the rows allow word loads and vector stores
    const uintptr_t srcBits = reinterpret_cast<uintptr_t>(kp.src) | static_cast<uintptr_t>(kp.sRow)
                            | static_cast<uintptr_t>(kp.sSample);
    const uintptr_t dstBits = reinterpret_cast<uintptr_t>(kp.dst) | static_cast<uintptr_t>(kp.dRow)
                            | static_cast<uintptr_t>(kp.dSample);
    if (kp.srcElem == 1 && (srcBits & 3) == 0 && (dstBits & (4 * kp.dstElem - 1)) == 0 && g_kernelPath.load() != 1)
    {
        dim3 lutGrid(((kp.rowElems + 3) / 4 + 127) / 128, 1, grid.z);
        lutGrid.y = lut_grid_rows(kp.height, kp.dstElem == 4 ? 16 : 32, lutGrid.x * lutGrid.z);
        if (kp.dstElem == 4)
            convert_lut_kernel<4><<<lutGrid, block, 0, stream>>>(kp);
        else if (kp.dstElem == 2)
            convert_lut_kernel<2><<<lutGrid, block, 0, stream>>>(kp);
        else
            convert_lut_kernel<1><<<lutGrid, block, 0, stream>>>(kp);
        return check_launch("ConvertTo");
    }
    if (kp.srcType == B200PP_F32 && (srcBits & 15) == 0 && (dstBits & (4 * kp.dstElem - 1)) == 0 && g_kernelPath.load() != 1)
    {
        dim3 vecGrid(((kp.rowElems + 3) / 4 + 63) / 64, grid.y, grid.z);
        if (kp.dstElem == 4)
            convert_f32_kernel<4><<<vecGrid, block, 0, stream>>>(kp);
        else if (kp.dstElem == 2)
            convert_f32_kernel<2><<<vecGrid, block, 0, stream>>>(kp);
        else
            convert_f32_kernel<1><<<vecGrid, block, 0, stream>>>(kp);
        return check_launch("ConvertTo");
    }
    convert_kernel<<<grid, block, 0, stream>>>(kp);
    return check_launch("ConvertTo");
}

// ================================================================================================ stand-alone CopyMakeBorder

namespace b200pp {

// One pixel's bytes for the constant border: each channel value converted from float to the element type the way a C++
// static_cast does inside the type's range (toward zero), clamped to the range outside it.
static void border_fill_bytes(int dtype, int channels, const float value[4], unsigned (&fill)[4])
{
    uint8_t   bytes[16] = {};
    const int es        = elem_size(dtype);
    for (int c = 0; c < channels; ++c)
    {
        const float v = value ? value[c] : 0.f;
        if (dtype == B200PP_F32)
        {
            std::memcpy(bytes + c * es, &v, 4);
            continue;
        }
        double lo = 0, hi = 255;
        switch (dtype)
        {
        case B200PP_S8:
            lo = -128, hi = 127;
            break;
        case B200PP_U16:
            hi = 65535;
            break;
        case B200PP_S16:
            lo = -32768, hi = 32767;
            break;
        case B200PP_S32:
            lo = -2147483648.0, hi = 2147483647.0;
            break;
        default:
            break;
        }
        double d = v != v ? 0.0 : std::trunc(static_cast<double>(v));
        d        = d < lo ? lo : (d > hi ? hi : d);
        const long long i = static_cast<long long>(d);
        std::memcpy(bytes + c * es, &i, es); // little-endian: the low bytes are the two's-complement element
    }
    std::memcpy(fill, bytes, 16);
}

template<int PB>
static void launch_border(dim3 grid, dim3 block, cudaStream_t stream, const BorderKParams &kp)
{
    copy_make_border_kernel<PB><<<grid, block, 0, stream>>>(kp);
}

} // namespace b200pp

extern "C" int b200ppCopyMakeBorder(const B200ppImageSet *src, const B200ppImageSet *dst, int32_t top, int32_t left,
                                    const int32_t *topList, const int32_t *leftList, int32_t borderMode,
                                    const float borderValue[4], cudaStream_t stream)
{
    if (!src || !dst)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    // Checks and order of the reference operator (src/cvcuda/priv/legacy/copy_make_border.cu:98-166 for tensors,
    // copy_make_border_var_shape.cu:150-222 for variable-shape batches).
    if (src->dtype != dst->dtype)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataType between input and output");
    if (src->channels != dst->channels)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output channels are different");
    if (src->channels > 4 || src->channels < 1)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid channel number %d", src->channels);
    if (!(src->dtype == B200PP_U8 || src->dtype == B200PP_U16 || src->dtype == B200PP_S16 || src->dtype == B200PP_F32
          || src->dtype == B200PP_S8 || src->dtype == B200PP_S32))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataType %d", src->dtype);
    if (borderMode < B200PP_BORDER_CONSTANT || borderMode > B200PP_BORDER_REFLECT101)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid borderType %d", borderMode);
    if (src->numSamples != dst->numSamples)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output samples are different");
    if ((topList == nullptr) != (leftList == nullptr))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Top and left must both be lists or both be single values");
    if (!dst->imageList && src->imageList && !topList)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Variable-shape input needs per-sample top and left");
    if (!src->imageList && !dst->imageList && !topList
        && !(top >= 0 && dst->height >= top + src->height && left >= 0 && dst->width >= left + src->width))
        return fail(B200PP_ERROR_INVALID_ARGUMENT,
                    "Invalid border %d %d %d %d, top >= 0 && bottom >= 0 && left >= 0 && right >= 0, in resolution: %dx%d, "
                    "out resolution: %dx%d",
                    top, dst->height - top - src->height, left, dst->width - left - src->width, src->height, src->width,
                    dst->height, dst->width);
    if (src->numSamples < 0)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Negative batch size");
    if (src->numSamples == 0)
        return B200PP_SUCCESS;
    if ((!src->base && !src->imageList) || (!dst->base && !dst->imageList))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be cuda-accessible, pitch-linear memory");
    const int gw = dst->imageList ? dst->maxWidth : dst->width, gh = dst->imageList ? dst->maxHeight : dst->height;
    if (gw < 0 || gh < 0 || (!src->imageList && (src->width < 0 || src->height < 0)))
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Invalid image size");
    if (gw == 0 || gh == 0)
        return B200PP_SUCCESS;

    BorderKParams kp{};
    kp.src        = plain_side(src);
    kp.dst        = plain_side(dst);
    kp.numSamples = src->numSamples;
    kp.top        = top;
    kp.left       = left;
    kp.topList    = topList;
    kp.leftList   = leftList;
    kp.border     = borderMode;
    border_fill_bytes(src->dtype, src->channels, borderValue, kp.fill);
    const int       pixBytes = elem_size(src->dtype) * src->channels;
    const long long rowBytes = static_cast<long long>(gw) * pixBytes;
    if (rowBytes > 0x7fffffffll)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output size exceeds 2147483647. Tensor is too large.");
    dim3 block(32, 8);
    dim3 grid(static_cast<unsigned>((rowBytes + 511) / 512), (gh + 8 * kBorderRows - 1) / (8 * kBorderRows),
              std::min(src->numSamples, 65535));
    if (grid.y > 65535u)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Input or output tensors are too large");
    switch (pixBytes)
    {
    case 1:
        launch_border<1>(grid, block, stream, kp);
        break;
    case 2:
        launch_border<2>(grid, block, stream, kp);
        break;
    case 3:
        launch_border<3>(grid, block, stream, kp);
        break;
    case 4:
        launch_border<4>(grid, block, stream, kp);
        break;
    case 6:
        launch_border<6>(grid, block, stream, kp);
        break;
    case 8:
        launch_border<8>(grid, block, stream, kp);
        break;
    case 12:
        launch_border<12>(grid, block, stream, kp);
        break;
    default:
        launch_border<16>(grid, block, stream, kp);
        break;
    }
    return check_launch("CopyMakeBorder");
}

// Device parameter buffers of operator objects that draw per-sample parameters on the host (RandomResizedCrop): the
// handle layer (cvcuda_ops.cpp) does not include the CUDA runtime, so allocation and upload live here.
extern "C" int b200ppParamBufferCreate(void **dev, size_t bytes)
{
    if (!dev)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    *dev = nullptr;
    if (bytes == 0)
        return B200PP_SUCCESS;
    if (cudaMalloc(dev, bytes) != cudaSuccess)
    {
        cudaGetLastError();
        return fail(B200PP_ERROR_INTERNAL, "Cannot allocate %zu bytes of device memory for operator parameters", bytes);
    }
    return B200PP_SUCCESS;
}

extern "C" void b200ppParamBufferDestroy(void *dev)
{
    if (dev)
        cudaFree(dev);
}

// Copy from pageable host memory: the runtime stages it before returning, so the caller may reuse `host` at once.
extern "C" int b200ppParamBufferUpload(void *dev, const void *host, size_t bytes, cudaStream_t stream)
{
    if (bytes == 0)
        return B200PP_SUCCESS;
    if (!dev || !host)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    const cudaError_t e = cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess)
        return fail(B200PP_ERROR_INTERNAL, "Parameter upload failed: %s", cudaGetErrorString(e));
    return B200PP_SUCCESS;
}

extern "C" const char *b200ppGetLastErrorMessage(void)
{
    return t_lastError;
}

extern "C" int b200ppSetKernelPath(int path)
{
    return g_kernelPath.exchange(path);
}

extern "C" uint64_t b200ppGetLaunchCount(void)
{
    return g_launchCount.load();
}

extern "C" int b200ppSelfTestWaitTimeout(uint32_t limitMs, cudaStream_t stream)
{
    if (limitMs == 0 || limitMs > 1000)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "The wait limit of the self-test must be 1..1000 ms");
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess)
        device_facts(dev); // sets up the host view of the error word on first use
    wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(static_cast<unsigned long long>(limitMs) * 1000000ull);
    return check_launch("wait self-test");
}

extern "C" int b200ppReadDeviceError(uint32_t *outError)
{
    if (!outError)
        return fail(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_deviceError, sizeof(v)) != cudaSuccess
        || cudaMemcpyToSymbol(g_deviceError, &zero, sizeof(zero)) != cudaSuccess)
    {
        cudaGetLastError();
        return fail(B200PP_ERROR_INTERNAL, "Could not read the device error word");
    }
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess)
        if (volatile unsigned int *w = device_facts(dev).errorMirror)
            *w = 0;
    *outError = v;
    return B200PP_SUCCESS;
}
