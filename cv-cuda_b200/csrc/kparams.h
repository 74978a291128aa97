// Kernel argument blocks shared by the host dispatch code and the device kernels.
#ifndef CVCUDA_B200_KPARAMS_H
#define CVCUDA_B200_KPARAMS_H

#include <cuda_runtime.h>
#include <cvcuda_b200/preproc.h>

#include <stdint.h>

namespace b200pp {

enum DstKind
{
    DST_U8  = 0,
    DST_F32 = 1,
    DST_F16 = 2
};

// Arguments of the resize kernels (passed by value in the kernel parameter space).
struct ResizeKParams
{
    // source: dense tensor, or a device list of image descriptors when `list` is not null
    const uint8_t           *srcBase;
    long long                srcSampleStride, srcRowStride;
    int                      srcW, srcH;
    const B200ppImageBuffer *list;
    const int               *roi;
    long long                roiStride; // bytes
    const int               *flip;
    int                      numSamples;
    // srcW / resizeW and srcH / resizeH in float32, worked out on the host for sources without per-sample sizes
    // (the same correctly rounded quotient the device would compute)
    float                    denseScaleW, denseScaleH;

    // geometry
    int   resizeW, resizeH, cropX, cropY, srcCast;
    int   dstX, dstY, regionW, regionH;
    float padValue;

    // affine step; constants indexed by source channel
    int   perChannel;
    float scale, offset;
    float base[3], mul[3];
    float gscale, shift;
    int   mapC[3]; // output channel of source channel c

    // destination
    uint8_t  *dst;
    long long dSample, dRow, dPix, dChan; // bytes
    int       dstW, dstH;
};

// Shape of the staged pipeline, chosen on the host.
struct StagedCfg
{
    int       stages;       // ring depth
    int       segBytes;     // shared-memory bytes reserved per staged source row (multiple of 128)
    int       rowsPerStage; // source row segments per destination row: 2 for linear, 1 for nearest
    int       unitRows;     // destination rows per work unit (1..4)
    int       chunkCols;    // destination columns per work unit (at most 128 * colBlocks)
    int       colBlocks;    // 128-column blocks per unit; the warps of a consumer team are a multiple of it
    int       teams;        // consumer teams per CTA; team t consumes the CTA's units t, t + teams, ...
    int       chunksPerRow;
    long long totalUnits;   // numSamples * ceil(dstH / unitRows) * chunksPerRow
    long long blockUnits;   // consecutive units dealt to a CTA at a time
    int       probe;        // test hook: consumers skip the taps and the arithmetic and store the pad value (memory-only run)
};

// Arguments of the crop/flip/normalise kernel.
struct SliceKParams
{
    const uint8_t           *srcBase; // dense (not reachable through the public operator, used by tests)
    long long                srcSampleStride, srcRowStride, srcPlaneStride;
    int                      srcW, srcH;
    const B200ppImageBuffer *list;
    int                      srcPlanar, channels, numSamples;

    const int *cropRect;
    long long  cropRectStride;
    const int *flip;
    int        border;
    float      borderAsSrc; // border value after static_cast to the source type, promoted back to float

    const float *base;
    long long    baseChanStride;
    int          baseCh;
    const float *scale;
    long long    scaleChanStride;
    int          scaleCh;
    float        gscale, shift, epsilon;
    int          stddev;

    uint8_t  *dst;
    long long dSample, dRow, dPix, dChan;
    int       dstW, dstH;
};

} // namespace b200pp

#endif
