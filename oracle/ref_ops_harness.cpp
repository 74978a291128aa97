// TEST / BASELINE INFRASTRUCTURE ONLY -- never part of the product library.
//
// A small driver written against the reference's own header-only C++ API (nvcv::Tensor, nvcv::ImageBatchVarShape,
// cvcuda::ResizeCropConvertReformat, cvcuda::CropFlipNormalizeReformat, ... from src/nvcv/src/include and
// src/cvcuda/include of the reference tree) and its real object-model library (libnvcv_types, compiled from the reference
// tree by build_oracle.py::build_ref_ops). It is compiled twice from this one source:
//
//   libharness_b200.so  linked against libcvcuda_b200.so  -- the operator symbols resolve to the B200 library, so the
//                       reference's wrappers, its real tensor / image-batch handles and the lazy descriptor upload of
//                       ImageBatchVarShape::exportData (src/nvcv/src/priv/ImageBatchVarShape.cpp:215-254) run under it;
//   libharness_ref.so   linked against libcvcuda_ref.so   -- the reference's own operators (sm_100a build) behind the very
//                       same calls: the "reference CUDA operator on the same GPU" baseline.
//
// Every entry point takes and returns HOST arrays; device memory is allocated by the nvcv objects themselves. A failed call
// returns the NVCVStatus the wrapper threw (or -1) and keeps the message for h_last_message().
#include <cuda_runtime.h>

#include <cvcuda/OpConvertTo.hpp>
#include <cvcuda/OpCopyMakeBorder.hpp>
#include <cvcuda/OpCropFlipNormalizeReformat.hpp>
#include <cvcuda/OpNormalize.hpp>
#include <cvcuda/OpRandomResizedCrop.hpp>
#include <cvcuda/OpReformat.hpp>
#include <cvcuda/OpResize.hpp>
#include <cvcuda/OpResizeCropConvertReformat.hpp>
#include <nvcv/Image.hpp>
#include <nvcv/ImageBatch.hpp>
#include <nvcv/Tensor.hpp>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#ifdef HARNESS_B200
#    include <cvcuda_b200/preproc.h>
extern "C" NVCVStatus cvcudaB200FusedPreprocessSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                                      NVCVTensorHandle out, const B200ppResizeOp *op);
extern "C" NVCVStatus cvcudaB200FusedPreprocessVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                              NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                              const B200ppResizeOp *op);
#endif

namespace {

thread_local std::string t_message;

template<class F>
int guarded(F &&f)
{
    try
    {
        f();
        return 0;
    }
    catch (const nvcv::Exception &e)
    {
        t_message = e.what();
        return static_cast<int>(e.code());
    }
    catch (const std::exception &e)
    {
        t_message = e.what();
        return -1;
    }
}

void check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess)
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// element type codes shared with the Python side: 0 u8, 1 s8, 2 u16, 3 s16, 4 u32, 5 s32, 6 f32, 7 f16
nvcv::DataType dtype_of(int code)
{
    switch (code)
    {
    case 0:
        return nvcv::TYPE_U8;
    case 1:
        return nvcv::TYPE_S8;
    case 2:
        return nvcv::TYPE_U16;
    case 3:
        return nvcv::TYPE_S16;
    case 4:
        return nvcv::TYPE_U32;
    case 5:
        return nvcv::TYPE_S32;
    case 6:
        return nvcv::TYPE_F32;
    case 7:
        return nvcv::TYPE_F16;
    }
    throw std::runtime_error("unknown element type code");
}

int elem_size(int code)
{
    return code <= 1 ? 1 : (code <= 3 || code == 7 ? 2 : 4);
}

// Interleaved / planar image formats by (element type, channels, planar).
nvcv::ImageFormat format_of(int code, int channels, bool planar)
{
    if (code == 0 && channels == 1)
        return nvcv::FMT_U8;
    if (code == 0 && channels == 3)
        return planar ? nvcv::FMT_RGB8p : nvcv::FMT_RGB8;
    if (code == 0 && channels == 4)
        return planar ? nvcv::FMT_RGBA8p : nvcv::FMT_RGBA8;
    if (code == 6 && channels == 1)
        return nvcv::FMT_F32;
    if (code == 6 && channels == 3)
        return planar ? nvcv::FMT_RGBf32p : nvcv::FMT_RGBf32;
    if (code == 6 && channels == 4)
        return planar ? nvcv::FMT_RGBAf32p : nvcv::FMT_RGBAf32;
    if (code == 5 && channels == 1)
        return nvcv::FMT_S32;
    if (code == 3 && channels == 1)
        return nvcv::FMT_S16;
    if (code == 2 && channels == 1)
        return nvcv::FMT_U16;
    throw std::runtime_error("no image format for this element type / channel count");
}

// A rank-4 image tensor, NHWC or NCHW, created by the reference's allocator (pitch rules of src/nvcv/src/priv/Tensor.cpp).
nvcv::Tensor make_tensor(int n, int h, int w, int c, bool planar, int code)
{
    if (planar)
        return nvcv::Tensor(nvcv::TensorShape({n, c, h, w}, "NCHW"), dtype_of(code));
    return nvcv::Tensor(nvcv::TensorShape({n, h, w, c}, "NHWC"), dtype_of(code));
}

// Host <-> device copies of a whole rank-4 tensor: the last two dimensions of NHWC and the last one of NCHW are packed, the
// dimension before them is the pitched row.
void copy_tensor(const nvcv::Tensor &t, void *host, bool toDevice)
{
    auto data = t.exportData<nvcv::TensorDataStridedCuda>();
    if (!data)
        throw std::runtime_error("tensor is not strided CUDA memory");
    const int  rank = data->rank();
    const auto es   = static_cast<size_t>(data->dtype().strideBytes());
    auto      *dev  = reinterpret_cast<uint8_t *>(data->basePtr());
    auto      *hst  = static_cast<uint8_t *>(host);
    if (rank == 1)
    {
        const size_t bytes = static_cast<size_t>(data->shape(0)) * es;
        check(toDevice ? cudaMemcpy(dev, hst, bytes, cudaMemcpyHostToDevice) : cudaMemcpy(hst, dev, bytes, cudaMemcpyDeviceToHost),
              "cudaMemcpy");
        return;
    }
    if (rank != 4)
        throw std::runtime_error("copy_tensor handles rank 1 and rank 4");
    const bool   nhwc     = data->layout() == nvcv::TENSOR_NHWC;
    const int    rowDim   = nhwc ? 1 : 2;
    const size_t rowBytes = (nhwc ? data->shape(2) * data->shape(3) : data->shape(3)) * es;
    const int    outer1   = nhwc ? 1 : static_cast<int>(data->shape(1));
    const int    rows     = static_cast<int>(data->shape(rowDim));
    for (int n = 0; n < data->shape(0); ++n)
        for (int p = 0; p < outer1; ++p)
        {
            uint8_t *d = dev + n * data->stride(0) + (nhwc ? 0 : p * data->stride(1));
            uint8_t *s = hst + (static_cast<size_t>(n) * outer1 + p) * rows * rowBytes;
            check(toDevice ? cudaMemcpy2D(d, data->stride(rowDim), s, rowBytes, rowBytes, rows, cudaMemcpyHostToDevice)
                           : cudaMemcpy2D(s, rowBytes, d, data->stride(rowDim), rowBytes, rows, cudaMemcpyDeviceToHost),
                  "cudaMemcpy2D");
        }
}

// One nvcv::Image per host image, allocated by the reference's allocator (its own pitch, its own cudaMalloc).
std::vector<nvcv::Image> make_images(const void *const *images, const int *ws, const int *hs, int n, int code, int channels,
                                     bool planar)
{
    std::vector<nvcv::Image> out;
    const auto               fmt = format_of(code, channels, planar);
    const size_t             es  = elem_size(code);
    for (int i = 0; i < n; ++i)
    {
        nvcv::Image img(nvcv::Size2D{ws[i], hs[i]}, fmt);
        auto        data = img.exportData<nvcv::ImageDataStridedCuda>();
        if (!data)
            throw std::runtime_error("image is not strided CUDA memory");
        const int    planes   = data->numPlanes();
        const size_t rowBytes = static_cast<size_t>(ws[i]) * (planar ? 1 : channels) * es;
        for (int p = 0; p < planes; ++p)
        {
            const auto &pl = data->plane(p);
            check(cudaMemcpy2D(pl.basePtr, pl.rowStride, static_cast<const uint8_t *>(images[i]) + p * hs[i] * rowBytes, rowBytes,
                               rowBytes, hs[i], cudaMemcpyHostToDevice),
                  "cudaMemcpy2D");
        }
        out.push_back(img);
    }
    return out;
}

struct Stream
{
    cudaStream_t s = nullptr;

    Stream()
    {
        check(cudaStreamCreate(&s), "cudaStreamCreate");
    }

    ~Stream()
    {
        if (s)
            cudaStreamDestroy(s);
    }
};

} // namespace

static void fill_bytes(const nvcv::Tensor &t, unsigned seed)
{
    auto                 data = t.exportData<nvcv::TensorDataStridedCuda>();
    const size_t         bytes = static_cast<size_t>(data->stride(0)) * data->shape(0);
    std::vector<uint8_t> host(std::min<size_t>(bytes, size_t(64) << 20));
    unsigned             x = seed * 2654435761u + 12345u;
    for (auto &b : host)
    {
        x ^= x << 13;
        x ^= x >> 17;
        x ^= x << 5;
        b = static_cast<uint8_t>(x >> 11);
    }
    for (size_t off = 0; off < bytes; off += host.size())
        check(cudaMemcpy(reinterpret_cast<uint8_t *>(data->basePtr()) + off, host.data(), std::min(host.size(), bytes - off),
                         cudaMemcpyHostToDevice),
              "cudaMemcpy");
}

template<class F>
static float time_passes(cudaStream_t s, int warmup, int iters, F &&pass)
{
    for (int i = 0; i < warmup; ++i) pass();
    cudaEvent_t a, b;
    check(cudaEventCreate(&a), "cudaEventCreate");
    check(cudaEventCreate(&b), "cudaEventCreate");
    check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    check(cudaEventRecord(a, s), "cudaEventRecord");
    for (int i = 0; i < iters; ++i) pass();
    check(cudaEventRecord(b, s), "cudaEventRecord");
    check(cudaEventSynchronize(b), "cudaEventSynchronize");
    float ms = 0.f;
    check(cudaEventElapsedTime(&ms, a, b), "cudaEventElapsedTime");
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    return ms / static_cast<float>(iters);
}

// Chain legs time the whole chain (stage < 0) or one of its operators alone (stage = 0, 1, ...: the others are not run inside
// the timed region; every intermediate was produced once by the warm-up passes of the whole chain).
static int g_stage = -1;

static const float kMean[3] = {123.675f, 116.28f, 103.53f};
static const float kStd[3]  = {58.395f, 57.12f, 57.375f};

extern "C"
{
void h_select_stage(int stage)
{
    g_stage = stage;
}

const char *h_last_message()
{
    return t_message.c_str();
}

const char *h_which()
{
#ifdef HARNESS_B200
    return "b200";
#else
    return "reference";
#endif
}

// cvcuda::ResizeCropConvertReformat on a real NHWC uint8 tensor. dstCode: 0 u8, 6 f32, 7 f16.
int h_rccr_tensor(const uint8_t *src, int n, int h, int w, void *dst, int dstCode, int planar, int ow, int oh, int rw, int rh,
                  int interp, int cx, int cy, int manip, float scale, float offset, int srcCast)
{
    return guarded([&] {
        nvcv::Tensor in  = make_tensor(n, h, w, 3, false, 0);
        nvcv::Tensor out = make_tensor(n, oh, ow, 3, planar != 0, dstCode);
        copy_tensor(in, const_cast<uint8_t *>(src), true);
        Stream                            st;
        cvcuda::ResizeCropConvertReformat op;
        op(st.s, in, out, NVCVSize2D{rw, rh}, static_cast<NVCVInterpolationType>(interp), int2{cx, cy},
           static_cast<NVCVChannelManip>(manip), scale, offset, srcCast != 0);
        check(cudaStreamSynchronize(st.s), "cudaStreamSynchronize");
        copy_tensor(out, dst, false);
    });
}

// The same through a real ImageBatchVarShape of nvcv::Image objects. `pushLate` > 0 pushes that many of the images only after
// a first call on the shorter batch, so that exportData has to upload descriptors a second time, on this call's stream.
int h_rccr_varshape(const void *const *images, const int *ws, const int *hs, int n, void *dst, int dstCode, int planar, int ow,
                    int oh, int rw, int rh, int interp, int cx, int cy, int manip, float scale, float offset, int srcCast,
                    int pushLate)
{
    return guarded([&] {
        std::vector<nvcv::Image> keep  = make_images(images, ws, hs, n, 0, 3, false);
        const int                first = n - std::max(0, std::min(pushLate, n - 1));
        nvcv::ImageBatchVarShape batch(n);
        for (int i = 0; i < first; ++i) batch.pushBack(keep[i]);
        Stream                            st;
        cvcuda::ResizeCropConvertReformat op;
        if (first < n)
        {
            nvcv::Tensor part = make_tensor(first, oh, ow, 3, planar != 0, dstCode);
            op(st.s, batch, part, NVCVSize2D{rw, rh}, static_cast<NVCVInterpolationType>(interp), int2{cx, cy},
               static_cast<NVCVChannelManip>(manip), scale, offset, srcCast != 0);
            for (int i = first; i < n; ++i) batch.pushBack(keep[i]);
        }
        nvcv::Tensor out = make_tensor(n, oh, ow, 3, planar != 0, dstCode);
        op(st.s, batch, out, NVCVSize2D{rw, rh}, static_cast<NVCVInterpolationType>(interp), int2{cx, cy},
           static_cast<NVCVChannelManip>(manip), scale, offset, srcCast != 0);
        check(cudaStreamSynchronize(st.s), "cudaStreamSynchronize");
        copy_tensor(out, dst, false);
    });
}

// cvcuda::CropFlipNormalizeReformat with the tensors the reference's test builds
// (tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:200-330): cropRect int32 [N,1,1,4] NHWC, flipCode int32 [N],
// base / scale float32 [1,1,1,C'] NHWC.
int h_cfnr(const void *const *images, const int *ws, const int *hs, int n, int srcCode, int channels, int srcPlanar, void *dst,
           int dstCode, int dstPlanar, int ow, int oh, const int32_t *rects, int border, float borderValue, const int32_t *flips,
           const float *base, int baseC, const float *scale, int scaleC, float gscale, float shift, float epsilon, uint32_t flags)
{
    return guarded([&] {
        std::vector<nvcv::Image> keep = make_images(images, ws, hs, n, srcCode, channels, srcPlanar != 0);
        nvcv::ImageBatchVarShape batch(n);
        batch.pushBack(keep.begin(), keep.end());
        nvcv::Tensor             out   = make_tensor(n, oh, ow, channels, dstPlanar != 0, dstCode);
        nvcv::Tensor             tRect(nvcv::TensorShape({n, 1, 1, 4}, "NHWC"), nvcv::TYPE_S32);
        nvcv::Tensor             tFlip(nvcv::TensorShape({n}, "N"), nvcv::TYPE_S32);
        nvcv::Tensor             tBase(nvcv::TensorShape({1, 1, 1, baseC}, "NHWC"), nvcv::TYPE_F32);
        nvcv::Tensor             tScale(nvcv::TensorShape({1, 1, 1, scaleC}, "NHWC"), nvcv::TYPE_F32);
        copy_tensor(tRect, const_cast<int32_t *>(rects), true);
        copy_tensor(tFlip, const_cast<int32_t *>(flips), true);
        copy_tensor(tBase, const_cast<float *>(base), true);
        copy_tensor(tScale, const_cast<float *>(scale), true);
        Stream                            st;
        cvcuda::CropFlipNormalizeReformat op;
        op(st.s, batch, out, tRect, static_cast<NVCVBorderType>(border), borderValue, tFlip, tBase, tScale, gscale, shift, epsilon,
           flags);
        check(cudaStreamSynchronize(st.s), "cudaStreamSynchronize");
        copy_tensor(out, dst, false);
    });
}

// ---------------------------------------------------------------------------------------------------------------- timing
//
// Device-resident batches of seeded bytes, CUDA events on the launching stream around `iters` passes after `warmup`.
// chain = 1: the pass as the reference's users have to write it, a chain of its operators with real intermediates.
// chain = 0 (b200 build only): the one-pass extended entry point on the same real handles.

// Classification-style pass: n images of h x w -> resize (rw, rh) -> crop (cx, cy) of ow x oh -> per-channel (v - mean) / std
// -> float32 NCHW. Chain: ResizeCropConvertReformat (float32 NHWC, scale 1) -> Normalize (stddev flag) -> Reformat, with
// the source split into groups of at most `maxPerCall` images (the reference refuses inputs above 2 GiB,
// src/cvcuda/priv/OpResizeCropConvertReformat.cu:515-519). Returns ms per pass in *ms and the launches per pass in *launches.
int h_time_classify(int n, int h, int w, int rw, int rh, int cx, int cy, int ow, int oh, int interp, int chain, int maxPerCall,
                    int warmup, int iters, float *ms, int *launches)
{
    return guarded([&] {
        Stream                    st;
        const int                 groups = (n + maxPerCall - 1) / maxPerCall;
        std::vector<nvcv::Tensor> in, mid, norm, out;
        for (int g = 0; g < groups; ++g)
        {
            const int m = std::min(maxPerCall, n - g * maxPerCall);
            in.push_back(make_tensor(m, h, w, 3, false, 0));
            fill_bytes(in.back(), 1234u + g);
            out.push_back(make_tensor(m, oh, ow, 3, true, 6));
            if (chain)
            {
                mid.push_back(make_tensor(m, oh, ow, 3, false, 6));
                norm.push_back(make_tensor(m, oh, ow, 3, false, 6));
            }
        }
        nvcv::Tensor tBase(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        nvcv::Tensor tScale(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        copy_tensor(tBase, const_cast<float *>(kMean), true);
        copy_tensor(tScale, const_cast<float *>(kStd), true);
        cvcuda::ResizeCropConvertReformat rccr;
        cvcuda::Normalize                 normalize;
        cvcuda::Reformat                  reformat;
        if (chain)
        {
            auto pass = [&](int stage) {
                for (int g = 0; g < groups; ++g)
                {
                    if (stage < 0 || stage == 0)
                        rccr(st.s, in[g], mid[g], NVCVSize2D{rw, rh}, static_cast<NVCVInterpolationType>(interp), int2{cx, cy},
                             NVCV_CHANNEL_NO_OP, 1.f, 0.f, false);
                    if (stage < 0 || stage == 1)
                        normalize(st.s, mid[g], tBase, tScale, norm[g], 1.f, 0.f, 0.f, CVCUDA_NORMALIZE_SCALE_IS_STDDEV);
                    if (stage < 0 || stage == 2)
                        reformat(st.s, norm[g], out[g]);
                }
            };
            pass(-1);
            *launches = (g_stage < 0 ? 3 : 1) * groups;
            *ms       = time_passes(st.s, warmup, iters, [&] { pass(g_stage); });
        }
        else
        {
#ifdef HARNESS_B200
            B200ppResizeOp op;
            std::memset(&op, 0, sizeof(op));
            op.resizeW = rw, op.resizeH = rh, op.cropX = cx, op.cropY = cy, op.interp = interp, op.srcCast = 0;
            op.perChannel = 1, op.gscale = 1.f, op.shift = 0.f, op.scale = 1.f;
            for (int c = 0; c < 3; ++c) op.base[c] = kMean[c], op.mul[c] = 1.0f / kStd[c];
            *launches = groups;
            *ms       = time_passes(st.s, warmup, iters, [&] {
                for (int g = 0; g < groups; ++g)
                    nvcv::detail::CheckThrow(cvcudaB200FusedPreprocessSubmit(rccr.handle(), st.s, in[g].handle(), out[g].handle(), &op));
            });
#else
            throw std::runtime_error("the one-pass entry point exists in the B200 library only");
#endif
        }
    });
}

// The stock variable-shape operator on a list of n equal-sized images: ResizeCropConvertReformat(batch) -> float32 NCHW, x scale.
// Identical call in both builds (src/cvcuda/include/cvcuda/OpResizeCropConvertReformat.hpp: the ImageBatchVarShape overload).
int h_time_rccr_list(int n, int h, int w, int rw, int rh, int cx, int cy, int ow, int oh, int interp, float scale, int warmup,
                     int iters, float *ms)
{
    return guarded([&] {
        Stream                   st;
        std::vector<nvcv::Image> keep;
        nvcv::ImageBatchVarShape batch(n);
        for (int i = 0; i < n; ++i)
        {
            nvcv::Image img(nvcv::Size2D{w, h}, nvcv::FMT_RGB8);
            auto        data = img.exportData<nvcv::ImageDataStridedCuda>();
            check(cudaMemset2D(data->plane(0).basePtr, data->plane(0).rowStride, 37 + i, static_cast<size_t>(w) * 3, h), "cudaMemset2D");
            keep.push_back(img);
            batch.pushBack(img);
        }
        nvcv::Tensor                      out = make_tensor(n, oh, ow, 3, true, 6);
        cvcuda::ResizeCropConvertReformat rccr;
        *ms = time_passes(st.s, warmup, iters, [&] {
            rccr(st.s, batch, out, NVCVSize2D{rw, rh}, static_cast<NVCVInterpolationType>(interp), int2{cx, cy}, NVCV_CHANNEL_NO_OP,
                 scale, 0.f, false);
        });
    });
}

// Letterbox pass: n images of h x w -> resize to rw x rh -> placed at (0, top) of a cw x ch canvas padded with 114 -> x / 255
// -> float32 NCHW. Chain: Resize -> CopyMakeBorder -> ConvertTo -> Reformat (the channel swap of the one-pass form would be a
// fifth operator and is left out of the chain).
int h_time_letterbox(int n, int h, int w, int rw, int rh, int cw, int ch, int top, int chain, int warmup, int iters, float *ms,
                     int *launches)
{
    return guarded([&] {
        Stream       st;
        nvcv::Tensor in = make_tensor(n, h, w, 3, false, 0);
        fill_bytes(in, 4321u);
        nvcv::Tensor out = make_tensor(n, ch, cw, 3, true, 6);
        if (chain)
        {
            nvcv::Tensor            small = make_tensor(n, rh, rw, 3, false, 0), padded = make_tensor(n, ch, cw, 3, false, 0);
            nvcv::Tensor            asFloat = make_tensor(n, ch, cw, 3, false, 6);
            cvcuda::Resize          resize;
            cvcuda::CopyMakeBorder  border;
            cvcuda::ConvertTo       convert;
            cvcuda::Reformat        reformat;
            auto pass = [&](int stage) {
                if (stage < 0 || stage == 0)
                    resize(st.s, in, small, NVCV_INTERP_LINEAR);
                if (stage < 0 || stage == 1)
                    border(st.s, small, padded, top, 0, NVCV_BORDER_CONSTANT, float4{114.f, 114.f, 114.f, 0.f});
                if (stage < 0 || stage == 2)
                    convert(st.s, padded, asFloat, 1.0 / 255.0, 0.0);
                if (stage < 0 || stage == 3)
                    reformat(st.s, asFloat, out);
            };
            pass(-1);
            *launches = g_stage < 0 ? 4 : 1;
            *ms       = time_passes(st.s, warmup, iters, [&] { pass(g_stage); });
        }
        else
        {
#ifdef HARNESS_B200
            cvcuda::ResizeCropConvertReformat rccr;
            B200ppResizeOp                    op;
            std::memset(&op, 0, sizeof(op));
            op.resizeW = rw, op.resizeH = rh, op.interp = 1, op.srcCast = 1, op.manip = 1, op.scale = 1.0f / 255.0f;
            op.dstX = 0, op.dstY = top, op.regionW = rw, op.regionH = rh, op.padValue = 114.f;
            *launches = 1;
            *ms       = time_passes(st.s, warmup, iters, [&] {
                nvcv::detail::CheckThrow(cvcudaB200FusedPreprocessSubmit(rccr.handle(), st.s, in.handle(), out.handle(), &op));
            });
#else
            throw std::runtime_error("the one-pass entry point exists in the B200 library only");
#endif
        }
    });
}

// Variable-shape pass: n images (sizes ws / hs) -> one random rectangle each -> 224 x 224 -> flip -> per-channel normalise
// -> float32 NCHW. Chain: RandomResizedCrop (variable-shape, draws its own rectangles: an equal-work stand-in) ->
// CropFlipNormalizeReformat. One pass (b200 only): rectangles and flip codes given by the caller.
int h_time_varshape(const int *ws, const int *hs, int n, int ow, int oh, const int32_t *rects, const int32_t *flips, int chain,
                    int warmup, int iters, float *ms, int *launches)
{
    return guarded([&] {
        Stream                   st;
        std::vector<nvcv::Image> keep, keepSmall;
        nvcv::ImageBatchVarShape batch(n), small(n);
        for (int i = 0; i < n; ++i)
        {
            nvcv::Image img(nvcv::Size2D{ws[i], hs[i]}, nvcv::FMT_RGB8);
            auto        data = img.exportData<nvcv::ImageDataStridedCuda>();
            check(cudaMemset2D(data->plane(0).basePtr, data->plane(0).rowStride, 37 + i, static_cast<size_t>(ws[i]) * 3, hs[i]),
                  "cudaMemset2D");
            keep.push_back(img);
            batch.pushBack(img);
            nvcv::Image s(nvcv::Size2D{ow, oh}, nvcv::FMT_RGB8);
            keepSmall.push_back(s);
            small.pushBack(s);
        }
        nvcv::Tensor out = make_tensor(n, oh, ow, 3, true, 6);
        nvcv::Tensor tRect(nvcv::TensorShape({n, 1, 1, 4}, "NHWC"), nvcv::TYPE_S32);
        nvcv::Tensor tFlip(nvcv::TensorShape({n}, "N"), nvcv::TYPE_S32);
        nvcv::Tensor tBase(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        nvcv::Tensor tScale(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        copy_tensor(tFlip, const_cast<int32_t *>(flips), true);
        copy_tensor(tBase, const_cast<float *>(kMean), true);
        copy_tensor(tScale, const_cast<float *>(kStd), true);
        if (chain)
        {
            std::vector<int32_t> full(static_cast<size_t>(n) * 4);
            for (int i = 0; i < n; ++i) full[4 * i] = 0, full[4 * i + 1] = 0, full[4 * i + 2] = ow, full[4 * i + 3] = oh;
            copy_tensor(tRect, full.data(), true);
            cvcuda::RandomResizedCrop         crop(0.08, 1.0, 0.75, 4.0 / 3.0, n, 1234u);
            cvcuda::CropFlipNormalizeReformat cfnr;
            *launches = 2;
            *ms       = time_passes(st.s, warmup, iters, [&] {
                crop(st.s, batch, small, NVCV_INTERP_LINEAR);
                cfnr(st.s, small, out, tRect, NVCV_BORDER_CONSTANT, 0.f, tFlip, tBase, tScale, 1.f, 0.f, 0.f,
                     CVCUDA_NORMALIZE_SCALE_IS_STDDEV);
            });
        }
        else
        {
#ifdef HARNESS_B200
            copy_tensor(tRect, const_cast<int32_t *>(rects), true);
            auto                              rectData = tRect.exportData<nvcv::TensorDataStridedCuda>();
            auto                              flipData = tFlip.exportData<nvcv::TensorDataStridedCuda>();
            cvcuda::ResizeCropConvertReformat rccr;
            B200ppResizeOp                    op;
            std::memset(&op, 0, sizeof(op));
            op.resizeW = ow, op.resizeH = oh, op.interp = 1, op.srcCast = 1, op.perChannel = 1, op.gscale = 1.f, op.scale = 1.f;
            for (int c = 0; c < 3; ++c) op.base[c] = kMean[c], op.mul[c] = 1.0f / kStd[c];
            op.roi       = reinterpret_cast<const int32_t *>(rectData->basePtr());
            op.roiStride = rectData->stride(0);
            op.flipCode  = reinterpret_cast<const int32_t *>(flipData->basePtr());
            *launches    = 1;
            *ms          = time_passes(st.s, warmup, iters, [&] {
                nvcv::detail::CheckThrow(
                    cvcudaB200FusedPreprocessVarShapeSubmit(rccr.handle(), st.s, batch.handle(), out.handle(), &op));
            });
#else
            (void)rects;
            throw std::runtime_error("the one-pass entry point exists in the B200 library only");
#endif
        }
    });
}
// CropFlipNormalizeReformat alone, on the shape of the reference's own benchmark (bench/BenchCropFlipNormalizeReformat.cpp:
// crop = the whole image, flip both axes, REFLECT101) with RGB uint8 images of w x h -> float32 NCHW.
int h_time_cfnr(int n, int h, int w, int warmup, int iters, float *ms, int *launches)
{
    return guarded([&] {
        Stream                   st;
        std::vector<nvcv::Image> keep;
        nvcv::ImageBatchVarShape batch(n);
        for (int i = 0; i < n; ++i)
        {
            nvcv::Image img(nvcv::Size2D{w, h}, nvcv::FMT_RGB8);
            auto        data = img.exportData<nvcv::ImageDataStridedCuda>();
            check(cudaMemset2D(data->plane(0).basePtr, data->plane(0).rowStride, 11 + i, static_cast<size_t>(w) * 3, h),
                  "cudaMemset2D");
            keep.push_back(img);
            batch.pushBack(img);
        }
        nvcv::Tensor out = make_tensor(n, h, w, 3, true, 6);
        nvcv::Tensor tRect(nvcv::TensorShape({n, 1, 1, 4}, "NHWC"), nvcv::TYPE_S32);
        nvcv::Tensor tFlip(nvcv::TensorShape({n}, "N"), nvcv::TYPE_S32);
        nvcv::Tensor tBase(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        nvcv::Tensor tScale(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        std::vector<int32_t> rects(static_cast<size_t>(n) * 4), flips(n, -1);
        for (int i = 0; i < n; ++i) rects[4 * i] = 0, rects[4 * i + 1] = 0, rects[4 * i + 2] = w, rects[4 * i + 3] = h;
        copy_tensor(tRect, rects.data(), true);
        copy_tensor(tFlip, flips.data(), true);
        copy_tensor(tBase, const_cast<float *>(kMean), true);
        copy_tensor(tScale, const_cast<float *>(kStd), true);
        cvcuda::CropFlipNormalizeReformat cfnr;
        *launches = 1;
        *ms       = time_passes(st.s, warmup, iters, [&] {
            cfnr(st.s, batch, out, tRect, NVCV_BORDER_REFLECT101, 0.f, tFlip, tBase, tScale, 1.f, 0.f, 0.f,
                 CVCUDA_NORMALIZE_SCALE_IS_STDDEV);
        });
    });
}
// End to end through the handle API: page-locked HOST memory wrapped as nvcv tensors (nvcv::TensorWrapData; the kernels take
// any device-accessible address), one extended-entry-point call per pass reading the tapped source rows over PCIe and writing
// the result rows into the page-locked result. n images of h x w -> resize (rw, rh) -> crop -> per-channel normalise -> float32
// NCHW. B200 build only.
int h_time_classify_e2e_host(int n, int h, int w, int rw, int rh, int cx, int cy, int ow, int oh, int interp, int warmup,
                             int iters, float *ms)
{
    return guarded([&] {
#ifdef HARNESS_B200
        Stream       st;
        const size_t srcBytes = static_cast<size_t>(n) * h * w * 3, dstBytes = static_cast<size_t>(n) * 3 * oh * ow * sizeof(float);
        uint8_t     *hsrc     = nullptr;
        float       *hdst     = nullptr;
        check(cudaHostAlloc(reinterpret_cast<void **>(&hsrc), srcBytes, cudaHostAllocDefault), "cudaHostAlloc");
        check(cudaHostAlloc(reinterpret_cast<void **>(&hdst), dstBytes, cudaHostAllocDefault), "cudaHostAlloc");
        unsigned x = 2463534242u;
        for (size_t i = 0; i < srcBytes; i += 4)
        {
            x ^= x << 13, x ^= x >> 17, x ^= x << 5;
            std::memcpy(hsrc + i, &x, std::min<size_t>(4, srcBytes - i));
        }
        {
            nvcv::TensorDataStridedCuda::Buffer bi{}, bo{};
            bi.strides[3] = 1, bi.strides[2] = 3, bi.strides[1] = static_cast<int64_t>(w) * 3, bi.strides[0] = static_cast<int64_t>(h) * w * 3;
            bi.basePtr    = reinterpret_cast<NVCVByte *>(hsrc);
            bo.strides[3] = 4, bo.strides[2] = static_cast<int64_t>(ow) * 4, bo.strides[1] = static_cast<int64_t>(oh) * ow * 4;
            bo.strides[0] = 3 * bo.strides[1];
            bo.basePtr    = reinterpret_cast<NVCVByte *>(hdst);
            nvcv::Tensor in  = nvcv::TensorWrapData(nvcv::TensorDataStridedCuda(nvcv::TensorShape({n, h, w, 3}, "NHWC"), nvcv::TYPE_U8, bi));
            nvcv::Tensor out = nvcv::TensorWrapData(nvcv::TensorDataStridedCuda(nvcv::TensorShape({n, 3, oh, ow}, "NCHW"), nvcv::TYPE_F32, bo));
            cvcuda::ResizeCropConvertReformat rccr;
            B200ppResizeOp                    op;
            std::memset(&op, 0, sizeof(op));
            op.resizeW = rw, op.resizeH = rh, op.cropX = cx, op.cropY = cy, op.interp = interp, op.srcCast = 0;
            op.perChannel = 1, op.gscale = 1.f, op.shift = 0.f, op.scale = 1.f;
            for (int c = 0; c < 3; ++c) op.base[c] = kMean[c], op.mul[c] = 1.0f / kStd[c];
            *ms = time_passes(st.s, warmup, iters, [&] {
                nvcv::detail::CheckThrow(cvcudaB200FusedPreprocessSubmit(rccr.handle(), st.s, in.handle(), out.handle(), &op));
            });
        }
        cudaFreeHost(hsrc);
        cudaFreeHost(hdst);
#else
        (void)n, (void)h, (void)w, (void)rw, (void)rh, (void)cx, (void)cy, (void)ow, (void)oh, (void)interp, (void)warmup, (void)iters, (void)ms;
        throw std::runtime_error("the one-pass entry point exists in the B200 library only");
#endif
    });
}
// Stand-alone operators alone, on dense RGB uint8 / float32 tensors of n x h x w: op 0 = Resize to rw x rh (interp), 1 = Normalize
// uint8 -> float32 with per-channel mean / std, 2 = ConvertTo uint8 -> float32 (x 1/255), 3 = Reformat float32 NHWC -> NCHW,
// 4 = CopyMakeBorder (32 pixels on every side, constant).
int h_time_single_op(int op, int n, int h, int w, int rw, int rh, int interp, int warmup, int iters, float *ms)
{
    return guarded([&] {
        Stream       st;
        nvcv::Tensor in = make_tensor(n, h, w, 3, false, op == 3 ? 6 : 0);
        fill_bytes(in, 99u);
        nvcv::Tensor tBase(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        nvcv::Tensor tScale(nvcv::TensorShape({1, 1, 1, 3}, "NHWC"), nvcv::TYPE_F32);
        copy_tensor(tBase, const_cast<float *>(kMean), true);
        copy_tensor(tScale, const_cast<float *>(kStd), true);
        if (op == 0)
        {
            nvcv::Tensor   out = make_tensor(n, rh, rw, 3, false, 0);
            cvcuda::Resize resize;
            *ms = time_passes(st.s, warmup, iters, [&] { resize(st.s, in, out, static_cast<NVCVInterpolationType>(interp)); });
        }
        else if (op == 1)
        {
            nvcv::Tensor      out = make_tensor(n, h, w, 3, false, 6);
            cvcuda::Normalize normalize;
            *ms = time_passes(st.s, warmup, iters,
                              [&] { normalize(st.s, in, tBase, tScale, out, 1.f, 0.f, 0.f, CVCUDA_NORMALIZE_SCALE_IS_STDDEV); });
        }
        else if (op == 2)
        {
            nvcv::Tensor      out = make_tensor(n, h, w, 3, false, 6);
            cvcuda::ConvertTo convert;
            *ms = time_passes(st.s, warmup, iters, [&] { convert(st.s, in, out, 1.0 / 255.0, 0.0); });
        }
        else if (op == 3)
        {
            nvcv::Tensor     out = make_tensor(n, h, w, 3, true, 6);
            cvcuda::Reformat reformat;
            *ms = time_passes(st.s, warmup, iters, [&] { reformat(st.s, in, out); });
        }
        else
        {
            nvcv::Tensor           out = make_tensor(n, h + 64, w + 64, 3, false, 0);
            cvcuda::CopyMakeBorder border;
            *ms = time_passes(st.s, warmup, iters,
                              [&] { border(st.s, in, out, 32, 32, NVCV_BORDER_CONSTANT, float4{1.f, 2.f, 3.f, 0.f}); });
        }
    });
}
}
