// Handle-based operator entry points: the symbols the reference's libcvcuda exports for the fused pre-processing
// path, implemented on top of the plain-C launch layer (library.cu).
//
// Tensor / image-batch handles belong to the reference's object-model library (libnvcv_types). This file never looks
// inside them: it asks that library, found in the running process, to export their contents
// (reference call sites: src/cvcuda/priv/OpResizeCropConvertReformat.cu:423-438,561-583,
//  src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:373-428).
#include <cvcuda_b200/cvcuda_ops.h>

#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <mutex>
#include <new>

namespace {

// ---------------------------------------------------------------------------------------------- object-model functions

enum DataKind // NVCVDataKind (nvcv/DataLayout.h:260-267)
{
    KIND_UNSIGNED = 0,
    KIND_SIGNED   = 1,
    KIND_FLOAT    = 2,
    KIND_COMPLEX  = 3
};

struct NvcvApi
{
    NVCVStatus (*tensorExportData)(NVCVTensorHandle, NVCVTensorData *)                     = nullptr;
    NVCVStatus (*imageBatchExportData)(NVCVImageBatchHandle, cudaStream_t, NVCVImageBatchData *) = nullptr;
    NVCVStatus (*dataTypeGetDataKind)(NVCVDataType, int *)                                  = nullptr;
    NVCVStatus (*dataTypeGetBitsPerChannel)(NVCVDataType, int32_t *)                        = nullptr;
    NVCVStatus (*imageFormatGetDataKind)(NVCVImageFormat, int *)                            = nullptr;
    NVCVStatus (*imageFormatGetBitsPerChannel)(NVCVImageFormat, int32_t *)                  = nullptr;
    NVCVStatus (*imageFormatGetNumChannels)(NVCVImageFormat, int32_t *)                     = nullptr;
    NVCVStatus (*imageFormatGetNumPlanes)(NVCVImageFormat, int32_t *)                       = nullptr;
    void (*setThreadStatus)(NVCVStatus, const char *, ...)                                  = nullptr;
    // per-image sizes of a variable-shape batch on the host (RandomResizedCrop draws its rectangles from them)
    NVCVStatus (*imageBatchVarShapeGetImages)(NVCVImageBatchHandle, int32_t, NVCVImageHandle *, int32_t) = nullptr;
    NVCVStatus (*imageGetSize)(NVCVImageHandle, int32_t *, int32_t *)                       = nullptr;
    NVCVStatus (*imageDecRef)(NVCVImageHandle, int *)                                       = nullptr;
    bool ok                                                                                 = false;
};

const NvcvApi &nvcv()
{
    static NvcvApi        api;
    static std::once_flag once;
    std::call_once(once, [] {
        auto find = [](const char *name) -> void * {
            if (void *p = dlsym(RTLD_DEFAULT, name))
                return p;
            // not yet in the process: load the object-model library the way libcvcuda depends on it
            for (const char *lib : {"libnvcv_types.so.0", "libnvcv_types.so"})
                if (void *h = dlopen(lib, RTLD_NOW | RTLD_GLOBAL))
                    if (void *p = dlsym(h, name))
                        return p;
            return nullptr;
        };
#define B200_BIND(field, symbol) api.field = reinterpret_cast<decltype(api.field)>(find(symbol))
        B200_BIND(tensorExportData, "nvcvTensorExportData");
        B200_BIND(imageBatchExportData, "nvcvImageBatchExportData");
        B200_BIND(dataTypeGetDataKind, "nvcvDataTypeGetDataKind");
        B200_BIND(dataTypeGetBitsPerChannel, "nvcvDataTypeGetBitsPerChannel");
        B200_BIND(imageFormatGetDataKind, "nvcvImageFormatGetDataKind");
        B200_BIND(imageFormatGetBitsPerChannel, "nvcvImageFormatGetBitsPerChannel");
        B200_BIND(imageFormatGetNumChannels, "nvcvImageFormatGetNumChannels");
        B200_BIND(imageFormatGetNumPlanes, "nvcvImageFormatGetNumPlanes");
        B200_BIND(setThreadStatus, "nvcvSetThreadStatus");
        B200_BIND(imageBatchVarShapeGetImages, "nvcvImageBatchVarShapeGetImages");
        B200_BIND(imageGetSize, "nvcvImageGetSize");
        B200_BIND(imageDecRef, "nvcvImageDecRef");
#undef B200_BIND
        api.ok = api.tensorExportData && api.imageBatchExportData && api.dataTypeGetDataKind
              && api.dataTypeGetBitsPerChannel && api.imageFormatGetDataKind && api.imageFormatGetBitsPerChannel
              && api.imageFormatGetNumChannels && api.imageFormatGetNumPlanes;
    });
    return api;
}

// Sets the thread's last status the way nvcv::ProtectCall does (nvcv/Exception.hpp:162-222) and returns it.
NVCVStatus report(NVCVStatus status, const char *fmt, ...)
{
    char    msg[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    if (nvcv().setThreadStatus)
        nvcv().setThreadStatus(status, "%s", msg);
    return status;
}

// Success leaves the thread's status untouched, as nvcv::ProtectCall does (nvcv/Exception.hpp:209-222).
NVCVStatus forward(int status)
{
    if (status == B200PP_SUCCESS)
        return B200PP_SUCCESS;
    return report(status, "%s", b200ppGetLastErrorMessage());
}

// ---------------------------------------------------------------------------------------------- operator objects

constexpr uint64_t kMagic = 0xB2000C0DA0F5ED01ull;

enum OpKind
{
    OP_RESIZE_CROP_CONVERT_REFORMAT  = 1,
    OP_CROP_FLIP_NORMALIZE_REFORMAT = 2,
    OP_RESIZE                       = 3,
    OP_NORMALIZE                    = 4,
    OP_REFORMAT                     = 5,
    OP_CONVERT_TO                   = 6,
    OP_COPY_MAKE_BORDER             = 7,
    OP_RANDOM_RESIZED_CROP          = 8
};

// The handle is the object pointer itself, as in the reference (src/cvcuda/priv/IOperator.hpp:37-40). Operators hold
// no mutable state, so one handle may be used from any number of threads and streams.
struct Operator
{
    uint64_t magic;
    int      kind;
    // RandomResizedCrop only (the one operator with state: its generator advances with every call, as in the
    // reference; calls on one such handle must not overlap)
    B200ppRandomCrop *generator   = nullptr;
    int32_t          *rectsDevice = nullptr;
    int32_t          *rectsHost   = nullptr;
    int               maxBatch    = 0;
};

NVCVStatus create(NVCVOperatorHandle *handle, int kind)
{
    if (handle == nullptr)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Pointer to NVCVOperator handle must not be NULL");
    Operator *op = new (std::nothrow) Operator{kMagic, kind};
    if (!op)
        return report(7 /* NVCV_ERROR_OUT_OF_MEMORY */, "Not enough memory to create the operator");
    *handle = reinterpret_cast<NVCVOperatorHandle>(op);
    return forward(B200PP_SUCCESS);
}

// NULL -> INVALID_ARGUMENT, another operator's handle -> NOT_COMPATIBLE (src/cvcuda/priv/IOperator.hpp:56-73).
NVCVStatus check_handle(NVCVOperatorHandle handle, int kind)
{
    if (handle == nullptr)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Handle cannot be NULL");
    const Operator *op = reinterpret_cast<const Operator *>(handle);
    if (op->magic != kMagic || op->kind != kind)
        return report(B200PP_ERROR_NOT_COMPATIBLE,
                      "Handle doesn't correspond to the requested object or was already destroyed.");
    return B200PP_SUCCESS;
}

// ---------------------------------------------------------------------------------------------- handle unpacking

int element_type(int kind, int bits)
{
    if (kind == KIND_UNSIGNED)
        return bits == 8 ? B200PP_U8 : bits == 16 ? B200PP_U16 : bits == 32 ? B200PP_U32 : -1;
    if (kind == KIND_SIGNED)
        return bits == 8 ? B200PP_S8 : bits == 16 ? B200PP_S16 : bits == 32 ? B200PP_S32 : -1;
    if (kind == KIND_FLOAT)
        return bits == 32 ? B200PP_F32 : bits == 16 ? B200PP_F16 : -1;
    return -1;
}

// Image view of a tensor: the rules of nvcv::TensorDataAccessStridedImagePlanar
// (nvcv/TensorDataAccess.hpp:389-458,564-605; accepted layouts nvcv/TensorShapeInfo.hpp:334-361).
struct ImageView
{
    bool     valid = false;
    int      samples = 1, channels = 1, rows = 1, cols = 1;
    bool     channelLast = true; // interleaved
    int64_t  sampleStride = 0, rowStride = 0, colStride = 0, chanStride = 0;
    uint8_t *base = nullptr;
    int      dtype = -1;
    int      elemChannels = 1; // channels carried by the element type itself (3U8 -> 3)
    int64_t  elements = 0;     // product of the shape, whatever the layout
    char     layout[NVCV_TENSOR_MAX_RANK + 1] = "";
};

bool export_tensor(NVCVTensorHandle h, ImageView &v, const char *what, NVCVStatus &status)
{
    NVCVTensorData d;
    std::memset(&d, 0, sizeof(d));
    if (h == nullptr || nvcv().tensorExportData(h, &d) != B200PP_SUCCESS || d.bufferType != 1)
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "%s must be a cuda-accessible, pitch-linear tensor", what);
        return false;
    }
    int kind = -1, bits[4] = {0, 0, 0, 0};
    nvcv().dataTypeGetDataKind(d.dtype, &kind);
    nvcv().dataTypeGetBitsPerChannel(d.dtype, bits);
    v.dtype = element_type(kind, bits[0]);
    for (int k = 1; k < 4; ++k) v.elemChannels += bits[k] != 0;
    v.base  = d.strided.basePtr;
    std::memcpy(v.layout, d.layout.data, sizeof(v.layout));
    v.layout[NVCV_TENSOR_MAX_RANK] = 0;
    v.elements = d.rank >= 1 ? 1 : 0;
    for (int i = 0; i < d.rank; ++i) v.elements *= d.shape[i];

    int iN = -1, iC = -1, iH = -1, iW = -1;
    for (int i = 0; i < d.rank; ++i)
    {
        switch (d.layout.data[i])
        {
        case 'N':
            iN = i;
            break;
        case 'C':
            iC = i;
            break;
        case 'H':
            iH = i;
            break;
        case 'W':
            iW = i;
            break;
        }
    }
    v.valid = d.rank >= 1 && iW >= 0 && (iN <= 0);
    if (!v.valid)
        return true; // exported, but not an image-like tensor: callers decide what that means
    v.samples      = iN >= 0 ? static_cast<int>(d.shape[iN]) : 1;
    v.channels     = iC >= 0 ? static_cast<int>(d.shape[iC]) : 1;
    v.rows         = iH >= 0 ? static_cast<int>(d.shape[iH]) : 1;
    v.cols         = static_cast<int>(d.shape[iW]);
    v.channelLast  = iC < 0 || iC == d.rank - 1;
    v.sampleStride = iN >= 0 ? d.strided.strides[iN] : 0;
    v.rowStride    = iH >= 0 ? d.strided.strides[iH] : 0;
    v.colStride    = d.strided.strides[iW];
    v.chanStride   = iC >= 0 ? d.strided.strides[iC] : 0;
    return true;
}

bool layout_is(const ImageView &v, const char *a, const char *b = nullptr, const char *c = nullptr,
               const char *d = nullptr)
{
    for (const char *s : {a, b, c, d})
        if (s && std::strcmp(v.layout, s) == 0)
            return true;
    return false;
}

void fill_dest(const ImageView &o, B200ppDest &d)
{
    d.base         = o.base;
    d.dtype        = o.dtype;
    d.channels     = o.channels;
    d.width        = o.cols;
    d.height       = o.rows;
    d.sampleStride = o.sampleStride;
    d.rowStride    = o.rowStride;
    d.pixStride    = o.colStride;
    d.chanStride   = o.chanStride;
}

// Output checks shared by both resize entry points
// (src/cvcuda/priv/OpResizeCropConvertReformat.cu:446-498 / :591-640).
NVCVStatus check_resize_output(const ImageView &o, int samples, int channels, bool allowHalf)
{
    if (samples != o.samples)
        return report(B200PP_ERROR_INVALID_ARGUMENT,
                      "Input and output must have the same batch size (i.e., same number of images): Provided %d "
                      "input and %d output images / samples",
                      samples, o.samples);
    if (channels != o.channels)
        return report(B200PP_ERROR_NOT_COMPATIBLE,
                      "Input and output must have same number of channels: Provided %d input and %d output channels",
                      channels, o.channels);
    if (channels != 3)
        return report(B200PP_ERROR_NOT_COMPATIBLE,
                      "Only three-channel input is currently supported: Provided %d input channels", channels);
    if (!(o.dtype == B200PP_U8 || o.dtype == B200PP_F32 || (allowHalf && o.dtype == B200PP_F16)))
        return report(B200PP_ERROR_NOT_COMPATIBLE, "Output must be of data type uchar or float.");
    return B200PP_SUCCESS;
}

NVCVStatus check_output_layout(const ImageView &o)
{
    if (!layout_is(o, "NHWC", "HWC", "NCHW", "CHW"))
        return report(B200PP_ERROR_NOT_COMPATIBLE,
                      "Output tensor must have 'NHWC', 'NCHW', 'HWC', or 'CHW' layout: Layout provided %s", o.layout);
    return B200PP_SUCCESS;
}

NVCVStatus resize_tensor(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in, NVCVTensorHandle out,
                         const B200ppResizeOp &op, bool extended)
{
    if (NVCVStatus st = check_handle(handle, OP_RESIZE_CROP_CONVERT_REFORMAT))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  i, o;
    if (!export_tensor(in, i, "Input", st) || !export_tensor(out, o, "Output", st))
        return st;
    if (!i.valid || !o.valid)
        return report(B200PP_ERROR_NOT_COMPATIBLE, "Input and output must be image-like tensors");
    if ((st = check_resize_output(o, i.samples, i.channels, extended)))
        return st;
    if (i.dtype != B200PP_U8)
        return report(B200PP_ERROR_NOT_COMPATIBLE, "Input must be of data type uchar.");
    if (!layout_is(i, "NHWC", "HWC"))
        return report(B200PP_ERROR_NOT_COMPATIBLE, "Input tensor must have 'NHWC' or 'HWC' layout: Layout provided %s",
                      i.layout);
    if ((st = check_output_layout(o)))
        return st;

    B200ppSource s;
    std::memset(&s, 0, sizeof(s));
    s.dtype        = i.dtype;
    s.channels     = i.channels;
    s.planar       = 0;
    s.numSamples   = i.samples;
    s.base         = i.base;
    s.sampleStride = i.sampleStride;
    s.rowStride    = i.rowStride;
    s.width        = i.cols;
    s.height       = i.rows;
    B200ppDest d;
    fill_dest(o, d);
    // Unlike the reference (src/cvcuda/priv/OpResizeCropConvertReformat.cu:515-519) inputs beyond 2 GiB are accepted:
    // sample offsets are 64-bit.
    return forward(b200ppResizeCropConvertReformat(&s, &d, &op, stream));
}

NVCVStatus resize_varshape(NVCVOperatorHandle handle, cudaStream_t stream, NVCVImageBatchHandle in,
                           NVCVTensorHandle out, const B200ppResizeOp &op, bool extended)
{
    if (NVCVStatus st = check_handle(handle, OP_RESIZE_CROP_CONVERT_REFORMAT))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVImageBatchData b;
    std::memset(&b, 0, sizeof(b));
    if (in == nullptr || nvcv().imageBatchExportData(in, stream, &b) != B200PP_SUCCESS || b.bufferType != 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input data must be a cuda-accessible, varshape image batch");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  o;
    if (!export_tensor(out, o, "Output", st))
        return st;
    if (b.varShapeStrided.uniqueFormat == 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT,
                      "All input images in a batch must have the same format (including number of channels)");
    if (!o.valid)
        return report(B200PP_ERROR_NOT_COMPATIBLE, "Output must be an image-like tensor");
    int channels = 0, planes = 0, kind = -1, bits[4] = {0, 0, 0, 0};
    nvcv().imageFormatGetNumChannels(b.varShapeStrided.uniqueFormat, &channels);
    nvcv().imageFormatGetNumPlanes(b.varShapeStrided.uniqueFormat, &planes);
    nvcv().imageFormatGetDataKind(b.varShapeStrided.uniqueFormat, &kind);
    nvcv().imageFormatGetBitsPerChannel(b.varShapeStrided.uniqueFormat, bits);
    if ((st = check_resize_output(o, b.numImages, channels, extended)))
        return st;
    if (element_type(kind, bits[0]) != B200PP_U8)
        return report(B200PP_ERROR_NOT_COMPATIBLE, "Input must be of data type uchar.");
    if (planes > 1)
        return report(B200PP_ERROR_NOT_COMPATIBLE, "Input must be non-planar (i.e., interleaved).");
    if ((st = check_output_layout(o)))
        return st;

    B200ppSource s;
    std::memset(&s, 0, sizeof(s));
    s.dtype      = B200PP_U8;
    s.channels   = channels;
    s.planar     = 0;
    s.numSamples = b.numImages;
    s.imageList  = b.varShapeStrided.imageList;
    s.maxWidth   = b.varShapeStrided.maxWidth;
    s.maxHeight  = b.varShapeStrided.maxHeight;
    B200ppDest d;
    fill_dest(o, d);
    return forward(b200ppResizeCropConvertReformat(&s, &d, &op, stream));
}

B200ppResizeOp reference_op(NVCVSize2D resizeDim, int interp, int2 cropPos, int manip, float scale, float offset,
                            bool srcCast)
{
    B200ppResizeOp op;
    std::memset(&op, 0, sizeof(op));
    op.resizeW = resizeDim.w;
    op.resizeH = resizeDim.h;
    op.cropX   = cropPos.x;
    op.cropY   = cropPos.y;
    op.interp  = interp;
    op.srcCast = srcCast ? 1 : 0;
    op.manip   = manip;
    op.scale   = scale;
    op.offset  = offset;
    return op;
}

// ---------------------------------------------------------------------------------------------- stand-alone Resize

// The reference accepts the channel count either in the tensor shape or baked into the element type (3U8 ...),
// src/cvcuda/priv/OpResize.cu:455-486: ImageView::elemChannels carries the latter.
NVCVStatus plain_resize_tensor(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in, NVCVTensorHandle out,
                               int interp)
{
    if (NVCVStatus st = check_handle(handle, OP_RESIZE))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  i, o;
    if (!export_tensor(in, i, "Input", st) || !export_tensor(out, o, "Output", st))
        return st;
    // order and codes of src/cvcuda/priv/OpResize.cu:501-541
    if (i.dtype != o.dtype || i.elemChannels != o.elemChannels)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input and output data type are different");
    if (std::strcmp(i.layout, o.layout) != 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input and output data layout are different");
    if (!layout_is(i, "HWC", "NHWC"))
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input must have (N)HWC layout");
    if (!i.valid || !o.valid)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input and output must be image-like tensors");
    B200ppImageSet s, d;
    std::memset(&s, 0, sizeof(s));
    std::memset(&d, 0, sizeof(d));
    const ImageView *views[2] = {&i, &o};
    B200ppImageSet  *sets[2]  = {&s, &d};
    for (int k = 0; k < 2; ++k)
    {
        sets[k]->base         = views[k]->base;
        sets[k]->dtype        = views[k]->dtype;
        sets[k]->channels     = views[k]->channels * views[k]->elemChannels;
        sets[k]->numSamples   = views[k]->samples;
        sets[k]->width        = views[k]->cols;
        sets[k]->height       = views[k]->rows;
        sets[k]->rowStride    = views[k]->rowStride;
        sets[k]->sampleStride = views[k]->sampleStride;
    }
    return forward(b200ppResize(&s, &d, interp, stream));
}

NVCVStatus plain_resize_varshape(NVCVOperatorHandle handle, cudaStream_t stream, NVCVImageBatchHandle in,
                                 NVCVImageBatchHandle out, int interp)
{
    if (NVCVStatus st = check_handle(handle, OP_RESIZE))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVImageBatchData bi, bo;
    std::memset(&bi, 0, sizeof(bi));
    std::memset(&bo, 0, sizeof(bo));
    if (in == nullptr || nvcv().imageBatchExportData(in, stream, &bi) != B200PP_SUCCESS || bi.bufferType != 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input must be cuda-accessible, varshape pitch-linear image batch");
    if (out == nullptr || nvcv().imageBatchExportData(out, stream, &bo) != B200PP_SUCCESS || bo.bufferType != 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Output must be cuda-accessible, varshape pitch-linear image batch");
    if (bi.varShapeStrided.uniqueFormat == 0 || bo.varShapeStrided.uniqueFormat == 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Images in the input and output batches must all have the same format");
    if (bi.varShapeStrided.uniqueFormat != bo.varShapeStrided.uniqueFormat)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input and output data type are different");
    int channels = 0, planes = 0, kind = -1, bits[4] = {0, 0, 0, 0};
    nvcv().imageFormatGetNumChannels(bi.varShapeStrided.uniqueFormat, &channels);
    nvcv().imageFormatGetNumPlanes(bi.varShapeStrided.uniqueFormat, &planes);
    nvcv().imageFormatGetDataKind(bi.varShapeStrided.uniqueFormat, &kind);
    nvcv().imageFormatGetBitsPerChannel(bi.varShapeStrided.uniqueFormat, bits);
    if (planes > 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Image batches must hold interleaved (single-plane) images");
    B200ppImageSet s, d;
    std::memset(&s, 0, sizeof(s));
    std::memset(&d, 0, sizeof(d));
    s.dtype = d.dtype = element_type(kind, bits[0]);
    s.channels = d.channels = channels;
    s.numSamples            = bi.numImages;
    d.numSamples            = bo.numImages;
    s.imageList             = bi.varShapeStrided.imageList;
    d.imageList             = bo.varShapeStrided.imageList;
    s.maxWidth              = bi.varShapeStrided.maxWidth;
    s.maxHeight             = bi.varShapeStrided.maxHeight;
    d.maxWidth              = bo.varShapeStrided.maxWidth;
    d.maxHeight             = bo.varShapeStrided.maxHeight;
    return forward(b200ppResize(&s, &d, interp, stream));
}

// ---------------------------------------------------------------------------------------------- stand-alone Normalize

// base / scale tensor -> pointer and the four broadcast strides (a dimension of extent 1 gets stride 0). Every extent must
// be 1 or the input's (src/cvcuda/priv/legacy/normalize.cu:300-306, checkParamShape); rows / cols < 0 stands for a
// variable-shape input, whose images have no common size, so only extent 1 fits there.
bool param_tensor(NVCVTensorHandle h, const char *what, int samples, int rows, int cols, int channels, const float *&ptr,
                  int64_t (&stride)[4], NVCVStatus &status)
{
    ImageView v;
    char      msg[96];
    std::snprintf(msg, sizeof(msg), "Input %s", what);
    if (!export_tensor(h, v, msg, status))
        return false;
    if (!v.valid || v.dtype != B200PP_F32 || !v.channelLast)
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "Input %s must be a float32 (N)HWC tensor", what);
        return false;
    }
    if (!(v.samples == 1 || v.samples == samples) || !(v.channels == 1 || v.channels == channels)
        || !(v.rows == 1 || v.rows == rows) || !(v.cols == 1 || v.cols == cols))
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT,
                        "Input %s has shape [%d,%d,%d,%d]: every extent must be 1 or equal to the input's", what, v.samples,
                        v.rows, v.cols, v.channels);
        return false;
    }
    ptr       = reinterpret_cast<const float *>(v.base);
    stride[0] = v.samples == 1 ? 0 : v.sampleStride;
    stride[1] = v.rows == 1 ? 0 : v.rowStride;
    stride[2] = v.cols == 1 ? 0 : v.colStride;
    stride[3] = v.channels == 1 ? 0 : v.chanStride;
    return true;
}

NVCVStatus normalize_common(NVCVOperatorHandle handle, cudaStream_t stream, const B200ppImageSet &s, const B200ppImageSet &d,
                            NVCVTensorHandle base, NVCVTensorHandle scale, float gscale, float shift, float epsilon,
                            uint32_t flags)
{
    (void)handle;
    NVCVStatus        st = B200PP_SUCCESS;
    B200ppNormalizeOp op;
    std::memset(&op, 0, sizeof(op));
    const int rows = s.imageList ? -1 : s.height, cols = s.imageList ? -1 : s.width;
    if (!param_tensor(base, "base", s.numSamples, rows, cols, s.channels, op.base, op.baseStride, st)
        || !param_tensor(scale, "scale", s.numSamples, rows, cols, s.channels, op.scale, op.scaleStride, st))
        return st;
    op.gscale  = gscale;
    op.shift   = shift;
    op.epsilon = epsilon;
    op.flags   = flags;
    return forward(b200ppNormalize(&s, &d, &op, stream));
}

NVCVStatus normalize_tensor(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in, NVCVTensorHandle base,
                            NVCVTensorHandle scale, NVCVTensorHandle out, float gscale, float shift, float epsilon,
                            uint32_t flags)
{
    if (NVCVStatus st = check_handle(handle, OP_NORMALIZE))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  i, o;
    if (!export_tensor(in, i, "Input", st) || !export_tensor(out, o, "Output", st))
        return st;
    // src/cvcuda/priv/legacy/normalize.cu:314-326
    if (std::strcmp(i.layout, o.layout) != 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataFormat between input (%s) and output (%s)", i.layout, o.layout);
    if (!layout_is(i, "NHWC", "HWC") || !i.valid || !o.valid)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input DataFormat %s, the valid DataFormats are: \"NHWC\", \"HWC\"",
                      i.layout);
    B200ppImageSet s, d;
    std::memset(&s, 0, sizeof(s));
    std::memset(&d, 0, sizeof(d));
    const ImageView *views[2] = {&i, &o};
    B200ppImageSet  *sets[2]  = {&s, &d};
    for (int k = 0; k < 2; ++k)
    {
        sets[k]->base         = views[k]->base;
        sets[k]->dtype        = views[k]->dtype;
        sets[k]->channels     = views[k]->channels * views[k]->elemChannels;
        sets[k]->numSamples   = views[k]->samples;
        sets[k]->width        = views[k]->cols;
        sets[k]->height       = views[k]->rows;
        sets[k]->rowStride    = views[k]->rowStride;
        sets[k]->sampleStride = views[k]->sampleStride;
    }
    return normalize_common(handle, stream, s, d, base, scale, gscale, shift, epsilon, flags);
}

NVCVStatus normalize_varshape(NVCVOperatorHandle handle, cudaStream_t stream, NVCVImageBatchHandle in, NVCVTensorHandle base,
                              NVCVTensorHandle scale, NVCVImageBatchHandle out, float gscale, float shift, float epsilon,
                              uint32_t flags)
{
    if (NVCVStatus st = check_handle(handle, OP_NORMALIZE))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVImageBatchData bi, bo;
    std::memset(&bi, 0, sizeof(bi));
    std::memset(&bo, 0, sizeof(bo));
    if (in == nullptr || nvcv().imageBatchExportData(in, stream, &bi) != B200PP_SUCCESS || bi.bufferType != 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input must be cuda-accessible, varshape pitch-linear image batch");
    if (out == nullptr || nvcv().imageBatchExportData(out, stream, &bo) != B200PP_SUCCESS || bo.bufferType != 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Output must be cuda-accessible, varshape pitch-linear image batch");
    if (bi.varShapeStrided.uniqueFormat == 0 || bo.varShapeStrided.uniqueFormat == 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Images in the input and output batches must all have the same format");
    B200ppImageSet s, d;
    std::memset(&s, 0, sizeof(s));
    std::memset(&d, 0, sizeof(d));
    const NVCVImageBatchData *batches[2] = {&bi, &bo};
    B200ppImageSet           *sets[2]    = {&s, &d};
    for (int k = 0; k < 2; ++k)
    {
        int channels = 0, planes = 0, kind = -1, bits[4] = {0, 0, 0, 0};
        nvcv().imageFormatGetNumChannels(batches[k]->varShapeStrided.uniqueFormat, &channels);
        nvcv().imageFormatGetNumPlanes(batches[k]->varShapeStrided.uniqueFormat, &planes);
        nvcv().imageFormatGetDataKind(batches[k]->varShapeStrided.uniqueFormat, &kind);
        nvcv().imageFormatGetBitsPerChannel(batches[k]->varShapeStrided.uniqueFormat, bits);
        if (planes > 1)
            return report(B200PP_ERROR_INVALID_ARGUMENT, "Image batches must hold interleaved (single-plane) images");
        sets[k]->dtype      = element_type(kind, bits[0]);
        sets[k]->channels   = channels;
        sets[k]->numSamples = batches[k]->numImages;
        sets[k]->imageList  = batches[k]->varShapeStrided.imageList;
        sets[k]->maxWidth   = batches[k]->varShapeStrided.maxWidth;
        sets[k]->maxHeight  = batches[k]->varShapeStrided.maxHeight;
    }
    return normalize_common(handle, stream, s, d, base, scale, gscale, shift, epsilon, flags);
}

// ---------------------------------------------------------------------------------------------- stand-alone Reformat

NVCVStatus reformat_tensor(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in, NVCVTensorHandle out)
{
    if (NVCVStatus st = check_handle(handle, OP_REFORMAT))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  i, o;
    if (!export_tensor(in, i, "Input", st) || !export_tensor(out, o, "Output", st))
        return st;
    // layouts and combinations of src/cvcuda/priv/legacy/reformat.cu:120-179
    if (!layout_is(i, "NHWC", "HWC", "NCHW", "CHW") || !layout_is(o, "NHWC", "HWC", "NCHW", "CHW") || !i.valid || !o.valid
        || (std::strlen(i.layout) != std::strlen(o.layout)))
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid combination of input format %s and output format %s", i.layout,
                      o.layout);
    if (i.dtype != o.dtype || i.elemChannels != o.elemChannels)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "DataType of input and output must be equal");
    if (i.samples != o.samples)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input and output samples are different");
    if (i.elemChannels != 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataType: channels must be a tensor dimension");
    B200ppDest s, d;
    fill_dest(i, s);
    fill_dest(o, d);
    return forward(b200ppReformat(&s, &d, i.samples, stream));
}

// ---------------------------------------------------------------------------------------------- stand-alone ConvertTo

NVCVStatus convert_tensor(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in, NVCVTensorHandle out,
                          double alpha, double beta)
{
    if (NVCVStatus st = check_handle(handle, OP_CONVERT_TO))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  i, o;
    if (!export_tensor(in, i, "Input", st) || !export_tensor(out, o, "Output", st))
        return st;
    // src/cvcuda/priv/legacy/convert_to.cu:140-160: both sides (N)HWC
    if (!layout_is(i, "NHWC", "HWC") || !layout_is(o, "NHWC", "HWC") || !i.valid || !o.valid)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataFormat: input and output must be kNHWC or kHWC");
    B200ppImageSet s, d;
    std::memset(&s, 0, sizeof(s));
    std::memset(&d, 0, sizeof(d));
    const ImageView *views[2] = {&i, &o};
    B200ppImageSet  *sets[2]  = {&s, &d};
    for (int k = 0; k < 2; ++k)
    {
        sets[k]->base         = views[k]->base;
        sets[k]->dtype        = views[k]->dtype;
        sets[k]->channels     = views[k]->channels * views[k]->elemChannels;
        sets[k]->numSamples   = views[k]->samples;
        sets[k]->width        = views[k]->cols;
        sets[k]->height       = views[k]->rows;
        sets[k]->rowStride    = views[k]->rowStride;
        sets[k]->sampleStride = views[k]->sampleStride;
    }
    return forward(b200ppConvertTo(&s, &d, alpha, beta, stream));
}

} // namespace

// ---------------------------------------------------------------------------------------------- stand-alone CopyMakeBorder

void image_set_from_view(const ImageView &v, B200ppImageSet &s)
{
    std::memset(&s, 0, sizeof(s));
    s.base         = v.base;
    s.dtype        = v.dtype;
    s.channels     = v.channels * v.elemChannels;
    s.numSamples   = v.samples;
    s.width        = v.cols;
    s.height       = v.rows;
    s.rowStride    = v.rowStride;
    s.sampleStride = v.sampleStride;
}

bool image_set_from_batch(NVCVImageBatchHandle h, cudaStream_t stream, const char *what, B200ppImageSet &s, NVCVStatus &status)
{
    NVCVImageBatchData b;
    std::memset(&b, 0, sizeof(b));
    if (h == nullptr || nvcv().imageBatchExportData(h, stream, &b) != B200PP_SUCCESS || b.bufferType != 1)
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "%s must be varshape image batch", what);
        return false;
    }
    if (b.varShapeStrided.uniqueFormat == 0)
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "Images in the %s batch must all have the same format", what);
        return false;
    }
    int channels = 0, planes = 0, kind = -1, bits[4] = {0, 0, 0, 0};
    nvcv().imageFormatGetNumChannels(b.varShapeStrided.uniqueFormat, &channels);
    nvcv().imageFormatGetNumPlanes(b.varShapeStrided.uniqueFormat, &planes);
    nvcv().imageFormatGetDataKind(b.varShapeStrided.uniqueFormat, &kind);
    nvcv().imageFormatGetBitsPerChannel(b.varShapeStrided.uniqueFormat, bits);
    if (planes > 1)
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "%s batch must hold interleaved (single-plane) images", what);
        return false;
    }
    std::memset(&s, 0, sizeof(s));
    s.dtype      = element_type(kind, bits[0]);
    s.channels   = channels;
    s.numSamples = b.numImages;
    s.imageList  = b.varShapeStrided.imageList;
    s.maxWidth   = b.varShapeStrided.maxWidth;
    s.maxHeight  = b.varShapeStrided.maxHeight;
    return true;
}

// top / left of the variable-shape forms: int32 (N)HWC tensors with one value per image along the width
// (src/cvcuda/priv/legacy/copy_make_border_var_shape.cu:195-219 and the kernel's ptr(0, 0, image) at :41-42).
bool offset_tensor(NVCVTensorHandle h, const char *what, int samples, const int32_t *&ptr, NVCVStatus &status)
{
    ImageView v;
    if (!export_tensor(h, v, what, status))
        return false;
    if (v.dtype != B200PP_S32)
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid %s DataType", what);
        return false;
    }
    if (!v.valid || !layout_is(v, "HWC", "NHWC"))
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid %s DataFormat", what);
        return false;
    }
    if (v.cols < samples || (v.cols > 1 && v.colStride != 4))
    {
        status = report(B200PP_ERROR_INVALID_ARGUMENT, "%s must hold one packed int32 per image along its width", what);
        return false;
    }
    ptr = reinterpret_cast<const int32_t *>(v.base);
    return true;
}

NVCVStatus border_tensor(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in, NVCVTensorHandle out, int top,
                         int left, int borderMode, const float4 &value)
{
    if (NVCVStatus st = check_handle(handle, OP_COPY_MAKE_BORDER))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  i, o;
    if (!export_tensor(in, i, "Input", st) || !export_tensor(out, o, "Output", st))
        return st;
    // order of src/cvcuda/priv/legacy/copy_make_border.cu:102-122
    if (std::strcmp(i.layout, o.layout) != 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataFormat between input (%s) and output (%s)", i.layout, o.layout);
    if (!layout_is(i, "HWC", "NHWC") || !i.valid || !o.valid)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input DataFormat %s, the valid DataFormats are: \"NHWC\", \"HWC\"",
                      i.layout);
    if (i.dtype != o.dtype || i.elemChannels != o.elemChannels)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataType between input and output");
    B200ppImageSet s, d;
    image_set_from_view(i, s);
    image_set_from_view(o, d);
    const float v[4] = {value.x, value.y, value.z, value.w};
    return forward(b200ppCopyMakeBorder(&s, &d, top, left, nullptr, nullptr, borderMode, v, stream));
}

// Variable-shape input; the output is a variable-shape batch (outBatch) or a tensor (outTensor: the "stack" form).
NVCVStatus border_varshape(NVCVOperatorHandle handle, cudaStream_t stream, NVCVImageBatchHandle in,
                           NVCVImageBatchHandle outBatch, NVCVTensorHandle outTensor, NVCVTensorHandle top,
                           NVCVTensorHandle left, int borderMode, const float4 &value)
{
    if (NVCVStatus st = check_handle(handle, OP_COPY_MAKE_BORDER))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVStatus     st = B200PP_SUCCESS;
    B200ppImageSet s, d;
    if (!image_set_from_batch(in, stream, "Input", s, st))
        return st;
    if (outBatch)
    {
        if (!image_set_from_batch(outBatch, stream, "Output", d, st))
            return st;
    }
    else
    {
        ImageView o;
        if (!export_tensor(outTensor, o, "Output", st))
            return st;
        if (!o.valid || !layout_is(o, "HWC", "NHWC"))
            return report(B200PP_ERROR_INVALID_ARGUMENT,
                          "Invalid input DataFormat %s, the valid DataFormats are: \"NHWC\", \"HWC\"", o.layout);
        image_set_from_view(o, d);
    }
    const int32_t *topPtr = nullptr, *leftPtr = nullptr;
    if (!offset_tensor(left, "Left", s.numSamples, leftPtr, st) || !offset_tensor(top, "Top", s.numSamples, topPtr, st))
        return st;
    const float v[4] = {value.x, value.y, value.z, value.w};
    return forward(b200ppCopyMakeBorder(&s, &d, 0, 0, topPtr, leftPtr, borderMode, v, stream));
}

// ---------------------------------------------------------------------------------------------- RandomResizedCrop

NVCVStatus random_crop_create(NVCVOperatorHandle *handle, double minScale, double maxScale, double minRatio, double maxRatio,
                              int32_t maxBatch, uint32_t seed)
{
    if (handle == nullptr)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Pointer to NVCVOperator handle must not be NULL");
    // src/cvcuda/priv/legacy/random_resized_crop.cu:300-304
    if (minScale > maxScale || minRatio > maxRatio)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid Parameter: scale and ratio should be of kind (min, max)");
    Operator *op = new (std::nothrow) Operator{kMagic, OP_RANDOM_RESIZED_CROP};
    if (!op)
        return report(7 /* NVCV_ERROR_OUT_OF_MEMORY */, "Not enough memory to create the operator");
    op->maxBatch = maxBatch > 0 ? maxBatch : 0;
    int st       = b200ppRandomCropCreate(&op->generator, minScale, maxScale, minRatio, maxRatio, seed);
    if (st == B200PP_SUCCESS && op->maxBatch > 0)
    {
        op->rectsHost = new (std::nothrow) int32_t[4 * static_cast<size_t>(op->maxBatch)];
        st            = op->rectsHost ? b200ppParamBufferCreate(reinterpret_cast<void **>(&op->rectsDevice),
                                                                16 * static_cast<size_t>(op->maxBatch))
                                      : B200PP_ERROR_INTERNAL;
    }
    if (st != B200PP_SUCCESS)
    {
        nvcvOperatorDestroy(reinterpret_cast<NVCVOperatorHandle>(op));
        return report(st, "Cannot create the RandomResizedCrop operator: %s", b200ppGetLastErrorMessage());
    }
    *handle = reinterpret_cast<NVCVOperatorHandle>(op);
    return B200PP_SUCCESS;
}

// Checks shared by both forms, in the reference's order (random_resized_crop.cu:410-436): channel count, element
// type, equal types, interpolation.
NVCVStatus random_crop_checks(const B200ppImageSet &s, const B200ppImageSet &d, int interp)
{
    if (s.channels > 4)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid channel number %d", s.channels);
    if (!(s.dtype == B200PP_U8 || s.dtype == B200PP_U16 || s.dtype == B200PP_S16 || s.dtype == B200PP_F32))
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataType");
    if (s.dtype != d.dtype)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "DataType of input and output must be equal");
    if (interp == 2 /* NVCV_INTERP_CUBIC */)
        return report(B200PP_ERROR_NOT_IMPLEMENTED, "Interpolation not implemented: NVCV_INTERP_CUBIC");
    if (interp != B200PP_INTERP_NEAREST && interp != B200PP_INTERP_LINEAR)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid interpolation %d", interp);
    return B200PP_SUCCESS;
}

NVCVStatus random_crop_launch(Operator *op, cudaStream_t stream, const B200ppImageSet &s, const B200ppImageSet &d, int interp)
{
    if (int st = b200ppParamBufferUpload(op->rectsDevice, op->rectsHost, 16 * static_cast<size_t>(s.numSamples), stream))
        return forward(st);
    return forward(b200ppResizedCrop(&s, &d, op->rectsDevice, interp, stream));
}

NVCVStatus random_crop_tensor(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in, NVCVTensorHandle out,
                              int interp)
{
    if (NVCVStatus st = check_handle(handle, OP_RANDOM_RESIZED_CROP))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    Operator  *op = reinterpret_cast<Operator *>(handle);
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  i, o;
    if (!export_tensor(in, i, "Input", st) || !export_tensor(out, o, "Output", st))
        return st;
    // random_resized_crop.cu:395-408
    if (std::strcmp(i.layout, o.layout) != 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid DataFormat between input (%s) and output (%s)", i.layout, o.layout);
    if (!layout_is(i, "HWC", "NHWC") || !i.valid || !o.valid)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input DataFormat %s, the valid DataFormats are: \"NHWC\", \"HWC\"",
                      i.layout);
    B200ppImageSet s, d;
    image_set_from_view(i, s);
    image_set_from_view(o, d);
    if ((st = random_crop_checks(s, d, interp)))
        return st;
    if (s.numSamples > op->maxBatch)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Batch of %d images exceeds the operator's maxBatchSize %d", s.numSamples,
                      op->maxBatch);
    for (int k = 0; k < s.numSamples; ++k)
        if (b200ppRandomCropNext(op->generator, s.height, s.width, op->rectsHost + 4 * k) != B200PP_SUCCESS)
            return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid input size %dx%d", s.width, s.height);
    return random_crop_launch(op, stream, s, d, interp);
}

NVCVStatus random_crop_varshape(NVCVOperatorHandle handle, cudaStream_t stream, NVCVImageBatchHandle in,
                                NVCVImageBatchHandle out, int interp)
{
    if (NVCVStatus st = check_handle(handle, OP_RANDOM_RESIZED_CROP))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    if (!nvcv().imageBatchVarShapeGetImages || !nvcv().imageGetSize)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types lacks nvcvImageBatchVarShapeGetImages / nvcvImageGetSize");
    Operator      *op = reinterpret_cast<Operator *>(handle);
    NVCVStatus     st = B200PP_SUCCESS;
    B200ppImageSet s, d;
    if (!image_set_from_batch(in, stream, "Input", s, st) || !image_set_from_batch(out, stream, "Output", d, st))
        return st;
    if ((st = random_crop_checks(s, d, interp)))
        return st;
    if (s.numSamples != d.numSamples)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input and output samples are different");
    if (s.numSamples > op->maxBatch)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Batch of %d images exceeds the operator's maxBatchSize %d", s.numSamples,
                      op->maxBatch);
    // one rectangle per image from that image's own size (random_resized_crop_var_shape.cu:366-380)
    for (int k = 0; k < s.numSamples; ++k)
    {
        NVCVImageHandle image = nullptr;
        int32_t         w = 0, h = 0;
        if (nvcv().imageBatchVarShapeGetImages(in, k, &image, 1) != B200PP_SUCCESS || image == nullptr)
            return report(B200PP_ERROR_INVALID_ARGUMENT, "Cannot access image %d of the input batch", k);
        const NVCVStatus sizeStatus = nvcv().imageGetSize(image, &w, &h);
        if (nvcv().imageDecRef)
            nvcv().imageDecRef(image, nullptr);
        if (sizeStatus != B200PP_SUCCESS || b200ppRandomCropNext(op->generator, h, w, op->rectsHost + 4 * k) != B200PP_SUCCESS)
            return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid size of input image %d", k);
    }
    return random_crop_launch(op, stream, s, d, interp);
}

// ================================================================================================ exported symbols

extern "C" NVCVStatus cvcudaRandomResizedCropCreate(NVCVOperatorHandle *handle, double minScale, double maxScale,
                                                    double minRatio, double maxRatio, int32_t maxBatchSize, uint32_t seed)
{
    return random_crop_create(handle, minScale, maxScale, minRatio, maxRatio, maxBatchSize, seed);
}

extern "C" NVCVStatus cvcudaRandomResizedCropSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                                    NVCVTensorHandle out, const NVCVInterpolationType interpolation)
{
    return random_crop_tensor(handle, stream, in, out, static_cast<int>(interpolation));
}

extern "C" NVCVStatus cvcudaRandomResizedCropVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                            NVCVImageBatchHandle in, NVCVImageBatchHandle out,
                                                            const NVCVInterpolationType interpolation)
{
    return random_crop_varshape(handle, stream, in, out, static_cast<int>(interpolation));
}

extern "C" NVCVStatus cvcudaCopyMakeBorderCreate(NVCVOperatorHandle *handle)
{
    return create(handle, OP_COPY_MAKE_BORDER);
}

extern "C" NVCVStatus cvcudaCopyMakeBorderSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                                 NVCVTensorHandle out, int32_t top, int32_t left, NVCVBorderType borderMode,
                                                 const float4 borderValue)
{
    return border_tensor(handle, stream, in, out, top, left, static_cast<int>(borderMode), borderValue);
}

extern "C" NVCVStatus cvcudaCopyMakeBorderVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                         NVCVImageBatchHandle in, NVCVImageBatchHandle out,
                                                         NVCVTensorHandle top, NVCVTensorHandle left,
                                                         NVCVBorderType borderMode, const float4 borderValue)
{
    if (out == nullptr)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Output must be varshape image batch");
    return border_varshape(handle, stream, in, out, nullptr, top, left, static_cast<int>(borderMode), borderValue);
}

extern "C" NVCVStatus cvcudaCopyMakeBorderVarShapeStackSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                              NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                              NVCVTensorHandle top, NVCVTensorHandle left,
                                                              NVCVBorderType borderMode, const float4 borderValue)
{
    return border_varshape(handle, stream, in, nullptr, out, top, left, static_cast<int>(borderMode), borderValue);
}

extern "C" NVCVStatus cvcudaConvertToCreate(NVCVOperatorHandle *handle)
{
    return create(handle, OP_CONVERT_TO);
}

extern "C" NVCVStatus cvcudaConvertToSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                            NVCVTensorHandle out, const double alpha, const double beta)
{
    return convert_tensor(handle, stream, in, out, alpha, beta);
}

extern "C" NVCVStatus cvcudaReformatCreate(NVCVOperatorHandle *handle)
{
    return create(handle, OP_REFORMAT);
}

extern "C" NVCVStatus cvcudaReformatSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                           NVCVTensorHandle out)
{
    return reformat_tensor(handle, stream, in, out);
}

extern "C" NVCVStatus cvcudaNormalizeCreate(NVCVOperatorHandle *handle)
{
    return create(handle, OP_NORMALIZE);
}

extern "C" NVCVStatus cvcudaNormalizeSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                            NVCVTensorHandle base, NVCVTensorHandle scale, NVCVTensorHandle out,
                                            float global_scale, float shift, float epsilon, uint32_t flags)
{
    return normalize_tensor(handle, stream, in, base, scale, out, global_scale, shift, epsilon, flags);
}

extern "C" NVCVStatus cvcudaNormalizeVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVImageBatchHandle in,
                                                    NVCVTensorHandle base, NVCVTensorHandle scale, NVCVImageBatchHandle out,
                                                    float global_scale, float shift, float epsilon, uint32_t flags)
{
    return normalize_varshape(handle, stream, in, base, scale, out, global_scale, shift, epsilon, flags);
}

extern "C" NVCVStatus cvcudaResizeCreate(NVCVOperatorHandle *handle)
{
    return create(handle, OP_RESIZE);
}

extern "C" NVCVStatus cvcudaResizeSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVTensorHandle in,
                                         NVCVTensorHandle out, const NVCVInterpolationType interpolation)
{
    return plain_resize_tensor(handle, stream, in, out, static_cast<int>(interpolation));
}

extern "C" NVCVStatus cvcudaResizeVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream, NVCVImageBatchHandle in,
                                                 NVCVImageBatchHandle out, const NVCVInterpolationType interpolation)
{
    return plain_resize_varshape(handle, stream, in, out, static_cast<int>(interpolation));
}

extern "C" NVCVStatus cvcudaResizeCropConvertReformatCreate(NVCVOperatorHandle *handle)
{
    return create(handle, OP_RESIZE_CROP_CONVERT_REFORMAT);
}

extern "C" NVCVStatus cvcudaCropFlipNormalizeReformatCreate(NVCVOperatorHandle *handle)
{
    return create(handle, OP_CROP_FLIP_NORMALIZE_REFORMAT);
}

extern "C" void nvcvOperatorDestroy(NVCVOperatorHandle handle)
{
    Operator *op = reinterpret_cast<Operator *>(handle);
    if (op && op->magic == kMagic)
    {
        op->magic = 0;
        b200ppRandomCropDestroy(op->generator);
        b200ppParamBufferDestroy(op->rectsDevice);
        delete[] op->rectsHost;
        delete op;
    }
}

extern "C" NVCVStatus cvcudaResizeCropConvertReformatSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                            NVCVTensorHandle in, NVCVTensorHandle out,
                                                            const NVCVSize2D resizeDim,
                                                            const NVCVInterpolationType interpolation,
                                                            const int2 cropPos, const NVCVChannelManip manip,
                                                            const float scale, const float offset, const bool srcCast)
{
    return resize_tensor(handle, stream, in, out,
                         reference_op(resizeDim, interpolation, cropPos, manip, scale, offset, srcCast), false);
}

extern "C" NVCVStatus cvcudaResizeCropConvertReformatVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                                    NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                                    const NVCVSize2D resizeDim,
                                                                    const NVCVInterpolationType interpolation,
                                                                    const int2 cropPos, const NVCVChannelManip manip,
                                                                    const float scale, const float offset,
                                                                    const bool srcCast)
{
    return resize_varshape(handle, stream, in, out,
                           reference_op(resizeDim, interpolation, cropPos, manip, scale, offset, srcCast), false);
}

extern "C" NVCVStatus cvcudaB200FusedPreprocessSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                      NVCVTensorHandle in, NVCVTensorHandle out,
                                                      const B200ppResizeOp *op)
{
    if (!op)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    return resize_tensor(handle, stream, in, out, *op, true);
}

extern "C" NVCVStatus cvcudaB200FusedPreprocessVarShapeSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                              NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                              const B200ppResizeOp *op)
{
    if (!op)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Null argument");
    return resize_varshape(handle, stream, in, out, *op, true);
}

extern "C" NVCVStatus cvcudaCropFlipNormalizeReformatSubmit(NVCVOperatorHandle handle, cudaStream_t stream,
                                                            NVCVImageBatchHandle in, NVCVTensorHandle out,
                                                            NVCVTensorHandle cropRect, NVCVBorderType borderMode,
                                                            float borderValue, NVCVTensorHandle flipCode,
                                                            NVCVTensorHandle base, NVCVTensorHandle scale,
                                                            float global_scale, float shift, float epsilon,
                                                            uint32_t flags)
{
    if (NVCVStatus st = check_handle(handle, OP_CROP_FLIP_NORMALIZE_REFORMAT))
        return st;
    if (!nvcv().ok)
        return report(B200PP_ERROR_INTERNAL, "libnvcv_types is not loaded in this process");
    NVCVImageBatchData b;
    std::memset(&b, 0, sizeof(b));
    if (in == nullptr || nvcv().imageBatchExportData(in, stream, &b) != B200PP_SUCCESS || b.bufferType != 1)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input must be cuda-accessible, pitch-linear tensor");
    NVCVStatus st = B200PP_SUCCESS;
    ImageView  o, fc, bs, sc, cr;
    if (!export_tensor(out, o, "Output", st) || !export_tensor(flipCode, fc, "Input flipCode", st)
        || !export_tensor(base, bs, "Input base", st) || !export_tensor(scale, sc, "Input scale", st)
        || !export_tensor(cropRect, cr, "Input cropRect", st))
        return st;
    if (!o.valid || !bs.valid || !sc.valid || !cr.valid)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Output, base, scale and cropRect must be image-like tensors");

    // The reference reads these tensors through typed accessors without looking at their element types or extents
    // (OpCropFlipNormalizeReformat.cu:208-215); here a mismatch is refused before any pointer is reinterpreted.
    if (fc.dtype != B200PP_S32 || cr.dtype != B200PP_S32)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "flipCode and cropRect must be int32 tensors");
    if (bs.dtype != B200PP_F32 || sc.dtype != B200PP_F32)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "base and scale must be float32 tensors");
    if (fc.elements < b.numImages)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "flipCode must hold one code per input image: %lld for %d images",
                      static_cast<long long>(fc.elements), b.numImages);
    if (cr.samples < b.numImages || cr.elements < int64_t(4) * cr.samples)
        return report(B200PP_ERROR_INVALID_ARGUMENT,
                      "cropRect must hold four int32 values per input image: shape [N,1,1,4] with N >= %d", b.numImages);
    if (b.varShapeStrided.uniqueFormat == 0)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "All images of the input batch must have the same format");

    int channels = 0, planes = 0, kind = -1, bits[4] = {0, 0, 0, 0};
    nvcv().imageFormatGetNumChannels(b.varShapeStrided.uniqueFormat, &channels);
    nvcv().imageFormatGetNumPlanes(b.varShapeStrided.uniqueFormat, &planes);
    nvcv().imageFormatGetDataKind(b.varShapeStrided.uniqueFormat, &kind);
    nvcv().imageFormatGetBitsPerChannel(b.varShapeStrided.uniqueFormat, bits);
    if (kind == KIND_COMPLEX)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Input DataKind must be unsigned, signed or float");
    const int srcType = element_type(kind, bits[0]);
    // float16 is no input type of the reference's dispatch table (OpCropFlipNormalizeReformat.cu:453-458)
    if (srcType < 0 || srcType == B200PP_F16)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Unsupported input data type");
    // ... nor an output type (:335-341); the plain-C layer offers it as an addition
    if (o.dtype < 0 || o.dtype == B200PP_F16)
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Unsupported output data type");
    if (!layout_is(o, "NHWC", "NCHW"))
        return report(B200PP_ERROR_INVALID_ARGUMENT, "Invalid tensor layout in output");
    // The kernel writes numImages samples of the input's channel count (OpCropFlipNormalizeReformat.cu:264-267 sizes its
    // grid by the input batch): a smaller output would be overrun.
    if (o.samples < b.numImages || o.channels < channels)
        return report(B200PP_ERROR_INVALID_ARGUMENT,
                      "Output must have at least the input's samples and channels: %d x %d provided for %d x %d",
                      o.samples, o.channels, b.numImages, channels);

    B200ppSource s;
    std::memset(&s, 0, sizeof(s));
    s.dtype      = srcType;
    s.channels   = channels;
    s.planar     = planes > 1;
    s.numSamples = b.numImages;
    s.imageList  = b.varShapeStrided.imageList;
    s.maxWidth   = b.varShapeStrided.maxWidth;
    s.maxHeight  = b.varShapeStrided.maxHeight;
    B200ppDest d;
    fill_dest(o, d);
    d.channels = channels; // the kernel writes the input's channels (OpCropFlipNormalizeReformat.cu:264-267)

    B200ppSliceOp op;
    std::memset(&op, 0, sizeof(op));
    op.cropRect        = reinterpret_cast<const int32_t *>(cr.base);
    op.cropRectStride  = cr.sampleStride;
    op.flipCode        = reinterpret_cast<const int32_t *>(fc.base);
    op.border          = borderMode;
    op.borderValue     = borderValue;
    op.base            = reinterpret_cast<const float *>(bs.base);
    op.baseChannels    = bs.channels;
    op.baseChanStride  = bs.chanStride;
    op.scale           = reinterpret_cast<const float *>(sc.base);
    op.scaleChannels   = sc.channels;
    op.scaleChanStride = sc.chanStride;
    op.gscale          = global_scale;
    op.shift           = shift;
    op.epsilon         = epsilon;
    op.flags           = flags;
    return forward(b200ppCropFlipNormalizeReformat(&s, &d, &op, stream));
}
