// Test double of the reference's object-model library (libnvcv_types): just enough of its C API for the handle-based
// operator entry points to unpack tensors and image batches. Handles are pointers to heap copies of the exported
// structs. Type and format codes use this file's own encoding, which only the functions below interpret:
//   data type    = kind | bits << 8 | channels << 16
//   image format = kind | bits << 8 | channels << 16 | planes << 24     (0 = no unique format)
// TEST INFRASTRUCTURE ONLY.
#include <cvcuda_b200/cvcuda_ops.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#define FAKE_API extern "C" __attribute__((visibility("default")))

namespace {
thread_local NVCVStatus t_status = 0;
thread_local char       t_message[512] = "";
}

FAKE_API NVCVTensorHandle fakeTensorCreate(const NVCVTensorData *d)
{
    return reinterpret_cast<NVCVTensorHandle>(new NVCVTensorData(*d));
}

FAKE_API void fakeTensorDestroy(NVCVTensorHandle h)
{
    delete reinterpret_cast<NVCVTensorData *>(h);
}

namespace {
// The exported struct first, so a batch handle reads as one; then the host-side image sizes (width, height pairs)
// that the real library keeps in its image objects.
struct FakeBatch
{
    NVCVImageBatchData data;
    int32_t           *sizes;
};
} // namespace

FAKE_API NVCVImageBatchHandle fakeImageBatchCreate(const NVCVImageBatchData *d)
{
    return reinterpret_cast<NVCVImageBatchHandle>(new FakeBatch{*d, nullptr});
}

FAKE_API NVCVImageBatchHandle fakeImageBatchCreateSized(const NVCVImageBatchData *d, const int32_t *widthHeight)
{
    FakeBatch *b = new FakeBatch{*d, new int32_t[2 * (d->numImages > 0 ? d->numImages : 1)]};
    std::memcpy(b->sizes, widthHeight, sizeof(int32_t) * 2 * d->numImages);
    return reinterpret_cast<NVCVImageBatchHandle>(b);
}

FAKE_API void fakeImageBatchDestroy(NVCVImageBatchHandle h)
{
    FakeBatch *b = reinterpret_cast<FakeBatch *>(h);
    if (b)
        delete[] b->sizes;
    delete b;
}

// Image handles of this double are pointers to a batch's (width, height) pair; they carry no reference count.
FAKE_API NVCVStatus nvcvImageBatchVarShapeGetImages(NVCVImageBatchHandle h, int32_t begIndex, NVCVImageHandle *outImages,
                                                    int32_t numImages)
{
    FakeBatch *b = reinterpret_cast<FakeBatch *>(h);
    if (!b || !outImages || !b->sizes)
        return 2;
    if (begIndex < 0 || begIndex + numImages > b->data.numImages)
        return 10;
    for (int i = 0; i < numImages; ++i) outImages[i] = reinterpret_cast<NVCVImageHandle>(b->sizes + 2 * (begIndex + i));
    return 0;
}

FAKE_API NVCVStatus nvcvImageGetSize(NVCVImageHandle h, int32_t *width, int32_t *height)
{
    if (!h || !width || !height)
        return 2;
    *width  = reinterpret_cast<const int32_t *>(h)[0];
    *height = reinterpret_cast<const int32_t *>(h)[1];
    return 0;
}

FAKE_API NVCVStatus nvcvImageDecRef(NVCVImageHandle, int *newRefCount)
{
    if (newRefCount)
        *newRefCount = 1;
    return 0;
}

FAKE_API NVCVStatus fakeLastStatus()
{
    return t_status;
}

FAKE_API const char *fakeLastMessage()
{
    return t_message;
}

FAKE_API NVCVStatus nvcvTensorExportData(NVCVTensorHandle h, NVCVTensorData *out)
{
    if (!h || !out)
        return 2;
    *out = *reinterpret_cast<NVCVTensorData *>(h);
    return 0;
}

FAKE_API NVCVStatus nvcvImageBatchExportData(NVCVImageBatchHandle h, cudaStream_t, NVCVImageBatchData *out)
{
    if (!h || !out)
        return 2;
    *out = *reinterpret_cast<NVCVImageBatchData *>(h);
    return 0;
}

FAKE_API NVCVStatus nvcvDataTypeGetDataKind(NVCVDataType t, int *kind)
{
    *kind = static_cast<int>(t & 0xff);
    return 0;
}

FAKE_API NVCVStatus nvcvDataTypeGetBitsPerChannel(NVCVDataType t, int32_t *bits)
{
    const int ch = static_cast<int>((t >> 16) & 0xff);
    for (int i = 0; i < 4; ++i) bits[i] = i < ch ? static_cast<int>((t >> 8) & 0xff) : 0;
    return 0;
}

FAKE_API NVCVStatus nvcvImageFormatGetDataKind(NVCVImageFormat f, int *kind)
{
    return nvcvDataTypeGetDataKind(f, kind);
}

FAKE_API NVCVStatus nvcvImageFormatGetBitsPerChannel(NVCVImageFormat f, int32_t *bits)
{
    return nvcvDataTypeGetBitsPerChannel(f, bits);
}

FAKE_API NVCVStatus nvcvImageFormatGetNumChannels(NVCVImageFormat f, int32_t *n)
{
    *n = static_cast<int>((f >> 16) & 0xff);
    return 0;
}

FAKE_API NVCVStatus nvcvImageFormatGetNumPlanes(NVCVImageFormat f, int32_t *n)
{
    *n = static_cast<int>((f >> 24) & 0xff);
    return 0;
}

FAKE_API void nvcvSetThreadStatus(NVCVStatus status, const char *fmt, ...)
{
    t_status = status;
    if (fmt)
    {
        va_list va;
        va_start(va, fmt);
        vsnprintf(t_message, sizeof(t_message), fmt, va);
        va_end(va);
    }
    else
    {
        t_message[0] = 0;
    }
}
