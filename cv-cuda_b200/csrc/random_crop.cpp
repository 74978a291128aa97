// Host side of RandomResizedCrop: draws one crop rectangle per image the way the reference operator does
// (src/cvcuda/priv/legacy/random_resized_crop.cu:336-390 -- up to ten tries of area x scale and log-uniform aspect
// ratio, a position uniform over what is left, else the central crop that respects the ratio limits), from a
// std::mt19937 seeded as at :314-322. The standard library's engine and distributions are used exactly as the
// reference uses them, so a given seed yields the reference's sequence of rectangles on the same standard library.
#include "cvcuda_b200/preproc.h"

#include <cmath>
#include <cstdint>
#include <new>
#include <random>

struct B200ppRandomCrop
{
    double       minScale, maxScale, minRatio, maxRatio;
    std::mt19937 generator;
};

extern "C" int b200ppRandomCropCreate(B200ppRandomCrop **gen, double minScale, double maxScale, double minRatio,
                                      double maxRatio, uint32_t seed)
{
    if (gen == nullptr)
        return B200PP_ERROR_INVALID_ARGUMENT;
    *gen = nullptr;
    // :300-304
    if (minScale > maxScale || minRatio > maxRatio)
        return B200PP_ERROR_INVALID_ARGUMENT;
    B200ppRandomCrop *g = new (std::nothrow) B200ppRandomCrop;
    if (g == nullptr)
        return B200PP_ERROR_INTERNAL;
    g->minScale = minScale;
    g->maxScale = maxScale;
    g->minRatio = minRatio;
    g->maxRatio = maxRatio;
    if (seed == 0) // :314-318: a seed of 0 asks for a non-deterministic one
    {
        std::random_device dev;
        g->generator = std::mt19937(dev());
    }
    else
    {
        g->generator = std::mt19937(seed);
    }
    *gen = g;
    return B200PP_SUCCESS;
}

extern "C" void b200ppRandomCropDestroy(B200ppRandomCrop *gen)
{
    delete gen;
}

extern "C" int b200ppRandomCropNext(B200ppRandomCrop *gen, int32_t rows, int32_t cols, int32_t rect[4])
{
    if (gen == nullptr || rect == nullptr || rows < 1 || cols < 1)
        return B200PP_ERROR_INVALID_ARGUMENT;
    const double area        = rows * cols;
    const double logMinRatio = std::log(gen->minRatio);
    const double logMaxRatio = std::log(gen->maxRatio);

    std::uniform_real_distribution<double> scaleDist(gen->minScale, gen->maxScale);
    std::uniform_real_distribution<double> ratioDist(logMinRatio, logMaxRatio);

    int cropCols = 0, cropRows = 0;
    for (int attempt = 0; attempt < 10; ++attempt)
    {
        const int    targetArea  = area * scaleDist(gen->generator); // truncated to int, as at :352
        const double aspectRatio = std::exp(ratioDist(gen->generator));
        cropCols                 = int(std::round(std::sqrt(targetArea * aspectRatio)));
        cropRows                 = int(std::round(std::sqrt(targetArea / aspectRatio)));
        if (cropCols > 0 && cropCols <= cols && cropRows > 0 && cropRows <= rows)
        {
            std::uniform_int_distribution<int> rowDist(0, rows - cropRows);
            std::uniform_int_distribution<int> colDist(0, cols - cropCols);
            rect[1] = rowDist(gen->generator); // top first, then left: the order of the draws matters
            rect[0] = colDist(gen->generator);
            rect[2] = cropCols;
            rect[3] = cropRows;
            return B200PP_SUCCESS;
        }
    }
    // no fit in ten tries: central crop (:367-389)
    const double inRatio = double(cols) / double(rows);
    if (inRatio < gen->minRatio)
    {
        cropCols = cols;
        cropRows = int(std::round(cropCols / gen->minRatio));
    }
    else if (inRatio > gen->maxRatio)
    {
        cropRows = rows;
        cropCols = int(std::round(cropRows * gen->maxRatio));
    }
    else
    {
        cropCols = cols;
        cropRows = rows;
    }
    rect[0] = (cols - cropCols) / 2;
    rect[1] = (rows - cropRows) / 2;
    rect[2] = cropCols;
    rect[3] = cropRows;
    return B200PP_SUCCESS;
}
