"""B200-native fused image pre-processing (ResizeCropConvertReformat, CropFlipNormalizeReformat).

The package directory name contains a hyphen, so load it with ``__graft_entry__.load_package()`` (or
``importlib``) under the module name ``cvcuda_b200``.

Everything computes in ``libcvcuda_b200.so`` (hand-written sm_100a kernels); there is no CPU or PyTorch fallback:
importing the operator functions fails loudly when the library has not been built.
"""
from . import ops as _ops
from . import cvcuda  # noqa: F401  (the reference-style object surface: cvcuda = nvcv = cvcuda_b200.cvcuda)
from . import sharding  # noqa: F401
from .ops import (  # noqa: F401
    Border,
    ChannelManip,
    ImageBatchVarShape,
    Interp,
    NORMALIZE_SCALE_IS_STDDEV,
    RectI,
    convertto,
    convertto_into,
    copymakeborder,
    copymakeborder_into,
    copymakeborderstack,
    copymakeborderstack_into,
    crop_flip_normalize_reformat,
    crop_flip_normalize_reformat_into,
    fused_preprocess_into,
    last_error,
    launch_count,
    lib,
    lib_path,
    normalize,
    normalize_into,
    read_device_error,
    reformat,
    reformat_into,
    random_crop_rects,
    random_resized_crop,
    random_resized_crop_into,
    resize,
    resized_crop_into,
    resize_into,
    resize_crop_convert_reformat,
    resize_crop_convert_reformat_into,
    self_test_wait_timeout,
    set_kernel_path,
)

__all__ = [n for n in dir(_ops) if not n.startswith("_")]
