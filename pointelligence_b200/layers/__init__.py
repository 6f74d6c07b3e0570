from .contract import TripletContract
from .conv import GeneralConv, PointConv3d, conv_with_stride
from .downsample import downsample
from .metadata import MetaData
from .triplets import (build_triplets, build_triplets_segmented, full_cover_radius_scaler,
                       handle_stride_and_build_triplets, minimum_full_cover_kernel_size,
                       radius_scaler_for_kernel_size, should_use_direct_segmented_triplets, voxelize_3d)

__all__ = ["TripletContract", "GeneralConv", "PointConv3d", "conv_with_stride", "downsample", "MetaData",
           "build_triplets", "build_triplets_segmented", "full_cover_radius_scaler",
           "handle_stride_and_build_triplets", "minimum_full_cover_kernel_size",
           "radius_scaler_for_kernel_size", "should_use_direct_segmented_triplets", "voxelize_3d"]
