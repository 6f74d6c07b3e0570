from .contract import TripletContract
from .conv import (GeneralConv, GenerativePointConv3d, PointConv3d, conv_with_stride, conv_with_stride_disjoint,
                   conv_with_stride_full_cover)
from .downsample import downsample
from .generative import (CoordinateGenerator, GeneratedSites, KernelStampGenerator, SubdivisionGenerator,
                         build_generative_triplets)
from .metadata import MetaData
from .norm import RaggedBatchNorm, RaggedGroupNorm, RaggedInstanceNorm, RaggedLayerNorm, RaggedNorm
from .pooling import GlobalPool, max_pool3d
from .upsample import Upsample, recompute_cached_upsample_k
from .triplets import (FullCoverStridedRulebook, build_full_cover_strided_rulebook, build_triplets,
                       build_triplets_segmented, full_cover_radius_scaler,
                       handle_stride_and_build_triplets, handle_stride_disjoint_and_build_triplets,
                       minimum_full_cover_kernel_size, partition_slots, radius_scaler_for_kernel_size, should_use_direct_segmented_triplets, voxelize_3d)

__all__ = ["TripletContract", "GeneralConv", "GenerativePointConv3d", "CoordinateGenerator", "GeneratedSites",
           "KernelStampGenerator", "SubdivisionGenerator", "build_generative_triplets", "PointConv3d", "conv_with_stride", "conv_with_stride_disjoint",
           "handle_stride_disjoint_and_build_triplets", "partition_slots", "conv_with_stride_full_cover", "FullCoverStridedRulebook",
           "build_full_cover_strided_rulebook", "downsample", "MetaData", "Upsample", "recompute_cached_upsample_k",
           "build_triplets", "build_triplets_segmented", "full_cover_radius_scaler",
           "handle_stride_and_build_triplets", "minimum_full_cover_kernel_size",
           "radius_scaler_for_kernel_size", "should_use_direct_segmented_triplets", "voxelize_3d",
           "RaggedNorm", "RaggedBatchNorm", "RaggedInstanceNorm", "RaggedLayerNorm", "RaggedGroupNorm",
           "GlobalPool", "max_pool3d"]
