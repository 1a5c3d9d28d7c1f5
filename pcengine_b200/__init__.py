"""pcengine_b200: a Blackwell (sm_100a) sparse-convolution inference engine behind
PCEngine's operator surface (spTensor, conv3d, BatchNorm, ReLU/LeakyReLU and the
five ``backend`` entry points).  Importing the package loads libpce_b200.so and
fails if it has not been built; there is no CPU or PyTorch fallback."""
from . import _lib  # noqa: F401  (loads the shared library, raises when missing)
from . import backend, functional  # noqa: F401
from .activation import LeakyReLU, ReLU
from .batchnorm import BatchNorm, bn_scale_shift
from .functional import FusedEpilogue, invalidate_packed
from .kmap import KernelMap
from .minkunet import MinkUNet, randomize_batchnorm
from .planner import MapPlan
from .spconv import conv3d, conv_func
from .sptensor import SparseTensor, spTensor
from .utils import (cat, conv_info_decoder, conv_info_encoder, fapply, init_layer_scheduler, output_stride_compute,
                    sparse_collate, sparse_collate_fn, sparse_quantize)

__version__ = "0.1.0"
