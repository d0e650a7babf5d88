"""Native ops: every function dispatches on the tensor's device -- CPU tensors run the C++ oracle,
CUDA tensors run the hand-written sm_100a kernel.  There is no PyTorch fallback on a GPU."""
from . import _native, bn, conv, gemm, head, linalg, packing, philox, quant, topk
from .bn import bn_act
from .conv import conv_bn_act
from .head import head_loss
from ._native import NativeError, launches
from .linalg import gram_schmidt_, topk_abs_indices
from .packing import bytepack, byteunpack, varpack, varunpack
from .quant import (MODE_BIASED, MODE_NU, MODE_NU_BIASED, MODE_STOCHASTIC, absmax, dequantize_levels, mag_width,
                    pack_levels, packed_sizes, pad128, plane_pack, plane_unpack, qsgd_pack, qsgd_unpack_dequant,
                    quantize_levels, randk_gather, randk_indices, randk_scatter, scale_, sgd_step,
                    sum_container_dtype, unpack_levels)
