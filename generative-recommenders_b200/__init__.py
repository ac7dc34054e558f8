"""B200-native HSTU jagged attention: the reference's operator API over hand-written sm_100a
kernels in libb200_hstu.so (C ABI in include/b200_hstu.h)."""

from . import _cabi, hstu_compute
from .common import HammerKernel
from .hstu_attention import delta_hstu_mha, hstu_mha, set_attention_impl
from .hstu_attention_fp8 import hstu_mha_fp8, quantize_e4m3_block
from .hstu_compute import (
    hstu_compute_output,
    hstu_compute_uqvk,
    hstu_norm_mul_dropout,
    hstu_preprocess_and_attention,
)
from .jagged_tensors import (
    concat_2D_jagged,
    hstu_concat_l2_embeddings,
    hstu_split_l2_embeddings,
    split_2D_jagged,
)
from .layer_norm import layer_norm
from .mm import addmm
from .position import add_timestamp_positional_embeddings
from .positional_encoder import HSTUPositionalEncoder
from .stu import STULayer, STULayerConfig, STUStack
from .integration import install, uninstall

__all__ = [
    "HammerKernel",
    "delta_hstu_mha",
    "hstu_mha",
    "hstu_mha_fp8",
    "quantize_e4m3_block",
    "hstu_compute_uqvk",
    "hstu_compute_output",
    "hstu_norm_mul_dropout",
    "hstu_preprocess_and_attention",
    "layer_norm",
    "concat_2D_jagged",
    "split_2D_jagged",
    "hstu_split_l2_embeddings",
    "hstu_concat_l2_embeddings",
    "add_timestamp_positional_embeddings",
    "addmm",
    "HSTUPositionalEncoder",
    "STULayer",
    "STULayerConfig",
    "STUStack",
    "set_attention_impl",
    "install",
    "uninstall",
]
