"""torch_int for NVIDIA B200: the W8A8 operator set of torch-int behind the
reference's Python surface (torch_int/__init__.py:1 exports ``nn``).

    torch_int._CUDA        native ops (sm_100a kernels through a C ABI)
    torch_int.nn           W8A8 linear / BMM / LayerNorm-quantise modules
    torch_int.functional   quantisation helpers and thin op aliases
    torch_int.models.opt   Int8 OPT attention / decoder layer / causal LM
"""
from . import nn  # noqa: F401
