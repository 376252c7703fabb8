"""B200 (sm_100a) implementation of fused exponent-decode + BF16 GEMV for losslessly compressed
linear layers, with the Python surface of ``lszxb/bf16_huffman_infer``:

    from bf16_huffman_infer_b200 import convert_all_linear, get_graphed_model, get_model_size

There is no CPU or non-CUDA code path: importing the package loads the native libraries and
fails if they have not been built (``python -m bf16_huffman_infer_b200._build``).
"""
from .functional import *  # noqa: F401,F403
from .functional import mv_ans, mv_huffman  # noqa: F401
from .cudagraph_utils import get_graphed_model  # noqa: F401
from .utils import get_model_size  # noqa: F401
