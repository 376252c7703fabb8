"""B200 (sm_100a) implementation of fused exponent-decode + BF16 GEMV for losslessly compressed
linear layers, with the Python surface of ``lszxb/bf16_huffman_infer``:

    from bf16_huffman_infer_b200 import convert_all_linear, get_graphed_model, get_model_size

There is no CPU or non-CUDA code path: importing the package loads the native libraries and
fails if they have not been built (``python bf16_huffman_infer_b200/_build.py``).
"""
from .functional import *  # noqa: F401,F403
from .functional import mv_ans, mv_huffman  # noqa: F401
from .cudagraph_utils import get_graphed_model  # noqa: F401
from .utils import get_model_size  # noqa: F401
from .checkpoint import load_compressed, save_compressed  # noqa: F401

import os as _os
from . import ops as _ops_mod

# Consecutive fused kernels may overlap their weight-only prologues (see ops.set_launch_overlap).
# Everything this package writes into weight buffers is followed by a stream synchronisation, so
# the default is on; BHI_LAUNCH_OVERLAP=0 turns it off.
_ops_mod.set_launch_overlap(_os.environ.get("BHI_LAUNCH_OVERLAP", "1") != "0")
