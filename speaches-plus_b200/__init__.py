"""B200 (sm_100a) NVFP4 weight-only linear path: ctypes binding of libnvk_b200.so plus a
host-side mirror of the reference's `Linear` / MoE operator interface for that path.

There is no CPU or PyTorch fallback: every operator calls the CUDA library and raises if the
library is missing or a launcher refuses the call.
"""
from . import _ffi as ffi  # noqa: F401
from .linear import Nvfp4Linear, Bf16Linear, Nvfp4Mlp, quantize_weight_nvfp4, swizzled_scale_bytes  # noqa: F401
from .moe import (MoeGroupedWeights, GroupedDecodeContext, forward_grouped_decode, forward_grouped,  # noqa: F401
                  plan_routing, MoeBlock, MoeConfig, TiledDecodeContext, forward_grouped_decode_into)
from . import weights  # noqa: F401,E402
from . import runner  # noqa: F401,E402
from . import backend  # noqa: F401,E402
from .weights import Nvfp4Tensor  # noqa: F401,E402
from .stack import DecodeStep  # noqa: F401,E402
