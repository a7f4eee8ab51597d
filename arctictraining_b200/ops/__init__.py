# SPDX-License-Identifier: Apache-2.0
from . import reference
from .functional import IGNORE_INDEX
from .functional import COMM_COUNTER
from .functional import LAUNCH_COUNTER
from .functional import accumulate_lp_grad
from .functional import adamw_step
from .functional import attention
from .functional import fused_linear_cross_entropy
from .functional import fused_linear_logprobs
from .functional import gemm
from .functional import linear
from .functional import linear_swiglu
from .functional import mlp_swiglu
from .functional import rms_norm
from .functional import rope
from .functional import rope_attention
from .functional import rope_qkv
from .functional import set_gemm_backend
from .functional import sumsq
from .functional import swiglu_interleaved

__all__ = [
    "reference", "IGNORE_INDEX", "LAUNCH_COUNTER", "COMM_COUNTER", "accumulate_lp_grad", "adamw_step", "attention",
    "fused_linear_cross_entropy", "fused_linear_logprobs", "gemm", "linear", "linear_swiglu", "mlp_swiglu", "rms_norm", "rope", "rope_attention", "rope_qkv", "set_gemm_backend",
    "sumsq", "swiglu_interleaved",
]
