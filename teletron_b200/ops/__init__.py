"""Op layer: every op has a PyTorch reference (`*_ref`, also the CPU path) and an sm_100a kernel."""
from . import _lib  # noqa: F401
from .attention import (attention, attention_bwd, attention_fwd, attention_ref,  # noqa: F401
                        self_attention_core)
from .flow import add_noise, add_noise_ref, flow_mse, flow_mse_ref  # noqa: F401
from .gemm import gemm, gemm_ag, gemm_ag_gather, gemm_ref, gemm_rs_scatter, tp_reduce_rows  # noqa: F401
from .linear import colsum, ffn, linear, linear_residual  # noqa: F401
from .norm import (adaln, adaln_ref, adaln_res, layernorm_affine, rmsnorm_rope, rmsnorm_rope_ref,  # noqa: F401
                   rope_ref)
from .optim import adamw_ref, adamw_step, grad_norm  # noqa: F401
