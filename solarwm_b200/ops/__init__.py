"""Hot-path operators: ctypes front ends of the sm_100a kernels plus their PyTorch oracles."""
from . import reference  # noqa: F401
from ._lib import COUNTERS, NativeError, available, count, reset_counters, total_launches  # noqa: F401
from .attention import attention, get_backend, set_backend  # noqa: F401
from .functional import (  # noqa: F401
    NN, NT, TN, accumulate_main_grad, add_noise, adamw_, check_status, colsum, read_status, euler_step,
    flow_to_x0, gated_residual, gelu, gemm, head_norm_rope_prope, linear, norm_modulate, rgb8, rmsnorm_rope, set_gemm_backend, status_word,
    sumsq, swiglu, weighted_masked_mse,
)
