"""Hot-path operators: hand-written sm_100a kernels behind plain functions and autograd
Functions, each with an fp32 PyTorch oracle that also serves CPU execution."""
from .gemm import gemm, linear  # noqa: F401
from .norm import lincomb_rmsnorm, rms_norm, rms_norm_weighted, rms_norm_ref  # noqa: F401
from .rope import rotary_freqs, apply_rotary, qkv_post, rope_norm  # noqa: F401
from .ce import lm_head_ce, softcap, softcap_ce_  # noqa: F401
from .attention import attention, attention_ref, attention_packed  # noqa: F401
from . import embed  # noqa: F401,E402
