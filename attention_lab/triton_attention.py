"""Historical module name kept so ``from attention_lab.triton_attention import attention`` keeps working; the implementation is the sm_100a CUDA kernel, not Triton."""

from systems_for_llms_b200.attention.flash import *  # noqa: F401,F403
from systems_for_llms_b200.attention.flash import __doc__ as _target_doc  # noqa: F401
