"""Import-compatible name for ``systems_for_llms_b200.attention.backward``."""

from systems_for_llms_b200.attention.backward import *  # noqa: F401,F403
from systems_for_llms_b200.attention.backward import StructuredAttention, training_attention  # noqa: F401
from systems_for_llms_b200.attention.masks import transpose_schedule  # noqa: F401
