"""Import-compatible name for ``systems_for_llms_b200.config`` (same public functions as the reference's module of this name)."""

from systems_for_llms_b200.config import *  # noqa: F401,F403
from systems_for_llms_b200.config import __doc__ as _target_doc  # noqa: F401
