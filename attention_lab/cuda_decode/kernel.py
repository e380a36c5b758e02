"""Import-compatible name for ``systems_for_llms_b200.attention.decode``."""

from systems_for_llms_b200.attention.decode import PreparedDecode, decode, prepare  # noqa: F401
