"""Reference module path ``attention_lab.block_benchmark``; the implementation is ``systems_for_llms_b200.attention.block_benchmark``."""

from systems_for_llms_b200.attention.block_benchmark import *  # noqa: F401,F403
from systems_for_llms_b200.attention import block_benchmark as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
