"""Reference module path ``attention_lab.search``; the implementation is ``systems_for_llms_b200.attention.search``."""

from systems_for_llms_b200.attention.search import *  # noqa: F401,F403
from systems_for_llms_b200.attention import search as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
