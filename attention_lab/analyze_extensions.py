"""Reference module path ``attention_lab.analyze_extensions``; the implementation is ``systems_for_llms_b200.attention.analyze_extensions``."""

from systems_for_llms_b200.attention.analyze_extensions import *  # noqa: F401,F403
from systems_for_llms_b200.attention import analyze_extensions as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
