"""Reference module path ``attention_lab.analyze_study``; the implementation is ``systems_for_llms_b200.attention.analyze_study``."""

from systems_for_llms_b200.attention.analyze_study import *  # noqa: F401,F403
from systems_for_llms_b200.attention import analyze_study as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
