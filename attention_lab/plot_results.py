"""Reference module path ``attention_lab.plot_results``; the implementation is ``systems_for_llms_b200.attention.plot_results``."""

from systems_for_llms_b200.attention.plot_results import *  # noqa: F401,F403
from systems_for_llms_b200.attention import plot_results as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
