"""Reference module path ``attention_lab.backward_study``; the implementation is ``systems_for_llms_b200.attention.backward_study``."""

from systems_for_llms_b200.attention.backward_study import *  # noqa: F401,F403
from systems_for_llms_b200.attention import backward_study as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
