"""Reference module path ``attention_lab.run_modal``; the implementation is ``systems_for_llms_b200.attention.launcher``."""

from systems_for_llms_b200.attention.launcher import *  # noqa: F401,F403
from systems_for_llms_b200.attention import launcher as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
