"""Reference module path ``attention_lab.validate``; the implementation is ``systems_for_llms_b200.attention.validate``."""

from systems_for_llms_b200.attention.validate import *  # noqa: F401,F403
from systems_for_llms_b200.attention import validate as _impl

if hasattr(_impl, "main") and __name__ == "__main__":
    raise SystemExit(_impl.main())
