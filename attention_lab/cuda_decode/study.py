"""Reference module path ``attention_lab.cuda_decode.study``; the implementation is ``systems_for_llms_b200.attention.decode_study``."""

from systems_for_llms_b200.attention.decode_study import *  # noqa: F401,F403
from systems_for_llms_b200.attention import decode_study as _impl

if __name__ == "__main__":
    _impl.main()
