"""Import-compatible name for ``systems_for_llms_b200.parallel.train`` (same public functions as the reference's module of this name)."""

from systems_for_llms_b200.parallel.train import *  # noqa: F401,F403
from systems_for_llms_b200.parallel.train import __doc__ as _target_doc  # noqa: F401
from systems_for_llms_b200.parallel.train import (MODES, evaluate, fsdp_clip_grad_norm, run, state_hash,  # noqa: F401
                                                tensor_bytes, train_step, validate_layout)

from systems_for_llms_b200.parallel.train import main

if __name__ == "__main__":
    main()
