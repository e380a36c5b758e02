"""Import-compatible name for ``systems_for_llms_b200.train`` (same public functions as the reference's module of this name)."""

from systems_for_llms_b200.train import *  # noqa: F401,F403
from systems_for_llms_b200.train import __doc__ as _target_doc  # noqa: F401
from systems_for_llms_b200.train import (autocast, check_precision, evaluate, get_device, learning_rate,  # noqa: F401
                                       resume_config, run, source_identity, synchronize, train_step)

from systems_for_llms_b200.train import main

if __name__ == "__main__":
    main()
