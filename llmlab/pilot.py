"""Import-compatible name for ``systems_for_llms_b200.pilot``."""

from systems_for_llms_b200.pilot import *  # noqa: F401,F403
from systems_for_llms_b200.pilot import (aggregate_results, execute_plan, main, make_plan,  # noqa: F401
                                         summarize_case, write_plan)

if __name__ == "__main__":
    main()
