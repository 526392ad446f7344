"""Names of the reference's ``performance/comm_model.py``; implementation: ``plexus_b200/perf/comm_model.py``."""

from plexus_b200.perf.comm_model import (  # noqa: F401
    compute_config_costs,
    get_bw,
    split_into_three_powers_of_two,
)
