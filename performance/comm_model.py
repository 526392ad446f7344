from plexus_b200.perf.comm_model import (  # noqa: F401
    compute_config_costs,
    get_bw,
    split_into_three_powers_of_two,
)
