from plexus_b200.perf.comp_model import comp_model, split_into_three_powers_of_two, spmm_time_b200  # noqa: F401
