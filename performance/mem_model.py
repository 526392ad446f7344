"""Names of the reference's ``performance/mem_model.py``; implementation: ``plexus_b200/perf/mem_model.py``."""

from plexus_b200.perf.mem_model import compute_config_mem, split_into_three_powers_of_two  # noqa: F401
