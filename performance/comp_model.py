"""Names of the reference's ``performance/comp_model.py`` plus the B200 SpMM bandwidth model;
implementation: ``plexus_b200/perf/comp_model.py``."""

from plexus_b200.perf.comp_model import comp_model, split_into_three_powers_of_two, spmm_time_b200  # noqa: F401
