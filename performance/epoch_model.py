"""Per-region epoch-time model of this framework on B200 (no counterpart in the reference's ``performance/``);
implementation: ``plexus_b200/perf/epoch_model.py``."""

from plexus_b200.perf.epoch_model import predict_epoch_ms, rank_grids  # noqa: F401
