from plexus_b200.perf.epoch_model import predict_epoch_ms, rank_grids  # noqa: F401
