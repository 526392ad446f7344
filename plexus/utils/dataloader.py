"""Name of the reference's ``plexus/utils/dataloader.py`` (``DataLoader(data_dir, num_gcn_layers).load()``);
implementation: ``plexus_b200/utils/dataloader.py``."""

from plexus_b200.utils.dataloader import DataLoader  # noqa: F401
