from plexus_b200.utils.dataloader import DataLoader  # noqa: F401
