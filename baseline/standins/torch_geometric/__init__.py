"""Container-only stand-in: the reference's loader imports `torch_geometric.data.Data`."""
