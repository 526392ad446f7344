import torch
import torch.distributed as dist


def _drop(t, group):
    """Keep this rank's block of the last dimension."""
    p, r = dist.get_world_size(group), dist.get_rank(group)
    n = t.shape[-1] // p
    return t[..., r * n:(r + 1) * n]


@torch.no_grad()
def extract_local_params_from_full_params(params, out_features_group, in_features_group, depth_group):
    params = _drop(params, in_features_group)
    params = _drop(params.t().contiguous(), out_features_group).t().contiguous()
    flat = params.reshape(-1)
    p, r = dist.get_world_size(depth_group), dist.get_rank(depth_group)
    n = flat.numel() // p
    return flat[r * n:(r + 1) * n].clone()
