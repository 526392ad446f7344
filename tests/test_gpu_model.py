"""End-to-end single-GPU GCN step versus the CPU oracle (bf16 storage tolerances)."""

import pytest
import torch

from helpers import oracle, small_processed_graph

pytestmark = pytest.mark.gpu


def _run(device, data, nc, fuse):
    import plexus_b200 as plx
    from plexus_b200.models.cross_entropy import parallel_cross_entropy
    from plexus_b200.models.net import Net
    from plexus_b200.utils.dataloader import DataLoader

    plx.init(1, 1, 1, device=device, dtype=torch.bfloat16, channel_align=8)
    dev = torch.device("cuda", 0) if device is None else torch.device("cpu")
    adj, feats, labels, N, F, C = DataLoader(None, 3, data=(data, nc), device=dev).load()
    model = Net(3, F, 64, C, fuse_layers=fuse, seed=3).to(dev)
    out = model(feats, adj)
    loss = parallel_cross_entropy(out, labels, 3, N, C)
    loss.backward()
    return dict(loss=loss.item(), logits=out.detach().float().cpu(), gx=feats.grad.float().cpu(),
                gw=[l.weight.grad.float().cpu() for l in model.layers], N=N, F=F, C=C, model=model)


def _rel(a, b):
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


@pytest.mark.parametrize("fuse", [True, False])
def test_one_gpu_epoch_matches_cpu_pipeline_and_oracle(fuse):
    """GPU kernels vs the same bf16-storage pipeline in plain torch on the CPU (tight), and vs
    the fp64 dense oracle (loose: bf16 rounding accumulates over three layers)."""
    from plexus_b200.ops import cuda as opc

    data, nc = small_processed_graph(n=3000, e=24000, f=100, c=47, seed=7)
    cpu = _run("cpu", data, nc, fuse)
    gpu = _run(None, data, nc, fuse)
    opc.check_status()

    assert abs(gpu["loss"] - cpu["loss"]) < 5e-3 * abs(cpu["loss"])
    assert _rel(gpu["logits"], cpu["logits"]) < 2e-2
    for l in range(3):
        assert _rel(gpu["gw"][l], cpu["gw"][l]) < 3e-2, l
    assert _rel(gpu["gx"], cpu["gx"]) < 3e-2

    ref_loss, ref_gw, ref_gx, ref_logits = oracle(data, nc, 3, 64, seed=3)
    N, F, C = gpu["N"], gpu["F"], gpu["C"]
    assert abs(gpu["loss"] - ref_loss.item()) < 2e-2 * abs(ref_loss.item())
    assert _rel(gpu["logits"][:N, :C], ref_logits.float()) < 5e-2
    for l, layer in enumerate(gpu["model"].layers):
        got = gpu["gw"][l].view(layer.in_channels, layer.out_channels)
        want = torch.zeros_like(got)
        want[: ref_gw[l].shape[0], : ref_gw[l].shape[1]] = ref_gw[l].float()
        assert _rel(got, want) < 0.35, l
    assert _rel(gpu["gx"].view(N, -1)[:, :F], ref_gx.float()) < 0.35


def test_training_reduces_loss_with_fused_adam():
    import plexus_b200 as plx
    from plexus_b200.models.cross_entropy import parallel_cross_entropy
    from plexus_b200.models.net import Net
    from plexus_b200.optim import FusedAdamW
    from plexus_b200.utils.dataloader import DataLoader

    plx.init(1, 1, 1)
    data, nc = small_processed_graph(n=2000, e=16000, f=32, c=8, seed=1, unlabeled=0.0)
    adj, feats, labels, N, F, C = DataLoader(None, 2, data=(data, nc)).load()
    model = Net(2, F, 32, C, seed=1)
    opt = FusedAdamW(list(model.parameters()) + [feats], lr=1e-2)
    losses = []
    for _ in range(30):
        opt.zero_grad(set_to_none=True)
        loss = parallel_cross_entropy(model(feats, adj), labels, 2, N, C)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.9 * losses[0], losses
