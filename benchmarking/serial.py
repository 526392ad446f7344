"""Serial single-process GCN on the same processed data, for validating a parallel run.

Prints ``Epoch: NNN, Train Loss: X`` per epoch exactly like ``examples/train.py`` so the two
logs can be compared line by line (the reference validates against a PyG script by eye,
benchmarking/pyg_serial.py:48-119; this one needs no PyG: the layer is ``A @ x @ W`` on a torch
CSR matrix with the same weight initialisation as the parallel ``GCNConv``).

    python benchmarking/serial.py --data_dir <dir with processed_*.pt> [--num_epochs 10]
    python benchmarking/serial.py --synthetic 16384,262144,128,16 --num_gcn_layers 2
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from plexus_b200.data import graph_ops  # noqa: E402
from plexus_b200.data.container import load_processed  # noqa: E402
from plexus_b200.models.net import SerialGCN, serial_loss  # noqa: E402
from plexus_b200.utils.general import set_seed  # noqa: E402


def create_parser():
    p = argparse.ArgumentParser()
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--data_dir", "--download_path", dest="data_dir", type=str, default=None,
                   help="directory with one processed .pt file (--download_path is the reference's name for it)")
    p.add_argument("--synthetic", type=str, default=None, help="nodes,undirected_edges,features,classes")
    p.add_argument("--num_epochs", type=int, default=10)
    p.add_argument("--num_gcn_layers", type=int, default=3)
    p.add_argument("--hidden_size", type=int, default=128)
    p.add_argument("--lr", type=float, default=3e-3)
    p.add_argument("--weight_decay", type=float, default=0.0)
    return p


def csr_of(ei, ew, n, device):
    crow, col, val = graph_ops.coo_to_csr(ei[0], ei[1], ew, n, n, index_dtype=torch.int64)
    return graph_ops.csr_tensor(crow, col, val, (n, n)).to(device)


def main(argv=None):
    args = create_parser().parse_args(argv)
    set_seed(args.seed)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if args.synthetic:
        from plexus_b200.data.synthetic import synthetic_graph
        from plexus_b200.utils.dataset import preprocess_data

        n, e, f, c = (int(v) for v in args.synthetic.split(",")[:4])
        raw, _ = synthetic_graph(n, e, f, c, seed=args.seed)
        data, num_classes = preprocess_data(raw, c, double_perm=True, normalized=True, seed=args.seed)
    else:
        pt = [f for f in os.listdir(args.data_dir) if f.endswith(".pt")]
        data, num_classes = load_processed(os.path.join(args.data_dir, pt[0]))
    n = data.x.shape[0]
    adjs = [csr_of(data.edge_index, data.edge_weight, n, dev)]
    if hasattr(data, "edge_index_2"):
        adjs.append(csr_of(data.edge_index_2, data.edge_weight_2, n, dev))
    labels = (data.y_2 if (hasattr(data, "y_2") and args.num_gcn_layers % 2 == 0) else data.y).to(dev)
    x = data.x.to(dev).float().requires_grad_()
    model = SerialGCN(args.num_gcn_layers, x.shape[1], args.hidden_size, num_classes, seed=args.seed).to(dev)
    opt = torch.optim.AdamW(list(model.parameters()) + [x], lr=args.lr, weight_decay=args.weight_decay)
    losses = []
    for i in range(args.num_epochs):
        opt.zero_grad()
        loss = serial_loss(model(x, adjs), labels, n)
        loss.backward()
        opt.step()
        losses.append(loss.item())
        print("Epoch: {:03d}, Train Loss: {:.4f}".format(i, loss))
    return losses


if __name__ == "__main__":
    main()
