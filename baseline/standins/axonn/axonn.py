"""`from axonn import axonn as ax`: init, comm_handle, get_timers.

Rank order is Y (column) fastest, then X (row), then Z (depth); one process group per grid line.
"""

import torch
import torch.distributed as dist

comm_handle = None


class _Handle:
    pass


class _Timers:
    """CUDA-event region timers keyed by the stack of open region names."""

    def __init__(self):
        self.enabled = False
        self.stack, self.open, self.pending, self.counts = [], {}, [], {}

    def __call__(self):  # both ax.get_timers() and ax.get_timers work
        return self

    def start(self, name):
        if not self.enabled:
            return
        self.stack.append(name)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.open[tuple(self.stack)] = ev

    def stop(self, name):
        if not self.enabled:
            return
        key = tuple(self.stack)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.pending.append((key, self.open.pop(key), ev))
        self.counts[key] = self.counts.get(key, 0) + 1
        self.stack.pop()

    def get_times(self):
        torch.cuda.synchronize()
        totals = {}
        for key, b, e in self.pending:
            totals[key] = totals.get(key, 0.0) + b.elapsed_time(e)
        counts, self.pending, self.counts = self.counts, [], {}
        return totals, counts


get_timers = _Timers()


def init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=1, gpus_per_node=None,
         enable_internal_timers=False, **_):
    global comm_handle
    world, rank = dist.get_world_size(), dist.get_rank()
    X, Y, Z = G_intra_r, G_intra_c, G_intra_d
    assert G_inter * G_data * X * Y * Z == world
    if gpus_per_node is None:
        gpus_per_node = torch.cuda.device_count()
    torch.cuda.set_device(rank % gpus_per_node)
    h = _Handle()
    h.G_intra_r, h.G_intra_c, h.G_intra_d = X, Y, Z
    y, x, z = rank % Y, (rank // Y) % X, rank // (X * Y)
    h.intra_layer_row_parallel_rank = x
    h.intra_layer_column_parallel_rank = y
    h.intra_layer_depth_parallel_rank = z

    def rk(x_, y_, z_):
        return z_ * X * Y + x_ * Y + y_

    def line_groups(lines):
        mine = None
        for members in lines:
            g = dist.new_group(ranks=members)
            if rank in members:
                mine = g
        return mine

    h.outer_intra_layer_parallel_group = line_groups(
        [[rk(i, b, c) for i in range(X)] for c in range(Z) for b in range(Y)])
    h.inner_intra_layer_parallel_group = line_groups(
        [[rk(a, i, c) for i in range(Y)] for c in range(Z) for a in range(X)])
    h.depth_intra_layer_parallel_group = line_groups(
        [[rk(a, b, i) for i in range(Z)] for b in range(Y) for a in range(X)])
    comm_handle = h
    get_timers.enabled = bool(enable_internal_timers)
