"""Restart-from-checkpoint supervisor for the training application.

    python examples/supervise.py --nproc 8 --max_restarts 3 -- \\
        --synthetic 2449029,60634000,100,47 --hidden_size 256 --grid auto --comm fused \\
        --num_epochs 100 --checkpoint_dir ckpt --checkpoint_every 10 --epoch_timeout 60

Runs ``train.py`` under ``torch.distributed.run``.  A run that ends with a non-zero exit code - a
rank that died, the per-epoch watchdog (exit code 43), a peer-failure or device-status exception -
is started again with ``--resume``, which loads the last complete sharded checkpoint (or starts
over if none was written yet).  ``--restart_grid XxYxZ`` resumes on a different grid from the
consolidated checkpoint instead (``--consolidated FILE`` must be among the training flags).

A supervised job expects ranks to disappear, so its ranks never bind memory to an NVLink multicast
object: the children run with ``PLEXUS_NVLS=0`` and ``NCCL_NVLS_ENABLE=0`` unless the caller set
these variables (a rank that dies while its buffers are multicast-bound can fault its peers' GPUs).

The reference has no failure handling: a lost rank leaves the job hanging until the batch system's
time limit (its examples/run_4.sh:2).  Fault injection for tests is host-side only
(``PLEXUS_INJECT_FAILURE=rank:epoch[:exit|raise|stall]``, honoured by the first attempt).
"""

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--max_restarts", type=int, default=2)
    ap.add_argument("--master_port", type=int, default=29500)
    ap.add_argument("--restart_grid", type=str, default=None)
    ap.add_argument("train_args", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    train_args = [a for a in args.train_args if a != "--"]
    rc = 1
    for attempt in range(args.max_restarts + 1):
        env = dict(os.environ)
        env.setdefault("PLEXUS_NVLS", "0")
        env.setdefault("NCCL_NVLS_ENABLE", "0")
        extra = []
        if attempt > 0:
            env.pop("PLEXUS_INJECT_FAILURE", None)
            if "--resume" not in train_args:
                extra.append("--resume")
            if args.restart_grid:
                extra += ["--grid", args.restart_grid]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(args.master_port + attempt),
               os.path.join(HERE, "train.py")] + train_args + extra
        rc = subprocess.call(cmd, env=env)
        if rc == 0:
            if attempt:
                print(f"[supervise] finished after {attempt} restart(s)", flush=True)
            return 0
        print(f"[supervise] attempt {attempt} ended with exit code {rc}"
              + ("; restarting from the last checkpoint" if attempt < args.max_restarts else "; giving up"),
              flush=True)
    return rc


if __name__ == "__main__":
    sys.exit(main())
