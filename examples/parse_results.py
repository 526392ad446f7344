"""``process_log_file(filename, warmup) -> (epoch_ms, comm_ms)``; CLI prints both.

Same entry point as the reference's ``examples/parse_results.py``; implementation:
``plexus_b200/utils/parse_results.py``."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from plexus_b200.utils.parse_results import extract_avg_time, process_log_file  # noqa: E402,F401

if __name__ == "__main__":
    ep, comm = process_log_file(sys.argv[1], int(sys.argv[2]) if len(sys.argv) > 2 else 0)
    print(f"epoch_ms={ep:.3f} comm_ms={comm:.3f}")
