"""Names of the reference's ``plexus/utils/general.py`` (seeding, padding, process-group info, CSR stats,
timer report); implementation: ``plexus_b200/utils/general.py``."""

from plexus_b200.utils.general import (  # noqa: F401
    Node,
    analyze_csr_tensor,
    color,
    get_process_groups_info,
    pad_dimension,
    print_axonn_timer_data,
    set_seed,
)
