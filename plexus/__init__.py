"""Import-compatible facade: the module names of hpcgroup/plexus over plexus_b200."""
