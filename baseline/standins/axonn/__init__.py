"""Minimal stand-in for the parts of AxoNN that hpcgroup/plexus imports (baseline runs only)."""
