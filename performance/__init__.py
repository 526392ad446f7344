"""Stand-alone cost models under the reference's module names."""
