"""Utility modules under the reference's ``plexus.utils`` names."""
