"""Callers of the two drop-in entry points, after the reference's examples/."""
