"""Utilities: profiling ranges and tables, roofline arithmetic, timing helpers."""
