"""Kernel libraries (built on first use) and their Python faces."""
