"""Kernel launchers."""
