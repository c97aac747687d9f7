"""Offline checkpoint tools (not part of the serving runtime)."""
