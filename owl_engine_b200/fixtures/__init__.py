"""Measurement and evaluation fixtures that drive a running server or a set of ranks (not runtime code)."""
