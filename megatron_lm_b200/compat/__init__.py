"""Opt-in import aliases for code written against the reference's module paths."""
