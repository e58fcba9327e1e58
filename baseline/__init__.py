"""Seeded input generators shared by bench.py, the tests and the smoke run (not part of the product package)."""
