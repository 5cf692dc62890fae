"""Harness code that drives the unmodified reference (installed under ``baseline/_ref``) for A/B runs."""
