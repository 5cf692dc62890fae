"""Calibration: importance statistics and bit allocation (imatrix, AlphaQ, expert-wise MILP solver, scheme artefact)."""
