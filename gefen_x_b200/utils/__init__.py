"""Subpackage of gefen_x_b200."""
