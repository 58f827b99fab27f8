"""Architectures: each module turns its typed configuration into a ModelSpec and registers
itself under its config.json name."""
