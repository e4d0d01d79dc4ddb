"""Architectures: each module turns its typed config into a ``ModelSpec`` and registers itself."""
