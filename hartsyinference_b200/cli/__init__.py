"""Command-line interface (``python -m hartsyinference_b200.cli``)."""
