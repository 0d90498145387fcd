"""Command-line tools: corpus preparation, held-out / long-context evaluation, router checks.

Run as ``python -m nestor_b200.scripts.<name> --help``.
"""
