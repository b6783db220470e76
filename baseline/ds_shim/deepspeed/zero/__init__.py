"""ZeRO stage-3 construction context: accepted and ignored (parameters are built whole)."""
import contextlib


class Init(contextlib.AbstractContextManager):
    def __init__(self, *a, **k):
        pass

    def __exit__(self, *exc):
        return False
