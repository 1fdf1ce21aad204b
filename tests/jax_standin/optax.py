"""optax is absent: any use of it skips the calling test."""
import pytest


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)

    def missing(*_a, **_k):
        pytest.skip(f"optax.{name}: optax is not installed")

    return missing
