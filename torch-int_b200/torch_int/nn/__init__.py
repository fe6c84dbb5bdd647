# The reference re-exports exactly these two names (torch_int/nn/__init__.py:1).
from .linear import W8A16Linear, W8FakeA8Linear  # noqa: F401
