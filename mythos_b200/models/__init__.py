"""Model definitions."""
from .config import NAMED_CONFIGS, TransformerConfig  # noqa: F401
from .dense import DenseModel  # noqa: F401
