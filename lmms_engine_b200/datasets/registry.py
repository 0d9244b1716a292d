"""Imports every dataset / processor module so that their ``@register_*`` decorators run."""
from . import synthetic  # noqa: F401

try:
    from . import iterable, naive, processor  # noqa: F401
    from . import extra  # noqa: F401
except ImportError:  # pragma: no cover
    pass
