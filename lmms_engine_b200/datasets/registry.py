"""Imports every dataset / processor module so that their ``@register_*`` decorators run.  A module that
fails to import is an error: a dataset type that silently is not registered would only surface later as
an unknown ``dataset_type``."""
from . import synthetic  # noqa: F401
from . import iterable, naive, processor  # noqa: F401
from . import extra  # noqa: F401
from . import families  # noqa: F401
from . import codec_video  # noqa: F401
from . import realtime  # noqa: F401
