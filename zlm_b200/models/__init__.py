"""Architectures this build knows.  Importing the package fills the registry."""
from . import qwen3   # noqa: F401
from . import nuvilorn   # noqa: F401
from . import zekazen   # noqa: F401
from . import lodevik   # noqa: F401
from . import sudupel   # noqa: F401
