"""Architectures.  Importing this package registers every one of them."""
from . import fidolix  # noqa: F401
from . import kedelorn  # noqa: F401
from . import llama  # noqa: F401
from . import povusun  # noqa: F401
from . import zepavik  # noqa: F401
