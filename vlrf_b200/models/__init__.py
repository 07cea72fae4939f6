"""Architectures.  Importing this package registers them."""
from . import gpt2  # noqa: F401
from . import kuvusun  # noqa: F401
from . import kotisun  # noqa: F401
from . import rakelorn  # noqa: F401
from . import suposun  # noqa: F401
