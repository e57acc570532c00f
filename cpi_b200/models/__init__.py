"""Architectures: each module turns its typed configuration into a ModelSpec and registers itself."""
from . import llama4  # noqa: F401
from . import veredra  # noqa: F401
from . import savenex  # noqa: F401
from . import nogapel  # noqa: F401
from . import kikerax  # noqa: F401
