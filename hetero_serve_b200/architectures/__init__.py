"""Importing this package registers every architecture the framework ships."""
from . import gpt2  # noqa: F401
from . import pedorax  # noqa: F401
from . import putelix  # noqa: F401
from . import roritar  # noqa: F401
from . import mafuzen  # noqa: F401
