"""Parts of a decoder. Importing the package registers the standard parts."""
from . import base, plan, standard  # noqa: F401
