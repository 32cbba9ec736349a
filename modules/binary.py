"""Drop-in import path of the reference project (``from modules.binary import *``)."""
from nesgpu_b200.binary import *  # noqa: F401,F403
