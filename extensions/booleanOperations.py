"""Drop-in import path of the reference project (``from extensions import booleanOperations``)."""
from nesgpu_b200.boolean_operations import *  # noqa: F401,F403
