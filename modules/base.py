"""Drop-in import path of the reference project (``from modules.base import *``)."""
from nesgpu_b200.base import *  # noqa: F401,F403
from nesgpu_b200.base import Perturbed, Permuted, PerturbedModel  # noqa: F401
