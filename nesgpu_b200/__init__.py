"""nesgpu_b200: B200-native kernels behind the NESgpu perturbed-layer API.

``nesgpu_b200.base`` mirrors the reference's ``modules/base.py``, ``nesgpu_b200.binary`` its
``modules/binary.py`` and ``nesgpu_b200.boolean_operations`` its
``extensions/booleanOperations.py``; the top-level ``modules`` and ``extensions`` packages of
this repository re-export them under the reference's import paths.  Importing the layer
modules loads ``lib/libnesgpu_b200.so`` and fails if it has not been built
(``python -m nesgpu_b200.build``).
"""
__version__ = "0.1.0"
