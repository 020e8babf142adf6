"""odla_b200: a B200-native ODLA platform library (libodla_b200.so) and its Python host mirror.

The product is the shared library built from ``csrc/`` (``build.build()``); ``odla`` binds its C ABI
with ctypes and ``halo_models`` holds HALO-style model descriptions that drive it.  Importing the
package never builds anything and never falls back to a CPU implementation: every compute call
goes through libodla_b200.so and fails loudly when the library or a GPU is missing.
"""
from . import build, odla  # noqa: F401
from .odla import Graph, OdlaLib, default_library_path  # noqa: F401


def load():
    """Loads libodla_b200.so (raises FileNotFoundError with the build command if it is absent)."""
    return OdlaLib(default_library_path())
