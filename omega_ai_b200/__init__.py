"""B200-native mixture-of-experts FFN forward for the Omega-AI engine.

The product is ``libomoe.so`` (CUDA for sm_100a behind the C ABI in
``include/omoe.h``); this package binds it and mirrors the engine's
Layer/Tensor surface for it.  Importing the package does not load the library;
the first use does, and fails loudly if it has not been built.
"""
from .native import OMOE_BF16, OMOE_F32, OmoeError, build  # noqa: F401


def __getattr__(name):
    if name in ("MoELayer", "Tensor", "Layer"):
        from . import layer

        return getattr(layer, name)
    raise AttributeError(name)
