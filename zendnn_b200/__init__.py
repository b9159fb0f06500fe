"""zendnn_b200: B200-native (sm_100a) implementation of ZenDNN's LowOHA W8A8 hot path.

`zendnn_b200.capi` binds the C ABI of libb200dnn.so and raises ImportError when the library has
not been built (`python -m zendnn_b200.build`).  There is no CPU or PyTorch fallback.
"""
import importlib

__all__ = ["capi", "build"]


def __getattr__(name):
    if name in ("capi", "build", "lowoha"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
