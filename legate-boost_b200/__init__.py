"""B200-native tree-building kernels behind legate-boost's tree-model interface.

``Tree`` mirrors ``legateboost.models.Tree`` (same constructor, ``fit(X, g, h)``, ``predict``,
``batch_predict``); it drives hand-written sm_100a CUDA kernels through the C ABI declared in
``include/lbk.h`` (``liblbk.so``).  There is no CPU fallback: importing works anywhere, every
compute call needs the built library and a CUDA device.
"""
from . import library  # noqa: F401
from .tree import BaseModel, Sketch, Tree  # noqa: F401
from .estimator import LBClassifier, LBRegressor  # noqa: F401

__all__ = ["Tree", "BaseModel", "Sketch", "LBRegressor", "LBClassifier", "library"]
