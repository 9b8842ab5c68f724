"""optimi_b200 — the optimizer-step hot path of optimi as hand-written sm_100a CUDA kernels.

Drop-in for `optimi`'s optimizers: same classes, functional API, gradient release, optimizer
accumulation and checkpoint layout; the step itself runs as multi-tensor CUDA kernels from
liboptimi_b200.so (C ABI in include/optimi_b200.h).  CUDA tensors only — there is no CPU path.
"""

__version__ = "0.1.0"

from . import _lib  # noqa: F401  loads the kernel library; raises if it is missing and cannot be built
from .functional import adam, adamw, adan, lion, radam, ranger, sgd, stableadamw
from .gradientrelease import prepare_for_gradient_release, remove_gradient_release
from .optimizer import SGD, Adam, AdamW, Adan, Lion, OptimiOptimizer, RAdam, Ranger, StableAdamW
from .utils import param_groups_weight_decay, to_low_precision

__all__ = [
    "Adam", "AdamW", "Adan", "Lion", "RAdam", "Ranger", "SGD", "StableAdamW", "OptimiOptimizer",
    "adam", "adamw", "adan", "lion", "radam", "ranger", "sgd", "stableadamw",
    "prepare_for_gradient_release", "remove_gradient_release", "param_groups_weight_decay", "to_low_precision",
]  # fmt: skip
