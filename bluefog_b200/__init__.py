"""bluefog_b200: decentralized training for a single 8xB200 NVSwitch machine.

``import bluefog_b200.torch as bf`` gives the public API (same names as ``bluefog.torch``)."""
import torch as _torch  # noqa: F401  (loads libc10/libtorch, which the native extension ``_C`` links against)

__version__ = "0.1.0"
