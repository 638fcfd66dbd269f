"""bluefog_b200: decentralized training for a single 8xB200 NVSwitch machine.

``import bluefog_b200.torch as bf`` gives the public API (same names as ``bluefog.torch``)."""
import torch as _torch  # noqa: F401  (loads libc10/libtorch, which the native extension ``_C`` links against)

__version__ = "0.1.0"


def _load_alternate_native():
    """BLUEFOG_B200_NATIVE=/path/to/_C*.so: use that build of the native module instead of the one beside this file
    (a ThreadSanitizer build of the host runtime, for instance; see the Makefile's ``tsan`` target)."""
    import importlib.util
    import os
    import sys
    path = os.environ.get("BLUEFOG_B200_NATIVE")
    if not path:
        return
    spec = importlib.util.spec_from_file_location("bluefog_b200._C", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["bluefog_b200._C"] = module
    spec.loader.exec_module(module)
    globals()["_C"] = module


_load_alternate_native()
