"""bluefog_b200: decentralized training for a single 8xB200 NVSwitch machine.

``import bluefog_b200.torch as bf`` gives the public API (same names as ``bluefog.torch``)."""
__version__ = "0.1.0"
