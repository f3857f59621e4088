"""etha_b200 — M-to-N DTensor redistribution for B200 (sm_100a) over NVLink 5 / NVSwitch.

Sub-packages are imported on first attribute access so that `import etha_b200.comm` does not pull in
the agent runtime (the reference imports everything eagerly, src/etha/__init__.py:1-8).
"""

import importlib

__all__ = ["comm", "tensor_bus", "kvstore", "ops", "parallel", "models", "utils"]
__version__ = "0.1.0"


def __getattr__(name):
    if name in __all__:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
