"""``RansManager`` under the module name the reference reserves for it
(comp_inference/rans_manager.py is an empty file there; the class itself is
ccore.RansManager, src/python_bindings.cpp:222-471)."""
from .ccore import RansManager  # noqa: F401
